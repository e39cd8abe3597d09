// Split-K decode attention over the four-segment KV cache, one launch.
//
//   segments per (batch, kv-head):  INT4 prefix (64 B K + 64 B V + 2x fp16 scale
//   per token) | BF16 vertical-line tokens | BF16 staging | BF16 window
//
// Roofline: HBM-bound.  Algorithmic bytes per call
//   BH_KV * (132 * n_quant + 512 * (n_topk + n_staging + n_window)) + 512 * BH_Q.
//
// Work decomposition.  Each head's tokens are cut into ~4 KB "units" (32 INT4
// tokens, or 8 BF16 tokens), so units are balanced in BYTES across segment
// kinds.  A CTA (one per SM, 16 warps) owns a contiguous range of one head's
// units; its warps take units round-robin.  Every warp runs its own 3-slot ring:
// lane 0 issues 1-D bulk copies (TMA engine, mbarrier complete_tx) for the units
// ahead, the warp consumes the current one straight from shared memory.  No
// CTA-wide barrier is needed before or in the main loop: every warp reads the
// query fragments it needs straight from global memory.
//
// Math.  Scores are computed transposed, S^T = K Q^T, with tokens on the MMA M
// axis and the kv-group's query heads on the N axis (N = 8 per tile, so GQA
// ratios 4 and 8 fit one tile and 16 two tiles).  INT4 codes are expanded to
// fp16 in registers with the 0x6400 magic-number trick and fed to
// mma.sync.m16n8k16.f16.  For K the magic offset is NOT subtracted per element:
// the MMA sees 1032 + code (low nibbles) or 1152 + 16 code (high nibbles, with
// q/16 on the other operand) and the per-head constant 1032 sum(q_even) +
// 1152 sum(q_odd/16) is subtracted from the fp32 score, which removes half of
// the conversion instructions.  V codes reach the MMA as fp16 SUBNORMALS: the
// field (code + h) of an element, left where it is in the low 8 bits of a 16-bit
// lane, is the fp16 value (code + h) 2^-24 (bits 0-3), 2^-20 (bits 4-7) and so on,
// exactly, with no conversion arithmetic at all.  The small offset h (8 at 4 bits)
// is taken off once at the end as h * sum(p~), that sum coming from one extra MMA
// per 16 tokens against an all-ones operand; the power of two is a per-tile
// constant (tiles are built from fields of one position) applied at the end too,
// and the BF16 segments feed the same accumulators with P scaled by it.  The
// per-token K scale multiplies the fp32 score, the per-token V scale is folded
// into P before the PV product.
// BF16 segments use mma.sync bf16.  All segments share one online softmax in
// base 2 with a lazily updated reference maximum.  O^T = V^T P^T accumulates in
// fp32 registers.  Warps merge through shared memory, CTAs through a fp32
// workspace with an atomic ticket: the last CTA of a head does the
// log-sum-exp merge and writes the output, so there is no second launch.
#include "hq_decode_kernel.cuh"

namespace hq {

// ---- host side ---------------------------------------------------------------

// Tensor map of the code planes as {unit bytes (in 8-byte elements, so that a whole unit of up to 2 KB is one row of
// the box), units per plane, planes}, box {unit, 1, 2}, no swizzle.  The last few maps are kept (a cache's buffers change only when it grows), since encoding one costs about as much
// host time as the launch.
static int kv_tensor_map(CUtensorMap* out, const void* base, int row_bytes, int64_t plane_tokens, int64_t planes, int unit_tokens) {
  struct Entry { const void* base; int row; int64_t tokens, planes; int unit; CUtensorMap map; };
  constexpr int kKeep = 8;
  static thread_local Entry kept[kKeep];
  static thread_local int next = 0;
  for (int i = 0; i < kKeep; ++i)
    if (kept[i].base == base && kept[i].row == row_bytes && kept[i].tokens == plane_tokens && kept[i].planes == planes &&
        kept[i].unit == unit_tokens) { *out = kept[i].map; return HQ_OK; }
  tc::EncodeTiledFn fn = tc::encode_fn();
  HQ_REQUIRE(fn != nullptr, HQ_ERR_CUDA, "hq_decode_splitk: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t unit_bytes = (cuuint64_t)row_bytes * (cuuint64_t)unit_tokens;
  const cuuint64_t dims[3] = {unit_bytes / 8, (cuuint64_t)plane_tokens / (cuuint64_t)unit_tokens, (cuuint64_t)planes};
  const cuuint64_t strides[2] = {unit_bytes, (cuuint64_t)row_bytes * (cuuint64_t)plane_tokens};
  const cuuint32_t box[3] = {(cuuint32_t)(unit_bytes / 8), 1u, 2u};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HQ_REQUIRE(r == CUDA_SUCCESS, HQ_ERR_CUDA, "hq_decode_splitk: cuTensorMapEncodeTiled failed with %d (row %d, %lld tokens, %lld planes)",
             (int)r, row_bytes, (long long)plane_tokens, (long long)planes);
  kept[next] = Entry{base, row_bytes, plane_tokens, planes, unit_tokens, *out};
  next = (next + 1) % kKeep;
  return HQ_OK;
}

static int max_ctas() { return 4 * sm_count(); }

static int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

}  // namespace hq

extern "C" int hq_decode_workspace_bytes(int BH_KV, int kv_repeat, int64_t* bytes) {
  using namespace hq;
  HQ_REQUIRE(bytes && BH_KV > 0 && kv_repeat > 0 && kv_repeat <= 16, HQ_ERR_INVALID,
             "hq_decode_workspace_bytes: BH_KV>0 and 1<=kv_repeat<=16 required");
  const int64_t ctas = (int64_t)BH_KV + max_ctas();
  *bytes = kWsHeaderBytes + align_up((int64_t)BH_KV * 4, 256) + ctas * kv_repeat * (128 + 2) * 4 + 256;
  return HQ_OK;
}

extern "C" int hq_decode_splitk(const hq_decode_args* a, void* stream) {
  using namespace hq;
  HQ_REQUIRE(a != nullptr, HQ_ERR_INVALID, "hq_decode_splitk: null args");
  HQ_REQUIRE(a->struct_bytes == (int32_t)sizeof(hq_decode_args), HQ_ERR_INVALID,
             "hq_decode_splitk: struct_bytes %d != %d", a->struct_bytes, (int)sizeof(hq_decode_args));
  HQ_REQUIRE(a->head_dim == 128, HQ_ERR_UNSUPPORTED, "hq_decode_splitk: head_dim %d (only 128 is built)", a->head_dim);
  HQ_REQUIRE(a->kv_repeat >= 1 && a->kv_repeat <= 16, HQ_ERR_UNSUPPORTED,
             "hq_decode_splitk: kv_repeat %d outside 1..16", a->kv_repeat);
  HQ_REQUIRE(a->BH_KV >= 0 && a->n_quant >= 0 && a->n_topk >= 0 && a->n_staging >= 0 && a->n_window >= 0,
             HQ_ERR_INVALID, "hq_decode_splitk: negative size");
  if (a->BH_KV == 0) return HQ_OK;
  HQ_REQUIRE(a->q != nullptr, HQ_ERR_INVALID, "hq_decode_splitk: q is null");
  const bool partial = a->partial_acc != nullptr;
  HQ_REQUIRE(partial ? (a->partial_m && a->partial_l) : (a->out != nullptr), HQ_ERR_INVALID,
             "hq_decode_splitk: output pointer(s) missing");
  HQ_REQUIRE(a->out_dtype == HQ_BF16 || a->out_dtype == HQ_F16 || a->out_dtype == HQ_F32, HQ_ERR_UNSUPPORTED,
             "hq_decode_splitk: out_dtype %d", a->out_dtype);

  HQ_REQUIRE(((uintptr_t)a->q & 7) == 0 && a->q_stride % 4 == 0, HQ_ERR_ALIGNMENT,
             "hq_decode_splitk: q rows must be 8-byte aligned");
  const int k_bits = a->k_bits == 0 ? 4 : a->k_bits, v_bits = a->v_bits == 0 ? 4 : a->v_bits;
  HQ_REQUIRE((k_bits == 2 || k_bits == 4 || k_bits == 8) && (v_bits == 2 || v_bits == 4 || v_bits == 8), HQ_ERR_UNSUPPORTED,
             "hq_decode_splitk: bit widths must be 2, 4 or 8 (K%d V%d)", k_bits, v_bits);
  DecodeParams p{};
  p.q = (const __nv_bfloat16*)a->q; p.q_stride = a->q_stride;
  p.n_quant = a->n_quant;
  if (a->n_quant > 0) {
    HQ_REQUIRE(a->k_packed && a->v_packed && a->k_scale && a->v_scale, HQ_ERR_INVALID, "hq_decode_splitk: null quantised segment");
    HQ_REQUIRE(aligned16(a->k_packed) && aligned16(a->v_packed) && a->kp_stride_bh % 16 == 0 && a->vp_stride_bh % 16 == 0,
               HQ_ERR_ALIGNMENT, "hq_decode_splitk: packed K/V must be 16-byte aligned with 16-byte head strides");
  }
  p.k_packed = (const uint8_t*)a->k_packed; p.v_packed = (const uint8_t*)a->v_packed;
  p.kp_stride_bh = a->kp_stride_bh; p.vp_stride_bh = a->vp_stride_bh;
  p.k_scale = (const __half*)a->k_scale; p.v_scale = (const __half*)a->v_scale;
  p.ks_stride_bh = a->ks_stride_bh; p.vs_stride_bh = a->vs_stride_bh;
  const bool has_new = a->k_new != nullptr || a->v_new != nullptr;
  if (has_new) {
    HQ_REQUIRE(a->k_new && a->v_new && a->k_staging && a->v_staging && a->n_staging < HQ_GROUP_SIZE, HQ_ERR_INVALID,
               "hq_decode_splitk: a new token needs k_new, v_new, the staging buffers and a free staging slot");
    HQ_REQUIRE(aligned16(a->k_staging) && aligned16(a->v_staging) && a->kg_stride_bh % 8 == 0 && a->vg_stride_bh % 8 == 0,
               HQ_ERR_ALIGNMENT, "hq_decode_splitk: staging buffers must be 16-byte aligned");
  }
  const void* ks[4] = {a->k_topk, a->k_staging, a->k_window, a->k_new};
  const void* vs[4] = {a->v_topk, a->v_staging, a->v_window, a->v_new};
  const int64_t kst[4] = {a->kt_stride_bh, a->kg_stride_bh, a->kw_stride_bh, a->kn_stride};
  const int64_t vst[4] = {a->vt_stride_bh, a->vg_stride_bh, a->vw_stride_bh, a->vn_stride};
  const int ns[4] = {a->n_topk, a->n_staging, a->n_window, has_new ? 1 : 0};
  p.stage_k = (__nv_bfloat16*)a->k_staging; p.stage_v = (__nv_bfloat16*)a->v_staging;
  const int kUnitQ = unit_tokens(k_bits, v_bits);
  p.uq = (a->n_quant + kUnitQ - 1) / kUnitQ;
  p.units = p.uq;
  for (int s = 0; s < 4; ++s) {
    p.nseg[s] = ns[s];
    p.useg[s] = (ns[s] + kUnitB - 1) / kUnitB;
    p.units += p.useg[s];
    p.kseg[s] = (const __nv_bfloat16*)ks[s]; p.vseg[s] = (const __nv_bfloat16*)vs[s];
    p.kseg_stride[s] = kst[s]; p.vseg_stride[s] = vst[s];
    if (ns[s] > 0) {
      HQ_REQUIRE(ks[s] && vs[s], HQ_ERR_INVALID, "hq_decode_splitk: null BF16 segment %d", s);
      HQ_REQUIRE(aligned16(ks[s]) && aligned16(vs[s]) && kst[s] % 8 == 0 && vst[s] % 8 == 0, HQ_ERR_ALIGNMENT,
                 "hq_decode_splitk: BF16 segment %d must be 16-byte aligned with head strides multiple of 8", s);
    }
  }
  HQ_REQUIRE((a->flags & ~HQ_DECODE_OVERLAP_PREVIOUS) == 0, HQ_ERR_INVALID, "hq_decode_splitk: unknown flags 0x%x", a->flags);
  p.overlap = (a->flags & HQ_DECODE_OVERLAP_PREVIOUS) ? 1 : 0;
  p.R = a->kv_repeat;
  p.out_dtype = a->out_dtype;
  p.sml = a->sm_scale * 1.44269504f;
  p.out = a->out; p.out_stride = a->out_stride;
  p.pm = a->partial_m; p.pl = a->partial_l; p.pacc = a->partial_acc;
  p.lengths = a->lengths;
  p.rope_cos = (const __nv_bfloat16*)a->rope_cos; p.rope_sin = (const __nv_bfloat16*)a->rope_sin;
  p.rope_stride = a->rope_stride; p.heads_per_batch = a->rope_heads_per_batch > 0 ? a->rope_heads_per_batch : 1;
  HQ_REQUIRE((a->rope_cos == nullptr) == (a->rope_sin == nullptr), HQ_ERR_INVALID, "hq_decode_splitk: rope_cos and rope_sin go together");
  if (a->rope_cos != nullptr) {
    HQ_REQUIRE(aligned16(a->rope_cos) && aligned16(a->rope_sin) && a->rope_stride % 8 == 0 && a->rope_heads_per_batch > 0 &&
                   a->BH_KV % a->rope_heads_per_batch == 0, HQ_ERR_INVALID,
               "hq_decode_splitk: rotary factors must be 16-byte aligned rows, rope_heads_per_batch must divide BH_KV");
  }
  HQ_REQUIRE(a->lengths == nullptr || (((uintptr_t)a->lengths & 3) == 0 && a->k_staging && a->v_staging), HQ_ERR_INVALID,
             "hq_decode_splitk: lengths must be 4-byte aligned and needs the staging buffers");
  p.peer.world = 0;
  if (a->peer_world > 1) {
    HQ_REQUIRE(!partial && a->out != nullptr, HQ_ERR_INVALID, "hq_decode_splitk: a peer exchange writes the merged result to out");
    HQ_REQUIRE(a->peer_world <= kPeerMaxWorld && a->peer_rank >= 0 && a->peer_rank < a->peer_world && a->peer_bufs != nullptr &&
                   a->peer_seq != 0, HQ_ERR_INVALID, "hq_decode_splitk: peer_world %d peer_rank %d (seq starts at 1)",
               a->peer_world, a->peer_rank);
    for (int j = 0; j < a->peer_world; ++j) {
      HQ_REQUIRE(a->peer_bufs[j] != nullptr && ((uintptr_t)a->peer_bufs[j] & 255) == 0, HQ_ERR_ALIGNMENT,
                 "hq_decode_splitk: peer buffer %d null or not 256-byte aligned", j);
      p.peer.bufs[j] = (uint8_t*)a->peer_bufs[j];
    }
    p.peer.world = a->peer_world; p.peer.rank = a->peer_rank; p.peer.seq = a->peer_seq;
    p.peer.rows = a->BH_KV * a->kv_repeat;
    p.peer.timeout_ns = a->peer_timeout_ns > 0 ? a->peer_timeout_ns : 2000000000ll;
  }

  // splits: one wave of blocks, one per SM, about one unit per warp at least; the blocks' partials live in the
  // workspace (sized for BH + 4 x SMs blocks), the merge of a head's splits needs no staging memory
  const int sms = sm_count();
  const int NT = a->kv_repeat <= 8 ? 1 : 2;
  const int kWarps = warps_of(NT);
  const int split_cap = (int)(((int64_t)a->BH_KV + max_ctas()) / a->BH_KV);
  bool force_direct_scales = false, force_split_kv = false;
  int nsplit = a->num_splits;
  int last_share = 256;
  int cluster = 1;                 // candidate cluster size (checked against the device below)
  if (nsplit <= 0) {
    const int by_grid = sms / a->BH_KV;
    const int by_work = (p.units + kWarps - 1) / kWarps;
    nsplit = by_grid < by_work ? by_grid : by_work;
    if (nsplit > split_cap) nsplit = split_cap;
    // A head's splits as one thread-block cluster (at most 8 blocks) merge through distributed shared memory, which
    // saves the partial store, the ticket and the last block's merge: taken when the plain plan has no more splits
    // than a cluster has blocks (short prefixes, or enough heads).
    // Not in partial mode: a sequence shard's state is bit for bit what the exchanging kernel sends, in either form.
    // A short prefix is better off with eight blocks of half-empty warps than with four full ones (1K: 5.8 against
    // 6.4 us), and even cluster sizes measured better than odd ones.
    if (nsplit <= 8 && p.peer.world <= 1 && !partial) {
      int c = by_grid < 8 ? by_grid : 8;
      if (c > p.units) c = p.units;
      if (c > split_cap) c = split_cap;
      if (c > 2 && (c & 1)) --c;
      if (c >= 2) cluster = c;
    }
    // SMs left over by an even split (sms - BH * nsplit) take one more, small split of every head: a fraction
    // 0.8 * spare / sms of the head (the 0.8 pays for the fixed cost of the extra blocks), if that is worth a block
    const int spare = sms - a->BH_KV * nsplit;
    if (nsplit >= 1 && nsplit == by_grid && nsplit + 1 <= split_cap && spare * 16 >= sms) {
      const double f = 0.8 * spare / sms;
      if (f * p.units >= 4.0 * kWarps) {
        last_share = (int)(f * nsplit * 256.0 / (1.0 - f) + 0.5);
        nsplit += 1;
      }
    }
  }
#ifdef HQ_DEC_FAST_BUILD
  if (const char* e = getenv("HQ_DEC_NSPLIT")) nsplit = atoi(e);
  if (getenv("HQ_DEC_NOSCALETMA")) force_direct_scales = true;
  if (getenv("HQ_DEC_SPLITKV")) force_split_kv = true;
#endif
  if (nsplit < 1) nsplit = 1;
  if (nsplit > p.units && p.units > 0) nsplit = p.units;
  if (nsplit > split_cap) nsplit = split_cap;
  if (nsplit < 1) nsplit = 1;
  p.nsplit = nsplit;
  p.BH = a->BH_KV;
  p.last_share = last_share;
  p.cluster = 1;
#ifdef HQ_DEC_FAST_BUILD
  if (const char* e = getenv("HQ_DEC_LAST")) p.last_share = atoi(e);
#endif
  int64_t need = 0;
  hq_decode_workspace_bytes(a->BH_KV, a->kv_repeat, &need);
  HQ_REQUIRE(a->workspace && a->workspace_bytes >= need, HQ_ERR_WORKSPACE,
             "hq_decode_splitk: workspace of %lld bytes needed, %lld given", (long long)need, (long long)a->workspace_bytes);
  HQ_REQUIRE(((uintptr_t)a->workspace & 255) == 0, HQ_ERR_ALIGNMENT, "hq_decode_splitk: workspace must be 256-byte aligned");
  uint8_t* ws = (uint8_t*)a->workspace;
  p.status = (int*)ws;
  p.counters = (int*)(ws + kWsHeaderBytes);
  float* f = (float*)(ws + kWsHeaderBytes + align_up((int64_t)a->BH_KV * 4, 256));
  const int64_t rows = (int64_t)a->BH_KV * nsplit * a->kv_repeat;
  p.ws_m = f; p.ws_l = f + rows; p.ws_acc = f + 2 * rows;
  // keep ws_acc 16-byte aligned
  p.ws_acc = (float*)(((uintptr_t)p.ws_acc + 15) & ~(uintptr_t)15);

  // scales can ride in the bulk copies when every 32-token group of a row starts on a
  // 16-byte boundary and a row has room for the round-up of its tail to 8 tokens
  const int64_t nq8 = ((int64_t)a->n_quant + 7) & ~(int64_t)7;
  p.scale_tma = !force_direct_scales && a->n_quant > 0 && aligned16(a->k_scale) && aligned16(a->v_scale) && a->ks_stride_bh % 8 == 0 &&
                a->vs_stride_bh % 8 == 0 && a->ks_stride_bh >= nq8 && a->vs_stride_bh >= nq8;
  // K and V codes as two planes of one tensor (what DStageLayerCache allocates when K and V have the same width):
  // v_packed lies one plane after k_packed and a head is two planes.  Then a unit's codes are one box of a 3-D
  // tensor map {row bytes, tokens of a plane, 2 * BH planes}.
  CUtensorMap kv_map;
  memset(&kv_map, 0, sizeof(kv_map));
  p.kv_fused = 0;
  if (k_bits == v_bits && a->n_quant >= kUnitQ && p.peer.world <= 1 && !force_split_kv) {
    const int64_t row = 16 * k_bits;
    const int64_t plane = (const uint8_t*)a->v_packed - (const uint8_t*)a->k_packed;
    if (plane > 0 && plane % row == 0 && plane % 16 == 0 && a->kp_stride_bh == 2 * plane && a->vp_stride_bh == 2 * plane &&
        plane / row >= a->n_quant && plane / row < (1ll << 31) && (kUnitQ * row) % 16 == 0 && kUnitQ * row <= 2048) {
      const int rm = kv_tensor_map(&kv_map, a->k_packed, (int)row, plane / row, 2 * (int64_t)a->BH_KV, kUnitQ);
      if (rm != HQ_OK) return rm;
      p.kv_fused = 1;
    }
  }
  cudaStream_t st = (cudaStream_t)stream;
  auto dispatch = [&](const DecodeParams& pp, dim3 grid, int* clusters_out) -> int {
    const DecodeParams& p = pp;
#ifdef HQ_DEC_FAST_BUILD      // development builds: the K4/V4 instantiations only
    HQ_REQUIRE(k_bits == 4 && v_bits == 4 && p.peer.world <= 1, HQ_ERR_UNSUPPORTED, "hq_decode_splitk: development build (K4/V4, no peers)");
    if (p.cluster > 1) {
      if (!p.scale_tma) { if (clusters_out) *clusters_out = 0; return clusters_out ? HQ_OK : HQ_ERR_INVALID; }
      return NT == 1 ? launch_decode<1, true, 4, 4, 2>(p, kv_map, grid, st, clusters_out) : launch_decode<2, true, 4, 4, 2>(p, kv_map, grid, st, clusters_out);
    }
    if (NT == 1) return p.scale_tma ? launch_decode<1, true, 4, 4, 0>(p, kv_map, grid, st, clusters_out) : launch_decode<1, false, 4, 4, 0>(p, kv_map, grid, st, clusters_out);
    return p.scale_tma ? launch_decode<2, true, 4, 4, 0>(p, kv_map, grid, st, clusters_out) : launch_decode<2, false, 4, 4, 0>(p, kv_map, grid, st, clusters_out);
#else
    switch (k_bits * 16 + v_bits) {
      case 0x44: return launch_decode_k4v4(p, kv_map, NT, grid, st, clusters_out);
      case 0x88: return launch_decode_k8v8(p, kv_map, NT, grid, st, clusters_out);
      case 0x84: return launch_decode_k8v4(p, kv_map, NT, grid, st, clusters_out);
      case 0x82: return launch_decode_k8v2(p, kv_map, NT, grid, st, clusters_out);
      case 0x48: return launch_decode_k4v8(p, kv_map, NT, grid, st, clusters_out);
      case 0x42: return launch_decode_k4v2(p, kv_map, NT, grid, st, clusters_out);
      case 0x28: return launch_decode_k2v8(p, kv_map, NT, grid, st, clusters_out);
      case 0x24: return launch_decode_k2v4(p, kv_map, NT, grid, st, clusters_out);
      default: return launch_decode_k2v2(p, kv_map, NT, grid, st, clusters_out);
    }
#endif
  };
#ifdef HQ_DEC_FAST_BUILD
  if (const char* e = getenv("HQ_DEC_CLUSTER")) cluster = atoi(e);
#endif
  if (cluster > 1 && cluster <= p.units) {
    // the device must hold every head's cluster at once (one block per SM, clusters do not span GPCs)
    DecodeParams pc = p;
    pc.cluster = cluster;
    pc.nsplit = cluster;
    pc.last_share = 256;
    int held = 0;
    const int rq = dispatch(pc, dim3((unsigned)(a->BH_KV * cluster)), &held);
    if (rq != HQ_OK) return rq;
    if (held >= a->BH_KV) return dispatch(pc, dim3((unsigned)(a->BH_KV * cluster)), nullptr);
  }
  return dispatch(p, dim3((unsigned)(a->BH_KV * nsplit)), nullptr);
}

// ---- decode without caller-provided scratch -----------------------------------------------
namespace hq {
constexpr int64_t kStaticScratchBytes = 4 << 20;     // 4 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];
}  // namespace hq

// Same computation as hq_decode_splitk, for callers that cannot hand over device memory of
// their own (a plugin host that forbids cudaMalloc in its callbacks, a process whose memory
// pool is owned by another runtime): the split-K partials and tickets live in a fixed 4 MiB
// array inside the library image.  `workspace` / `workspace_bytes` of the argument block are
// ignored.  The first call on each device looks up the array's device address (with that
// device current); make that first call outside any stream capture.  Every call shares the one
// array, so two calls that may overlap on the GPU (different streams, or different host threads
// without ordering between their streams) race; keep them in one stream.  The ticket words are
// cleared in-stream before each launch; the status word (bit 0: a bounded wait ran out) is NOT,
// so it accumulates over calls until hq_decode_static_status reads and clears it.  A shape whose
// scratch need exceeds 4 MiB is rejected with HQ_ERR_WORKSPACE.  No cudaMalloc / cudaFree or
// allocating library call is made.
namespace hq {
// Device address of the array on the current device.  The table is filled without locking: two threads
// that race here both store the same address, which the runtime returns for the lifetime of the context.
static int static_scratch(void** out) {
  constexpr int kMaxDev = 64;
  static void* dev_ptr[kMaxDev] = {nullptr};
  int dev = 0;
  HQ_CUDA(cudaGetDevice(&dev));
  HQ_REQUIRE(dev >= 0 && dev < kMaxDev, HQ_ERR_UNSUPPORTED, "hq_decode_splitk_static: device index %d", dev);
  if (dev_ptr[dev] == nullptr) {
    void* p = nullptr;
    HQ_CUDA(cudaGetSymbolAddress(&p, g_decode_scratch));   // the host-side name is not a device address
    HQ_REQUIRE(p != nullptr, HQ_ERR_CUDA, "hq_decode_splitk_static: no device address for the scratch array");
    dev_ptr[dev] = p;
  }
  *out = dev_ptr[dev];
  return HQ_OK;
}
}  // namespace hq

extern "C" int hq_decode_splitk_static(const hq_decode_args* a, void* stream) {
  using namespace hq;
  HQ_REQUIRE(a != nullptr, HQ_ERR_INVALID, "hq_decode_splitk_static: null args");
  HQ_REQUIRE(a->struct_bytes == (int32_t)sizeof(hq_decode_args), HQ_ERR_INVALID,
             "hq_decode_splitk_static: struct_bytes %d != %d", a->struct_bytes, (int)sizeof(hq_decode_args));
  HQ_REQUIRE((a->flags & ~HQ_DECODE_OVERLAP_PREVIOUS) == 0, HQ_ERR_INVALID, "hq_decode_splitk_static: unknown flags 0x%x", a->flags);
  if (a->BH_KV == 0) return HQ_OK;
  int64_t need = 0;
  const int rc = hq_decode_workspace_bytes(a->BH_KV, a->kv_repeat, &need);
  if (rc != HQ_OK) return rc;
  HQ_REQUIRE(need <= kStaticScratchBytes, HQ_ERR_WORKSPACE,
             "hq_decode_splitk_static: this shape needs %lld bytes of scratch, the built-in array holds %lld; "
             "use hq_decode_splitk with a caller workspace", (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  const int rs = static_scratch(&scratch);
  if (rs != HQ_OK) return rs;
  // the tickets (one word per head, after the header that holds the status word) must start at zero
  HQ_CUDA(cudaMemsetAsync((uint8_t*)scratch + kWsHeaderBytes, 0, (size_t)align_up((int64_t)a->BH_KV * 4, 256), (cudaStream_t)stream));
  hq_decode_args b = *a;
  b.flags = 0;                       // the kernel's predecessor in the stream is the memset above
  b.workspace = scratch;
  b.workspace_bytes = kStaticScratchBytes;
  return hq_decode_splitk(&b, stream);
}

// Synchronising read-and-clear of the status word of the built-in scratch array on the current device
// (0 = every bounded wait of the hq_decode_splitk_static calls since the last read completed; bit 0 = one ran
// out, and the output of that call is not valid).
extern "C" int hq_decode_static_status(int* status) {
  using namespace hq;
  HQ_REQUIRE(status != nullptr, HQ_ERR_INVALID, "hq_decode_static_status: null pointer");
  void* scratch = nullptr;
  const int rs = static_scratch(&scratch);
  if (rs != HQ_OK) return rs;
  HQ_CUDA(cudaMemcpy(status, scratch, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) HQ_CUDA(cudaMemset(scratch, 0, sizeof(int)));
  return HQ_OK;
}

