// The split-K decode kernel and its launch: included by hq_decode.cu (the entry points) and by the files that
// instantiate it for the (K bits, V bits) pairs, hq_decode_k8.cu, hq_decode_k4.cu and hq_decode_k2.cu - one kernel
// source, compiled side by side.  The design is described at the top of hq_decode.cu.
#pragma once
#include <stdlib.h>

#include "hq_common.cuh"
#include "hq_peer.cuh"
#include "hq_tc05.cuh"      // the tensor-map encoder
#include <string.h>

namespace hq {

// One CTA per SM.  Warps per CTA: 16 with one n8 tile of query heads (GQA ratio <= 8; 128 registers per thread fill
// the register file), 12 with two tiles (ratios 9..16: 32 fp32 accumulators more per thread, <= 168 registers).  Half
// as many CTAs as two per SM would give means half as many split-K partials to merge per head.
#ifndef HQ_DEC_WARPS1
#define HQ_DEC_WARPS1 16
#endif
#ifndef HQ_DEC_WARPS2
#define HQ_DEC_WARPS2 12
#endif
__host__ __device__ constexpr int warps_of(int NT) { return NT == 2 ? HQ_DEC_WARPS2 : HQ_DEC_WARPS1; }
constexpr int kSlots = 3;
constexpr int kScaleLanes = 8;            // lanes of a warp that fetch a unit's scales (16 bytes each)
// quantised tokens per unit: 32, or 16 when 32 rows of K and V codes would not fit the 4 KB of a BF16 unit (every pair
// with an 8-bit side), so that every pair keeps a 4224-byte slot and two CTAs per SM
__host__ __device__ constexpr int unit_tokens(int kb, int vb) { return 32 * 16 * (kb + vb) > 4096 ? 16 : 32; }
constexpr int kUnitB = 8;                 // BF16 tokens per unit
constexpr float kLazyRescale = 4.0f;      // rescale only if the max grows by > 2^4
constexpr int kWsHeaderBytes = 256;       // [0] status word
// Between the main loop and the final stores every 128-channel row (warp merge area, split-K partials in the workspace,
// the last block's sums) is kept in POSITION order: channel 16 g + c sits at position 8 c + g.  The 8 lanes g of an MMA
// row group then write 8 consecutive words (rows padded to 132 words keep the two head pairs of a warp apart), where
// channel order put them 16 words apart, on two banks.  Channel order comes back at the stores that leave the kernel.
constexpr int kMrgStride = 132;
__host__ __device__ constexpr int chan_of_pos(int pos) { return 16 * (pos & 7) + (pos >> 3); }

struct DecodeParams {
  const __nv_bfloat16* q; int64_t q_stride;
  const uint8_t* k_packed; const uint8_t* v_packed; int64_t kp_stride_bh, vp_stride_bh;
  const __half* k_scale; const __half* v_scale; int64_t ks_stride_bh, vs_stride_bh;
  const __nv_bfloat16* kseg[4]; const __nv_bfloat16* vseg[4]; int64_t kseg_stride[4], vseg_stride[4];
  int nseg[4];                            // tokens in topk / staging / window / the step's new token (0 or 1)
  int n_quant;
  int uq;                                 // INT4 units
  int useg[4];                            // BF16 units per segment
  int units;                              // total units per head
  int nsplit;
  int BH;                                 // heads of the call (grid = BH * nsplit blocks, split-major)
  int last_share;                         // share of a head's last split in 1/256 of an even share
  int cluster;                            // > 1: the nsplit (= cluster) blocks of a head are one thread-block cluster
  int R;                                  // kv_repeat
  int out_dtype;
  float sml;                              // sm_scale * log2(e)
  void* out; int64_t out_stride;
  float* pm; float* pl; float* pacc;      // partial mode outputs (or null)
  PeerGroup peer;                         // peer.world > 1: exchange the state with the other sequence shards and merge
  __nv_bfloat16* stage_k; __nv_bfloat16* stage_v;   // staging buffers, written only when the call carries a new token
  int scale_tma;                          // scales ride in the bulk copies (aligned rows) or are loaded directly
  int kv_fused;                           // K and V codes of a head are two planes of one tensor: one request per unit
  int overlap;                            // launched with programmatic stream serialisation
  const int* lengths;                     // device {n_quant, n_staging} overriding the values above (or null)
  const __nv_bfloat16* rope_cos; const __nv_bfloat16* rope_sin;   // [batch, 128] rotary factors of the step (or null)
  int64_t rope_stride; int heads_per_batch;
  int* status; int* counters;             // workspace
  float* ws_m; float* ws_l; float* ws_acc;
};

// Shared-memory slot of one unit for a (K bits, V bits) pair.  Quantised unit: 32 token rows of K codes, then 32
// rows of V codes, then (past the larger of that and a BF16 unit) 32 fp16 K scales and 32 fp16 V scales.  BF16 unit:
// 8 K rows at 0, 8 V rows at 2048.  K4/V4: K 2048 | V 2048 | k_scale 64 | v_scale 64 = 4224 bytes.
template <int KB, int VB>
struct Fmt {
  static constexpr int kRowK = 16 * KB, kRowV = 16 * VB;                  // bytes per token row (128 channels)
  static constexpr int kUnitQ = unit_tokens(KB, VB), kChunks = kUnitQ / 16;   // 16-token MMA chunks per unit
  static constexpr int kQuant = kUnitQ * (kRowK + kRowV);
  static constexpr int kData = kQuant > 4096 ? kQuant : 4096;
  static constexpr int kVOff = kUnitQ * kRowK;
  static constexpr int kSlot = kData + 128;
};

// How the V codes of a (bit width) reach the P V product as fp16 subnormals, and which channel lands where.
// This lane handles channels 16 g .. 16 g + 15 (g = lane / 4) of the tokens of its MMA k-slots.  Output tile mt
// (0..7) has two rows per lane (MMA rows g and g + 8); tile mt, row r holds local channel chan(mt, r), every element
// of the tile carries the factor 2^-exp2(mt) and the code offset kOff:
//   8 bits: byte + 128 in bits 0-7            -> one factor; tile mt = channels 2 mt, 2 mt + 1
//   4 bits: (nibble ^ 8) in bits 0-3 / 4-7    -> tile 2 p + b: nibble b and nibble b + 2 of 16-bit group p
//   2 bits: (field ^ 2) in bits 2 f, 2 f + 1  -> tile 4 hl + f: field f of the low and of the high byte of group hl
template <int VB> struct VFmt;
template <> struct VFmt<8> {
  static constexpr float kOff = 128.f;
  static constexpr int kScales = 1;
  __host__ __device__ static constexpr int exp2(int) { return 24; }
  __host__ __device__ static constexpr int chan(int mt, int r) { return 2 * mt + r; }
  __host__ __device__ static constexpr int scale_idx(int) { return 0; }
};
template <> struct VFmt<4> {
  static constexpr float kOff = 8.f;
  static constexpr int kScales = 2;
  __host__ __device__ static constexpr int exp2(int mt) { return (mt & 1) ? 20 : 24; }
  __host__ __device__ static constexpr int chan(int mt, int r) { return 4 * (mt >> 1) + 2 * r + (mt & 1); }
  __host__ __device__ static constexpr int scale_idx(int mt) { return mt & 1; }
};
template <> struct VFmt<2> {
  static constexpr float kOff = 2.f;
  static constexpr int kScales = 4;
  __host__ __device__ static constexpr int exp2(int mt) { return 24 - 2 * (mt & 3); }
  __host__ __device__ static constexpr int chan(int mt, int r) { return 8 * (mt >> 2) + 4 * r + (mt & 3); }
  __host__ __device__ static constexpr int scale_idx(int mt) { return mt & 3; }
};

struct Unit {
  const uint8_t* k; const uint8_t* v;
  int kind;       // 0 = quantised, 1 = BF16
  int ntok;       // valid tokens
  int tok0;       // first token within its segment
  int seg;        // BF16 units: 0 vertical lines, 1 staging, 2 window, 3 the step's new token
};

// The lengths that change from step to step.  They come with the launch (host values) or, when the call names a device
// record, from there: a launch captured in a CUDA graph then stays valid while the cache grows.
struct Lens {
  int n_quant, n_stg;     // quantised prefix tokens, live staging tokens
  int uq, useg1, units;   // quantised units, staging units, all units of a head
  int uq_stable;          // quantised units that the kernel just before this one cannot have written
};

template <int KB, int VB>
__device__ __forceinline__ Unit unit_of(const DecodeParams& p, const Lens& L, int head, int u) {
  Unit r;
  if (u < L.uq) {
    constexpr int kUnitQ = Fmt<KB, VB>::kUnitQ;
    r.kind = 0; r.seg = -1; r.tok0 = u * kUnitQ; r.ntok = min(kUnitQ, L.n_quant - r.tok0);
    r.k = p.k_packed + head * p.kp_stride_bh + (int64_t)r.tok0 * Fmt<KB, VB>::kRowK;
    r.v = p.v_packed + head * p.vp_stride_bh + (int64_t)r.tok0 * Fmt<KB, VB>::kRowV;
    return r;
  }
  u -= L.uq;
  int s = 0;
  if (u >= p.useg[0]) {
    u -= p.useg[0]; s = 1;
    if (u >= L.useg1) { u -= L.useg1; s = 2; if (u >= p.useg[2]) { u -= p.useg[2]; s = 3; } }
  }
  r.kind = 1; r.seg = s; r.tok0 = u * kUnitB; r.ntok = min(kUnitB, (s == 1 ? L.n_stg : p.nseg[s]) - r.tok0);
  r.k = reinterpret_cast<const uint8_t*>(p.kseg[s] + head * p.kseg_stride[s] + (int64_t)r.tok0 * 128);
  r.v = reinterpret_cast<const uint8_t*>(p.vseg[s] + head * p.vseg_stride[s] + (int64_t)r.tok0 * 128);
  return r;
}

// ---- register-level helpers -------------------------------------------------

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Each 16-bit lane of w carries four two's-complement nibbles.  Result k is the
// fp16x2 (lane_lo nibble k, lane_hi nibble k) with the exact integer values.
__device__ __forceinline__ void cvt_nibbles_f16(uint32_t w, uint32_t (&h)[4]) {
  const uint32_t w8 = w >> 8;
  const __half2 c1032 = u32_as_h2(0x64086408u);
  const __half2 c16th = u32_as_h2(0x2C002C00u);     // 1/16
  const __half2 cm72 = u32_as_h2(0xD480D480u);      // -72
  h[0] = h2_as_u32(__hsub2(u32_as_h2(lop3_and_xor(w, 0x000F000Fu, 0x64086408u)), c1032));
  h[1] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_xor(w, 0x00F000F0u, 0x64806480u)), c16th, cm72));
  h[2] = h2_as_u32(__hsub2(u32_as_h2(lop3_and_xor(w8, 0x000F000Fu, 0x64086408u)), c1032));
  h[3] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_xor(w8, 0x00F000F0u, 0x64806480u)), c16th, cm72));
}

// Same lanes, without removing the magic offset: result k holds 1032 + code for
// k = 0, 2 (low nibbles) and 1152 + 16 code for k = 1, 3 (high nibbles).
__device__ __forceinline__ void cvt_nibbles_biased(uint32_t w, uint32_t (&h)[4]) {
  const uint32_t w8 = w >> 8;
  h[0] = lop3_and_xor(w, 0x000F000Fu, 0x64086408u);
  h[1] = lop3_and_xor(w, 0x00F000F0u, 0x64806480u);
  h[2] = lop3_and_xor(w8, 0x000F000Fu, 0x64086408u);
  h[3] = lop3_and_xor(w8, 0x00F000F0u, 0x64806480u);
}

// Byte b of `wa` and of `wb` (two's-complement codes of two tokens) -> result b = fp16x2 (code of wa, code of wb), exact.
__device__ __forceinline__ void cvt_byte_pairs_f16(uint32_t wa, uint32_t wb, uint32_t (&h)[4]) {
  const uint32_t m01 = prmt(wa, wb, 0x5140u) ^ 0x80808080u;    // a0 b0 a1 b1, each + 128
  const uint32_t m23 = prmt(wa, wb, 0x7362u) ^ 0x80808080u;    // a2 b2 a3 b3
  const __half2 c1152 = u32_as_h2(0x64806480u);
  h[0] = h2_as_u32(__hsub2(u32_as_h2(prmt(m01, 0x64646464u, 0x4140u)), c1152));
  h[1] = h2_as_u32(__hsub2(u32_as_h2(prmt(m01, 0x64646464u, 0x4342u)), c1152));
  h[2] = h2_as_u32(__hsub2(u32_as_h2(prmt(m23, 0x64646464u, 0x4140u)), c1152));
  h[3] = h2_as_u32(__hsub2(u32_as_h2(prmt(m23, 0x64646464u, 0x4342u)), c1152));
}

// Each 16-bit lane of w carries 2-bit two's-complement codes in its low byte (fields f = 0..3 at bits 2f, 2f+1).
// Result f is the fp16x2 (lane_lo field f, lane_hi field f) as 1024 + 4^f (2 + code): the magic offset stays in.
__device__ __forceinline__ void cvt_crumbs_biased(uint32_t w, uint32_t (&h)[4]) {
  h[0] = lop3_and_xor(w, 0x00030003u, 0x64026402u);
  h[1] = lop3_and_xor(w, 0x000C000Cu, 0x64086408u);
  h[2] = lop3_and_xor(w, 0x00300030u, 0x64206420u);
  h[3] = lop3_and_xor(w, 0x00C000C0u, 0x64806480u);
}
// Same fields with the exact integer values.
__device__ __forceinline__ void cvt_crumbs_f16(uint32_t w, uint32_t (&h)[4]) {
  uint32_t b[4];
  cvt_crumbs_biased(w, b);
  h[0] = h2_as_u32(__hsub2(u32_as_h2(b[0]), u32_as_h2(0x64026402u)));                               // - 1026
  h[1] = h2_as_u32(__hfma2(u32_as_h2(b[1]), u32_as_h2(0x34003400u), u32_as_h2(0xDC08DC08u)));       // / 4 - 258
  h[2] = h2_as_u32(__hfma2(u32_as_h2(b[2]), u32_as_h2(0x2C002C00u), u32_as_h2(0xD420D420u)));       // / 16 - 66
  h[3] = h2_as_u32(__hfma2(u32_as_h2(b[3]), u32_as_h2(0x24002400u), u32_as_h2(0xCC80CC80u)));       // / 64 - 18
}

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return h2_as_u32(h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float group_max(float v) {   // over the 8 lanes sharing lane%4
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
  return v;
}
__device__ __forceinline__ float group_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

// Online-softmax bookkeeping shared by both unit kinds.  `mx` is the group-wide
// maximum of the new scores for this thread's two heads of tile nt.
template <int NT>
__device__ __forceinline__ void lazy_rescale(const float (&mx)[NT][2], float (&m_ref)[NT][2], float (&l_part)[NT][2],
                                             float (&O)[NT][8][4], float (&Lt)[NT][4]) {
  bool need = false;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < 2; ++j) need |= (mx[nt][j] > m_ref[nt][j] + kLazyRescale);
  if (__any_sync(0xffffffffu, need)) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float nm = fmaxf(m_ref[nt][j], mx[nt][j]);
        const float alpha = (nm == -INFINITY) ? 1.0f : ex2f(m_ref[nt][j] - nm);   // m_ref=-inf -> 0
        m_ref[nt][j] = nm;
        l_part[nt][j] *= alpha;
        Lt[nt][j] *= alpha; Lt[nt][2 + j] *= alpha;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) { O[nt][mt][j] *= alpha; O[nt][mt][2 + j] *= alpha; }
      }
  }
}

// Sequence-sharded call: channel d of query row `row` of this shard's un-normalised state goes to every peer, the
// peers' arrive in this rank's exchange buffer, and the merged, normalised value is the output.
// The rows of a thread are handled in two passes - first every row is sent, then every row is awaited - so that the
// one-way NVLink latency is paid once per call and not once per row.
__device__ __forceinline__ void peer_send(const DecodeParams& p, int row, int d, float m, float l, float acc) {
  const PeerLayout L = peer_layout(p.peer.world, p.peer.rows);
  peer_push(p.peer, L, 2 * (int64_t)p.peer.rows + (int64_t)row * 128 + d, acc);
  if (d == 0) { peer_push(p.peer, L, row, m); peer_push(p.peer, L, p.peer.rows + row, l); }
}
// Floats of shared-memory scratch peer_receive_all needs for `world` ranks and R query heads per kv head.
__host__ __device__ constexpr int peer_scratch_floats(int world, int R) { return 3 * (world - 1) * R + 3 * R + R * 128; }

// Second pass for the R rows of kv-head `head`, by the whole CTA: (1) the peers' m and l words are polled by all threads
// in parallel into shared memory, (2) one thread per row turns them into merge weights and the denominator, (3) every
// thread keeps sixteen acc loads in flight over its (row, peer) pairs and accumulates into its own shared-memory
// cells.  `local(hd, d, m, l, acc)` recomputes this rank's values of row hd at POSITION d (channel chan_of_pos(d)): rows are
// held in position order inside the kernel, the exchange buffers are in channel order.
template <int kThreads, class LocalFn>
__device__ __forceinline__ void peer_receive_all(const DecodeParams& p, float* sm, int head, int tid, LocalFn local) {
  const PeerGroup& g = p.peer;
  const PeerLayout L = peer_layout(g.world, g.rows);
  const int R = p.R, np = g.world - 1;
  float* s_m = sm; float* s_l = s_m + np * R; float* s_w = s_l + np * R;
  float* s_M = s_w + np * R; float* s_den = s_M + R; float* s_w0 = s_den + R; float* s_acc = s_w0 + R;
  const uint2* recv = reinterpret_cast<const uint2*>(g.bufs[g.rank] + L.recv_off) + (int64_t)(g.seq & 1u) * g.world * L.msg;
  const int64_t row0 = (int64_t)head * R;
  bool expired = false;
  for (int idx = tid; idx < np * R * 2; idx += kThreads) {
    const int jj = idx / (2 * R), rem = idx - jj * 2 * R, which = rem >= R ? 1 : 0, row = rem - which * R;
    const int j = jj < g.rank ? jj : jj + 1;
    const float v = wait_pair(recv + j * L.msg + (int64_t)which * g.rows + row0 + row, g.seq, g.timeout_ns, &expired);
    (which ? s_l : s_m)[jj * R + row] = v;
  }
  __syncthreads();
  if (tid < R) {
    float m, l, a;
    local(tid, 0, m, l, a);
    float M = m;
    for (int jj = 0; jj < np; ++jj) M = fmaxf(M, s_m[jj * R + tid]);
    const float w0 = (m == -INFINITY) ? 0.f : ex2f(m - M);
    float den = w0 * l;
    for (int jj = 0; jj < np; ++jj) {
      const float mj = s_m[jj * R + tid];
      const float w = (mj == -INFINITY) ? 0.f : ex2f(mj - M);
      s_w[jj * R + tid] = w;
      den += w * s_l[jj * R + tid];
    }
    s_w0[tid] = w0; s_den[tid] = den;
  }
  __syncthreads();
  constexpr int kRowThreads = kThreads / 128 * 128, G = kRowThreads / 128;
  if (tid < kRowThreads) {
    const int d = tid & 127, g0 = tid >> 7;
    int mine = 0;
    for (int hd = g0; hd < R; hd += G, ++mine) {
      float m, l, a;
      local(hd, d, m, l, a);
      s_acc[hd * 128 + d] = s_w0[hd] * a;
    }
    const int n_items = mine * np;
    constexpr int kFly = 16;
    for (int it0 = 0; it0 < n_items; it0 += kFly) {
      uint2 v[kFly];
#pragma unroll
      for (int u = 0; u < kFly; ++u) {
        const int it = it0 + u < n_items ? it0 + u : n_items - 1;
        const int k = it / np, jj = it - k * np, hd = g0 + k * G, j = jj < g.rank ? jj : jj + 1;
        v[u] = ld_pair_sys(recv + j * L.msg + 2 * (int64_t)g.rows + (row0 + hd) * 128 + chan_of_pos(d));
      }
#pragma unroll
      for (int u = 0; u < kFly; ++u) {
        const int it = it0 + u;
        if (it < n_items) {
          const int k = it / np, jj = it - k * np, hd = g0 + k * G, j = jj < g.rank ? jj : jj + 1;
          const float val = v[u].y == g.seq ? __uint_as_float(v[u].x)
                                            : wait_pair(recv + j * L.msg + 2 * (int64_t)g.rows + (row0 + hd) * 128 + chan_of_pos(d), g.seq,
                                                        g.timeout_ns, &expired);
          s_acc[hd * 128 + d] += s_w[jj * R + hd] * val;
        }
      }
    }
    for (int hd = g0; hd < R; hd += G) {
      const float den = s_den[hd];
      store_out(p.out, (row0 + hd) * p.out_stride + chan_of_pos(d), den > 0.f ? s_acc[hd * 128 + d] / den : 0.f, p.out_dtype);
    }
  }
  if (expired) atomicOr(reinterpret_cast<int*>(g.bufs[g.rank]), 2);
}

// Rotary position embedding as Hugging Face models apply it (rotate_half form, the arithmetic of apply_rotary_pos_emb
// that the reference's patched forwards call before the cache, src/patch/patch_llama.py:58-65): out = x cos + rot sin with
// rot[d] = -x[d + 64] for d < 64 and x[d - 64] otherwise, every product and the sum rounded to bf16 as eager bf16
// arithmetic does.  `x`, `other`: two bf16 values each (this channel pair and the pair 64 channels away); `neg`: this pair is in
// the lower half.
__device__ __forceinline__ uint32_t rope_pair(uint32_t x, uint32_t other, uint32_t cs, uint32_t sn, bool neg) {
  auto lo = [](uint32_t w) { return __uint_as_float(w << 16); };
  auto hi = [](uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); };
  auto rb = [](float f) { return __bfloat162float(__float2bfloat16_rn(f)); };
  const float r0 = neg ? -lo(other) : lo(other), r1 = neg ? -hi(other) : hi(other);
  const float o0 = rb(rb(lo(x) * lo(cs)) + rb(r0 * lo(sn))), o1 = rb(rb(hi(x) * hi(cs)) + rb(r1 * hi(sn)));
  return pack_bf16x2(o0, o1);
}

// ---- the kernel -------------------------------------------------------------

// The four 16-bit-lane fields of a word as fp16 subnormals, offset binary: result k = ((nibble k) ^ 8) * 2^-24 for k = 0, 2
// (bits 0-3) and * 2^-20 for k = 1, 3 (bits 4-7).
__device__ __forceinline__ void cvt_nibbles_subnormal(uint32_t w, uint32_t (&h)[4]) {
  const uint32_t w8 = w >> 8;
  h[0] = lop3_and_xor(w, 0x000F000Fu, 0x00080008u);
  h[1] = lop3_and_xor(w, 0x00F000F0u, 0x00800080u);
  h[2] = lop3_and_xor(w8, 0x000F000Fu, 0x00080008u);
  h[3] = lop3_and_xor(w8, 0x00F000F0u, 0x00800080u);
}
// 2-bit fields f = 0..3 of the low byte of each 16-bit lane: result f = ((field f) ^ 2) * 2^(2 f - 24)
__device__ __forceinline__ void cvt_crumbs_subnormal(uint32_t w, uint32_t (&h)[4]) {
  h[0] = lop3_and_xor(w, 0x00030003u, 0x00020002u);
  h[1] = lop3_and_xor(w, 0x000C000Cu, 0x00080008u);
  h[2] = lop3_and_xor(w, 0x00300030u, 0x00200020u);
  h[3] = lop3_and_xor(w, 0x00C000C0u, 0x00800080u);
}

// Cluster-wide barrier: orders the blocks' shared-memory writes before it against the other blocks' reads after it.
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// fp32 at shared-memory address `addr` (of this block's window) in block `rank` of the cluster
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr, int rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// kMode: 0 = the splits of a head merge through the workspace; 1 = the same, followed by the exchange with the other
// sequence shards over peer memory; 2 = the splits of a head are one thread-block cluster and merge through
// distributed shared memory.  Instantiated apart, so that each form costs the others no registers.
template <int NT, bool kScaleTma, int KB, int VB, int kMode>
__global__ void __launch_bounds__(warps_of(NT) * 32, 1)
decode_splitk_kernel(const __grid_constant__ CUtensorMap kv_map, const DecodeParams p) {
  constexpr bool kPeer = kMode == 1, kCluster = kMode == 2;
  using F = Fmt<KB, VB>;
  using VF = VFmt<VB>;
  constexpr int kWarps = warps_of(NT), kThreads = kWarps * 32;
  constexpr int kSlotBytes = F::kSlot, kUnitQ = F::kUnitQ, kChunks = F::kChunks;
  constexpr int kQItems = NT * 8;                                   // (tile, head) pairs whose query row is loaded
  constexpr int kQIter = (kQItems + kWarps - 1) / kWarps;           // per warp: items warp, warp + kWarps, ...
  extern __shared__ __align__(128) uint8_t smem[];
  // layout: ring [kWarps][kSlots][kSlotBytes] | fragH [NT][8][2][32] u32 | fragB same |
  //         headC [NT*8] f32 | mbarriers [kWarps][kSlots]
  uint8_t* ring = smem;
  uint32_t* fragH = reinterpret_cast<uint32_t*>(smem + kWarps * kSlots * kSlotBytes);
  uint32_t* fragB = fragH + NT * 512;
  float* headC = reinterpret_cast<float*>(fragB + NT * 512);
  uint64_t* bars = reinterpret_cast<uint64_t*>(headC + NT * 8);
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  // Blocks are numbered split-major, so that the blocks the hardware starts last are the LAST split of every head, and
  // that split may be a small one (p.last_share / 256 of an even share, the other splits the rest): when the heads
  // do not fill the SMs evenly (128 heads on 148 SMs), the SMs left over work through the small splits while the others
  // each do one large one.
  // In cluster mode the splits of a head are the blocks of one cluster (consecutive block numbers).
  const int split = kCluster ? (int)(blockIdx.x % p.cluster) : (int)(blockIdx.x / p.BH);
  const int head = kCluster ? (int)(blockIdx.x / p.cluster) : (int)(blockIdx.x - split * p.BH);
  Lens L;
  L.n_quant = p.n_quant; L.n_stg = p.nseg[1];
  if (p.lengths != nullptr) {       // written before the kernel that precedes this one started (see hq_decode_args.lengths)
    L.n_quant = __ldg(p.lengths); L.n_stg = __ldg(p.lengths + 1);
  }
  L.uq = (L.n_quant + kUnitQ - 1) / kUnitQ;
  L.useg1 = (L.n_stg + kUnitB - 1) / kUnitB;
  L.units = L.uq + p.useg[0] + L.useg1 + p.useg[2] + p.useg[3];
  L.uq_stable = L.n_quant > 128 ? (L.n_quant - 128) / kUnitQ : 0;
  int u_begin, u_end;
  {
    const int64_t parts = (int64_t)(p.nsplit - 1) * 256 + p.last_share;          // in 1/256 of an even share
    u_begin = (int)(((int64_t)split * 256 * L.units) / parts);
    u_end = split + 1 == p.nsplit ? L.units : (int)(((int64_t)(split + 1) * 256 * L.units) / parts);
  }
  const int n_my = (u_end - u_begin - warp + kWarps - 1) / kWarps;   // units u_begin + warp + kWarps i
  uint8_t* my_ring = ring + warp * (kSlots * kSlotBytes);
  uint64_t* my_bar = bars + warp * kSlots;

  // ---- 1. barriers
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kSlots; ++s) mbar_init(&my_bar[s], kScaleTma ? 1 + kScaleLanes : 1);
    fence_mbar_init();
  }
  __syncwarp();

  // Requested by lane 0 of the warp that consumes it.  (One producer warp serving every ring, a lane per ring, was
  // measured slower: the bulk-copy instructions of one warp issue one after the other and cannot keep 15 rings fed.)
  // The lane's instructions are a serial chain that holds up its warp, so the common case - a full quantised unit -
  // is kept to one multiply-add per address on bases computed once.
  const uint8_t* const kq_base = p.k_packed + head * p.kp_stride_bh;
  const uint8_t* const vq_base = p.v_packed + head * p.vp_stride_bh;
  const __half* const ks_base = p.k_scale + head * p.ks_stride_bh;
  const __half* const vs_base = p.v_scale + head * p.vs_stride_bh;
  const uint32_t ring_u32 = smem_u32(my_ring), bar_u32 = smem_u32(my_bar);
  const int uq_full = L.n_quant / kUnitQ;            // quantised units with all their tokens
  auto bulk_raw = [](uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar) : "memory");
  };
  // The two code tensors of a unit travel as bulk copies (lane 0).  Its scales - 64 bytes each - do not: the copy
  // engine takes about as long to accept a 64-byte request as a 2 KB one, and at four requests per unit it is the
  // requests, not the bytes, that it runs out of.  Lanes 0..7 fetch them as 16-byte asynchronous copies (lanes 0-3
  // the K scales, 4-7 the V scales) and let the slot's barrier count their completion (one arrival per lane, which
  // the barrier's arrival count includes; a lane with nothing to copy arrives at once).
  auto scale_copies = [&](int slot, int64_t tok0, int ntok) {     // lanes 0..7, kScaleTma only
    const int c = lane & 3;
    if (8 * c < ntok) {
      const __half* src = (lane < 4 ? ks_base : vs_base) + tok0 + 8 * c;
      const uint32_t dst = ring_u32 + slot * kSlotBytes + F::kData + (lane < 4 ? 0 : 64) + 16 * c;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_u32 + slot * 8) : "memory");
  };
  auto issue = [&](int i) {   // the whole warp
    const int u = u_begin + warp + kWarps * i;
    const int slot = i % kSlots;
    if (u < uq_full) {
      const int64_t tok0 = (int64_t)u * kUnitQ;
      if (lane == 0) {
        const uint32_t dst = ring_u32 + slot * kSlotBytes, bar = bar_u32 + slot * 8;
        constexpr uint32_t kb = kUnitQ * F::kRowK, vb = kUnitQ * F::kRowV;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kb + vb) : "memory");
        if (KB == VB && p.kv_fused) {
          // the unit's K rows and V rows are one box {unit bytes, 1 unit, 2 planes} of the head's code tensor:
          // one request to the copy engine instead of two, landing as [K rows | V rows] like the two bulk copies
          asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                       ::"r"(dst), "l"(&kv_map), "r"(0), "r"(u), "r"(2 * head), "r"(bar) : "memory");
        } else {
          bulk_raw(dst, kq_base + tok0 * F::kRowK, kb, bar);
          bulk_raw(dst + F::kVOff, vq_base + tok0 * F::kRowV, vb, bar);
        }
      }
      if (kScaleTma && lane < kScaleLanes) scale_copies(slot, tok0, kUnitQ);
      return;
    }
    const Unit un = unit_of<KB, VB>(p, L, head, u);
    if (kScaleTma && lane < kScaleLanes) scale_copies(slot, un.kind == 0 ? un.tok0 : 0, un.kind == 0 ? un.ntok : 0);
    if (lane != 0) return;
    uint8_t* dst = my_ring + slot * kSlotBytes;
    if (un.kind == 0) {
      const uint32_t kbytes = (uint32_t)un.ntok * F::kRowK, vbytes = (uint32_t)un.ntok * F::kRowV;
      mbar_expect_tx(&my_bar[slot], kbytes + vbytes);
      bulk_g2s(dst, un.k, kbytes, &my_bar[slot]);
      bulk_g2s(dst + F::kVOff, un.v, vbytes, &my_bar[slot]);
    } else {
      const uint32_t bytes = (uint32_t)un.ntok * 256u;
      mbar_expect_tx(&my_bar[slot], 2 * bytes);
      bulk_g2s(dst, un.k, bytes, &my_bar[slot]);
      bulk_g2s(dst + 2048, un.v, bytes, &my_bar[slot]);
    }
  };
  // A unit is stable when the kernel running just before this one cannot have written it:
  // quantised tokens older than the newest 128, vertical-line tokens, window tokens (not staging, not the new token).
  auto stable = [&](int i) -> bool {
    const int u = u_begin + warp + kWarps * i;
    if (u < L.uq) return u < L.uq_stable;
    const int ub = u - L.uq;
    return ub < p.useg[0] || (ub >= p.useg[0] + L.useg1 && ub < p.useg[0] + L.useg1 + p.useg[2]);
  };

  // ---- 2. the query rows and the first bulk copies.
  // Plain launch: the small query loads go first, or they queue behind megabytes of cache
  // traffic.  Overlapped launch: the previous kernel may still be running, so only stable
  // units are requested; then this grid waits for the previous one to complete (its q,
  // staging and workspace writes are visible after that) and requests the rest.
  uint2 qraw[kQIter];
  auto load_q = [&]() {
#pragma unroll
    for (int k = 0; k < kQIter; ++k) {
      const int hd = warp + k * kWarps;
      qraw[k] = make_uint2(0u, 0u);
      if (hd < kQItems && hd < p.R)
        qraw[k] = __ldg(reinterpret_cast<const uint2*>(p.q + (int64_t)(head * p.R + hd) * p.q_stride) + lane);
      if (p.rope_cos != nullptr) {     // the query arrives unrotated: this lane's channels 4 lane .. + 3 pair with lane ^ 16's
        const int64_t ro = (int64_t)(head / p.heads_per_batch) * p.rope_stride;
        const uint2 cs = __ldg(reinterpret_cast<const uint2*>(p.rope_cos + ro) + lane);
        const uint2 sn = __ldg(reinterpret_cast<const uint2*>(p.rope_sin + ro) + lane);
        const uint32_t ox = __shfl_xor_sync(0xffffffffu, qraw[k].x, 16), oy = __shfl_xor_sync(0xffffffffu, qraw[k].y, 16);
        qraw[k].x = rope_pair(qraw[k].x, ox, cs.x, sn.x, lane < 16);
        qraw[k].y = rope_pair(qraw[k].y, oy, cs.y, sn.y, lane < 16);
      }
    }
  };
  if (!p.overlap) {
    // a kernel launched behind this one as a programmatic dependent (the exchange of sequence shards) may take its place
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    load_q();
    for (int i = 0; i < kSlots && i < n_my; ++i) issue(i);
  } else {
    int early = 0;
    while (early < kSlots && early < n_my && stable(early)) { issue(early); ++early; }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    load_q();
    for (int i = early; i < kSlots && i < n_my; ++i) issue(i);
  }

  // The step's new token, if the call carries one, is attended to from where the caller has it (segment 3) and
  // copied into its staging slot for the calls to come: one warp per head, 16 bytes per lane.
  if (p.nseg[3] > 0 && split == 0 && warp == 0) {
    const __nv_bfloat16* src = (lane < 16 ? p.kseg[3] : p.vseg[3]) + head * (lane < 16 ? p.kseg_stride[3] : p.vseg_stride[3]);
    __nv_bfloat16* dst = (lane < 16 ? p.stage_k : p.stage_v) + head * (lane < 16 ? p.kseg_stride[1] : p.vseg_stride[1]) +
                         (int64_t)L.n_stg * 128;
    uint4 w = __ldg(reinterpret_cast<const uint4*>(src) + (lane & 15));
    if (p.rope_cos != nullptr) {       // the new K row is stored rotated (lanes 0..15 hold it, 8 channels each; V is left alone)
      const int64_t ro = (int64_t)(head / p.heads_per_batch) * p.rope_stride;
      const uint4 cs = __ldg(reinterpret_cast<const uint4*>(p.rope_cos + ro) + (lane & 15));
      const uint4 sn = __ldg(reinterpret_cast<const uint4*>(p.rope_sin + ro) + (lane & 15));
      const uint4 o = make_uint4(__shfl_xor_sync(0xffffffffu, w.x, 8), __shfl_xor_sync(0xffffffffu, w.y, 8),
                                 __shfl_xor_sync(0xffffffffu, w.z, 8), __shfl_xor_sync(0xffffffffu, w.w, 8));
      if (lane < 16) {
        const bool neg = lane < 8;
        w = make_uint4(rope_pair(w.x, o.x, cs.x, sn.x, neg), rope_pair(w.y, o.y, cs.y, sn.y, neg),
                       rope_pair(w.z, o.z, cs.z, sn.z, neg), rope_pair(w.w, o.w, cs.w, sn.w, neg));
      }
    }
    reinterpret_cast<uint4*>(dst)[lane & 15] = w;
  }

  // ---- 3. query fragments (B operands of S^T = K Q^T) scattered straight into fragment
  // order, permuted along the channel axis to match the order in which channels fall out
  // of the K loads; plus the per-head offset constant of the biased K codes.
  // This thread holds channels 4*lane + x (x = 0..3) of head hd = warp + k * kWarps (tile hd / 8, column hd % 8).
#pragma unroll
  for (int k = 0; k < kQIter; ++k) {
    const int hd = warp + k * kWarps;
    if (hd >= kQItems) break;
    const int nt = hd >> 3, col = hd & 7;
    const float qv[4] = {__uint_as_float(qraw[k].x << 16), __uint_as_float(qraw[k].x & 0xFFFF0000u),
                         __uint_as_float(qraw[k].y << 16), __uint_as_float(qraw[k].y & 0xFFFF0000u)};
    // Quantised path.  K codes reach the MMA as 1024 + k (h + code) in fp16, h = 2^(bits - 1) (k = 1 for bytes and low
    // nibbles, 16 for high nibbles, 1 / 4 / 16 / 64 for the four 2-bit fields of a byte), so the query value is divided
    // by k and the head's constant sum((1024 + k h) * q / k) is taken off the fp32 score.  The channel that lands in MMA chunk
    // c, register r, k-slot thread tt, half e depends on how the lanes read a token row:
    //   8 bits: channel = 64 (c >> 2) + 16 tt + 4 (c & 3) + 2 r + e
    //   4 bits: channel = 32 tt + 8 (c >> 1) + 4 e + 2 (c & 1) + r            (r = 1: high nibbles)
    //   2 bits: channel = 32 tt + 16 (c >> 2) + 8 e + 4 ((c >> 1) & 1) + 2 (c & 1) + r   (field 2 (c & 1) + r)
    {
      __half* fh = reinterpret_cast<__half*>(fragH);
      float c = 0.f;
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int chn = 4 * lane + x;
        int cc, r, tt, e;
        float inv, bias;
        if (KB == 8) {
          cc = 4 * (chn >> 6) + ((chn >> 2) & 3); tt = (chn >> 4) & 3; r = (chn >> 1) & 1; e = chn & 1;
          inv = 1.0f; bias = 1152.f;
        } else if (KB == 4) {
          tt = chn >> 5; cc = 2 * ((chn >> 3) & 3) + ((chn >> 1) & 1); e = (chn >> 2) & 1; r = chn & 1;
          inv = r ? 0.0625f : 1.0f; bias = r ? 1152.f : 1032.f;
        } else {
          tt = chn >> 5; cc = 4 * ((chn >> 4) & 1) + 2 * ((chn >> 2) & 1) + ((chn >> 1) & 1); e = (chn >> 3) & 1; r = chn & 1;
          const int f = 2 * ((chn >> 1) & 1) + r;        // field within the byte: weight 4^f
          inv = f == 0 ? 1.0f : f == 1 ? 0.25f : f == 2 ? 0.0625f : 0.015625f;
          bias = f == 0 ? 1026.f : f == 1 ? 1032.f : f == 2 ? 1056.f : 1152.f;
        }
        const float v = fminf(fmaxf(qv[x] * inv, -65504.f), 65504.f);
        const __half hv = __float2half_rn(v);
        fh[((((nt * 8 + cc) * 2 + r) * 32) + 4 * col + tt) * 2 + e] = hv;
        c += bias * __half2float(hv);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
      if (lane == 0) headC[hd] = c;
    }
    // BF16 path: 16-byte chunk j = 4 i + tt of a token row covers channels 8 j .. 8 j + 7;
    // chunk c = 2 i + odd takes channels 4 odd + (0,1 | 2,3) of it.
    {
      const int j = lane >> 1, tt = j & 3, i = j >> 2, odd = lane & 1;
      fragB[((nt * 8 + 2 * i + odd) * 2 + 0) * 32 + 4 * col + tt] = qraw[k].x;
      fragB[((nt * 8 + 2 * i + odd) * 2 + 1) * 32 + 4 * col + tt] = qraw[k].y;
    }
  }
  __syncthreads();

  float O[NT][8][4];
  float m_ref[NT][2], l_part[NT][2];
  float Lt[NT][4];          // sum of the fp16 P~ values the quantised V tiles were multiplied with ([0], [1]: heads 2t, 2t+1)
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int j = 0; j < 2; ++j) { m_ref[nt][j] = -INFINITY; l_part[nt][j] = 0.f; }
#pragma unroll
    for (int x = 0; x < 4; ++x) Lt[nt][x] = 0.f;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
      for (int x = 0; x < 4; ++x) O[nt][mt][x] = 0.f;
  }

  bool failed = false;
  int i = 0;

  // ======================= quantised units ==================================
  {
    uint32_t Qh[NT][8][2];
    float hc[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int r = 0; r < 2; ++r) Qh[nt][c][r] = fragH[((nt * 8 + c) * 2 + r) * 32 + lane];
      hc[nt][0] = headC[nt * 8 + 2 * t];
      hc[nt][1] = headC[nt * 8 + 2 * t + 1];
    }

    // direct-load path only: per-lane packed (k_scale, v_scale) of token `lane` of a unit
    auto load_scales = [&](int ii) -> uint32_t {
      if (kScaleTma || ii >= n_my) return 0u;
      const int u = u_begin + warp + kWarps * ii;
      if (u >= L.uq) return 0u;
      const int tok = u * kUnitQ + lane;
      if (lane >= kUnitQ || tok >= L.n_quant) return 0u;
      const uint16_t ks = __half_as_ushort(p.k_scale[head * p.ks_stride_bh + tok]);
      const uint16_t vs = __half_as_ushort(p.v_scale[head * p.vs_stride_bh + tok]);
      return (uint32_t)ks | ((uint32_t)vs << 16);
    };
    uint32_t sc_cur = load_scales(0);

    for (; i < n_my; ++i) {
      const int u = u_begin + warp + kWarps * i;
      if (u >= L.uq) break;
      const int ntok = min(kUnitQ, L.n_quant - u * kUnitQ);
      const uint32_t sc_next = load_scales(i + 1);
      const int slot = i % kSlots;
      if (!mbar_wait_bounded(&my_bar[slot], (uint32_t)((i / kSlots) & 1))) { failed = true; break; }
      const uint8_t* Ks = my_ring + slot * kSlotBytes;
      const uint8_t* Vs = Ks + F::kVOff;
      const __half* kss = reinterpret_cast<const __half*>(Ks + F::kData);
      const __half* vss = reinterpret_cast<const __half*>(Ks + F::kData + 64);

      // scores of both 16-token chunks: this lane holds tokens g, g+8, 16+g, 24+g
      float s[kChunks][NT][4];
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int x = 0; x < 4; ++x) s[ch][nt][x] = 0.f;
      if constexpr (KB == 4) {
        uint4 kw[kChunks][2];
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          kw[ch][0] = *reinterpret_cast<const uint4*>(Ks + (16 * ch + g) * 64 + t * 16);
          kw[ch][1] = *reinterpret_cast<const uint4*>(Ks + (16 * ch + g + 8) * 64 + t * 16);
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch) {
            const uint32_t wa = w == 0 ? kw[ch][0].x : w == 1 ? kw[ch][0].y : w == 2 ? kw[ch][0].z : kw[ch][0].w;
            const uint32_t wb = w == 0 ? kw[ch][1].x : w == 1 ? kw[ch][1].y : w == 2 ? kw[ch][1].z : kw[ch][1].w;
            uint32_t ha[4], hb[4];
            cvt_nibbles_biased(wa, ha);
            cvt_nibbles_biased(wb, hb);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              mma_f16_16816(s[ch][nt], ha[0], hb[0], ha[1], hb[1], Qh[nt][2 * w][0], Qh[nt][2 * w][1]);
              mma_f16_16816(s[ch][nt], ha[2], hb[2], ha[3], hb[3], Qh[nt][2 * w + 1][0], Qh[nt][2 * w + 1][1]);
            }
          }
        }
      } else if constexpr (KB == 8) {
        // a 128-byte row: 16 bytes at 64 h + 16 t; word w of it holds channels 64 h + 16 t + 4 w + (0..3)
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 ka = *reinterpret_cast<const uint4*>(Ks + (16 * ch + g) * 128 + 64 * h + t * 16);
            const uint4 kb = *reinterpret_cast<const uint4*>(Ks + (16 * ch + g + 8) * 128 + 64 * h + t * 16);
            const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w}, wb[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const uint32_t xa = wa[w] ^ 0x80808080u, xb = wb[w] ^ 0x80808080u;   // code + 128 in every byte
              const uint32_t a0 = prmt(xa, 0x64646464u, 0x4140u), a2 = prmt(xa, 0x64646464u, 0x4342u);
              const uint32_t a1 = prmt(xb, 0x64646464u, 0x4140u), a3 = prmt(xb, 0x64646464u, 0x4342u);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt)
                mma_f16_16816(s[ch][nt], a0, a1, a2, a3, Qh[nt][4 * h + w][0], Qh[nt][4 * h + w][1]);
            }
          }
      } else {
        // a 32-byte row: 8 bytes at 8 t; word x of it holds channels 32 t + 16 x + m, code m in bits 2m, 2m+1
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          const uint2 ka = *reinterpret_cast<const uint2*>(Ks + (16 * ch + g) * 32 + t * 8);
          const uint2 kb = *reinterpret_cast<const uint2*>(Ks + (16 * ch + g + 8) * 32 + t * 8);
          const uint32_t wa[2] = {ka.x, ka.y}, wb[2] = {kb.x, kb.y};
#pragma unroll
          for (int x = 0; x < 2; ++x)
#pragma unroll
            for (int sh = 0; sh < 2; ++sh) {
              const uint32_t ua = sh ? wa[x] >> 8 : wa[x], ub = sh ? wb[x] >> 8 : wb[x];
              uint32_t ra[4], rb[4];
              cvt_crumbs_biased(ua, ra);
              cvt_crumbs_biased(ub, rb);
#pragma unroll
              for (int pp = 0; pp < 2; ++pp)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                  mma_f16_16816(s[ch][nt], ra[2 * pp], rb[2 * pp], ra[2 * pp + 1], rb[2 * pp + 1],
                                Qh[nt][4 * x + 2 * sh + pp][0], Qh[nt][4 * x + 2 * sh + pp][1]);
            }
        }
      }
      float vsc[kChunks][2];
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        const int tokA = 16 * ch + g, tokB = tokA + 8;
        const bool okA = tokA < ntok, okB = tokB < ntok;
        float ksA, ksB;
        if (kScaleTma) {
          ksA = __half2float(kss[tokA]) * p.sml; ksB = __half2float(kss[tokB]) * p.sml;
          vsc[ch][0] = okA ? __half2float(vss[tokA]) : 0.f;
          vsc[ch][1] = okB ? __half2float(vss[tokB]) : 0.f;
        } else {
          const uint32_t scA = __shfl_sync(0xffffffffu, sc_cur, tokA);
          const uint32_t scB = __shfl_sync(0xffffffffu, sc_cur, tokB);
          ksA = __half2float(__ushort_as_half((uint16_t)(scA & 0xFFFFu))) * p.sml;
          ksB = __half2float(__ushort_as_half((uint16_t)(scB & 0xFFFFu))) * p.sml;
          vsc[ch][0] = __half2float(__ushort_as_half((uint16_t)(scA >> 16)));
          vsc[ch][1] = __half2float(__ushort_as_half((uint16_t)(scB >> 16)));
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          s[ch][nt][0] = okA ? (s[ch][nt][0] - hc[nt][0]) * ksA : -INFINITY;
          s[ch][nt][1] = okA ? (s[ch][nt][1] - hc[nt][1]) * ksA : -INFINITY;
          s[ch][nt][2] = okB ? (s[ch][nt][2] - hc[nt][0]) * ksB : -INFINITY;
          s[ch][nt][3] = okB ? (s[ch][nt][3] - hc[nt][1]) * ksB : -INFINITY;
        }
      }
      // one online-softmax step for the 32 tokens
      float mx[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j)
        {
          float v = fmaxf(s[0][nt][j], s[0][nt][2 + j]);
          if constexpr (kChunks == 2) v = fmaxf(v, fmaxf(s[kChunks - 1][nt][j], s[kChunks - 1][nt][2 + j]));
          mx[nt][j] = group_max(v);
        }
      lazy_rescale<NT>(mx, m_ref, l_part, O, Lt);

#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        uint32_t pb[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float pr[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float mu = m_ref[nt][x & 1];
            pr[x] = ex2f(s[ch][nt][x] - (mu == -INFINITY ? 0.f : mu));
          }
          l_part[nt][0] += pr[0] + pr[2];
          l_part[nt][1] += pr[1] + pr[3];
          const uint32_t pa = pack_f16x2(pr[0] * vsc[ch][0], pr[1] * vsc[ch][0]);   // token g
          const uint32_t pq = pack_f16x2(pr[2] * vsc[ch][1], pr[3] * vsc[ch][1]);   // token g + 8
          pb[nt][0] = movmatrix_trans(pa);    // (tokens 2t, 2t+1 ; head g)
          pb[nt][1] = movmatrix_trans(pq);    // (tokens 2t+8, 2t+9 ; head g)
          // sum over the chunk's tokens of the P~ values as the tensor core sees them, for the offset of the V codes
          mma_f16_16816(Lt[nt], 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, pb[nt][0], pb[nt][1]);
        }
        // V: this lane takes channels 16 g .. 16 g + 15 of tokens 2t, 2t+1, 2t+8, 2t+9 of the chunk; which of them
        // land in which output tile is VFmt<VB>::chan.  The codes are used where they lie, as fp16 subnormals.
        const uint8_t* vrow = Vs + (16 * ch + 2 * t) * F::kRowV + 2 * VB * g;
        if constexpr (VB == 4) {
          const uint2 vA = *reinterpret_cast<const uint2*>(vrow);
          const uint2 vB = *reinterpret_cast<const uint2*>(vrow + 64);
          const uint2 vC = *reinterpret_cast<const uint2*>(vrow + 8 * 64);
          const uint2 vD = *reinterpret_cast<const uint2*>(vrow + 9 * 64);
          const uint32_t wA[2] = {vA.x, vA.y}, wB[2] = {vB.x, vB.y}, wC[2] = {vC.x, vC.y}, wD[2] = {vD.x, vD.y};
#pragma unroll
          for (int w = 0; w < 2; ++w)
#pragma unroll
            for (int hl = 0; hl < 2; ++hl) {
              const uint32_t sel = hl ? 0x7632u : 0x5410u;
              uint32_t hab[4], hcd[4];
              cvt_nibbles_subnormal(prmt(wA[w], wB[w], sel), hab);
              cvt_nibbles_subnormal(prmt(wC[w], wD[w], sel), hcd);
              const int pidx = 2 * w + hl;      // 16-bit group: channels 16 g + 4 pidx + (0..3) = nibbles 0..3
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                mma_f16_16816(O[nt][2 * pidx], hab[0], hab[2], hcd[0], hcd[2], pb[nt][0], pb[nt][1]);       // nibbles 0, 2
                mma_f16_16816(O[nt][2 * pidx + 1], hab[1], hab[3], hcd[1], hcd[3], pb[nt][0], pb[nt][1]);   // nibbles 1, 3
              }
            }
        } else if constexpr (VB == 8) {
          const uint4 vA = *reinterpret_cast<const uint4*>(vrow);
          const uint4 vB = *reinterpret_cast<const uint4*>(vrow + 128);
          const uint4 vC = *reinterpret_cast<const uint4*>(vrow + 8 * 128);
          const uint4 vD = *reinterpret_cast<const uint4*>(vrow + 9 * 128);
          const uint32_t wA[4] = {vA.x, vA.y, vA.z, vA.w}, wB[4] = {vB.x, vB.y, vB.z, vB.w};
          const uint32_t wC[4] = {vC.x, vC.y, vC.z, vC.w}, wD[4] = {vD.x, vD.y, vD.z, vD.w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {      // word w: channels 16 g + 4 w + (0..3), one byte each
            const uint32_t ab01 = prmt(wA[w], wB[w], 0x5140u) ^ 0x80808080u;    // a0 b0 a1 b1, each + 128
            const uint32_t ab23 = prmt(wA[w], wB[w], 0x7362u) ^ 0x80808080u;    // a2 b2 a3 b3
            const uint32_t cd01 = prmt(wC[w], wD[w], 0x5140u) ^ 0x80808080u;
            const uint32_t cd23 = prmt(wC[w], wD[w], 0x7362u) ^ 0x80808080u;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              mma_f16_16816(O[nt][2 * w], prmt(ab01, 0u, 0x4140u), prmt(ab01, 0u, 0x4342u), prmt(cd01, 0u, 0x4140u),
                            prmt(cd01, 0u, 0x4342u), pb[nt][0], pb[nt][1]);
              mma_f16_16816(O[nt][2 * w + 1], prmt(ab23, 0u, 0x4140u), prmt(ab23, 0u, 0x4342u), prmt(cd23, 0u, 0x4140u),
                            prmt(cd23, 0u, 0x4342u), pb[nt][0], pb[nt][1]);
            }
          }
        } else {
          const uint32_t wA = *reinterpret_cast<const uint32_t*>(vrow);
          const uint32_t wB = *reinterpret_cast<const uint32_t*>(vrow + 32);
          const uint32_t wC = *reinterpret_cast<const uint32_t*>(vrow + 8 * 32);
          const uint32_t wD = *reinterpret_cast<const uint32_t*>(vrow + 9 * 32);
#pragma unroll
          for (int hl = 0; hl < 2; ++hl) {   // codes 8 hl .. 8 hl + 7 of the two tokens, one token per 16-bit half
            const uint32_t sel = hl ? 0x7632u : 0x5410u;
            const uint32_t mab = prmt(wA, wB, sel), mcd = prmt(wC, wD, sel);
            uint32_t ab0[4], ab1[4], cd0[4], cd1[4];       // low byte (codes 8 hl + 0..3) and high byte (8 hl + 4..7)
            cvt_crumbs_subnormal(mab, ab0);
            cvt_crumbs_subnormal(mab >> 8, ab1);
            cvt_crumbs_subnormal(mcd, cd0);
            cvt_crumbs_subnormal(mcd >> 8, cd1);
#pragma unroll
            for (int f = 0; f < 4; ++f)
#pragma unroll
              for (int nt = 0; nt < NT; ++nt)
                mma_f16_16816(O[nt][4 * hl + f], ab0[f], ab1[f], cd0[f], cd1[f], pb[nt][0], pb[nt][1]);
          }
        }
      }
      sc_cur = sc_next;
      __syncwarp();
      if (i + kSlots < n_my) issue(i + kSlots);
    }
  }

  // ======================= BF16 units =======================================
  if (!failed && i < n_my) {
    uint32_t Qb[NT][8][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int r = 0; r < 2; ++r) Qb[nt][c][r] = fragB[((nt * 8 + c) * 2 + r) * 32 + lane];

    for (; i < n_my; ++i) {
      const Unit un = unit_of<KB, VB>(p, L, head, u_begin + warp + kWarps * i);
      const int slot = i % kSlots;
      if (!mbar_wait_bounded(&my_bar[slot], (uint32_t)((i / kSlots) & 1))) { failed = true; break; }
      uint8_t* Ks = my_ring + slot * kSlotBytes;
      uint8_t* Vs = Ks + 2048;
      const bool patched = un.ntok < kUnitB;
      if (patched) {   // stale bytes past the copied rows must not reach the MMA as NaN/Inf
        const int n16 = (kUnitB - un.ntok) * 16;
        for (int x = lane; x < n16; x += 32) {
          reinterpret_cast<uint4*>(Ks + un.ntok * 256)[x] = make_uint4(0, 0, 0, 0);
          reinterpret_cast<uint4*>(Vs + un.ntok * 256)[x] = make_uint4(0, 0, 0, 0);
        }
        if (un.seg == 3 && p.rope_cos != nullptr) {     // the new token's K row came as the caller has it: rotate it here
          const int64_t ro = (int64_t)(head / p.heads_per_batch) * p.rope_stride;
          const uint2 cs = __ldg(reinterpret_cast<const uint2*>(p.rope_cos + ro) + lane);
          const uint2 sn = __ldg(reinterpret_cast<const uint2*>(p.rope_sin + ro) + lane);
          const uint2 mine = reinterpret_cast<const uint2*>(Ks)[lane], other = reinterpret_cast<const uint2*>(Ks)[lane ^ 16];
          __syncwarp();
          reinterpret_cast<uint2*>(Ks)[lane] = make_uint2(rope_pair(mine.x, other.x, cs.x, sn.x, lane < 16),
                                                          rope_pair(mine.y, other.y, cs.y, sn.y, lane < 16));
        }
        __syncwarp();
      }
      float s[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int x = 0; x < 4; ++x) s[nt][x] = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint4 kk = *reinterpret_cast<const uint4*>(Ks + g * 256 + (4 * w + t) * 16);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16_16816(s[nt], kk.x, 0u, kk.y, 0u, Qb[nt][2 * w][0], Qb[nt][2 * w][1]);
          mma_bf16_16816(s[nt], kk.z, 0u, kk.w, 0u, Qb[nt][2 * w + 1][0], Qb[nt][2 * w + 1][1]);
        }
      }
      const bool ok = g < un.ntok;
      float mx[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[nt][j] = ok ? s[nt][j] * p.sml : -INFINITY;
          mx[nt][j] = group_max(s[nt][j]);
        }
      lazy_rescale<NT>(mx, m_ref, l_part, O, Lt);
      // P^T operand once per factor the quantised tiles carry (the accumulators are shared with them)
      uint32_t pb[NT][VF::kScales];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float m0 = m_ref[nt][0] == -INFINITY ? 0.f : m_ref[nt][0];
        const float m1 = m_ref[nt][1] == -INFINITY ? 0.f : m_ref[nt][1];
        const float p0 = ex2f(s[nt][0] - m0), p1 = ex2f(s[nt][1] - m1);
        l_part[nt][0] += p0;
        l_part[nt][1] += p1;
#pragma unroll
        for (int sc = 0; sc < VF::kScales; ++sc) {
          const float f = VB == 8 ? 5.9604644775390625e-08f               // 2^-24
                                  : VB == 4 ? (sc ? 9.5367431640625e-07f : 5.9604644775390625e-08f)      // 2^-20, 2^-24
                                            : (sc == 0 ? 5.9604644775390625e-08f : sc == 1 ? 2.384185791015625e-07f
                                               : sc == 2 ? 9.5367431640625e-07f : 3.814697265625e-06f);   // 2^(2 sc - 24)
          pb[nt][sc] = movmatrix_trans(pack_bf16x2(p0 * f, p1 * f));     // (tokens 2t, 2t+1 ; head g)
        }
      }
      const uint8_t* va = Vs + (2 * t) * 256 + 32 * g;
      const uint4 a0 = *reinterpret_cast<const uint4*>(va);
      const uint4 a1 = *reinterpret_cast<const uint4*>(va + 16);
      const uint4 b0 = *reinterpret_cast<const uint4*>(va + 256);
      const uint4 b1 = *reinterpret_cast<const uint4*>(va + 256 + 16);
      const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};     // word m: channels 16 g + 2 m, + 1
      const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        const int c0 = VF::chan(mt, 0), c1 = VF::chan(mt, 1);          // local channels of the tile's two rows
        const uint32_t r0 = prmt(wa[c0 >> 1], wb[c0 >> 1], (c0 & 1) ? 0x7632u : 0x5410u);   // channel c0 of tokens (2t, 2t+1)
        const uint32_t r1 = prmt(wa[c1 >> 1], wb[c1 >> 1], (c1 & 1) ? 0x7632u : 0x5410u);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_bf16_1688(O[nt][mt], r0, r1, pb[nt][VF::scale_idx(mt)]);
      }
      __syncwarp();
      if (i + kSlots < n_my) {
        if (patched && lane == 0) fence_proxy_async_smem();   // generic-proxy writes above precede the next async write
        issue(i + kSlots);
      }
    }
  }
  if (failed && lane == 0) atomicOr(p.status, 1);

  // ======================= merge the warps ===================================
  // Two barriers: the warps' maxima first, then every warp writes its sums already weighted by 2^(m_warp - m_block), so
  // that a row of the block is a plain sum over the warps (one exponential per thread and head instead of one per
  // thread, head and warp).
  __syncthreads();   // every ring slot is drained (each issued unit was waited for) unless `failed`
  float* mrg_m = reinterpret_cast<float*>(smem);                 // [kWarps][NT*8]
  float* mrg_l = mrg_m + kWarps * NT * 8;                        // [kWarps][NT*8]
  float* mrg_o = mrg_l + kWarps * NT * 8;                        // [kWarps][NT*8][kMrgStride], position order
  if (g == 0) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) mrg_m[warp * NT * 8 + nt * 8 + 2 * t + j] = m_ref[nt][j];
  }
  __syncthreads();
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int hd = nt * 8 + 2 * t + j;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) M = fmaxf(M, mrg_m[w * NT * 8 + hd]);
      const float wt = (m_ref[nt][j] == -INFINITY) ? 0.f : ex2f(m_ref[nt][j] - M);
      const float lsum = group_sum(l_part[nt][j]);
      if (g == 0) mrg_l[warp * NT * 8 + hd] = lsum * wt;
      if (hd < p.R) {
        // true values: the tile's power of two back, the code offset times the sum of the quantised tokens' P~ off
        float* orow = mrg_o + ((size_t)(warp * NT * 8 + hd)) * kMrgStride + g;
        const float corr = VF::kOff * Lt[nt][j] * wt;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          const float up = (VF::exp2(mt) == 24 ? 16777216.f : VF::exp2(mt) == 22 ? 4194304.f : VF::exp2(mt) == 20 ? 1048576.f : 262144.f) * wt;
          orow[8 * VF::chan(mt, 0)] = fmaf(O[nt][mt][j], up, -corr);
          orow[8 * VF::chan(mt, 1)] = fmaf(O[nt][mt][2 + j], up, -corr);
        }
      }
    }
  __syncthreads();

  constexpr int kRowThreads = kThreads / 128 * 128;      // threads that write output rows, 128 per row at a time
  const int d = tid & 127;
  const bool single = (p.nsplit == 1);
  constexpr bool peers = kPeer;       // instantiated apart, so that the exchange code costs the plain kernel no registers
  // this CTA's state for head hd at position dd
  auto cta_row = [&](int hd, int dd, float& M, float& l, float& acc) {
    M = -INFINITY;
    acc = 0.f; l = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      M = fmaxf(M, mrg_m[w * NT * 8 + hd]);
      acc += mrg_o[((size_t)(w * NT * 8 + hd)) * kMrgStride + dd];
      l += mrg_l[w * NT * 8 + hd];
    }
  };
  if constexpr (kCluster) {
    // ======================= merge the splits inside the cluster ==============
    // Every block leaves its rows (position order) and their (m, l) in its own shared memory; after a cluster barrier
    // block r merges elements [r per, (r + 1) per) of the head's R x 128 outputs, reading the C blocks' values with
    // ld.shared::cluster (all in flight together), and writes them out.  A second barrier keeps every block's shared
    // memory alive until its readers are done.  Nothing goes through the workspace.
    const int C = p.cluster;
    float* cl_o = mrg_o + (size_t)kWarps * NT * 8 * kMrgStride;      // [R][128]
    float* cl_ml = cl_o + NT * 8 * 128;                              // [R][2]
    for (int hd = tid < kRowThreads ? tid >> 7 : p.R; hd < p.R; hd += kRowThreads / 128) {
      float M, l, acc;
      cta_row(hd, d, M, l, acc);
      cl_o[hd * 128 + d] = acc;
      if (d == 0) { cl_ml[2 * hd] = M; cl_ml[2 * hd + 1] = l; }
    }
    cluster_barrier();
    const int per = (p.R * 128 + C - 1) / C;
    for (int x = tid; x < per; x += kThreads) {
      const int e = split * per + x;
      if (e >= p.R * 128) break;
      const int hd = e >> 7, dd = e & 127;
      const uint32_t a_ml = smem_u32(cl_ml + 2 * hd), a_o = smem_u32(cl_o + e);
      float mc[8], lc[8], oc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        mc[c] = -INFINITY; lc[c] = 0.f; oc[c] = 0.f;
        if (c < C) {
          mc[c] = ld_cluster_f32(a_ml, c);
          lc[c] = ld_cluster_f32(a_ml + 4, c);
          oc[c] = ld_cluster_f32(a_o, c);
        }
      }
      float M = -INFINITY;
#pragma unroll
      for (int c = 0; c < 8; ++c) M = fmaxf(M, mc[c]);
      float den = 0.f, acc = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float wt = (mc[c] == -INFINITY) ? 0.f : ex2f(mc[c] - M);
        den = fmaf(wt, lc[c], den);
        acc = fmaf(wt, oc[c], acc);
      }
      const int64_t qrow = (int64_t)head * p.R + hd;
      store_out(p.out, qrow * p.out_stride + chan_of_pos(dd), den > 0.f ? acc / den : 0.f, p.out_dtype);
    }
    cluster_barrier();
    return;
  }
  for (int hd = tid < kRowThreads ? tid >> 7 : p.R; hd < p.R; hd += kRowThreads / 128) {
    float M, l, acc;
    cta_row(hd, d, M, l, acc);
    const int64_t qrow = (int64_t)head * p.R + hd;
    if (single) {
      if constexpr (peers) {
        peer_send(p, (int)qrow, chan_of_pos(d), M, l, acc);       // every row is sent before any is awaited
      } else if (p.pacc) {
        p.pacc[qrow * 128 + chan_of_pos(d)] = acc;
        if (d == 0) { p.pm[qrow] = M; p.pl[qrow] = l; }
      } else {
        store_out(p.out, qrow * p.out_stride + chan_of_pos(d), l > 0.f ? acc / l : 0.f, p.out_dtype);
      }
    } else {
      const int64_t prow = ((int64_t)head * p.nsplit + split) * p.R + hd;
      p.ws_acc[prow * 128 + d] = acc;
      if (d == 0) { p.ws_m[prow] = M; p.ws_l[prow] = l; }
    }
  }
  if (single) {
    if constexpr (peers) peer_receive_all<kThreads>(p, mrg_o + (size_t)kWarps * NT * 8 * kMrgStride, head, tid, cta_row);
    return;
  }

  // ======================= merge the splits (last CTA of the head) ===========
  // Ticket: the CTA barrier orders every thread's partial stores before thread 0's
  // release-add; the last arriver's acquire-add + barrier orders them before its loads.
  __syncthreads();
  if (tid == 0) {
    unsigned ticket;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.counters + head) : "memory");
    s_last = (ticket == (unsigned)(p.nsplit - 1));
  }
  __syncthreads();
  if (!s_last) return;
  // One warp per query head, no shared memory and no block barrier: lane s fetches (m, l) of split s, every lane the
  // four positions 4 lane .. 4 lane + 3 of every split's row - all requested before any is used, so the merge costs one
  // round trip to L2 - the weights 2^(m_s - M) are formed once per split and handed round by shuffles.  More splits
  // than a round holds go in several rounds with the usual running rescale.
  float* res = reinterpret_cast<float*>(smem);              // [R][kMrgStride] merged rows, for the exchange below only
  float* res_ml = res + (size_t)p.R * kMrgStride;            // [R][2]
  const int64_t base = (int64_t)head * p.nsplit * p.R;
  constexpr int kRound = 20;          // splits per round: their rows are all in flight at once (80 registers)
  for (int hd = warp; hd < p.R; hd += kWarps) {
    float M = -INFINITY, den = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < p.nsplit; s0 += kRound) {
      const int ns = min(kRound, p.nsplit - s0);
      float ms = -INFINITY, ls = 0.f;
      if (lane < ns) {
        ms = __ldcg(p.ws_m + base + (int64_t)(s0 + lane) * p.R + hd);
        ls = __ldcg(p.ws_l + base + (int64_t)(s0 + lane) * p.R + hd);
      }
      float4 v[kRound];
#pragma unroll
      for (int x = 0; x < kRound; ++x) {
        v[x] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (x < ns) v[x] = __ldcg(reinterpret_cast<const float4*>(p.ws_acc + (base + (int64_t)(s0 + x) * p.R + hd) * 128) + lane);
      }
      float Mc = ms;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) Mc = fmaxf(Mc, __shfl_xor_sync(0xffffffffu, Mc, o));
      const float Mn = fmaxf(M, Mc);
      const float keep = (M == -INFINITY) ? 0.f : ex2f(M - Mn);
      const float wt = (ms == -INFINITY) ? 0.f : ex2f(ms - Mn);
      float dl = wt * ls;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dl += __shfl_xor_sync(0xffffffffu, dl, o);
      den = den * keep + dl;
      acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
#pragma unroll
      for (int x = 0; x < kRound; ++x) {
        const float wx = __shfl_sync(0xffffffffu, wt, x);       // 0 for x >= ns
        acc.x += wx * v[x].x; acc.y += wx * v[x].y; acc.z += wx * v[x].z; acc.w += wx * v[x].w;
      }
      M = Mn;
    }
    const int64_t qrow = (int64_t)head * p.R + hd;
    const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
    if constexpr (peers) {
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        res[(size_t)hd * kMrgStride + 4 * lane + x] = a4[x];
        peer_send(p, (int)qrow, chan_of_pos(4 * lane + x), M, den, a4[x]);
      }
      if (lane == 0) { res_ml[2 * hd] = M; res_ml[2 * hd + 1] = den; }
    } else if (p.pacc) {
#pragma unroll
      for (int x = 0; x < 4; ++x) p.pacc[qrow * 128 + chan_of_pos(4 * lane + x)] = a4[x];
      if (lane == 0) { p.pm[qrow] = M; p.pl[qrow] = den; }
    } else {
      const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
      for (int x = 0; x < 4; ++x) store_out(p.out, qrow * p.out_stride + chan_of_pos(4 * lane + x), a4[x] * inv, p.out_dtype);
    }
  }
  if constexpr (peers) {
    __syncthreads();
    auto head_row = [&](int hd, int dd, float& M, float& l, float& acc) {
      M = res_ml[2 * hd]; l = res_ml[2 * hd + 1]; acc = res[(size_t)hd * kMrgStride + dd];
    };
    peer_receive_all<kThreads>(p, res_ml + 2 * p.R, head, tid, head_row);
  }
  if (tid == 0) p.counters[head] = 0;   // ready for the next launch on this workspace
}


// ---- launch ------------------------------------------------------------------

static size_t decode_smem_bytes(int NT, int slot_bytes) {
  const int w = warps_of(NT);
  return (size_t)w * kSlots * slot_bytes + (size_t)NT * 512 * 4 * 2 + (size_t)NT * 8 * 4 + (size_t)w * kSlots * 8;
}

template <int NT, bool kScaleTma, int KB, int VB, int kMode>
static int launch_decode(const DecodeParams& p, const CUtensorMap& kv_map, dim3 grid, cudaStream_t st, int* clusters_out) {
  const size_t smem = decode_smem_bytes(NT, Fmt<KB, VB>::kSlot);
  static thread_local int attr_dev = -1;
  int dev = 0;
  HQ_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    HQ_CUDA(cudaFuncSetAttribute(decode_splitk_kernel<NT, kScaleTma, KB, VB, kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    attr_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(warps_of(NT) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.overlap) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.cluster > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)p.cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (clusters_out != nullptr) {       // query only: how many clusters of this size the device holds at once
    *clusters_out = 0;
    if (kMode != 2) return HQ_OK;
    static thread_local int cached_dev = -1;
    static thread_local int cached[9];       // cluster sizes 2..8 (the portable ones)
    if (cached_dev != dev) { for (int i = 0; i < 9; ++i) cached[i] = -1; cached_dev = dev; }
    if (p.cluster > 8) return HQ_OK;
    if (cached[p.cluster] < 0) {
      int n = 0;
      cfg.numAttrs = 1;                 // the cluster dimension alone
      cudaLaunchAttribute only[1] = {attr[na - 1]};
      cfg.attrs = only;
      if (cudaOccupancyMaxActiveClusters(&n, decode_splitk_kernel<NT, kScaleTma, KB, VB, kMode>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      cached[p.cluster] = n;
    }
    *clusters_out = cached[p.cluster];
    return HQ_OK;
  }
  HQ_CUDA(cudaLaunchKernelEx(&cfg, decode_splitk_kernel<NT, kScaleTma, KB, VB, kMode>, kv_map, p));
  return HQ_OK;
}

template <int KB, int VB>
static int launch_decode_bits(const DecodeParams& p, const CUtensorMap& kv_map, int NT, dim3 grid, cudaStream_t st, int* clusters_out) {
  if (p.peer.world > 1) {   // the exchanging instantiations exist with directly loaded scales only (any alignment)
    return NT == 1 ? launch_decode<1, false, KB, VB, 1>(p, kv_map, grid, st, clusters_out) : launch_decode<2, false, KB, VB, 1>(p, kv_map, grid, st, clusters_out);
  }
  if (p.cluster > 1) {      // the cluster instantiations exist with scales riding in the bulk copies only
    if (!p.scale_tma) { if (clusters_out) *clusters_out = 0; return clusters_out ? HQ_OK : HQ_ERR_INVALID; }
    return NT == 1 ? launch_decode<1, true, KB, VB, 2>(p, kv_map, grid, st, clusters_out) : launch_decode<2, true, KB, VB, 2>(p, kv_map, grid, st, clusters_out);
  }
  if (NT == 1) return p.scale_tma ? launch_decode<1, true, KB, VB, 0>(p, kv_map, grid, st, clusters_out) : launch_decode<1, false, KB, VB, 0>(p, kv_map, grid, st, clusters_out);
  return p.scale_tma ? launch_decode<2, true, KB, VB, 0>(p, kv_map, grid, st, clusters_out) : launch_decode<2, false, KB, VB, 0>(p, kv_map, grid, st, clusters_out);
}

// One function per pair, each defined in the file that instantiates the pair's kernels.
#define HQ_DECODE_PAIRS(X) X(8, 8) X(8, 4) X(8, 2) X(4, 8) X(4, 4) X(4, 2) X(2, 8) X(2, 4) X(2, 2)
#define HQ_DECODE_DECLARE(kb, vb) \
  int launch_decode_k##kb##v##vb(const DecodeParams& p, const CUtensorMap& kv_map, int NT, dim3 grid, cudaStream_t st, int* clusters_out);
HQ_DECODE_PAIRS(HQ_DECODE_DECLARE)
#define HQ_DECODE_DEFINE(kb, vb) \
  int launch_decode_k##kb##v##vb(const DecodeParams& p, const CUtensorMap& kv_map, int NT, dim3 grid, cudaStream_t st, int* clusters_out) { \
    return launch_decode_bits<kb, vb>(p, kv_map, NT, grid, st, clusters_out); \
  }

}  // namespace hq
