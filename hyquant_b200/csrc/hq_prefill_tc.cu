// Hybrid-precision causal prefill attention on the Blackwell tensor path.
//
// Tile semantics as stated in hq_prefill.cu's header: for the 128-query
// block at s of query head h, keys below wla(s) are INT8 unless they are vertical lines of h
// (masked here, served from gathered BF16 tiles), keys in [wla(s), s + 128) are BF16 + causal mask.
//
// One CTA works on the same 128 queries of TWO query heads of one KV group (A and B), so every INT8 and
// window K / V tile that reaches shared memory feeds two score tiles, and the two heads' softmax chains
// interleave on the SM: while one head's threads are in their exponentials the tensor core runs the other
// head's products.  11 warps:
//   warp 8 (one lane)  producer: TMA tensor-map loads (128-byte swizzle) of both heads' Q once, then K tiles
//                      and transposed V tiles into two four-slot rings (a K slot is free again after the
//                      heads' Q K^T, a V slot after their P V).  INT8 and window items serve both heads;
//                      the gathered vertical-line tiles are per head.
//   warps 9, 10        (one lane each) issue tcgen05.mma for head A / B: S = Q K^T (kind::i8 with s32
//                      accumulators, or kind::f16 on bf16) into one of the head's two S buffers in tensor
//                      memory, two tiles ahead of O += P V (kind::f16, P read from tensor memory, V^T from
//                      shared memory); completion is signalled with tcgen05.commit.
//   warps 0-3 / 4-7    softmax of head A / B, one thread per query row: tcgen05.ld of the 64 scores,
//                      scales / masks, online softmax in base 2 with a lazily updated maximum (the O
//                      accumulator is rescaled in tensor memory only when the maximum grows by more than
//                      2^8), P as bf16 pairs written back over the first 32 columns of the same S buffer,
//                      final O / l from tensor memory.
// Tensor memory (512 columns): S_A0 | S_A1 | S_B0 | S_B1 (64 each) | O_A | O_B (128 each).
// All shared-memory operands are K-major: V is transposed once per call by the preparation pass.
// Every wait is bounded and abortable; a failed wait raises bit 1 of the status word.
#include "hq_tc05.cuh"

namespace hq {

struct PrefillTcParams {
  const float* q_scale; const float* k_scale;      // [B,H_Q,Npad], [B,H_KV,Npad]
  const float* v_scale;                            // FP8 P V: [B,H_KV,128], one per channel
  const int* nv_valid;
  void* out; int out_dtype; int64_t o_sb, o_sh, o_sn;
  int B, H_Q, H_KV, N, Npad, W, T, Tpad, nqb, nkb;
  float sml;
  int* status;
};

constexpr int kTcThreads = 352;            // 2 x 4 softmax warps + producer warp + one MMA warp per head
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256; // S buffer of head h, parity s: kColS + 128 h + 64 s; O of head h: kColO + 128 h

constexpr int kKStages = 3;    // depth of the K ring: Q K^T runs two tiles ahead of P V and frees its slot at once
constexpr int kVStages = 4;    // depth of the V ring
constexpr int kKsSlots = 6;    // ring of key-scale rows: a row is dead once P V of its item + 2 has been issued
constexpr int kKsBytes = 768;  // 64 key scales | 64 bias terms of head A | 64 bias terms of head B
struct TcSmem {              // offsets from a 1024-aligned base
  static constexpr int Qi = 0;                             // 2 x 16 KB  [head][128 rows][128 B] int8
  static constexpr int Qb = 32768;                         // 2 x 32 KB  [head][2 halves][128 rows][128 B] bf16
  static constexpr int K = 98304;                          // kKStages x 16 KB: int8 tile, or two bf16 halves
  static constexpr int V = K + kKStages * 16384;           // kVStages x 16 KB: V^T [128 d rows][128 B]
  static constexpr int Ks = V + kVStages * 16384;          // kKsSlots x kKsBytes
  static constexpr int Bar = Ks + kKsSlots * kKsBytes;     // barriers + scratch
  static constexpr int Total = Bar + 256;
};

// two fp32 lanes per instruction (sm_100 packed forms)
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return d;
}

struct TcPlan {
  int n_rest, n_win, nvert0, nvert1, nheads;
  __device__ __forceinline__ int nvert(int h) const { return h ? nvert1 : nvert0; }
  __device__ __forceinline__ int n_ops() const { return nheads * (n_rest + n_win) + nvert0 + nvert1; }
  __device__ __forceinline__ int n_tiles(int h) const { return h < nheads ? n_rest + nvert(h) + n_win : 0; }
  __device__ __forceinline__ int n_items() const { return n_rest + nvert0 + nvert1 + n_win; }
};

// The ring items of a CTA in load order, walked with counters only (the threads that walk it are single
// lanes whose instruction latency paces the pipeline): the INT8 tiles, then the vertical-line tiles of the
// two heads interleaved (A's j-th, B's j-th, ...), then the window tiles.  INT8 and window items feed both
// heads, a vertical item only its own head.
struct TcItemIter {
  int kind;     // 0 INT8, 1 vertical, 2 window, 3 = past the end
  int j;        // index within the kind
  int hh;       // owning head of a vertical item
  int stage;    // ring slot
  int depth;    // ring depth
  uint32_t par; // phase parity of the slot's "full" barrier for this item
  __device__ __forceinline__ bool valid(const TcPlan& pl) const {
    return kind == 0 ? j < pl.n_rest : kind == 1 ? j < pl.nvert(hh) : j < pl.n_win;
  }
  __device__ __forceinline__ void step(const TcPlan& pl) {
    if (kind == 1) { if (++hh == 2) { hh = 0; ++j; } } else ++j;
    const int lim = kind == 0 ? pl.n_rest : kind == 1 ? max(pl.nvert0, pl.nvert1) : pl.n_win;
    if (j >= lim) { ++kind; j = 0; hh = 0; }
  }
  __device__ __forceinline__ void begin(const TcPlan& pl, int ring_depth) {
    kind = 0; j = 0; hh = 0; stage = 0; par = 0u; depth = ring_depth;
    while (kind < 3 && !valid(pl)) step(pl);
  }
  __device__ __forceinline__ void next(const TcPlan& pl) {
    if (++stage == depth) { stage = 0; par ^= 1u; }
    // the common cases first (the lanes that walk the ring are single threads: every instruction here is latency)
    if (kind == 0 && j + 1 < pl.n_rest) { ++j; return; }
    if (kind == 2) { if (++j >= pl.n_win) kind = 3; return; }
    do step(pl); while (kind < 3 && !valid(pl));
  }
  __device__ __forceinline__ bool done() const { return kind >= 3; }
  __device__ __forceinline__ bool feeds(int h) const { return kind != 1 || hh == h; }
};

// The rare tile of a row whose P values against the current reference may be too large (or that has no
// reference yet): take the true maximum of the tile from the scores in tensor memory, rescale O and the row sum
// if the reference moves, and write the tile's P against the reference as it then stands.  Called by whole
// warps; kept out of line so that the common path keeps its registers.
struct TcSlowResult { float m_ref, l; bool ok; };
// FP8 P V (the arithmetic of the reference's sm_90 kernel, vendor/sageattention/csrc/qattn/attn_utils.cuh:30,354-458 and
// qk_int_sv_f8_cuda_sm90.cu:259-364): P~ = 2^(s - m + 8.807) against the EXACT running maximum m (so P~ <= 448, the largest
// e4m3 value), the row sum taken in fp32 before P~ is rounded to e4m3.
constexpr float kFp8Offset = 8.807f;
template <bool kFp8>
__device__ __noinline__ TcSlowResult tc_slow_tile(uint32_t tS, uint32_t tO, const float4* ks4, const float4* kb4, bool is_i8,
                                                  float esc, uint32_t mlo, uint32_t mhi, float m_ref, float l,
                                                  uint64_t* pv_bar, uint32_t pv_parity, volatile int* abort_flag) {
  TcSlowResult res;
  res.ok = true;
  uint32_t sr[64];
  float x[64];
  tc::tmem_ld32(tS, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
  tc::tmem_ld32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
  tc::tmem_wait_ld();
  if (is_i8) {
#pragma unroll
    for (int c4 = 0; c4 < 16; ++c4) {
      const float4 kk = ks4[c4], bb = kb4[c4];
      x[4 * c4] = fmaf(__int_as_float((int)sr[4 * c4] + 0x4B400000), kk.x, bb.x);
      x[4 * c4 + 1] = fmaf(__int_as_float((int)sr[4 * c4 + 1] + 0x4B400000), kk.y, bb.y);
      x[4 * c4 + 2] = fmaf(__int_as_float((int)sr[4 * c4 + 2] + 0x4B400000), kk.z, bb.z);
      x[4 * c4 + 3] = fmaf(__int_as_float((int)sr[4 * c4 + 3] + 0x4B400000), kk.w, bb.w);
    }
  } else {
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const uint32_t mw = c < 32 ? mlo : mhi;
      x[c] = ((mw >> (c & 31)) & 1u) ? -INFINITY : __uint_as_float(sr[c]);
    }
  }
  float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 64; ++c) m4[c & 3] = fmaxf(m4[c & 3], x[c]);
  const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * esc;      // esc > 0
  // Once here, move the reference all the way up to the maximum seen: with the reference left below it,
  // every later tile with a few scores near that maximum would bring the row back here.
  const bool grow = mx > m_ref;                              // also true for the first finite maximum
  if (__any_sync(0xffffffffu, grow)) {
    const float alpha = (m_ref == -INFINITY) ? 0.f : ex2f(m_ref - mx);
    if (pv_bar != nullptr) {   // O must be quiescent: every P V of this head issued so far has to be complete
      res.ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(pv_bar, pv_parity, abort_flag));
      if (!res.ok) { res.m_ref = m_ref; res.l = l; return res; }
      tc::fence_after_sync();
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t o[32];
        tc::tmem_ld32(tO + ch * 32, o);
        tc::tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * (grow ? alpha : 1.f));
        tc::tmem_st32(tO + ch * 32, o);
      }
      tc::tmem_wait_st();
    }
    if (grow) { l *= alpha; m_ref = mx; }
  }
  const float mu = m_ref == -INFINITY ? 0.f : m_ref;
  float rs[4] = {0.f, 0.f, 0.f, 0.f};
  if constexpr (kFp8) {
    uint32_t pk[16];
    const float off = kFp8Offset - mu;
#pragma unroll
    for (int c = 0; c < 64; c += 4) {
      const float p0 = ex2f(fmaf(x[c], esc, off)), p1 = ex2f(fmaf(x[c + 1], esc, off));
      const float p2 = ex2f(fmaf(x[c + 2], esc, off)), p3 = ex2f(fmaf(x[c + 3], esc, off));
      rs[0] += p0; rs[1] += p1; rs[2] += p2; rs[3] += p3;
      pk[c >> 2] = tc::pack_e4m3x4(p0, p1, p2, p3);
    }
    tc::tmem_st16(tS, pk);
  } else {
    uint32_t pk[32];
#pragma unroll
    for (int c = 0; c < 64; c += 2) {
      const float p0 = ex2f(fmaf(x[c], esc, -mu)), p1 = ex2f(fmaf(x[c + 1], esc, -mu));
      rs[c & 3] += p0; rs[(c & 3) + 1] += p1;
      __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);       // low half = even column
      pk[c >> 1] = *reinterpret_cast<uint32_t*>(&hh);
    }
    tc::tmem_st32(tS, pk);
  }
  tc::tmem_wait_st();
  res.m_ref = m_ref;
  res.l = l + (rs[0] + rs[1]) + (rs[2] + rs[3]);
  return res;
}

template <bool kFp8>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap mQi, const __grid_constant__ CUtensorMap mQb,
                  const __grid_constant__ CUtensorMap mKi, const __grid_constant__ CUtensorMap mKb,
                  const __grid_constant__ CUtensorMap mVt, const __grid_constant__ CUtensorMap mXk,
                  const __grid_constant__ CUtensorMap mXv, const __grid_constant__ CUtensorMap mKs,
                  const __grid_constant__ CUtensorMap mKbs, const PrefillTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TcSmem::Bar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;                   // [kKStages]
  uint64_t* k_empty = k_full + kKStages;         // [kKStages]
  uint64_t* v_full = k_empty + kKStages;         // [kVStages]
  uint64_t* v_empty = v_full + kVStages;         // [kVStages]
  uint64_t* s_full = v_empty + kVStages;         // [head][2]
  uint64_t* p_ready = s_full + 4;                // [head][2]
  uint64_t* pv_done = p_ready + 4;               // [head][2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(pv_done + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  __shared__ int s_skip;
  if (tid == 0) s_skip = *reinterpret_cast<volatile int*>(p.status) & 2;
  __syncthreads();
  if (s_skip) return;                         // an earlier CTA gave up: drain the grid quickly
  const int R = p.H_Q / p.H_KV, pairs = (R + 1) / 2;
  const int qb = p.nqb - 1 - blockIdx.x;     // heavy blocks first
  const int hkv = blockIdx.y / pairs, pr = blockIdx.y - hkv * pairs, b = blockIdx.z;
  const int s0 = qb * 128;
  TcPlan plan;
  plan.nheads = (2 * pr + 1 < R) ? 2 : 1;
  const int64_t bhk = (int64_t)b * p.H_KV + hkv;
  const int64_t bhq0 = (int64_t)b * p.H_Q + hkv * R + 2 * pr;
  const int wla = p.W > 0 ? (max(0, s0 - (p.W - 1)) / 64) * 64 : s0;
  plan.n_rest = wla / 64;
  const int win_end = min(p.N, s0 + 128);
  plan.n_win = (win_end - wla + 63) / 64;
  const int nv0 = p.T > 0 ? p.nv_valid[bhq0 * p.nqb + qb] : 0;
  const int nv1 = (p.T > 0 && plan.nheads == 2) ? p.nv_valid[(bhq0 + 1) * p.nqb + qb] : 0;
  plan.nvert0 = (nv0 + 63) / 64;
  plan.nvert1 = (nv1 + 63) / 64;

  if (tid == 0) {
    mbar_init(q_full, 1);
    // a slot comes back when every head has arrived
    for (int i = 0; i < kKStages; ++i) { mbar_init(k_full + i, 1); mbar_init(k_empty + i, plan.nheads); }
    for (int i = 0; i < kVStages; ++i) { mbar_init(v_full + i, 1); mbar_init(v_empty + i, plan.nheads); }
    for (int i = 0; i < 4; ++i) { mbar_init(s_full + i, 1); mbar_init(p_ready + i, 128); mbar_init(pv_done + i, 1); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 8) tc::tmem_alloc(tmem_slot, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tc::tma_prefetch_desc(&mQi); tc::tma_prefetch_desc(&mQb); tc::tma_prefetch_desc(&mKi);
      tc::tma_prefetch_desc(&mKb); tc::tma_prefetch_desc(&mVt); tc::tma_prefetch_desc(&mKs); tc::tma_prefetch_desc(&mKbs);
      mbar_expect_tx(q_full, (uint32_t)plan.nheads * (16384 + 32768));
      for (int h = 0; h < plan.nheads; ++h) {
        const int qrow = (int)((bhq0 + h) * p.N + s0);
        tc::tma_load_2d(smem + TcSmem::Qi + h * 16384, &mQi, 0, qrow, q_full);
        tc::tma_load_2d(smem + TcSmem::Qb + h * 32768, &mQb, 0, qrow, q_full);
        tc::tma_load_2d(smem + TcSmem::Qb + h * 32768 + 16384, &mQb, 64, qrow, q_full);
      }
      // K tiles and V tiles travel in rings of their own: a K slot comes back as soon as both heads' Q K^T
      // of its item have run, a V slot only after their P V, so K runs further ahead than V.  One thread
      // feeds both rings and never blocks on either.
      TcItemIter ck, cv;
      ck.begin(plan, kKStages);
      cv.begin(plan, kVStages);
      int ks_slot = 0;
      uint32_t idle = 0;
      while (!ck.done() || !cv.done()) {
        bool progress = false;
        if (!ck.done() && mbar_test_wait(k_empty + ck.stage, ck.par ^ 1u)) {
          uint8_t* sK = smem + TcSmem::K + ck.stage * 16384;
          uint64_t* full = k_full + ck.stage;
          if (ck.kind == 0) {
            uint8_t* sS = smem + TcSmem::Ks + ks_slot * kKsBytes;
            mbar_expect_tx(full, 8192 + 256 + 256 * (uint32_t)plan.nheads);
            tc::tma_load_2d(sK, &mKi, 0, (int)(bhk * p.N + ck.j * 64), full);
            tc::tma_load_2d(sS, &mKs, ck.j * 64, (int)bhk, full);
            for (int h = 0; h < plan.nheads; ++h) tc::tma_load_2d(sS + 256 + 256 * h, &mKbs, ck.j * 64, (int)(bhq0 + h), full);
            if (++ks_slot == kKsSlots) ks_slot = 0;
          } else {
            const CUtensorMap* m = ck.kind == 1 ? &mXk : &mKb;
            const int krow = ck.kind == 1 ? (int)((bhq0 + ck.hh) * p.Tpad + ck.j * 64) : (int)(bhk * p.N + wla + ck.j * 64);
            mbar_expect_tx(full, 16384);
            tc::tma_load_2d(sK, m, 0, krow, full);
            tc::tma_load_2d(sK + 8192, m, 64, krow, full);
          }
          ck.next(plan);
          progress = true;
        }
        if (!cv.done() && mbar_test_wait(v_empty + cv.stage, cv.par ^ 1u)) {
          uint8_t* sV = smem + TcSmem::V + cv.stage * 16384;
          uint64_t* full = v_full + cv.stage;
          mbar_expect_tx(full, kFp8 ? 8192 : 16384);      // FP8: V^T tiles of 64 one-byte keys
          if (cv.kind == 1) tc::tma_load_2d(sV, &mXv, cv.j * 64, (int)((bhq0 + cv.hh) * 128), full);
          else tc::tma_load_2d(sV, &mVt, (cv.kind == 0 ? 0 : wla) + cv.j * 64, (int)(bhk * 128), full);
          cv.next(plan);
          progress = true;
        }
        if (progress) { idle = 0; continue; }
        __nanosleep(64);
        if (*abort_flag) break;
        if (++idle > 2000000u) { *abort_flag = 1; break; }
      }
    }
  } else if (warp >= 9) {
    // ------------------------------------------------------------ MMA issuers: warp 9 for head A, warp 10 for head B
    // One lane per head issues, in the head's own order, Q K^T of tiles 0 and 1, then for every tile t:
    // P V of t, Q K^T of t + 2.  The S buffer that Q K^T of t + 2 overwrites held P of tile t, and the tensor
    // core runs one thread's operations in issue order, so the scores of the next tile are ready while the
    // head's softmax threads are still on the current one.  Ring slots come back when both heads are done
    // with them: a head arrives by tcgen05.commit for an item it used and by a plain arrive for a
    // vertical-line item of the other head, in ring order either way.
    const int h = warp - 9;
    if (lane == 0 && h < plan.nheads) {
      constexpr uint32_t idesc_i8 = tc::make_idesc(2, tc::kFmtS8, tc::kFmtS8, 128, 64);
      constexpr uint32_t idesc_qk = tc::make_idesc(1, tc::kFmtBF16, tc::kFmtBF16, 128, 64);
      constexpr uint32_t idesc_pv = tc::make_idesc(1, tc::kFmtBF16, tc::kFmtBF16, 128, 128);
      constexpr uint32_t idesc_pv8 = tc::make_idesc(1, tc::kFmtE4M3, tc::kFmtE4M3, 128, 128);
      bool ok = tc::mbar_wait_abortable(q_full, 0, abort_flag, 100);
      // operand descriptors differ only in their start-address field (16-byte units)
      const uint64_t dQi = tc::smem_desc_k128(smem + TcSmem::Qi + h * 16384, 0);
      const uint64_t dQb = tc::smem_desc_k128(smem + TcSmem::Qb + h * 32768, 0);
      const uint64_t dK = tc::smem_desc_k128(smem + TcSmem::K, 0);
      const uint64_t dV = kFp8 ? tc::smem_desc_k64(smem + TcSmem::V, 0) : tc::smem_desc_k128(smem + TcSmem::V, 0);
      const uint32_t tS = tmem_base + kColS + 128u * h, tO = tmem_base + kColO + 128u * h;
      const int n_t = plan.n_tiles(h);
      TcItemIter cq, cp;
      cq.begin(plan, kKStages);
      cp.begin(plan, kVStages);
      int tq = 0;
      auto qk_next = [&]() {
        for (;;) {          // the next item that feeds this head; hand back the other head's on the way
          ok = tc::mbar_wait_abortable(k_full + cq.stage, cq.par, abort_flag);
          if (!ok) return;
          if (cq.feeds(h)) break;
          tc::mbar_arrive(k_empty + cq.stage);
          cq.next(plan);
        }
        tc::fence_after_sync();
        const uint32_t dS = tS + 64u * (tq & 1);
        const uint64_t bK = dK + (uint64_t)(cq.stage * 1024);
        if (cq.kind == 0) {
#pragma unroll
          for (int k = 0; k < 4; ++k) tc::mma_s8_ss(dS, dQi + 2 * k, bK + 2 * k, idesc_i8, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            tc::mma_bf16_ss(dS, dQb + (k >> 2) * 1024 + 2 * (k & 3), bK + (k >> 2) * 512 + 2 * (k & 3), idesc_qk, k > 0);
        }
        tc::mma_commit(s_full + 2 * h + (tq & 1));
        tc::mma_commit(k_empty + cq.stage);
        ++tq;
        cq.next(plan);
      };
      if (ok && n_t > 0) qk_next();
      if (ok && n_t > 1) qk_next();
      for (int t = 0; ok && t < n_t; ++t) {
        for (;;) {
          ok = tc::mbar_wait_abortable(v_full + cp.stage, cp.par, abort_flag);
          if (!ok || cp.feeds(h)) break;
          tc::mbar_arrive(v_empty + cp.stage);
          cp.next(plan);
        }
        if (!ok) break;
        const int sl = 2 * h + (t & 1);
        ok = tc::mbar_wait_abortable(p_ready + sl, (uint32_t)((t >> 1) & 1), abort_flag);
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t aP = tS + 64u * (t & 1);
        const uint64_t bV = dV + (uint64_t)(cp.stage * 1024);
        if constexpr (kFp8) {     // 64 keys = two K steps of 32 e4m3: 8 columns of P, 32 bytes of a V^T row each
#pragma unroll
          for (int k = 0; k < 2; ++k) tc::mma_f8_ts(tO, aP + 8 * k, bV + 2 * k, idesc_pv8, (t > 0 || k > 0) ? 1u : 0u);
        } else if (t > 0) {
#pragma unroll
          for (int k = 0; k < 4; ++k) tc::mma_bf16_ts(tO, aP + 8 * k, bV + 2 * k, idesc_pv, 1u);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) tc::mma_bf16_ts(tO, aP + 8 * k, bV + 2 * k, idesc_pv, k > 0);
        }
        tc::mma_commit(pv_done + sl);
        tc::mma_commit(v_empty + cp.stage);
        cp.next(plan);
        if (t + 2 < n_t) qk_next();
      }
    }
  } else {
    // ------------------------------------------------------------ softmax: one thread per query row and head
    // Warps 0-3 serve head A, warps 4-7 head B; warp w reaches the tensor-memory lanes 32 (w % 4) .. + 31.
    const int h = warp >> 2, wq = warp & 3;
    const int n_tiles = plan.n_tiles(h);
    const int r = wq * 32 + lane;            // query row inside the block = tensor-memory lane
    const int row = s0 + r;
    const int64_t bhq = bhq0 + (h < plan.nheads ? h : 0);
    const uint32_t lane_base = tmem_base + ((uint32_t)(wq * 32) << 16);
    const uint32_t colS = kColS + 128 * h, colO = kColO + 128 * h;
    const int n_rest = plan.n_rest, n_vert = plan.nvert(h), nvh = h ? nv1 : nv0;
    // rows past N compute on a token scale, so that a masked column (-inf) times the scale stays -inf
    const float qs = (row < p.N && n_tiles > 0) ? p.q_scale[bhq * p.Npad + row] : 1e-30f;
    float m_ref = row < p.N ? -INFINITY : 0.f, l = 0.f;
    bool ok = true;
    int ks_slot = 0;
    for (int t = 0; t < n_tiles; ++t) {
      const int slot = t & 1, sl = 2 * h + slot;
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(s_full + sl, (uint32_t)((t >> 1) & 1), abort_flag));
      if (!ok) break;
      tc::fence_after_sync();
      const bool is_i8 = t < n_rest;
      const float esc = is_i8 ? qs : p.sml;                  // > 0
      const float4* ks4 = reinterpret_cast<const float4*>(smem + TcSmem::Ks + ks_slot * kKsBytes);
      const float4* kb4 = ks4 + 16 + 16 * h;
      if (is_i8 && ++ks_slot == kKsSlots) ks_slot = 0;
      uint32_t mlo = 0u, mhi = 0u;                           // BF16 tiles: bit c set = column c (of 64) is masked
      if (!is_i8) {
        int lim;                                             // columns <= lim are visible
        if (t < n_rest + n_vert) lim = min(64, nvh - (t - n_rest) * 64) - 1;
        else lim = min(row, p.N - 1) - (wla + (t - n_rest - n_vert) * 64);
        mlo = lim >= 31 ? 0u : lim < 0 ? 0xFFFFFFFFu : (0xFFFFFFFFu << (lim + 1));
        mhi = lim >= 63 ? 0u : lim < 32 ? 0xFFFFFFFFu : (0xFFFFFFFFu << (lim - 31));
      }
      // One fused pass per tile: score -> exponent units -> 2^(y - mu) against the reference maximum as it
      // stands -> row sum and bf16 P, two columns per instruction where the hardware has packed fp32 forms.
      // The row maximum is not computed: a P value above 2^8 would show in the row sum of the tile, which
      // is then > 2^8.  Only then (and for a row's first finite scores) the scores are read from tensor
      // memory again, the maximum is taken, O is rescaled, the reference moves and the pass is repeated.
      if constexpr (kFp8) {
        // FP8 P V: the exact running maximum is part of the arithmetic (P~ must not pass 448), so the tile's row
        // maximum is taken first; a row whose maximum grows goes through the out-of-line path, which rescales O.
        uint32_t pk8[16];
        float lsum;
        bool grow;
        {
          uint32_t sr[64];
          tc::tmem_ld32(lane_base + colS + slot * 64, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
          tc::tmem_ld32(lane_base + colS + slot * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
          tc::tmem_wait_ld();
          float* y = reinterpret_cast<float*>(sr);            // the scores in exponent units, in place
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          if (is_i8) {
#pragma unroll
            for (int c4 = 0; c4 < 16; ++c4) {
              const float4 kk = ks4[c4], bb = kb4[c4];
              const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, bv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                y[4 * c4 + e] = fmaf(__int_as_float((int)sr[4 * c4 + e] + 0x4B400000), kv[e], bv[e]) * esc;
                mx4[e] = fmaxf(mx4[e], y[4 * c4 + e]);
              }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 64; ++c) {
              const uint32_t mw = c < 32 ? mlo : mhi;
              y[c] = ((mw >> (c & 31)) & 1u) ? -INFINITY : y[c] * esc;
              mx4[c & 3] = fmaxf(mx4[c & 3], y[c]);
            }
          }
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          grow = mx > m_ref;                                   // also true for a row's first finite maximum
          const float off = kFp8Offset - (m_ref == -INFINITY ? 0.f : m_ref);
          float rs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int c = 0; c < 64; c += 4) {
            const float p0 = ex2f(y[c] + off), p1 = ex2f(y[c + 1] + off), p2 = ex2f(y[c + 2] + off), p3 = ex2f(y[c + 3] + off);
            rs[0] += p0; rs[1] += p1; rs[2] += p2; rs[3] += p3;
            pk8[c >> 2] = tc::pack_e4m3x4(p0, p1, p2, p3);
          }
          lsum = (rs[0] + rs[1]) + (rs[2] + rs[3]);
        }
        if (__any_sync(0xffffffffu, grow)) {
          const bool wait_pv = t > 0;
          const TcSlowResult sr2 = tc_slow_tile<true>(lane_base + colS + slot * 64, lane_base + colO, ks4, kb4, is_i8, esc, mlo, mhi, m_ref, l,
                                                      wait_pv ? pv_done + 2 * h + ((t - 1) & 1) : nullptr, (uint32_t)(((t - 1) >> 1) & 1),
                                                      abort_flag);
          ok = sr2.ok;
          if (!ok) break;
          m_ref = sr2.m_ref;
          l = sr2.l;
        } else {
          l += lsum;
          // P~ as e4m3 over the first 16 columns of the S buffer just read: row r in lane r, keys 4c .. 4c+3 in column c
          tc::tmem_st16(lane_base + colS + slot * 64, pk8);
          tc::tmem_wait_st();
        }
      } else {
        uint32_t pk[32];
        float lsum;
        {
          uint32_t sr[64];
          tc::tmem_ld32(lane_base + colS + slot * 64, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
          tc::tmem_ld32(lane_base + colS + slot * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
          tc::tmem_wait_ld();
          const float mu = m_ref == -INFINITY ? 0.f : m_ref;
          const float2 esc2 = make_float2(esc, esc), nmu2 = make_float2(-mu, -mu);
          float2 rsa = make_float2(0.f, 0.f), rsb = make_float2(0.f, 0.f);
          if (is_i8) {
            float* y = reinterpret_cast<float*>(sr);
#pragma unroll
            for (int c4 = 0; c4 < 16; ++c4) {
              const float4 kk = ks4[c4], bb = kb4[c4];
              const float2 a01 = make_float2(__int_as_float((int)sr[4 * c4] + 0x4B400000), __int_as_float((int)sr[4 * c4 + 1] + 0x4B400000));
              const float2 a23 = make_float2(__int_as_float((int)sr[4 * c4 + 2] + 0x4B400000), __int_as_float((int)sr[4 * c4 + 3] + 0x4B400000));
              const float2 y01 = ffma2(ffma2(a01, make_float2(kk.x, kk.y), make_float2(bb.x, bb.y)), esc2, nmu2);
              const float2 y23 = ffma2(ffma2(a23, make_float2(kk.z, kk.w), make_float2(bb.z, bb.w)), esc2, nmu2);
              y[4 * c4] = y01.x; y[4 * c4 + 1] = y01.y; y[4 * c4 + 2] = y23.x; y[4 * c4 + 3] = y23.y;
            }
#pragma unroll
            for (int c = 0; c < 64; ++c) y[c] = ex2f(y[c]);
            float2 rsc = make_float2(0.f, 0.f), rsd = make_float2(0.f, 0.f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
              rsa = fadd2(rsa, make_float2(y[8 * c8], y[8 * c8 + 1]));
              rsb = fadd2(rsb, make_float2(y[8 * c8 + 2], y[8 * c8 + 3]));
              rsc = fadd2(rsc, make_float2(y[8 * c8 + 4], y[8 * c8 + 5]));
              rsd = fadd2(rsd, make_float2(y[8 * c8 + 6], y[8 * c8 + 7]));
            }
            rsa = fadd2(rsa, rsc); rsb = fadd2(rsb, rsd);
#pragma unroll
            for (int c2 = 0; c2 < 32; ++c2) {
              __nv_bfloat162 h0 = __floats2bfloat162_rn(y[2 * c2], y[2 * c2 + 1]);
              pk[c2] = *reinterpret_cast<uint32_t*>(&h0);
            }
          } else {
  #pragma unroll
            for (int c2 = 0; c2 < 32; ++c2) {
              const uint32_t mw = c2 < 16 ? mlo : mhi;
              float2 y = ffma2(make_float2(__uint_as_float(sr[2 * c2]), __uint_as_float(sr[2 * c2 + 1])), esc2, nmu2);
              if ((mw >> ((2 * c2) & 31)) & 1u) y.x = -INFINITY;
              if ((mw >> ((2 * c2 + 1) & 31)) & 1u) y.y = -INFINITY;
              const float2 pp = make_float2(ex2f(y.x), ex2f(y.y));
              if (c2 & 1) rsb = fadd2(rsb, pp); else rsa = fadd2(rsa, pp);
              __nv_bfloat162 h0 = __floats2bfloat162_rn(pp.x, pp.y);
              pk[c2] = *reinterpret_cast<uint32_t*>(&h0);
            }
          }
          lsum = (rsa.x + rsa.y) + (rsb.x + rsb.y);
        }
        const bool need = m_ref == -INFINITY || !(lsum <= 256.f);
        if (__any_sync(0xffffffffu, need)) {
          // out of line: the maximum, the move of the reference and the tile's P against the new reference
          const bool wait_pv = t > 0;
          const TcSlowResult sr2 = tc_slow_tile<false>(lane_base + colS + slot * 64, lane_base + colO, ks4, kb4, is_i8, esc, mlo, mhi, m_ref, l,
                                                wait_pv ? pv_done + 2 * h + ((t - 1) & 1) : nullptr, (uint32_t)(((t - 1) >> 1) & 1),
                                                abort_flag);
          ok = sr2.ok;
          if (!ok) break;
          m_ref = sr2.m_ref;
          l = sr2.l;
        } else {
          l += lsum;
          // P over the first 32 columns of the S buffer just read: row r in lane r, keys 2c, 2c+1 in column c
          tc::tmem_st32(lane_base + colS + slot * 64, pk);
          tc::tmem_wait_st();
        }
      }
      tc::fence_before_sync();
      tc::mbar_arrive(p_ready + sl);
    }
    // ---- epilogue: O / l
    if (ok && n_tiles > 0)
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(pv_done + 2 * h + ((n_tiles - 1) & 1), (uint32_t)(((n_tiles - 1) >> 1) & 1), abort_flag));
    if (ok && n_tiles > 0) {
      tc::fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const float* vsc = kFp8 ? p.v_scale + bhk * 128 : nullptr;        // FP8 P V: the channel scales of V come back here
      const int hq = (int)(bhq - (int64_t)b * p.H_Q);
      const int64_t base = b * p.o_sb + hq * p.o_sh + (int64_t)row * p.o_sn;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t o[32];
        tc::tmem_ld32(lane_base + colO + ch * 32, o);
        tc::tmem_wait_ld();
        if constexpr (kFp8) {
#pragma unroll
          for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * __ldg(vsc + ch * 32 + x));
        }
        if (row < p.N) {
          if (p.out_dtype == HQ_BF16) {
            uint32_t w[16];
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
              w[x] = *reinterpret_cast<uint32_t*>(&hh);
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + base + ch * 32);
#pragma unroll
            for (int x = 0; x < 4; ++x) dst[x] = make_uint4(w[4 * x], w[4 * x + 1], w[4 * x + 2], w[4 * x + 3]);
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x) store_out(p.out, base + ch * 32 + x, __uint_as_float(o[x]) * inv, p.out_dtype);
          }
        }
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(p.status, 2);
  if (warp == 8) tc::tmem_dealloc(tmem_base, kTmemCols);
}

// ---- preparation for the tensor-memory kernel: transposed V tiles ---------------------------
// v [B,H_KV,N,128] (strided) -> vt [B,H_KV,128,Npad] bf16, columns >= N zero
__global__ void __launch_bounds__(256)
transpose_v_kernel(const __nv_bfloat16* __restrict__ v, int64_t sb, int64_t sh, int64_t sn, int H, int N, int Npad,
                   __nv_bfloat16* __restrict__ vt) {
  __shared__ __nv_bfloat16 tile[64][130];
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, key0 = blockIdx.x * 64, tid = threadIdx.x;
  for (int x = tid; x < 64 * 16; x += 256) {
    const int r = x >> 4, c = (x & 15) * 8;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (key0 + r < N) raw = __ldg(reinterpret_cast<const uint4*>(v + b * sb + h * sh + (int64_t)(key0 + r) * sn + c));
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[r][c + j] = e[j];
  }
  __syncthreads();
  for (int x = tid; x < 128 * 8; x += 256) {
    const int d = x >> 3, k8 = (x & 7) * 8;
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = tile[k8 + j][d];
    *reinterpret_cast<uint4*>(vt + ((int64_t)bh * 128 + d) * Npad + key0 + k8) = *reinterpret_cast<uint4*>(o);
  }
}

// gathered vertical rows: xk [B,H_Q,Tpad,128] (rows >= T zero), xvt [B,H_Q,128,Tpad] (transposed V rows)
__global__ void __launch_bounds__(256)
vertical_gather_t_kernel(const int* __restrict__ vasc, int T, int Tpad, int N, int H_Q, int H_KV,
                         const __nv_bfloat16* __restrict__ k_bf,
                         const __nv_bfloat16* __restrict__ v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                         __nv_bfloat16* __restrict__ xk, __nv_bfloat16* __restrict__ xvt) {
  __shared__ __nv_bfloat16 tile[64][130];
  const int64_t bhq = blockIdx.y;
  const int b = (int)(bhq / H_Q), hq = (int)(bhq - (int64_t)b * H_Q), hkv = hq / (H_Q / H_KV);
  const int j0 = blockIdx.x * 64, tid = threadIdx.x;
  for (int x = tid; x < 64 * 16; x += 256) {
    const int r = x >> 4, c = (x & 15) * 8;
    uint4 kr = make_uint4(0, 0, 0, 0), vr = make_uint4(0, 0, 0, 0);
    if (j0 + r < T) {
      const int src = min(max(vasc[bhq * T + j0 + r], 0), N - 1);
      kr = __ldg(reinterpret_cast<const uint4*>(k_bf + (((int64_t)b * H_KV + hkv) * N + src) * 128 + c));
      vr = __ldg(reinterpret_cast<const uint4*>(v + b * v_sb + hkv * v_sh + (int64_t)src * v_sn + c));
    }
    *reinterpret_cast<uint4*>(xk + (bhq * Tpad + j0 + r) * 128 + c) = kr;
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&vr);
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[r][c + j] = e[j];
  }
  __syncthreads();
  for (int x = tid; x < 128 * 8; x += 256) {
    const int d = x >> 3, k8 = (x & 7) * 8;
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = tile[k8 + j][d];
    *reinterpret_cast<uint4*>(xvt + (bhq * 128 + d) * Tpad + j0 + k8) = *reinterpret_cast<uint4*>(o);
  }
}

int prefill_tc_launch(const hq_prefill_args* a, cudaStream_t st) {
  const int N = a->N, Npad = (N + 63) / 64 * 64, T = a->T, Tpad = (T + 63) / 64 * 64;
  CUtensorMap mQi, mQb, mKi, mKb, mVt, mXk, mXv, mKs, mKbs;
  const uint64_t qrows = (uint64_t)a->B * a->H_Q * N, krows = (uint64_t)a->B * a->H_KV * N;
  int rc;
  if ((rc = tc::make_map_2d(&mQi, a->q_i8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128, qrows, 128, 128, 128))) return rc;
  if ((rc = tc::make_map_2d(&mQb, a->q_bf, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, qrows, 256, 64, 128))) return rc;
  if ((rc = tc::make_map_2d(&mKi, a->k_i8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128, krows, 128, 128, 64))) return rc;
  if ((rc = tc::make_map_2d(&mKb, a->k_bf, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, krows, 256, 64, 64))) return rc;
  const bool fp8 = a->pv_fp8 != 0;
  if (fp8) {       // V^T as e4m3 bytes: 64-key tiles are 64-byte rows, 64-byte swizzle
    if ((rc = tc::make_map_2d(&mVt, a->v_t8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)Npad, (uint64_t)a->B * a->H_KV * 128,
                              (uint64_t)Npad, 64, 128, 64))) return rc;
  } else if ((rc = tc::make_map_2d(&mVt, a->v_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)Npad, (uint64_t)a->B * a->H_KV * 128,
                                   (uint64_t)Npad * 2, 64, 128))) return rc;
  if ((rc = tc::make_map_2d(&mKs, a->k_scale, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)Npad, (uint64_t)a->B * a->H_KV,
                            (uint64_t)Npad * 4, 64, 1, false))) return rc;
  if ((rc = tc::make_map_2d(&mKbs, a->k_bias, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)Npad, (uint64_t)a->B * a->H_Q,
                            (uint64_t)Npad * 4, 64, 1, false))) return rc;
  if (T > 0) {
    if ((rc = tc::make_map_2d(&mXk, a->vert_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, (uint64_t)a->B * a->H_Q * Tpad, 256, 64, 64))) return rc;
    if (fp8) {
      if ((rc = tc::make_map_2d(&mXv, a->vert_vt8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)Tpad, (uint64_t)a->B * a->H_Q * 128,
                                (uint64_t)Tpad, 64, 128, 64))) return rc;
    } else if ((rc = tc::make_map_2d(&mXv, a->vert_vt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)Tpad, (uint64_t)a->B * a->H_Q * 128,
                                     (uint64_t)Tpad * 2, 64, 128))) return rc;
  } else {
    mXk = mKb; mXv = mVt;
  }
  PrefillTcParams p{};
  p.q_scale = a->q_scale; p.k_scale = a->k_scale; p.v_scale = a->v_scale8;
  p.nv_valid = a->nv_valid;
  p.out = a->out; p.out_dtype = a->out_dtype; p.o_sb = a->o_sb; p.o_sh = a->o_sh; p.o_sn = a->o_sn;
  p.B = a->B; p.H_Q = a->H_Q; p.H_KV = a->H_KV; p.N = N; p.Npad = Npad; p.W = a->window; p.T = T; p.Tpad = Tpad;
  p.nqb = (N + 127) / 128; p.nkb = (N + 63) / 64;
  p.sml = a->sm_scale * 1.44269504f;
  p.status = a->status;
  const size_t smem = TcSmem::Total + 1024;
  static thread_local int attr_dev = -1;
  int dev = 0;
  HQ_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    HQ_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    HQ_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_dev = dev;
  }
  const int R = a->H_Q / a->H_KV;
  dim3 grid((unsigned)p.nqb, (unsigned)(a->H_KV * ((R + 1) / 2)), (unsigned)a->B);   // two query heads of a KV group per CTA
  if (fp8) prefill_tc_kernel<true><<<grid, kTcThreads, smem, st>>>(mQi, mQb, mKi, mKb, mVt, mXk, mXv, mKs, mKbs, p);
  else prefill_tc_kernel<false><<<grid, kTcThreads, smem, st>>>(mQi, mQb, mKi, mKb, mVt, mXk, mXv, mKs, mKbs, p);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

// ---- FP8 P V: V^T as e4m3 with one scale per channel ----------------------------------------------------------
// The reference's per_channel_fp8 (vendor/sageattention/quant.py:134-166 with MeanScaleKernel, csrc/fused/fused.cu:318-429,
// smooth_v off): scale[b, h, d] = max_n |v[b, h, n, d]| / 448, code = e4m3(v * (448 / max)), stored transposed.
__global__ void __launch_bounds__(256)
v_amax_kernel(const __nv_bfloat16* __restrict__ v, int64_t sb, int64_t sh, int64_t sn, int H, int N, unsigned* __restrict__ amax_bits) {
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int d = threadIdx.x & 127, half = threadIdx.x >> 7;
  const int rows_per = (N + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per, r1 = min(N, r0 + rows_per);
  const __nv_bfloat16* base = v + b * sb + h * sh + d;
  float m = 0.f;
  for (int r = r0 + half; r < r1; r += 2) m = fmaxf(m, fabsf(__bfloat162float(base[(int64_t)r * sn])));
  atomicMax(amax_bits + (int64_t)bh * 128 + d, __float_as_uint(m));       // non-negative floats order like their bit patterns
}

// v [B,H_KV,N,128] (strided) -> vt8 [B,H_KV,128,Npad] e4m3 (columns >= N zero), scale [B,H_KV,128] = amax / 448
__global__ void __launch_bounds__(256)
transpose_v_fp8_kernel(const __nv_bfloat16* __restrict__ v, int64_t sb, int64_t sh, int64_t sn, int H, int N, int Npad,
                       const unsigned* __restrict__ amax_bits, uint8_t* __restrict__ vt8, float* __restrict__ scale) {
  __shared__ float tile[64][129];
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, key0 = blockIdx.x * 64, tid = threadIdx.x;
  for (int x = tid; x < 64 * 16; x += 256) {
    const int r = x >> 4, c = (x & 15) * 8;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (key0 + r < N) raw = __ldg(reinterpret_cast<const uint4*>(v + b * sb + h * sh + (int64_t)(key0 + r) * sn + c));
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[r][c + j] = __bfloat162float(e[j]);
  }
  __syncthreads();
  for (int x = tid; x < 128 * 4; x += 256) {
    const int d = x >> 2, k16 = (x & 3) * 16;
    const float amax = __uint_as_float(amax_bits[(int64_t)bh * 128 + d]);
    const float recip = amax > 0.f ? 448.f / amax : 0.f;
    if (blockIdx.x == 0 && k16 == 0) scale[(int64_t)bh * 128 + d] = amax / 448.f;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w[j] = tc::pack_e4m3x4(tile[k16 + 4 * j][d] * recip, tile[k16 + 4 * j + 1][d] * recip, tile[k16 + 4 * j + 2][d] * recip,
                             tile[k16 + 4 * j + 3][d] * recip);
    *reinterpret_cast<uint4*>(vt8 + ((int64_t)bh * 128 + d) * Npad + key0 + k16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// gathered vertical-line rows of V for FP8 P V: xvt8 [B,H_Q,128,Tpad] e4m3 (transposed; columns >= T zero), quantised with
// the kv-head's channel scales like the rest of V
__global__ void __launch_bounds__(256)
vertical_gather_v_fp8_kernel(const int* __restrict__ vasc, int T, int Tpad, int N, int H_Q, int H_KV,
                             const __nv_bfloat16* __restrict__ v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                             const float* __restrict__ v_scale, uint8_t* __restrict__ xvt8) {
  __shared__ float tile[64][129];
  const int64_t bhq = blockIdx.y;
  const int b = (int)(bhq / H_Q), hq = (int)(bhq - (int64_t)b * H_Q), hkv = hq / (H_Q / H_KV);
  const int j0 = blockIdx.x * 64, tid = threadIdx.x;
  for (int x = tid; x < 64 * 16; x += 256) {
    const int r = x >> 4, c = (x & 15) * 8;
    uint4 vr = make_uint4(0, 0, 0, 0);
    if (j0 + r < T) {
      const int src = min(max(vasc[bhq * T + j0 + r], 0), N - 1);
      vr = __ldg(reinterpret_cast<const uint4*>(v + b * v_sb + hkv * v_sh + (int64_t)src * v_sn + c));
    }
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&vr);
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[r][c + j] = __bfloat162float(e[j]);
  }
  __syncthreads();
  for (int x = tid; x < 128 * 4; x += 256) {
    const int d = x >> 2, k16 = (x & 3) * 16;
    const float sc = v_scale[((int64_t)b * H_KV + hkv) * 128 + d];
    const float recip = sc > 0.f ? 1.f / sc : 0.f;          // 448 / amax, the factor the V codes were formed with
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w[j] = tc::pack_e4m3x4(tile[k16 + 4 * j][d] * recip, tile[k16 + 4 * j + 1][d] * recip, tile[k16 + 4 * j + 2][d] * recip,
                             tile[k16 + 4 * j + 3][d] * recip);
    *reinterpret_cast<uint4*>(xvt8 + (bhq * 128 + d) * Tpad + j0 + k16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

int prefill_tc_gather_v_fp8(const int32_t* vasc, int B, int H_Q, int H_KV, int N, int T, const void* v, int64_t v_sb, int64_t v_sh,
                            int64_t v_sn, const float* v_scale, void* xvt8, cudaStream_t st) {
  const int Tpad = (T + 63) / 64 * 64;
  vertical_gather_v_fp8_kernel<<<dim3(Tpad / 64, B * H_Q), 256, 0, st>>>(vasc, T, Tpad, N, H_Q, H_KV, (const __nv_bfloat16*)v, v_sb,
                                                                        v_sh, v_sn, v_scale, (uint8_t*)xvt8);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

int prefill_tc_prepare_v_fp8(const void* v, int64_t sb, int64_t sh, int64_t sn, int B, int H_KV, int N, void* v_t8, float* v_scale,
                             void* amax_scratch, cudaStream_t st) {
  const int Npad = (N + 63) / 64 * 64;
  HQ_CUDA(cudaMemsetAsync(amax_scratch, 0, (size_t)B * H_KV * 128 * 4, st));
  v_amax_kernel<<<dim3(64, B * H_KV), 256, 0, st>>>((const __nv_bfloat16*)v, sb, sh, sn, H_KV, N, (unsigned*)amax_scratch);
  transpose_v_fp8_kernel<<<dim3(Npad / 64, B * H_KV), 256, 0, st>>>((const __nv_bfloat16*)v, sb, sh, sn, H_KV, N, Npad,
                                                                   (const unsigned*)amax_scratch, (uint8_t*)v_t8, v_scale);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

int prefill_tc_prepare_v(const void* v, int64_t sb, int64_t sh, int64_t sn, int B, int H_KV, int N, void* v_t, cudaStream_t st) {
  const int Npad = (N + 63) / 64 * 64;
  transpose_v_kernel<<<dim3(Npad / 64, B * H_KV), 256, 0, st>>>((const __nv_bfloat16*)v, sb, sh, sn, H_KV, N, Npad,
                                                               (__nv_bfloat16*)v_t);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

int prefill_tc_prepare_vertical(const int32_t* vasc, int B, int H_Q, int H_KV, int N, int T, const void* k_bf, const void* v,
                                int64_t v_sb, int64_t v_sh, int64_t v_sn, void* xk, void* xvt, cudaStream_t st) {
  const int Tpad = (T + 63) / 64 * 64;
  vertical_gather_t_kernel<<<dim3(Tpad / 64, B * H_Q), 256, 0, st>>>(vasc, T, Tpad, N, H_Q, H_KV, (const __nv_bfloat16*)k_bf,
                                                                    (const __nv_bfloat16*)v, v_sb, v_sh, v_sn,
                                                                    (__nv_bfloat16*)xk, (__nv_bfloat16*)xvt);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

}  // namespace hq
