// Hybrid-precision causal prefill attention on the Blackwell tensor path.
//
// Tile semantics as stated in hq_prefill.cu's header: for the 128-query
// block at s of query head h, keys below wla(s) are INT8 unless they are vertical lines of h
// (masked here, served from gathered BF16 tiles), keys in [wla(s), s + 128) are BF16 + causal mask.
//
// One CTA works on the same 128 queries of TWO query heads of one KV group (A and B), so every INT8 and
// window K / V tile that reaches shared memory feeds two score tiles, and the two heads' softmax chains
// interleave on the SM: while one head's threads are in their exponentials the tensor core runs the other
// head's products.  10 warps:
//   warp 8 (one lane)  producer: TMA tensor-map loads (128-byte swizzle) of both heads' Q once and of one
//                      item (a K tile + a transposed V tile) per step into a four-slot ring.  INT8 and
//                      window items serve both heads; the gathered vertical-line tiles are per head.
//   warp 9 (one lane)  issues tcgen05.mma in a fixed order of (head, tile) operations: S = Q K^T
//                      (kind::i8 with s32 accumulators, or kind::f16 on bf16) into one of the head's two
//                      S buffers in tensor memory, two operations ahead of O += P V (kind::f16, P read
//                      from tensor memory, V^T from shared memory); completion is signalled with
//                      tcgen05.commit.
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
  const unsigned long long* vmask; const int* nv_valid;
  void* out; int out_dtype; int64_t o_sb, o_sh, o_sn;
  int B, H_Q, H_KV, N, Npad, W, T, Tpad, nqb, nkb;
  float sml;
  int* status;
};

constexpr int kTcThreads = 320;            // 2 x 4 softmax warps + producer warp + MMA warp
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256; // S buffer of head h, parity s: kColS + 128 h + 64 s; O of head h: kColO + 128 h
constexpr float kTcLazy = 8.0f;

constexpr int kKvStages = 4;   // item ring depth: loads run this many items ahead of the MMAs
struct TcSmem {              // offsets from a 1024-aligned base
  static constexpr int Qi = 0;                             // 2 x 16 KB  [head][128 rows][128 B] int8
  static constexpr int Qb = 32768;                         // 2 x 32 KB  [head][2 halves][128 rows][128 B] bf16
  static constexpr int KV = 98304;                         // kKvStages x 32 KB: K 16 KB (int8 tile + scales at 8192,
                                                           // or two bf16 halves) | V^T 16 KB [128 d rows][128 B]
  static constexpr int Bar = KV + kKvStages * 32768;       // barriers + scratch
  static constexpr int Total = Bar + 512;
};

// One (head, tile) operation of the MMA issuer's fixed order.
struct TcOp {
  int h;        // head 0 / 1
  int item;     // ring item that holds its K / V
  int t;        // tile index within the head's own sequence
  int kind;     // 0 INT8, 1 vertical, 2 window
  bool first;   // first operation that uses the item (waits for the load)
  bool last;    // last operation that uses the item (frees the slot)
};

struct TcPlan {
  int n_rest, n_win, nvert[2], nheads;
  __device__ __forceinline__ int n_ops() const { return nheads * (n_rest + n_win) + nvert[0] + nvert[1]; }
  __device__ __forceinline__ int n_tiles(int h) const { return h < nheads ? n_rest + nvert[h] + n_win : 0; }
  __device__ __forceinline__ TcOp op(int n) const {
    TcOp o;
    const int a = nheads * n_rest;
    if (n < a) {
      o.kind = 0; o.item = n / nheads; o.h = n - o.item * nheads; o.t = o.item;
      o.first = o.h == 0; o.last = o.h == nheads - 1;
      return o;
    }
    n -= a;
    const int nvs = nvert[0] + nvert[1];
    if (n < nvs) {
      const int mn = min(nvert[0], nvert[1]);
      int j;
      if (n < 2 * mn) { j = n >> 1; o.h = n & 1; }
      else { j = mn + (n - 2 * mn); o.h = nvert[0] > nvert[1] ? 0 : 1; }
      o.kind = 1; o.item = n_rest + n; o.t = n_rest + j; o.first = true; o.last = true;
      return o;
    }
    n -= nvs;
    const int w = n / nheads;
    o.kind = 2; o.h = n - w * nheads; o.item = n_rest + nvs + w; o.t = n_rest + nvert[o.h] + w;
    o.first = o.h == 0; o.last = o.h == nheads - 1;
    return o;
  }
};

__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap mQi, const __grid_constant__ CUtensorMap mQb,
                  const __grid_constant__ CUtensorMap mKi, const __grid_constant__ CUtensorMap mKb,
                  const __grid_constant__ CUtensorMap mVt, const __grid_constant__ CUtensorMap mXk,
                  const __grid_constant__ CUtensorMap mXv, const __grid_constant__ CUtensorMap mKs,
                  const PrefillTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TcSmem::Bar);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;                  // [kKvStages]
  uint64_t* kv_empty = kv_full + kKvStages;      // [kKvStages]
  uint64_t* s_full = kv_empty + kKvStages;       // [head][2]
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
  int nv[2] = {0, 0};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (p.T > 0 && h < plan.nheads) nv[h] = p.nv_valid[(bhq0 + h) * p.nqb + qb];
    plan.nvert[h] = (nv[h] + 63) / 64;
  }

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kKvStages; ++i) { mbar_init(kv_full + i, 1); mbar_init(kv_empty + i, 1); }
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
      tc::tma_prefetch_desc(&mKb); tc::tma_prefetch_desc(&mVt); tc::tma_prefetch_desc(&mKs);
      mbar_expect_tx(q_full, (uint32_t)plan.nheads * (16384 + 32768));
      for (int h = 0; h < plan.nheads; ++h) {
        const int qrow = (int)((bhq0 + h) * p.N + s0);
        tc::tma_load_2d(smem + TcSmem::Qi + h * 16384, &mQi, 0, qrow, q_full);
        tc::tma_load_2d(smem + TcSmem::Qb + h * 32768, &mQb, 0, qrow, q_full);
        tc::tma_load_2d(smem + TcSmem::Qb + h * 32768 + 16384, &mQb, 64, qrow, q_full);
      }
      int it = 0;
      bool ok = true;
      auto acquire = [&]() -> uint8_t* {
        const int slot = it % kKvStages;
        ok = tc::mbar_wait_abortable(kv_empty + slot, (uint32_t)(((it / kKvStages) & 1) ^ 1), abort_flag, 200);
        return smem + TcSmem::KV + slot * 32768;
      };
      for (int i = 0; ok && i < plan.n_rest; ++i) {
        uint8_t* sK = acquire();
        if (!ok) break;
        uint64_t* full = kv_full + it % kKvStages;
        const int key0 = i * 64;
        mbar_expect_tx(full, 8192 + 256 + 16384);
        tc::tma_load_2d(sK, &mKi, 0, (int)(bhk * p.N + key0), full);
        tc::tma_load_2d(sK + 8192, &mKs, key0, (int)bhk, full);          // the tile's 64 key scales
        tc::tma_load_2d(sK + 16384, &mVt, key0, (int)(bhk * 128), full);
        ++it;
      }
      const int nvmax = max(plan.nvert[0], plan.nvert[1]);
      for (int j = 0; ok && j < nvmax; ++j) {
        for (int h = 0; ok && h < 2; ++h) {
          if (j >= plan.nvert[h]) continue;
          uint8_t* sK = acquire();
          if (!ok) break;
          uint64_t* full = kv_full + it % kKvStages;
          const int j0 = j * 64;
          mbar_expect_tx(full, 16384 + 16384);
          tc::tma_load_2d(sK, &mXk, 0, (int)((bhq0 + h) * p.Tpad + j0), full);
          tc::tma_load_2d(sK + 8192, &mXk, 64, (int)((bhq0 + h) * p.Tpad + j0), full);
          tc::tma_load_2d(sK + 16384, &mXv, j0, (int)((bhq0 + h) * 128), full);
          ++it;
        }
      }
      for (int w = 0; ok && w < plan.n_win; ++w) {
        uint8_t* sK = acquire();
        if (!ok) break;
        uint64_t* full = kv_full + it % kKvStages;
        const int key0 = wla + w * 64;
        mbar_expect_tx(full, 16384 + 16384);
        tc::tma_load_2d(sK, &mKb, 0, (int)(bhk * p.N + key0), full);
        tc::tma_load_2d(sK + 8192, &mKb, 64, (int)(bhk * p.N + key0), full);
        tc::tma_load_2d(sK + 16384, &mVt, key0, (int)(bhk * 128), full);
        ++it;
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_i8 = tc::make_idesc(2, tc::kFmtS8, tc::kFmtS8, 128, 64);
      constexpr uint32_t idesc_qk = tc::make_idesc(1, tc::kFmtBF16, tc::kFmtBF16, 128, 64);
      constexpr uint32_t idesc_pv = tc::make_idesc(1, tc::kFmtBF16, tc::kFmtBF16, 128, 128);
      bool ok = tc::mbar_wait_abortable(q_full, 0, abort_flag, 100);
      const int n_ops = plan.n_ops();
      auto issue_qk = [&](int n) {
        const TcOp o = plan.op(n);
        const int kvs = o.item % kKvStages;
        if (o.first) {
          ok = tc::mbar_wait_abortable(kv_full + kvs, (uint32_t)((o.item / kKvStages) & 1), abort_flag, 40);
          if (!ok) return;
        }
        tc::fence_after_sync();
        const uint32_t dS = tmem_base + kColS + (uint32_t)(128 * o.h + 64 * (o.t & 1));
        const uint8_t* sK = smem + TcSmem::KV + kvs * 32768;
        if (o.kind == 0) {
          const uint8_t* sQ = smem + TcSmem::Qi + o.h * 16384;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc::mma_s8_ss(dS, tc::smem_desc_k128(sQ, k * 32), tc::smem_desc_k128(sK, k * 32), idesc_i8, k > 0);
        } else {
          const uint8_t* sQ = smem + TcSmem::Qb + o.h * 32768;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            tc::mma_bf16_ss(dS, tc::smem_desc_k128(sQ + (k >> 2) * 16384, (k & 3) * 32),
                            tc::smem_desc_k128(sK + (k >> 2) * 8192, (k & 3) * 32), idesc_qk, k > 0);
        }
        tc::mma_commit(s_full + 2 * o.h + (o.t & 1));
      };
      auto issue_pv = [&](int n) {
        const TcOp o = plan.op(n);
        const int kvs = o.item % kKvStages, sl = 2 * o.h + (o.t & 1);
        ok = tc::mbar_wait_abortable(p_ready + sl, (uint32_t)((o.t >> 1) & 1), abort_flag, 40);
        if (!ok) return;
        tc::fence_after_sync();
        const uint32_t dO = tmem_base + kColO + (uint32_t)(128 * o.h);
        const uint32_t aP = tmem_base + kColS + (uint32_t)(128 * o.h + 64 * (o.t & 1));
        const uint8_t* sV = smem + TcSmem::KV + kvs * 32768 + 16384;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc::mma_bf16_ts(dO, aP + 8 * k, tc::smem_desc_k128(sV, k * 32), idesc_pv, (o.t > 0 || k > 0) ? 1u : 0u);
        tc::mma_commit(pv_done + sl);
        if (o.last) tc::mma_commit(kv_empty + kvs);
      };
      if (ok && n_ops > 0) issue_qk(0);
      if (ok && n_ops > 1) issue_qk(1);
      for (int n = 0; ok && n < n_ops; ++n) {
        issue_pv(n);
        if (ok && n + 2 < n_ops) issue_qk(n + 2);
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
    const int n_rest = plan.n_rest, n_vert = plan.nvert[h], nvh = nv[h];
    const float qs = (row < p.N && n_tiles > 0) ? p.q_scale[bhq * p.Npad + row] : 0.f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // the vertical-mask word of a tile is a fresh cache line every step: fetch it one step ahead
    const unsigned long long* vmrow = p.vmask + bhq * p.nkb;
    unsigned long long vm_next = (p.T > 0 && n_rest > 0 && n_tiles > 0) ? __ldg(vmrow) : 0ull;
    for (int t = 0; t < n_tiles; ++t) {
      const int slot = t & 1, sl = 2 * h + slot;
      const unsigned long long vm64 = vm_next;
      if (p.T > 0 && t + 1 < n_rest) vm_next = __ldg(vmrow + t + 1);
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(s_full + sl, (uint32_t)((t >> 1) & 1), abort_flag));
      if (!ok) break;
      tc::fence_after_sync();
      uint32_t sr[64];
      tc::tmem_ld32(lane_base + colS + slot * 64, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
      tc::tmem_ld32(lane_base + colS + slot * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
      tc::tmem_wait_ld();

      // scores in the exponent's units: v[c] * esc - mu, with esc folded into one FFMA per element
      float v[64];
      float esc;
      if (t < n_rest) {
        const float4* ks4 = reinterpret_cast<const float4*>(smem + TcSmem::KV + (t % kKvStages) * 32768 + 8192);
        esc = qs;
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 kk = ks4[c4];
          const float kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int c = 4 * c4 + x;
            // int32 -> float without the conversion unit: |score| < 2^22
            v[c] = (__int_as_float((int)sr[c] + 0x4B400000) - 12582912.0f) * kv[x];
          }
        }
        if (vm64 != 0ull) {
          const uint32_t lo = (uint32_t)vm64, hi = (uint32_t)(vm64 >> 32);
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if ((lo >> c) & 1u) v[c] = -INFINITY;
            if ((hi >> c) & 1u) v[32 + c] = -INFINITY;
          }
        }
      } else {
        esc = p.sml;
#pragma unroll
        for (int c = 0; c < 64; ++c) v[c] = __uint_as_float(sr[c]);
        int lim;                                             // columns <= lim are visible
        if (t < n_rest + n_vert) lim = min(64, nvh - (t - n_rest) * 64) - 1;
        else lim = min(row, p.N - 1) - (wla + (t - n_rest - n_vert) * 64);
        if (__any_sync(0xffffffffu, lim < 63)) {
#pragma unroll
          for (int c = 0; c < 64; ++c) if (c > lim) v[c] = -INFINITY;
        }
      }
      float mx;
      {
        float m8[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) m8[x] = v[x];
#pragma unroll
        for (int c = 8; c < 64; ++c) m8[c & 7] = fmaxf(m8[c & 7], v[c]);
        mx = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
      }
      mx *= esc;                                             // esc >= 0
      if (esc == 0.f) mx = -INFINITY;                        // rows past N
      const bool grow = mx > m_ref + kTcLazy;                // also true for the first finite maximum
      if (__any_sync(0xffffffffu, grow)) {
        const float nm = grow ? mx : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2f(m_ref - nm);
        if (t > 0) {     // O must be quiescent: every P V of this head issued so far has to be complete
          ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(pv_done + 2 * h + ((t - 1) & 1), (uint32_t)(((t - 1) >> 1) & 1), abort_flag));
          if (!ok) break;
          tc::fence_after_sync();
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[32];
            tc::tmem_ld32(lane_base + colO + ch * 32, o);
            tc::tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * (grow ? alpha : 1.f));
            tc::tmem_st32(lane_base + colO + ch * 32, o);
          }
          tc::tmem_wait_st();
        }
        if (grow) { l *= alpha; m_ref = nm; }
      }
      const float mu = m_ref == -INFINITY ? 0.f : m_ref;
      uint32_t pk[32];
      float rs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ex2f(fmaf(v[c], esc, -mu)), p1 = ex2f(fmaf(v[c + 1], esc, -mu));
        rs[c & 3] += p0; rs[(c & 3) + 1] += p1;
        __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);   // low half = even column
        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&hh);
      }
      l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
      // P over the first 32 columns of the S buffer just read: row r in lane r, keys 2c, 2c+1 in column c
      tc::tmem_st32(lane_base + colS + slot * 64, pk);
      tc::tmem_wait_st();
      tc::fence_before_sync();
      tc::mbar_arrive(p_ready + sl);
    }
    // ---- epilogue: O / l
    if (ok && n_tiles > 0)
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(pv_done + 2 * h + ((n_tiles - 1) & 1), (uint32_t)(((n_tiles - 1) >> 1) & 1), abort_flag));
    if (ok && n_tiles > 0) {
      tc::fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int hq = (int)(bhq - (int64_t)b * p.H_Q);
      const int64_t base = b * p.o_sb + hq * p.o_sh + (int64_t)row * p.o_sn;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t o[32];
        tc::tmem_ld32(lane_base + colO + ch * 32, o);
        tc::tmem_wait_ld();
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
  CUtensorMap mQi, mQb, mKi, mKb, mVt, mXk, mXv, mKs;
  const uint64_t qrows = (uint64_t)a->B * a->H_Q * N, krows = (uint64_t)a->B * a->H_KV * N;
  int rc;
  if ((rc = tc::make_map_2d(&mQi, a->q_i8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128, qrows, 128, 128, 128))) return rc;
  if ((rc = tc::make_map_2d(&mQb, a->q_bf, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, qrows, 256, 64, 128))) return rc;
  if ((rc = tc::make_map_2d(&mKi, a->k_i8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128, krows, 128, 128, 64))) return rc;
  if ((rc = tc::make_map_2d(&mKb, a->k_bf, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, krows, 256, 64, 64))) return rc;
  if ((rc = tc::make_map_2d(&mVt, a->v_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)Npad, (uint64_t)a->B * a->H_KV * 128,
                            (uint64_t)Npad * 2, 64, 128))) return rc;
  if ((rc = tc::make_map_2d(&mKs, a->k_scale, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)Npad, (uint64_t)a->B * a->H_KV,
                            (uint64_t)Npad * 4, 64, 1, false))) return rc;
  if (T > 0) {
    if ((rc = tc::make_map_2d(&mXk, a->vert_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, (uint64_t)a->B * a->H_Q * Tpad, 256, 64, 64))) return rc;
    if ((rc = tc::make_map_2d(&mXv, a->vert_vt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)Tpad, (uint64_t)a->B * a->H_Q * 128,
                              (uint64_t)Tpad * 2, 64, 128))) return rc;
  } else {
    mXk = mKb; mXv = mVt;
  }
  PrefillTcParams p{};
  p.q_scale = a->q_scale; p.k_scale = a->k_scale;
  p.vmask = (const unsigned long long*)a->vmask; p.nv_valid = a->nv_valid;
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
    HQ_CUDA(cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_dev = dev;
  }
  const int R = a->H_Q / a->H_KV;
  dim3 grid((unsigned)p.nqb, (unsigned)(a->H_KV * ((R + 1) / 2)), (unsigned)a->B);   // two query heads of a KV group per CTA
  prefill_tc_kernel<<<grid, kTcThreads, smem, st>>>(mQi, mQb, mKi, mKb, mVt, mXk, mXv, mKs, p);
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
