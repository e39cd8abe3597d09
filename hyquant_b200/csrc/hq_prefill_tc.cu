// Hybrid-precision causal prefill attention on the Blackwell tensor path.
//
// Tile semantics as stated in hq_prefill.cu's header: for the 128-query
// block at s of query head h, keys below wla(s) are INT8 unless they are vertical lines of h
// (masked here, served from gathered BF16 tiles), keys in [wla(s), s + 128) are BF16 + causal mask.
//
// Structure of one CTA (128 queries of one head, 10 warps):
//   warp 8 (one lane)  producer: TMA tensor-map loads (128-byte swizzle) of Q once and of a K tile
//                      + a transposed V tile per step into a four-slot ring;
//   warp 9 (one lane)  issues tcgen05.mma: S = Q K^T (kind::i8 with s32 accumulators or kind::f16 on
//                      bf16) into one of two S buffers in tensor memory, and O += P V (kind::f16) into
//                      the O accumulator in tensor memory; completion is signalled with tcgen05.commit;
//   warps 0-7          two threads per query row (half of the columns each): tcgen05.ld of the S row, scales / masks, online
//                      softmax in base 2 with a lazily updated maximum (the O accumulator is rescaled
//                      in tensor memory only when the maximum grows by more than 2^8), P to shared
//                      memory as the A operand of the next P V, final O / l from tensor memory.
// S is double-buffered so that Q K^T of tile i+1 runs while the softmax of tile i is in flight.
// All operands are K-major: V is transposed once per call by the preparation pass.
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

constexpr int kTcThreads = 320;        // 8 softmax warps + producer warp + MMA warp
constexpr uint32_t kTmemCols = 256;        // S0 [0,64) | S1 [64,128) | O [128,256)
constexpr float kTcLazy = 8.0f;

constexpr int kKvStages = 4;   // K / V^T ring depth: tile loads run this many tiles ahead of the MMAs
struct TcSmem {              // offsets from a 1024-aligned base
  static constexpr int Qi = 0;                             // 16 KB  [128 rows][128 B] int8
  static constexpr int Qb = 16384;                         // 32 KB  2 x [128 rows][128 B] bf16
  static constexpr int K = 49152;                          // kKvStages x 16 KB
  static constexpr int V = K + kKvStages * 16384;          // kKvStages x 16 KB  [128 d rows][128 B]
  static constexpr int P = V + kKvStages * 16384;          // 2 x 16 KB  [128 rows][128 B] bf16
  static constexpr int Bar = P + 32768;                    // barriers + scratch
  static constexpr int Xch = Bar + 256;                    // 3 x [2][128] floats: row maxima (two parities), row sums
  static constexpr int Total = Xch + 3072;
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
  uint64_t* s_full = bars + 1;       // [2]
  uint64_t* s_free = bars + 3;       // [2]
  uint64_t* p_ready = bars + 5;      // [2]
  uint64_t* pv_done = bars + 7;      // [2]
  uint64_t* kv_full = bars + 9;                  // [kKvStages]
  uint64_t* kv_empty = bars + 9 + kKvStages;     // [kKvStages]
  uint64_t* x_bar = bars + 9 + 2 * kKvStages;    // [3] row-maximum exchange (two parities) and row-sum exchange
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12 + 2 * kKvStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 13 + 2 * kKvStages);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  __shared__ int s_skip;
  if (tid == 0) s_skip = *reinterpret_cast<volatile int*>(p.status) & 2;
  __syncthreads();
  if (s_skip) return;                         // an earlier CTA gave up: drain the grid quickly
  const int qb = p.nqb - 1 - blockIdx.x;     // heavy blocks first
  const int hq = blockIdx.y, b = blockIdx.z, hkv = hq / (p.H_Q / p.H_KV);
  const int s0 = qb * 128;
  const int64_t bhq = (int64_t)b * p.H_Q + hq, bhk = (int64_t)b * p.H_KV + hkv;
  const int wla = p.W > 0 ? (max(0, s0 - (p.W - 1)) / 64) * 64 : s0;
  const int n_rest = wla / 64;
  const int nv = p.T > 0 ? p.nv_valid[bhq * p.nqb + qb] : 0;
  const int n_vert = (nv + 63) / 64;
  const int win_end = min(p.N, s0 + 128);
  const int n_win = (win_end - wla + 63) / 64;
  const int n_tiles = n_rest + n_vert + n_win;

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kKvStages; ++i) { mbar_init(kv_full + i, 1); mbar_init(kv_empty + i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(s_full + i, 1); mbar_init(s_free + i, 256); }
    for (int i = 0; i < 2; ++i) { mbar_init(p_ready + i, 256); mbar_init(pv_done + i, 1); mbar_init(x_bar + i, 256); }
    mbar_init(x_bar + 2, 256);
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
      tc::tma_prefetch_desc(&mKb); tc::tma_prefetch_desc(&mVt);
      mbar_expect_tx(q_full, 16384 + 32768);
      tc::tma_load_2d(smem + TcSmem::Qi, &mQi, 0, (int)(bhq * p.N + s0), q_full);
      tc::tma_load_2d(smem + TcSmem::Qb, &mQb, 0, (int)(bhq * p.N + s0), q_full);
      tc::tma_load_2d(smem + TcSmem::Qb + 16384, &mQb, 64, (int)(bhq * p.N + s0), q_full);
      for (int i = 0; i < n_tiles; ++i) {
        const int slot = i % kKvStages;
        if (!tc::mbar_wait_abortable(kv_empty + slot, (uint32_t)(((i / kKvStages) & 1) ^ 1), abort_flag, 200)) break;
        uint8_t* sK = smem + TcSmem::K + slot * 16384;
        uint8_t* sV = smem + TcSmem::V + slot * 16384;
        if (i < n_rest) {
          const int key0 = i * 64;
          mbar_expect_tx(kv_full + slot, 8192 + 256 + 16384);
          tc::tma_load_2d(sK, &mKi, 0, (int)(bhk * p.N + key0), kv_full + slot);
          tc::tma_load_2d(sK + 8192, &mKs, key0, (int)bhk, kv_full + slot);      // the tile's 64 key scales
          tc::tma_load_2d(sV, &mVt, key0, (int)(bhk * 128), kv_full + slot);
        } else if (i < n_rest + n_vert) {
          const int j0 = (i - n_rest) * 64;
          mbar_expect_tx(kv_full + slot, 16384 + 16384);
          tc::tma_load_2d(sK, &mXk, 0, (int)(bhq * p.Tpad + j0), kv_full + slot);
          tc::tma_load_2d(sK + 8192, &mXk, 64, (int)(bhq * p.Tpad + j0), kv_full + slot);
          tc::tma_load_2d(sV, &mXv, j0, (int)(bhq * 128), kv_full + slot);
        } else {
          const int key0 = wla + (i - n_rest - n_vert) * 64;
          mbar_expect_tx(kv_full + slot, 16384 + 16384);
          tc::tma_load_2d(sK, &mKb, 0, (int)(bhk * p.N + key0), kv_full + slot);
          tc::tma_load_2d(sK + 8192, &mKb, 64, (int)(bhk * p.N + key0), kv_full + slot);
          tc::tma_load_2d(sV, &mVt, key0, (int)(bhk * 128), kv_full + slot);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_i8 = tc::make_idesc(2, tc::kFmtS8, tc::kFmtS8, 128, 64);
      constexpr uint32_t idesc_qk = tc::make_idesc(1, tc::kFmtBF16, tc::kFmtBF16, 128, 64);
      constexpr uint32_t idesc_pv = tc::make_idesc(1, tc::kFmtBF16, tc::kFmtBF16, 128, 128);
      bool ok = tc::mbar_wait_abortable(q_full, 0, abort_flag, 100);
      for (int i = 0; ok && i <= n_tiles; ++i) {
        if (i < n_tiles) {
          const int slot = i & 1, kvs = i % kKvStages;
          ok = tc::mbar_wait_abortable(kv_full + kvs, (uint32_t)((i / kKvStages) & 1), abort_flag, 40) &&
               tc::mbar_wait_abortable(s_free + slot, (uint32_t)(((i >> 1) & 1) ^ 1), abort_flag, 40);
          if (!ok) break;
          tc::fence_after_sync();
          const uint32_t dS = tmem_base + (uint32_t)slot * 64;
          const uint8_t* sK = smem + TcSmem::K + kvs * 16384;
          if (i < n_rest) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc::mma_s8_ss(dS, tc::smem_desc_k128(smem + TcSmem::Qi, k * 32), tc::smem_desc_k128(sK, k * 32), idesc_i8, k > 0);
          } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              tc::mma_bf16_ss(dS, tc::smem_desc_k128(smem + TcSmem::Qb + (k >> 2) * 16384, (k & 3) * 32),
                              tc::smem_desc_k128(sK + (k >> 2) * 8192, (k & 3) * 32), idesc_qk, k > 0);
          }
          tc::mma_commit(s_full + slot);
        }
        if (i > 0) {
          const int j = i - 1, slot = j & 1;
          ok = tc::mbar_wait_abortable(p_ready + slot, (uint32_t)((j >> 1) & 1), abort_flag, 40);
          if (!ok) break;
          tc::fence_after_sync();
          const uint32_t dO = tmem_base + 128;
          const uint8_t* sV = smem + TcSmem::V + (j % kKvStages) * 16384;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc::mma_bf16_ss(dO, tc::smem_desc_k128(smem + TcSmem::P + slot * 16384, k * 32), tc::smem_desc_k128(sV, k * 32), idesc_pv,
                            (j > 0 || k > 0) ? 1u : 0u);
          tc::mma_commit(pv_done + slot);
          tc::mma_commit(kv_empty + (j % kKvStages));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax: two threads per query row
    // Warps w and w + 4 share the tensor-memory lanes 32 (w % 4) .. + 31 (the hardware ties a warp to the
    // lane quarter warp % 4) and split the row's 64 score columns / 128 output columns in halves, so every
    // scheduler has two softmax warps to interleave.  Row maxima meet through shared memory once per tile.
    const int half = warp >> 2, wq = warp & 3;
    const int r = wq * 32 + lane;            // query row inside the block = tensor-memory lane
    const int row = s0 + r;
    const uint32_t lane_base = tmem_base + ((uint32_t)(wq * 32) << 16);
    float* xmax = reinterpret_cast<float*>(smem + TcSmem::Xch);        // [2 parities][2 halves][128]
    float* xsum = xmax + 512;                                          // [2 halves][128]
    const float qs = row < p.N ? p.q_scale[bhq * p.Npad + row] : 0.f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // the vertical-mask word of a tile is a fresh cache line every step: fetch it one step ahead
    const unsigned long long* vmrow = p.vmask + bhq * p.nkb;
    unsigned long long vm_next = (p.T > 0 && n_rest > 0) ? __ldg(vmrow) : 0ull;
    for (int i = 0; i < n_tiles; ++i) {
      const int slot = i & 1;
      const unsigned long long vm64 = vm_next;
      if (p.T > 0 && i + 1 < n_rest) vm_next = __ldg(vmrow + i + 1);
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(s_full + slot, (uint32_t)((i >> 1) & 1), abort_flag));
      if (!ok) break;
      tc::fence_after_sync();
      uint32_t sr[32];
      tc::tmem_ld32(lane_base + slot * 64 + half * 32, sr);
      tc::tmem_wait_ld();
      tc::fence_before_sync();
      tc::mbar_arrive(s_free + slot);

      // scores in the exponent's units: t[c] * esc - mu, with esc folded into one FFMA per element
      float t[32];
      float esc;
      if (i < n_rest) {
        const float4* ks4 = reinterpret_cast<const float4*>(smem + TcSmem::K + (i % kKvStages) * 16384 + 8192) + half * 8;
        const uint32_t vm = (uint32_t)(vm64 >> (32 * half));
        esc = qs;
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 kk = ks4[c4];
          const float kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int c = 4 * c4 + x;
            // int32 -> float without the conversion unit: |score| < 2^22
            t[c] = (__int_as_float((int)sr[c] + 0x4B400000) - 12582912.0f) * kv[x];
          }
        }
        if (vm != 0u) {
#pragma unroll
          for (int c = 0; c < 32; ++c) if ((vm >> c) & 1u) t[c] = -INFINITY;
        }
      } else {
        esc = p.sml;
#pragma unroll
        for (int c = 0; c < 32; ++c) t[c] = __uint_as_float(sr[c]);
        int lim;                                             // columns (of the full tile) <= lim are visible
        if (i < n_rest + n_vert) lim = min(64, nv - (i - n_rest) * 64) - 1;
        else lim = min(row, p.N - 1) - (wla + (i - n_rest - n_vert) * 64);
        lim -= 32 * half;
        if (__any_sync(0xffffffffu, lim < 31)) {
#pragma unroll
          for (int c = 0; c < 32; ++c) if (c > lim) t[c] = -INFINITY;
        }
      }
      float mx;
      {
        float m8[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) m8[x] = t[x];
#pragma unroll
        for (int c = 8; c < 32; ++c) m8[c & 7] = fmaxf(m8[c & 7], t[c]);
        mx = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
      }
      mx *= esc;                                             // esc >= 0
      if (esc == 0.f) mx = -INFINITY;                        // rows past N
      // exchange the half-row maxima
      xmax[(slot * 2 + half) * 128 + r] = mx;
      tc::mbar_arrive(x_bar + slot);
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(x_bar + slot, (uint32_t)((i >> 1) & 1), abort_flag));
      if (!ok) break;
      mx = fmaxf(mx, xmax[(slot * 2 + (half ^ 1)) * 128 + r]);
      const bool grow = mx > m_ref + kTcLazy;                // also true for the first finite maximum
      if (__any_sync(0xffffffffu, grow)) {
        const float nm = grow ? mx : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2f(m_ref - nm);
        if (i > 0) {     // O must be quiescent: every P V issued so far has to be complete
          ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(pv_done + ((i - 1) & 1), (uint32_t)(((i - 1) >> 1) & 1), abort_flag));
          if (!ok) break;
          tc::fence_after_sync();
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t o[32];
            tc::tmem_ld32(lane_base + 128 + half * 64 + ch * 32, o);
            tc::tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * (grow ? alpha : 1.f));
            tc::tmem_st32(lane_base + 128 + half * 64 + ch * 32, o);
          }
          tc::tmem_wait_st();
          tc::fence_before_sync();
        }
        if (grow) { l *= alpha; m_ref = nm; }
      }
      const float mu = m_ref == -INFINITY ? 0.f : m_ref;
      uint32_t pk[16];
      float rs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float p0 = ex2f(fmaf(t[c], esc, -mu)), p1 = ex2f(fmaf(t[c + 1], esc, -mu));
        rs[c & 3] += p0; rs[(c & 3) + 1] += p1;
        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
      // the P buffer of this parity was last read by the P V of tile i - 2
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(pv_done + slot, (uint32_t)(((i >> 1) & 1) ^ 1), abort_flag));
      if (!ok) break;
      uint8_t* prow = smem + TcSmem::P + slot * 16384 + r * 128;
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int ch = 4 * half + x;
        *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
      }
      fence_proxy_async_smem();
      tc::fence_before_sync();
      tc::mbar_arrive(p_ready + slot);
    }
    // ---- epilogue: O / l, each half of the row's threads stores 64 output columns
    if (ok) {
      xsum[half * 128 + r] = l;
      tc::mbar_arrive(x_bar + 2);
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(x_bar + 2, 0, abort_flag));
    }
    if (ok && n_tiles > 0)
      ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(pv_done + ((n_tiles - 1) & 1), (uint32_t)(((n_tiles - 1) >> 1) & 1), abort_flag));
    if (ok) {
      tc::fence_after_sync();
      const float lt = xsum[r] + xsum[128 + r];
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      const int64_t base = b * p.o_sb + hq * p.o_sh + (int64_t)row * p.o_sn + half * 64;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t o[32];
        tc::tmem_ld32(lane_base + 128 + half * 64 + ch * 32, o);
        tc::tmem_wait_ld();
        if (row < p.N) {
          if (p.out_dtype == HQ_BF16) {
            uint32_t w[16];
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
              w[x] = *reinterpret_cast<uint32_t*>(&h);
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
  dim3 grid((unsigned)p.nqb, (unsigned)a->H_Q, (unsigned)a->B);
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
