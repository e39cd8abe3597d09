// Hybrid-precision causal prefill attention, GQA-native.
//
// For the 128-query block starting at s of query head h (kv head h / R):
//   keys j <  wla(s)          : INT8 QK^T (one scale per query row and per key row, smoothed K)
//                               unless j is a vertical line of head h -> masked here and taken
//                               from the gathered BF16 vertical tiles instead;
//   vertical lines < wla(s)   : BF16 QK^T on the gathered rows (ascending position);
//   keys in [wla(s), s + 128) : BF16 QK^T with the causal mask (local window + diagonal);
// with wla(s) = floor(max(0, s - (W - 1)) / 64) * 64 — the block rule of the reference kernel
// (src/ops/sage_unified.py:483-485, 538-544).  All tiles share one online softmax in base 2
// (sm_scale * log2 e is folded into the INT8 query scale and applied to the fp32 score of BF16 tiles) and one fp32 accumulator; P V runs in BF16.
// Unlike the reference nothing is expanded to query heads or physically reordered: K / V stay
// at kv-head granularity and a 64-bit mask word per (query head, 64-key block) removes the
// vertical columns from the INT8 pass.
//
// Tensor-bound.  FLOPs per call: 4 * B * H_Q * 128 * N (N + 1) / 2.
//
// This kernel drives the tensor cores through mma.sync (s8 and bf16 fragments from shared
// memory with ldmatrix); tiles are staged with cp.async in a two-stage ring.
#include "hq_common.cuh"

namespace hq {

struct PrefillParams {
  const int8_t* q_i8; const __nv_bfloat16* q_bf; const float* q_scale;        // [B,H_Q,N,128], [B,H_Q,N]
  const int8_t* k_i8; const __nv_bfloat16* k_bf; const float* k_scale;        // [B,H_KV,N,128], [B,H_KV,N]
  const __nv_bfloat16* v; int64_t v_sb, v_sh, v_sn;                            // [B,H_KV,N,128] strided
  const __nv_bfloat16* vert_k; const __nv_bfloat16* vert_v;                    // [B,H_Q,T,128] ascending position
  const unsigned long long* vmask;                                             // [B,H_Q,nkb]
  const int* nv_valid;                                                         // [B,H_Q,nqb]
  void* out; int out_dtype; int64_t o_sb, o_sh, o_sn;
  int B, H_Q, H_KV, N, Npad, W, T, nqb, nkb;
  float sml;      // sm_scale * log2(e), applied to the fp32 score of BF16 tiles
};

constexpr int kPfWarps = 8;
constexpr int kPfThreads = kPfWarps * 32;
constexpr int kBM = 128, kBN = 64;
constexpr int kStageBytes = 32768;   // K tile (<= 16 KB) | V tile (16 KB)

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = smem_u32(dst);
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// byte offset of 16-byte chunk `c` of row `r` in a tile whose rows are `row_bytes` long;
// chunks are XOR-swizzled with the row so that ldmatrix reads are bank-conflict free
__device__ __forceinline__ int swz(int r, int c, int row_bytes) { return r * row_bytes + ((c ^ (r & 7)) << 4); }

// copy `rows` x row_bytes from global (row stride src_stride bytes) into a swizzled tile; rows >= valid are zero
__device__ __forceinline__ void load_tile(uint8_t* dst, const uint8_t* src, int64_t src_stride, int rows, int valid,
                                          int row_bytes, int tid) {
  const int cpr = row_bytes >> 4;
  for (int x = tid; x < rows * cpr; x += kPfThreads) {
    const int r = x / cpr, c = x - r * cpr;
    const bool ok = r < valid;
    cp_async16(dst + swz(r, c, row_bytes), src + (ok ? (int64_t)r * src_stride + (c << 4) : 0), ok);
  }
}

struct PfTile { const uint8_t* k; const uint8_t* v; int64_t v_stride; int kind; int valid; int key0; int kblk; };

__global__ void __launch_bounds__(kPfThreads, 2)
prefill_hybrid_kernel(const PrefillParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQi = smem;                       // [128][128 B]
  uint8_t* sQb = smem + 16384;               // [128][256 B]
  uint8_t* sT = smem + 16384 + 32768;        // 2 stages x (K 16 KB | V 16 KB)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int qb = p.nqb - 1 - blockIdx.x;     // heavy blocks first
  const int hq = blockIdx.y, b = blockIdx.z, hkv = hq / (p.H_Q / p.H_KV);
  const int s0 = qb * kBM;
  const int64_t bhq = (int64_t)b * p.H_Q + hq, bhk = (int64_t)b * p.H_KV + hkv;
  const int wla = p.W > 0 ? (max(0, s0 - (p.W - 1)) / kBN) * kBN : s0;
  const int n_rest = wla / kBN;
  const int nv = p.T > 0 ? p.nv_valid[bhq * p.nqb + qb] : 0;
  const int n_vert = (nv + kBN - 1) / kBN;
  const int win_end = min(p.N, s0 + kBM);
  const int n_win = (win_end - wla + kBN - 1) / kBN;
  const int n_tiles = n_rest + n_vert + n_win;

  auto tile_of = [&](int i) -> PfTile {
    PfTile tl;
    if (i < n_rest) {
      tl.kind = 0; tl.key0 = i * kBN; tl.kblk = i; tl.valid = kBN;
      tl.k = reinterpret_cast<const uint8_t*>(p.k_i8 + (bhk * p.N + tl.key0) * 128);
      tl.v = reinterpret_cast<const uint8_t*>(p.v + b * p.v_sb + hkv * p.v_sh + (int64_t)tl.key0 * p.v_sn);
      tl.v_stride = p.v_sn * 2;
    } else if (i < n_rest + n_vert) {
      const int j = i - n_rest;
      tl.kind = 1; tl.key0 = j * kBN; tl.kblk = 0; tl.valid = min(kBN, nv - tl.key0);
      tl.k = reinterpret_cast<const uint8_t*>(p.vert_k + (bhq * p.T + tl.key0) * 128);
      tl.v = reinterpret_cast<const uint8_t*>(p.vert_v + (bhq * p.T + tl.key0) * 128);
      tl.v_stride = 256;
    } else {
      const int j = i - n_rest - n_vert;
      tl.kind = 2; tl.key0 = wla + j * kBN; tl.kblk = 0; tl.valid = min(kBN, p.N - tl.key0);
      tl.k = reinterpret_cast<const uint8_t*>(p.k_bf + (bhk * p.N + tl.key0) * 128);
      tl.v = reinterpret_cast<const uint8_t*>(p.v + b * p.v_sb + hkv * p.v_sh + (int64_t)tl.key0 * p.v_sn);
      tl.v_stride = p.v_sn * 2;
    }
    return tl;
  };
  auto issue_tile = [&](int i) {
    const PfTile tl = tile_of(i);
    uint8_t* st = sT + (i & 1) * kStageBytes;
    if (tl.kind == 0) {
      load_tile(st, tl.k, 128, kBN, tl.valid, 128, tid);
      if (tid < 64) {   // the 64 key scales of the tile ride behind the 8 KB of codes
        const uint32_t d = smem_u32(st + 8192 + tid * 4);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(p.k_scale + bhk * p.Npad + tl.key0 + tid) : "memory");
      }
    } else {
      load_tile(st, tl.k, 256, kBN, tl.valid, 256, tid);
    }
    load_tile(st + 16384, tl.v, tl.v_stride, kBN, tl.valid, 256, tid);
  };

  // queries of this block (rows past N are zero) + first tile
  {
    const int qvalid = min(kBM, p.N - s0);
    load_tile(sQi, reinterpret_cast<const uint8_t*>(p.q_i8 + (bhq * p.N + s0) * 128), 128, kBM, qvalid, 128, tid);
    load_tile(sQb, reinterpret_cast<const uint8_t*>(p.q_bf + (bhq * p.N + s0) * 128), 256, kBM, qvalid, 256, tid);
    if (n_tiles > 0) issue_tile(0);
    cp_async_commit();
  }
  float qsc[2];       // INT8 scales of this thread's accumulator rows g and g + 8
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = s0 + warp * 16 + g + 8 * r;
    qsc[r] = row < p.N ? p.q_scale[bhq * p.Npad + row] : 0.f;
  }

  float O[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) O[j][0] = O[j][1] = O[j][2] = O[j][3] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
  const int row_g = s0 + warp * 16 + g;       // absolute query position of accumulator rows g and g + 8

  for (int i = 0; i < n_tiles; ++i) {
    if (i + 1 < n_tiles) issue_tile(i + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const PfTile tl = tile_of(i);
    const uint8_t* sK = sT + (i & 1) * kStageBytes;
    const uint8_t* sV = sK + 16384;

    // ---- S = Q K^T for 16 rows x 64 keys
    float S[8][4];
    if (tl.kind == 0) {
      int Si[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) Si[j][0] = Si[j][1] = Si[j][2] = Si[j][3] = 0;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, sQi + swz(warp * 16 + (lane & 15), 2 * ks + (lane >> 4), 128));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bq[4];
          ldsm_x4(bq, sK + swz(16 * np + (lane & 7) + ((lane >> 4) << 3), 2 * ks + ((lane >> 3) & 1), 128));
          mma_s8(Si[2 * np], a, bq[0], bq[1]);
          mma_s8(Si[2 * np + 1], a, bq[2], bq[3]);
        }
      }
      const float* ksc = reinterpret_cast<const float*>(sK + 8192);
      const unsigned long long vm = p.T > 0 ? p.vmask[bhq * p.nkb + tl.kblk] : 0ull;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 kc = *reinterpret_cast<const float2*>(ksc + 8 * j + 2 * t);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int col = 8 * j + 2 * t + (x & 1);
          S[j][x] = ((vm >> col) & 1ull) ? -INFINITY : (float)Si[j][x] * (qsc[x >> 1] * ((x & 1) ? kc.y : kc.x));
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) S[j][0] = S[j][1] = S[j][2] = S[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, sQb + swz(warp * 16 + (lane & 15), 2 * ks + (lane >> 4), 256));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bq[4];
          ldsm_x4(bq, sK + swz(16 * np + (lane & 7) + ((lane >> 4) << 3), 2 * ks + ((lane >> 3) & 1), 256));
          mma_bf(S[2 * np], a, bq[0], bq[1]);
          mma_bf(S[2 * np + 1], a, bq[2], bq[3]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int x = 0; x < 4; ++x) S[j][x] *= p.sml;
      if (tl.kind == 1) {
        if (tl.valid < kBN) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int x = 0; x < 4; ++x)
              if (8 * j + 2 * t + (x & 1) >= tl.valid) S[j][x] = -INFINITY;
        }
      } else if (tl.key0 + kBN - 1 > s0 + warp * 16 || tl.valid < kBN) {   // causal / tail mask
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int key = tl.key0 + 8 * j + 2 * t + (x & 1);
            const int row = row_g + ((x >> 1) << 3);
            if (key > row || key >= p.N) S[j][x] = -INFINITY;
          }
      }
    }

    // ---- online softmax (rows g and g + 8 of this warp's 16)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mx[0] = fmaxf(mx[0], fmaxf(S[j][0], S[j][1]));
      mx[1] = fmaxf(mx[1], fmaxf(S[j][2], S[j][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float mu[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float nm = fmaxf(m_i[r], mx[r]);
      const float alpha = (nm == -INFINITY) ? 1.f : ex2f(m_i[r] - nm);
      m_i[r] = nm;
      mu[r] = (nm == -INFINITY) ? 0.f : nm;
      l_i[r] *= alpha;
#pragma unroll
      for (int j = 0; j < 16; ++j) { O[j][2 * r] *= alpha; O[j][2 * r + 1] *= alpha; }
    }
    uint32_t P[8][2];
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = ex2f(S[j][0] - mu[0]), p1 = ex2f(S[j][1] - mu[0]);
      const float p2 = ex2f(S[j][2] - mu[1]), p3 = ex2f(S[j][3] - mu[1]);
      rs[0] += p0 + p1; rs[1] += p2 + p3;
      P[j][0] = pack_bf(p0, p1);
      P[j][1] = pack_bf(p2, p3);
    }
    l_i[0] += rs[0]; l_i[1] += rs[1];       // per-thread partial row sums, reduced over t at the end

    // ---- O += P V   (k = 16 keys per step, 16 d-tiles of 8 channels)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a[4] = {P[2 * kk][0], P[2 * kk][1], P[2 * kk + 1][0], P[2 * kk + 1][1]};
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t bv[4];
        ldsm_x4_trans(bv, sV + swz(16 * kk + (lane & 7) + (((lane >> 3) & 1) << 3), 2 * dp + (lane >> 4), 256));
        mma_bf(O[2 * dp], a, bv[0], bv[1]);
        mma_bf(O[2 * dp + 1], a, bv[2], bv[3]);
      }
    }
    __syncthreads();     // this stage is overwritten by the copy issued at the top of the next iteration
  }
  cp_async_wait<0>();

  // ---- epilogue: O / l
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row_g + 8 * r;
    if (row >= p.N) continue;
    const float inv = l_i[r] > 0.f ? 1.f / l_i[r] : 0.f;
    const int64_t base = b * p.o_sb + hq * p.o_sh + (int64_t)row * p.o_sn;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float v0 = O[j][2 * r] * inv, v1 = O[j][2 * r + 1] * inv;
      const int c = 8 * j + 2 * t;
      if (p.out_dtype == HQ_BF16) {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(p.out) + base + c) = pack_bf(v0, v1);
      } else if (p.out_dtype == HQ_F16) {
        __half2 h = __floats2half2_rn(v0, v1);
        *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(p.out) + base + c) = h;
      } else {
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + base + c) = make_float2(v0, v1);
      }
    }
  }
}

// Vertical-line bookkeeping: for every (batch, query head) the ascending index list gives
//   vmask[blk]   bit j set  <=> key 64 blk + j is a vertical line of this head
//   nv_valid[qb] = number of vertical lines below wla(128 qb)
// (the role of the reference's reorder_kv_for_vertical counts, src/ops/sage_unified.py:537-544)
__global__ void vertical_meta_kernel(const int* __restrict__ vasc, int T, int N, int W, int nkb, int nqb,
                                     unsigned long long* __restrict__ vmask, int* __restrict__ nv_valid) {
  const int64_t bh = blockIdx.x;
  const int* a = vasc + bh * T;
  for (int blk = threadIdx.x; blk < nkb; blk += blockDim.x) {
    int lo = 0, hi = T;                    // lower_bound(64 blk)
    const int key0 = blk * 64;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (a[mid] < key0) lo = mid + 1; else hi = mid; }
    unsigned long long m = 0ull;
    for (int x = lo; x < T && a[x] < key0 + 64; ++x) m |= 1ull << (a[x] - key0);
    vmask[bh * nkb + blk] = m;
  }
  for (int qb = threadIdx.x; qb < nqb; qb += blockDim.x) {
    const int s0 = qb * 128;
    const int wla = W > 0 ? (max(0, s0 - (W - 1)) / 64) * 64 : s0;
    int lo = 0, hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (a[mid] < wla) lo = mid + 1; else hi = mid; }
    nv_valid[bh * nqb + qb] = lo;
  }
}

// gather rows `vasc` of k_bf (smoothed BF16 keys, kv-head granularity) and v into [B,H_Q,T,128]
__global__ void vertical_gather_kernel(const int* __restrict__ vasc, int T, int N, int H_Q, int H_KV,
                                       const __nv_bfloat16* __restrict__ k_bf,
                                       const __nv_bfloat16* __restrict__ v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                                       __nv_bfloat16* __restrict__ vert_k, __nv_bfloat16* __restrict__ vert_v) {
  const int64_t bhq = blockIdx.y;
  const int b = (int)(bhq / H_Q), hq = (int)(bhq - (int64_t)b * H_Q), hkv = hq / (H_Q / H_KV);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int j = blockIdx.x * (blockDim.x >> 5) + w;
  if (j >= T) return;
  int src = vasc[bhq * T + j];
  src = min(max(src, 0), N - 1);
  if (lane < 16) {
    const uint4* ks = reinterpret_cast<const uint4*>(k_bf + (((int64_t)b * H_KV + hkv) * N + src) * 128);
    reinterpret_cast<uint4*>(vert_k + (bhq * T + j) * 128)[lane] = __ldg(ks + lane);
  } else {
    const uint4* vs = reinterpret_cast<const uint4*>(v + b * v_sb + hkv * v_sh + (int64_t)src * v_sn);
    reinterpret_cast<uint4*>(vert_v + (bhq * T + j) * 128)[lane - 16] = __ldg(vs + (lane - 16));
  }
}

}  // namespace hq

namespace hq {
int prefill_tc_launch(const hq_prefill_args* a, cudaStream_t st);
int prefill_tc_prepare_v(const void* v, int64_t sb, int64_t sh, int64_t sn, int B, int H_KV, int N, void* v_t, cudaStream_t st);
int prefill_tc_prepare_vertical(const int32_t* vasc, int B, int H_Q, int H_KV, int N, int T, const void* k_bf, const void* v,
                                int64_t v_sb, int64_t v_sh, int64_t v_sn, void* xk, void* xvt, cudaStream_t st);
}

extern "C" int hq_prefill_transpose_v(const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn, int B, int H_KV, int N,
                                      void* v_t, void* stream) {
  using namespace hq;
  HQ_REQUIRE(v && v_t && B > 0 && H_KV > 0 && N > 0, HQ_ERR_INVALID, "hq_prefill_transpose_v: bad arguments");
  HQ_REQUIRE(aligned16(v) && aligned16(v_t) && v_sb % 8 == 0 && v_sh % 8 == 0 && v_sn % 8 == 0, HQ_ERR_ALIGNMENT,
             "hq_prefill_transpose_v: rows must be 16-byte aligned");
  return prefill_tc_prepare_v(v, v_sb, v_sh, v_sn, B, H_KV, N, v_t, (cudaStream_t)stream);
}

extern "C" int hq_prefill_vertical_prepare(const int32_t* vidx_asc, int B, int H_Q, int H_KV, int N, int window, int T,
                                           const void* k_bf, const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                                           void* vert_k, void* vert_v, void* vert_vt, uint64_t* vmask, int32_t* nv_valid,
                                           void* stream) {
  using namespace hq;
  HQ_REQUIRE(B > 0 && H_Q > 0 && H_KV > 0 && N > 0 && T >= 0 && window >= 0 && H_Q % H_KV == 0, HQ_ERR_INVALID,
             "hq_prefill_vertical_prepare: bad sizes");
  if (T == 0) return HQ_OK;
  HQ_REQUIRE(vidx_asc && k_bf && v && vert_k && (vert_v || vert_vt) && vmask && nv_valid, HQ_ERR_INVALID,
             "hq_prefill_vertical_prepare: null pointer");
  HQ_REQUIRE(aligned16(v) && aligned16(k_bf) && aligned16(vert_k) && aligned16(vert_v) && aligned16(vert_vt) && v_sb % 8 == 0 &&
                 v_sh % 8 == 0 && v_sn % 8 == 0, HQ_ERR_ALIGNMENT, "hq_prefill_vertical_prepare: rows must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int nkb = (N + 63) / 64, nqb = (N + 127) / 128;
  vertical_meta_kernel<<<B * H_Q, 256, 0, st>>>(vidx_asc, T, N, window, nkb, nqb, (unsigned long long*)vmask, nv_valid);
  if (vert_vt != nullptr)     // layout of the tensor-memory kernel: rows padded to 64, V rows transposed
    return prefill_tc_prepare_vertical(vidx_asc, B, H_Q, H_KV, N, T, k_bf, v, v_sb, v_sh, v_sn, vert_k, vert_vt, st);
  vertical_gather_kernel<<<dim3((T + 7) / 8, B * H_Q), 256, 0, st>>>(vidx_asc, T, N, H_Q, H_KV, (const __nv_bfloat16*)k_bf,
                                                                    (const __nv_bfloat16*)v, v_sb, v_sh, v_sn,
                                                                    (__nv_bfloat16*)vert_k, (__nv_bfloat16*)vert_v);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

extern "C" int hq_prefill_hybrid(const hq_prefill_args* a, void* stream) {
  using namespace hq;
  HQ_REQUIRE(a != nullptr, HQ_ERR_INVALID, "hq_prefill_hybrid: null args");
  HQ_REQUIRE(a->struct_bytes == (int32_t)sizeof(hq_prefill_args), HQ_ERR_INVALID, "hq_prefill_hybrid: struct_bytes %d != %d",
             a->struct_bytes, (int)sizeof(hq_prefill_args));
  HQ_REQUIRE(a->head_dim == 128, HQ_ERR_UNSUPPORTED, "hq_prefill_hybrid: head_dim %d (only 128 is built)", a->head_dim);
  HQ_REQUIRE(a->B > 0 && a->H_Q > 0 && a->H_KV > 0 && a->N > 0 && a->H_Q % a->H_KV == 0 && a->window >= 0 && a->T >= 0,
             HQ_ERR_INVALID, "hq_prefill_hybrid: bad sizes");
  HQ_REQUIRE(a->q_i8 && a->q_bf && a->q_scale && a->k_i8 && a->k_bf && a->k_scale && a->out, HQ_ERR_INVALID,
             "hq_prefill_hybrid: null pointer");
  HQ_REQUIRE(a->T == 0 || (a->vert_k && a->vmask && a->nv_valid), HQ_ERR_INVALID,
             "hq_prefill_hybrid: vertical arguments missing");
  HQ_REQUIRE(a->impl == 0 || (a->v && (a->T == 0 || a->vert_v)), HQ_ERR_INVALID, "hq_prefill_hybrid: v / vert_v missing");
  HQ_REQUIRE(aligned16(a->q_i8) && aligned16(a->q_bf) && aligned16(a->k_i8) && aligned16(a->k_bf) && aligned16(a->v) &&
                 a->v_sb % 8 == 0 && a->v_sh % 8 == 0 && a->v_sn % 8 == 0 && a->o_sn % 2 == 0 && a->o_sh % 2 == 0 && a->o_sb % 2 == 0,
             HQ_ERR_ALIGNMENT, "hq_prefill_hybrid: operand rows must be 16-byte aligned");
  HQ_REQUIRE(a->out_dtype == HQ_BF16 || a->out_dtype == HQ_F16 || a->out_dtype == HQ_F32, HQ_ERR_UNSUPPORTED,
             "hq_prefill_hybrid: out_dtype %d", a->out_dtype);
  if (a->impl == 0) return prefill_tc_launch(a, (cudaStream_t)stream);
  PrefillParams p{};
  p.q_i8 = (const int8_t*)a->q_i8; p.q_bf = (const __nv_bfloat16*)a->q_bf; p.q_scale = a->q_scale;
  p.k_i8 = (const int8_t*)a->k_i8; p.k_bf = (const __nv_bfloat16*)a->k_bf; p.k_scale = a->k_scale;
  p.v = (const __nv_bfloat16*)a->v; p.v_sb = a->v_sb; p.v_sh = a->v_sh; p.v_sn = a->v_sn;
  p.vert_k = (const __nv_bfloat16*)a->vert_k; p.vert_v = (const __nv_bfloat16*)a->vert_v;
  p.vmask = (const unsigned long long*)a->vmask; p.nv_valid = a->nv_valid;
  p.out = a->out; p.out_dtype = a->out_dtype; p.o_sb = a->o_sb; p.o_sh = a->o_sh; p.o_sn = a->o_sn;
  p.B = a->B; p.H_Q = a->H_Q; p.H_KV = a->H_KV; p.N = a->N; p.W = a->window; p.T = a->T;
  p.nqb = (a->N + 127) / 128; p.nkb = (a->N + 63) / 64; p.Npad = p.nkb * 64;
  p.sml = a->sm_scale * 1.44269504f;
  const size_t smem = 16384 + 32768 + 2 * kStageBytes;
  static thread_local int attr_dev = -1;
  int dev = 0;
  HQ_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    HQ_CUDA(cudaFuncSetAttribute(prefill_hybrid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_dev = dev;
  }
  dim3 grid((unsigned)p.nqb, (unsigned)a->H_Q, (unsigned)a->B);
  prefill_hybrid_kernel<<<grid, kPfThreads, smem, (cudaStream_t)stream>>>(p);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}
