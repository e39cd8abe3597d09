// Vertical-line identification: pooled-query scores over the candidate keys and
// an exact, deterministic top-k.
//
// Scores kernel — HBM-bound (one read of the candidate keys, 256 B per token per
// kv-head; 4 B per (token, query head) written).  scores^T[token, head] =
// K[token, :] . qbar[head, :] is computed with mma.sync bf16 (tokens on the M
// axis, the kv-group's query heads on the N axis), the pooled query being split
// into a bf16 high and low part so that an unrounded fp32 mean keeps ~16 bits.
// K fragments come straight from global memory as 16-byte loads; the channel
// axis is permuted consistently on both operands so that no shuffle is needed.
//
// Top-k kernel — one CTA per row: 4-pass radix select of the k-th largest key,
// order-preserving compaction (ties go to the lower index), bitonic sort of
// the selected (key, ~index) pairs in shared memory.
#include "hq_common.cuh"

namespace hq {

// ------------------------------------------------------------------ pooling
// `group` > 1: output head h is the mean of the input heads h group .. h group + group - 1, taken per token and rounded
// to the input dtype (what a 16-bit mean over the head axis gives) before the tokens are pooled.
template <typename T>
__global__ void pool_query_kernel(const T* __restrict__ q, int64_t sb, int64_t sh, int64_t sn, int H_Q, int n_q,
                                  int tail_len, int round_mode /*-1 none, else dtype*/, int group, int group_dtype,
                                  float* __restrict__ pooled) {
  const int bh = blockIdx.x, b = bh / H_Q, h = bh - b * H_Q, d = threadIdx.x;
  const T* base = q + b * sb + (int64_t)h * group * sh + (int64_t)(n_q - tail_len) * sn + d;
  float acc = 0.f;
  if (group <= 1) {
    for (int i = 0; i < tail_len; ++i) acc += load_as_float<T>(base + i * sn);
  } else {
    for (int i = 0; i < tail_len; ++i) {
      float s = 0.f;
      for (int r = 0; r < group; ++r) s += load_as_float<T>(base + r * sh + i * sn);
      acc += out_round(s / (float)group, group_dtype);
    }
  }
  float m = acc / (float)tail_len;
  if (round_mode >= 0) m = out_round(m, round_mode);
  pooled[(int64_t)bh * 128 + d] = m;
}

// ------------------------------------------------------------------ scores
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (kBf16) { __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&h); }
  __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&h);
}
template <bool kBf16>
__device__ __forceinline__ float round16(float v) {
  return kBf16 ? __bfloat162float(__float2bfloat16_rn(v)) : __half2float(__float2half_rn(v));
}

constexpr int kScoreWarps = 8;

// grid (chunks, B*H_KV).  K rows 128 elements wide, 16-bit dtype.
template <bool kBf16, int NT>
__global__ void __launch_bounds__(kScoreWarps * 32)
vertical_scores_kernel(const uint16_t* __restrict__ k, int64_t ksb, int64_t ksh, int64_t ksn, int H_KV, int R, int n_cand,
                       const float* __restrict__ pooled, int round_scores, float* __restrict__ scores) {
  const int bhk = blockIdx.y, b = bhk / H_KV, hk = bhk - b * H_KV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  // B fragments of qbar (hi and lo parts).  16-byte chunk j = 4 w + t of a key row
  // holds channels 8 j .. 8 j + 7; MMA chunk 2 w takes channels (0,1 | 2,3) of it,
  // chunk 2 w + 1 takes (4,5 | 6,7).
  uint32_t qh[NT][8][2], ql[NT][8][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int hd = nt * 8 + g;
    const float* qrow = pooled + ((int64_t)(b * H_KV + hk) * R + hd) * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int ch = 8 * (4 * (c >> 1) + t) + 4 * (c & 1) + 2 * r;
        float x0 = 0.f, x1 = 0.f;
        if (hd < R) { x0 = qrow[ch]; x1 = qrow[ch + 1]; }
        const float h0 = round16<kBf16>(x0), h1 = round16<kBf16>(x1);
        qh[nt][c][r] = pack2<kBf16>(h0, h1);
        ql[nt][c][r] = pack2<kBf16>(x0 - h0, x1 - h1);
      }
  }
  const uint16_t* kbase = k + b * ksb + hk * ksh;
  const int tiles = (n_cand + 15) / 16;
  const int tile_stride = gridDim.x * kScoreWarps;
  for (int tile = blockIdx.x * kScoreWarps + warp; tile < tiles; tile += tile_stride) {
    const int tokA = tile * 16 + g, tokB = tokA + 8;
    const bool okA = tokA < n_cand, okB = tokB < n_cand;
    uint4 ka[4], kb[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      ka[w] = okA ? __ldg(reinterpret_cast<const uint4*>(kbase + (int64_t)tokA * ksn + (4 * w + t) * 8)) : make_uint4(0, 0, 0, 0);
      kb[w] = okB ? __ldg(reinterpret_cast<const uint4*>(kbase + (int64_t)tokB * ksn + (4 * w + t) * 8)) : make_uint4(0, 0, 0, 0);
    }
    float s[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        if (kBf16) {
          mma_bf16(s[nt], ka[w].x, kb[w].x, ka[w].y, kb[w].y, ql[nt][2 * w][0], ql[nt][2 * w][1]);
          mma_bf16(s[nt], ka[w].z, kb[w].z, ka[w].w, kb[w].w, ql[nt][2 * w + 1][0], ql[nt][2 * w + 1][1]);
          mma_bf16(s[nt], ka[w].x, kb[w].x, ka[w].y, kb[w].y, qh[nt][2 * w][0], qh[nt][2 * w][1]);
          mma_bf16(s[nt], ka[w].z, kb[w].z, ka[w].w, kb[w].w, qh[nt][2 * w + 1][0], qh[nt][2 * w + 1][1]);
        } else {
          mma_f16(s[nt], ka[w].x, kb[w].x, ka[w].y, kb[w].y, ql[nt][2 * w][0], ql[nt][2 * w][1]);
          mma_f16(s[nt], ka[w].z, kb[w].z, ka[w].w, kb[w].w, ql[nt][2 * w + 1][0], ql[nt][2 * w + 1][1]);
          mma_f16(s[nt], ka[w].x, kb[w].x, ka[w].y, kb[w].y, qh[nt][2 * w][0], qh[nt][2 * w][1]);
          mma_f16(s[nt], ka[w].z, kb[w].z, ka[w].w, kb[w].w, qh[nt][2 * w + 1][0], qh[nt][2 * w + 1][1]);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int hd = nt * 8 + 2 * t + j;
        if (hd < R) {
          float* srow = scores + ((int64_t)(b * H_KV + hk) * R + hd) * n_cand;
          float vA = s[nt][j], vB = s[nt][2 + j];
          if (round_scores) { vA = round16<kBf16>(vA); vB = round16<kBf16>(vB); }
          if (okA) srow[tokA] = vA;
          if (okB) srow[tokB] = vB;
        }
      }
    }
  }
}

// ------------------------------------------------------------------- top-k
__device__ __forceinline__ uint32_t orderable(float f) {
  uint32_t u = (f == 0.0f) ? 0u : __float_as_uint(f);   // -0.0 and +0.0 compare equal, as in torch.topk
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kTopkThreads = 1024;
constexpr int kTopkMaxK = 16384;

__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
  // 1024 threads; returns exclusive prefix of v over the block, total in `total`
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();               // protect warp_sums reuse
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int ws = warp_sums[lane];
    int winc = ws;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    warp_sums[lane] = winc - ws;          // exclusive prefix of warp totals
    if (lane == 31) warp_sums[32] = winc;   // block total
  }
  __syncthreads();
  total = warp_sums[32];
  return warp_sums[warp] + inc - v;
}

__global__ void __launch_bounds__(kTopkThreads)
topk_kernel(const float* __restrict__ scores, int64_t stride, int n, int k, int kpad,
            int64_t* __restrict__ idx_desc, int32_t* __restrict__ idx_asc) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  unsigned long long* sel = reinterpret_cast<unsigned long long*>(smem_raw);   // [kpad]
  __shared__ int hist[256];
  __shared__ int warp_sums[33];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int s_count;
  const int tid = threadIdx.x;
  const float* row = scores + (int64_t)blockIdx.x * stride;

  // ---- radix select: find key T of the k-th largest element
  uint32_t prefix = 0, mask = 0;
  int remaining = k;   // rank (1-based from the top) within the current candidate set
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kTopkThreads) {
      const uint32_t key = orderable(__ldg(row + i));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFF], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int rem = remaining, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= rem) break;
        rem -= hist[b];
      }
      s_prefix = prefix | ((uint32_t)b << shift);
      s_remaining = rem;
    }
    __syncthreads();
    prefix = s_prefix;
    remaining = s_remaining;
    mask |= 0xFFu << shift;
    __syncthreads();
  }
  const uint32_t T = prefix;        // threshold key
  const int need_eq = remaining;    // how many elements equal to T to take (lowest indices first)

  // ---- order-preserving compaction into sel[]
  if (tid == 0) s_count = 0;
  __syncthreads();
  int eq_taken = 0;   // running number of == T elements seen in earlier tiles (block-uniform)
  int out_base = 0;   // running number of selected elements
  for (int base = 0; base < n; base += kTopkThreads) {
    const int i = base + tid;
    uint32_t key = 0;
    int is_gt = 0, is_eq = 0;
    if (i < n) {
      key = orderable(__ldg(row + i));
      is_gt = key > T;
      is_eq = key == T;
    }
    int eq_total;
    const int eq_rank = block_exclusive_scan(is_eq, warp_sums, eq_total);
    const int take = is_gt || (is_eq && (eq_taken + eq_rank) < need_eq);
    int take_total;
    const int pos = block_exclusive_scan(take, warp_sums, take_total);
    if (take) sel[out_base + pos] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)i);
    eq_taken += eq_total;
    out_base += take_total;
  }
  for (int i = out_base + tid; i < kpad; i += kTopkThreads) sel[i] = 0ull;   // smaller than any real entry
  __syncthreads();

  // ---- bitonic sort, descending
  for (int size = 2; size <= kpad; size <<= 1) {
    for (int strd = size >> 1; strd > 0; strd >>= 1) {
      for (int x = tid; x < (kpad >> 1); x += kTopkThreads) {
        const int lo = 2 * x - (x & (strd - 1));
        const int hi = lo + strd;
        const bool desc = ((lo & size) == 0);
        const unsigned long long a = sel[lo], b2 = sel[hi];
        if ((a < b2) == desc) { sel[lo] = b2; sel[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = tid; i < k; i += kTopkThreads)
    idx_desc[(int64_t)blockIdx.x * k + i] = (int64_t)(~(uint32_t)(sel[i] & 0xFFFFFFFFull));
  if (idx_asc == nullptr) return;
  __syncthreads();
  // ---- the same set in ascending position: sort the indices
  uint32_t* ids = reinterpret_cast<uint32_t*>(smem_raw) + 2 * kpad;   // after sel[]
  for (int i = tid; i < kpad; i += kTopkThreads) ids[i] = i < k ? ~(uint32_t)(sel[i] & 0xFFFFFFFFull) : 0xFFFFFFFFu;
  __syncthreads();
  for (int size = 2; size <= kpad; size <<= 1) {
    for (int strd = size >> 1; strd > 0; strd >>= 1) {
      for (int x = tid; x < (kpad >> 1); x += kTopkThreads) {
        const int lo = 2 * x - (x & (strd - 1));
        const int hi = lo + strd;
        const bool asc = ((lo & size) == 0);
        const uint32_t a = ids[lo], b2 = ids[hi];
        if ((a > b2) == asc) { ids[lo] = b2; ids[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = tid; i < k; i += kTopkThreads) idx_asc[(int64_t)blockIdx.x * k + i] = (int32_t)ids[i];
}

}  // namespace hq

namespace hq {
static int vertical_scores_impl(const void* q, int io_dtype, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                                int B, int H_Q, int n_q, int tail_len, int group,
                                const void* k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                                int H_KV, int n_cand, int round_mean, int round_scores,
                                float* pooled, float* scores, void* stream) {
  HQ_REQUIRE(B >= 0 && H_Q > 0 && H_KV > 0 && n_q > 0 && n_cand >= 0, HQ_ERR_INVALID, "hq_vertical_scores: bad sizes");
  HQ_REQUIRE(H_Q % H_KV == 0, HQ_ERR_INVALID, "hq_vertical_scores: H_Q %d not a multiple of H_KV %d", H_Q, H_KV);
  const int R = H_Q / H_KV;
  HQ_REQUIRE(R <= 16, HQ_ERR_UNSUPPORTED, "hq_vertical_scores: kv_repeat %d > 16", R);
  HQ_REQUIRE(tail_len >= 1 && tail_len <= n_q, HQ_ERR_INVALID, "hq_vertical_scores: tail_len %d outside 1..%d", tail_len, n_q);
  HQ_REQUIRE(io_dtype == HQ_BF16 || io_dtype == HQ_F16, HQ_ERR_UNSUPPORTED,
             "hq_vertical_scores: keys must be bf16 or fp16 on the device path");
  if (B == 0 || n_cand == 0) return HQ_OK;
  HQ_REQUIRE(q && k && pooled && scores, HQ_ERR_INVALID, "hq_vertical_scores: null pointer");
  HQ_REQUIRE(aligned16(k) && k_stride_b % 8 == 0 && k_stride_h % 8 == 0 && k_stride_n % 8 == 0, HQ_ERR_ALIGNMENT,
             "hq_vertical_scores: key rows must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int rm = round_mean ? io_dtype : -1;
  if (io_dtype == HQ_BF16)
    pool_query_kernel<__nv_bfloat16><<<B * H_Q, 128, 0, st>>>((const __nv_bfloat16*)q, q_stride_b, q_stride_h, q_stride_n, H_Q,
                                                              n_q, tail_len, rm, group, io_dtype, pooled);
  else
    pool_query_kernel<__half><<<B * H_Q, 128, 0, st>>>((const __half*)q, q_stride_b, q_stride_h, q_stride_n, H_Q, n_q,
                                                       tail_len, rm, group, io_dtype, pooled);
  HQ_CUDA(cudaGetLastError());
  const int tiles = (n_cand + 15) / 16;
  int chunks = (2 * sm_count() + B * H_KV - 1) / (B * H_KV);
  const int max_chunks = (tiles + kScoreWarps - 1) / kScoreWarps;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  dim3 grid((unsigned)chunks, (unsigned)(B * H_KV)), block(kScoreWarps * 32);
  const uint16_t* kk = (const uint16_t*)k;
  const bool bf = io_dtype == HQ_BF16;
  if (R <= 8) {
    if (bf) vertical_scores_kernel<true, 1><<<grid, block, 0, st>>>(kk, k_stride_b, k_stride_h, k_stride_n, H_KV, R, n_cand, pooled, round_scores, scores);
    else vertical_scores_kernel<false, 1><<<grid, block, 0, st>>>(kk, k_stride_b, k_stride_h, k_stride_n, H_KV, R, n_cand, pooled, round_scores, scores);
  } else {
    if (bf) vertical_scores_kernel<true, 2><<<grid, block, 0, st>>>(kk, k_stride_b, k_stride_h, k_stride_n, H_KV, R, n_cand, pooled, round_scores, scores);
    else vertical_scores_kernel<false, 2><<<grid, block, 0, st>>>(kk, k_stride_b, k_stride_h, k_stride_n, H_KV, R, n_cand, pooled, round_scores, scores);
  }
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}
}  // namespace hq

extern "C" int hq_vertical_scores(const void* q, int io_dtype, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                                  int B, int H_Q, int n_q, int tail_len,
                                  const void* k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                                  int H_KV, int n_cand, int round_mean, int round_scores,
                                  float* pooled, float* scores, void* stream) {
  return hq::vertical_scores_impl(q, io_dtype, q_stride_b, q_stride_h, q_stride_n, B, H_Q, n_q, tail_len, 1, k, k_stride_b,
                                  k_stride_h, k_stride_n, H_KV, n_cand, round_mean, round_scores, pooled, scores, stream);
}

// The selection of the cache's freeze: the saved queries of the `group` query heads of a kv-head are averaged first
// (per token, rounded to io_dtype), then pooled and scored per KV head.  q is [B, H_KV * group, n_q, 128].
extern "C" int hq_vertical_scores_grouped(const void* q, int io_dtype, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_n,
                                          int B, int H_KV, int group, int n_q, int tail_len,
                                          const void* k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_n,
                                          int n_cand, int round_mean, int round_scores,
                                          float* pooled, float* scores, void* stream) {
  using namespace hq;
  HQ_REQUIRE(group >= 1 && group <= 64, HQ_ERR_INVALID, "hq_vertical_scores_grouped: group %d outside 1..64", group);
  return vertical_scores_impl(q, io_dtype, q_stride_b, q_stride_h, q_stride_n, B, H_KV, n_q, tail_len, group, k, k_stride_b,
                              k_stride_h, k_stride_n, H_KV, n_cand, round_mean, round_scores, pooled, scores, stream);
}

extern "C" int hq_topk(const float* scores, int64_t scores_stride, int rows, int n, int k,
                       int64_t* idx_desc, int32_t* idx_asc, void* stream) {
  using namespace hq;
  HQ_REQUIRE(rows >= 0 && n >= 0 && k >= 0, HQ_ERR_INVALID, "hq_topk: negative size");
  if (rows == 0 || k == 0) return HQ_OK;
  HQ_REQUIRE(k <= n, HQ_ERR_INVALID, "hq_topk: k %d > n %d", k, n);
  HQ_REQUIRE(k <= kTopkMaxK, HQ_ERR_UNSUPPORTED, "hq_topk: k %d > %d", k, kTopkMaxK);
  HQ_REQUIRE(scores && idx_desc, HQ_ERR_INVALID, "hq_topk: null pointer");
  int kpad = 2;
  while (kpad < k) kpad <<= 1;
  const size_t smem = (size_t)kpad * 8 + (size_t)kpad * 4;
  static thread_local int attr_dev = -1;
  int dev = 0;
  HQ_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    HQ_CUDA(cudaFuncSetAttribute(topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTopkMaxK * 12));
    attr_dev = dev;
  }
  topk_kernel<<<rows, kTopkThreads, smem, (cudaStream_t)stream>>>(scores, scores_stride, n, k, kpad, idx_desc, idx_asc);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}
