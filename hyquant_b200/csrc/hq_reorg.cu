// Prefill -> decode cache reorganisation, and the cross-shard softmax merge.
//
// Reorganise — HBM-bound: reads K and V once (2 * 256 B per token per kv-head),
// writes INT4 codes + scales for the kept prefix rows, BF16 copies of the
// vertical-line rows and of the window.  The reference's
// scatter(-1)/sort/gather chain becomes: for source position p, rank(p) =
// number of vertical rows below p (looked up in the ascending index list, a
// per-tile slice of which sits in shared memory); p is dropped if it is itself
// vertical, else it lands at row p - rank(p) of the compact prefix, quantised
// on the way by the same warp-level routine the staging flush uses.
#include "hq_quant.cuh"

namespace hq {

constexpr int kReorgWarps = 8;
constexpr int kReorgTile = 128;   // source rows per CTA

__device__ __forceinline__ int lower_bound_i32(const int32_t* a, int n, int v) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(a + mid) < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ void copy_row_256B(const __nv_bfloat16* src, __nv_bfloat16* dst, int lane) {
  // 128 bf16 = 256 B: lanes 0..15 move 16 B each
  if (lane < 16) reinterpret_cast<uint4*>(dst)[lane] = __ldg(reinterpret_cast<const uint4*>(src) + lane);
}

// grid.x = prefix tiles + topk tiles + window tiles, grid.y = BH
__global__ void __launch_bounds__(kReorgWarps * 32)
cache_reorg_kernel(const __nv_bfloat16* __restrict__ keys, const __nv_bfloat16* __restrict__ values, int64_t kv_stride_bh,
                   int N, int prefix_len, int T, const int64_t* __restrict__ vidx_desc, const int32_t* __restrict__ vidx_asc,
                   __nv_bfloat16* __restrict__ k_topk, __nv_bfloat16* __restrict__ v_topk,
                   __nv_bfloat16* __restrict__ k_window, __nv_bfloat16* __restrict__ v_window,
                   uint8_t* __restrict__ k_packed, uint8_t* __restrict__ v_packed, int64_t kp_stride_bh, int64_t vp_stride_bh,
                   __half* __restrict__ k_scale, __half* __restrict__ v_scale, int64_t scale_stride_bh,
                   int k_bits, int v_bits, int scale_mode, int prefix_tiles, int topk_tiles) {
  __shared__ int32_t s_slice[kReorgTile];
  __shared__ int s_lo, s_hi;
  const int bh = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const __nv_bfloat16* K = keys + bh * kv_stride_bh;
  const __nv_bfloat16* V = values + bh * kv_stride_bh;
  int tile = blockIdx.x;
  if (tile < prefix_tiles) {
    const int p0 = tile * kReorgTile, p1 = min(p0 + kReorgTile, prefix_len);
    const int32_t* asc = vidx_asc + (int64_t)bh * T;
    if (threadIdx.x == 0) {
      s_lo = T > 0 ? lower_bound_i32(asc, T, p0) : 0;
      s_hi = T > 0 ? lower_bound_i32(asc, T, p1) : 0;
    }
    __syncthreads();
    const int lo = s_lo, cnt = s_hi - s_lo;   // cnt <= rows in tile (indices are distinct)
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) s_slice[i] = __ldg(asc + lo + i);
    __syncthreads();
    const int n_quant = prefix_len - T;
    // eight lanes per source row, four rows per warp and trip (every lane stays in step for the shuffles)
    const int sub = lane & 7;
    for (int pb = p0 + 4 * warp; pb < p1; pb += 4 * kReorgWarps) {
      const int p = pb + (lane >> 3);
      // rank within the slice: entries < p; hit: an entry == p
      int below = 0, hit = 0;
      for (int i = sub; i < cnt; i += 8) {
        const int v = s_slice[i];
        below += v < p;
        hit |= v == p;
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        below += __shfl_xor_sync(0xffffffffu, below, o);
        hit |= __shfl_xor_sync(0xffffffffu, hit, o);
      }
      const int dst = p - (lo + below);
      const bool live = p < p1 && !hit && dst >= 0 && dst < n_quant;     // dst out of range cannot happen for a consistent index list
      const int ps = p < p1 ? p : p1 - 1;
      float kv[16], vv[16];
      load16(K + (int64_t)ps * 128 + sub * 16, kv);
      load16(V + (int64_t)ps * 128 + sub * 16, vv);
      const int64_t d = live ? dst : 0;
      const __half sk = quant_store_row16(k_bits, kv, scale_mode, k_packed + bh * kp_stride_bh + d * (16 * k_bits), sub, live);
      const __half sv = quant_store_row16(v_bits, vv, scale_mode, v_packed + bh * vp_stride_bh + d * (16 * v_bits), sub, live);
      if (live && sub == 0) {
        k_scale[bh * scale_stride_bh + dst] = sk;
        v_scale[bh * scale_stride_bh + dst] = sv;
      }
    }
    return;
  }
  tile -= prefix_tiles;
  if (tile < topk_tiles) {
    const int j0 = tile * kReorgTile, j1 = min(j0 + kReorgTile, T);
    for (int j = j0 + warp; j < j1; j += kReorgWarps) {
      const int64_t src = __ldg(vidx_desc + (int64_t)bh * T + j);
      if (src < 0 || src >= N) continue;
      copy_row_256B(K + src * 128, k_topk + ((int64_t)bh * T + j) * 128, lane);
      copy_row_256B(V + src * 128, v_topk + ((int64_t)bh * T + j) * 128, lane);
    }
    return;
  }
  tile -= topk_tiles;
  {
    const int W = N - prefix_len;
    const int j0 = tile * kReorgTile, j1 = min(j0 + kReorgTile, W);
    for (int j = j0 + warp; j < j1; j += kReorgWarps) {
      copy_row_256B(K + (int64_t)(prefix_len + j) * 128, k_window + ((int64_t)bh * W + j) * 128, lane);
      copy_row_256B(V + (int64_t)(prefix_len + j) * 128, v_window + ((int64_t)bh * W + j) * 128, lane);
    }
  }
}

// ------------------------------------------------------------ cross-shard merge
__global__ void __launch_bounds__(128)
lse_merge_kernel(const float* __restrict__ m, const float* __restrict__ l, const float* __restrict__ acc, int64_t m_stride,
                 int64_t l_stride, int64_t acc_stride, int G, int rows, void* __restrict__ out, int out_dtype,
                 int64_t out_stride, float* __restrict__ out_m, float* __restrict__ out_l, float* __restrict__ out_acc) {
  const int r = blockIdx.x, d = threadIdx.x;
  float M = -INFINITY;
  for (int gI = 0; gI < G; ++gI) M = fmaxf(M, m[gI * m_stride + r]);
  float num = 0.f, den = 0.f;
  for (int gI = 0; gI < G; ++gI) {
    const float mg = m[gI * m_stride + r];
    const float w = (mg == -INFINITY) ? 0.f : ex2f(mg - M);
    num += w * acc[gI * acc_stride + (int64_t)r * 128 + d];
    den += w * l[gI * l_stride + r];
  }
  if (out_acc != nullptr) {
    out_acc[(int64_t)r * 128 + d] = num;
    if (d == 0) { out_m[r] = M; out_l[r] = den; }
  } else {
    store_out(out, (int64_t)r * out_stride + d, den > 0.f ? num / den : 0.f, out_dtype);
  }
}

}  // namespace hq

extern "C" int hq_cache_reorganize_bits(const void* keys, const void* values, int64_t kv_stride_bh,
                                   int BH, int N, int window, int T,
                                   const int64_t* vidx_desc, const int32_t* vidx_asc,
                                   void* k_topk, void* v_topk, void* k_window, void* v_window,
                                   void* k_packed, void* v_packed, int64_t kp_stride_bh, int64_t vp_stride_bh,
                                   void* k_scale, void* v_scale, int64_t scale_stride_bh,
                                   int k_bits, int v_bits, int scale_mode, void* stream) {
  using namespace hq;
  HQ_REQUIRE((k_bits == 2 || k_bits == 4 || k_bits == 8) && (v_bits == 2 || v_bits == 4 || v_bits == 8), HQ_ERR_UNSUPPORTED,
             "hq_cache_reorganize: bit widths must be 2, 4 or 8 (K%d V%d)", k_bits, v_bits);
  HQ_REQUIRE(BH >= 0 && N >= 0 && window >= 0 && window <= N && T >= 0 && T <= N - window, HQ_ERR_INVALID,
             "hq_cache_reorganize: need 0 <= window <= N and 0 <= T <= N - window (N=%d window=%d T=%d)", N, window, T);
  if (BH == 0 || N == 0) return HQ_OK;
  HQ_REQUIRE(keys && values, HQ_ERR_INVALID, "hq_cache_reorganize: null keys/values");
  HQ_REQUIRE(aligned16(keys) && aligned16(values) && kv_stride_bh % 8 == 0, HQ_ERR_ALIGNMENT,
             "hq_cache_reorganize: keys/values must be 16-byte aligned, head stride a multiple of 8 elements");
  HQ_REQUIRE(scale_mode == 0 || scale_mode == 1, HQ_ERR_INVALID, "hq_cache_reorganize: scale_mode must be 0 or 1");
  const int prefix_len = N - window;
  HQ_REQUIRE(T == 0 || (vidx_desc && vidx_asc && k_topk && v_topk), HQ_ERR_INVALID, "hq_cache_reorganize: null top-k argument");
  HQ_REQUIRE(window == 0 || (k_window && v_window), HQ_ERR_INVALID, "hq_cache_reorganize: null window output");
  HQ_REQUIRE(prefix_len - T == 0 || (k_packed && v_packed && k_scale && v_scale), HQ_ERR_INVALID,
             "hq_cache_reorganize: null quantised output");
  HQ_REQUIRE(((uintptr_t)k_packed % (2 * k_bits)) == 0 && ((uintptr_t)v_packed % (2 * v_bits)) == 0 && kp_stride_bh % (2 * k_bits) == 0 &&
                 vp_stride_bh % (2 * v_bits) == 0, HQ_ERR_ALIGNMENT,
             "hq_cache_reorganize: packed rows must be aligned to 2 * bits bytes (what one lane stores)");
  HQ_REQUIRE((T == 0 || (aligned16(k_topk) && aligned16(v_topk))) && (window == 0 || (aligned16(k_window) && aligned16(v_window))),
             HQ_ERR_ALIGNMENT, "hq_cache_reorganize: BF16 outputs must be 16-byte aligned");
  const int prefix_tiles = (prefix_len + kReorgTile - 1) / kReorgTile;
  const int topk_tiles = (T + kReorgTile - 1) / kReorgTile;
  const int window_tiles = (window + kReorgTile - 1) / kReorgTile;
  const int tiles = prefix_tiles + topk_tiles + window_tiles;
  if (tiles == 0) return HQ_OK;
  dim3 grid((unsigned)tiles, (unsigned)BH), block(kReorgWarps * 32);
  cache_reorg_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)keys, (const __nv_bfloat16*)values, kv_stride_bh, N, prefix_len, T, vidx_desc, vidx_asc,
      (__nv_bfloat16*)k_topk, (__nv_bfloat16*)v_topk, (__nv_bfloat16*)k_window, (__nv_bfloat16*)v_window,
      (uint8_t*)k_packed, (uint8_t*)v_packed, kp_stride_bh, vp_stride_bh, (__half*)k_scale, (__half*)v_scale, scale_stride_bh,
      k_bits, v_bits, scale_mode, prefix_tiles, topk_tiles);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

extern "C" int hq_cache_reorganize(const void* keys, const void* values, int64_t kv_stride_bh,
                                   int BH, int N, int window, int T,
                                   const int64_t* vidx_desc, const int32_t* vidx_asc,
                                   void* k_topk, void* v_topk, void* k_window, void* v_window,
                                   void* k_packed, void* v_packed, int64_t packed_stride_bh,
                                   void* k_scale, void* v_scale, int64_t scale_stride_bh,
                                   int scale_mode, void* stream) {
  return hq_cache_reorganize_bits(keys, values, kv_stride_bh, BH, N, window, T, vidx_desc, vidx_asc, k_topk, v_topk, k_window,
                                  v_window, k_packed, v_packed, packed_stride_bh, packed_stride_bh, k_scale, v_scale,
                                  scale_stride_bh, 4, 4, scale_mode, stream);
}

extern "C" int hq_lse_merge_strided(const float* m, const float* l, const float* acc, int64_t m_stride, int64_t l_stride,
                                    int64_t acc_stride, int G, int rows, void* out, int out_dtype, int64_t out_stride,
                                    void* stream) {
  using namespace hq;
  HQ_REQUIRE(G >= 1 && rows >= 0, HQ_ERR_INVALID, "hq_lse_merge: G >= 1 and rows >= 0 required");
  if (rows == 0) return HQ_OK;
  HQ_REQUIRE(m && l && acc && out, HQ_ERR_INVALID, "hq_lse_merge: null pointer");
  HQ_REQUIRE(out_dtype == HQ_BF16 || out_dtype == HQ_F16 || out_dtype == HQ_F32, HQ_ERR_UNSUPPORTED,
             "hq_lse_merge: out_dtype %d", out_dtype);
  lse_merge_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(m, l, acc, m_stride, l_stride, acc_stride, G, rows, out, out_dtype,
                                                           out_stride, nullptr, nullptr, nullptr);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

extern "C" int hq_lse_merge_partial(const float* m, const float* l, const float* acc, int64_t m_stride, int64_t l_stride,
                                    int64_t acc_stride, int G, int rows, float* out_m, float* out_l, float* out_acc,
                                    void* stream) {
  using namespace hq;
  HQ_REQUIRE(G >= 1 && rows >= 0, HQ_ERR_INVALID, "hq_lse_merge_partial: G >= 1 and rows >= 0 required");
  if (rows == 0) return HQ_OK;
  HQ_REQUIRE(m && l && acc && out_m && out_l && out_acc, HQ_ERR_INVALID, "hq_lse_merge_partial: null pointer");
  lse_merge_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(m, l, acc, m_stride, l_stride, acc_stride, G, rows, nullptr, HQ_F32, 0,
                                                           out_m, out_l, out_acc);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

extern "C" int hq_lse_merge(const float* m, const float* l, const float* acc, int G, int rows,
                            void* out, int out_dtype, int64_t out_stride, void* stream) {
  return hq_lse_merge_strided(m, l, acc, rows, rows, (int64_t)rows * 128, G, rows, out, out_dtype, out_stride, stream);
}
