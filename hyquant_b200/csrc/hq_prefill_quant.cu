// Operand preparation for the hybrid prefill kernel (one pass over Q and K):
//   * K smoothing: k_sm = k - mean_n(k) per (batch, kv-head, channel), formed in bf16
//     like the reference (src/ops/sage_unified.py:565-568);
//   * INT8 of k_sm and of q * sm_scale * log2(e) with scale = max|x| / 127 and
//     round-half-away-from-zero — the arithmetic of the reference's block quantiser
//     (src/ops/vendor/sageattention/triton/quant_per_block.py:21-47) applied with one scale
//     per token row instead of one per 64-key / 128-query block: an outlier row then costs
//     no precision in its neighbours, and the scales are applied to the fp32 score for free;
//   * a contiguous BF16 copy of the query for the BF16 tiles (unscaled: the kernel applies
//     sm_scale * log2(e) to the fp32 score, so no rounding is added to the query).
// HBM-bound: reads Q and K once, writes the INT8 and BF16 copies.
#include "hq_common.cuh"

namespace hq {

constexpr int kMeanChunks = 32;

// partial[bh][chunk][128] = sum over the chunk's rows
__global__ void __launch_bounds__(256)
kmean_partial_kernel(const __nv_bfloat16* __restrict__ k, int64_t sb, int64_t sh, int64_t sn, int H, int N,
                     float* __restrict__ partial) {
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, chunk = blockIdx.x;
  const int d = threadIdx.x & 127, half = threadIdx.x >> 7;
  const int rows_per = (N + kMeanChunks - 1) / kMeanChunks;
  const int r0 = chunk * rows_per, r1 = min(N, r0 + rows_per);
  const __nv_bfloat16* base = k + b * sb + h * sh + d;
  float acc = 0.f;
  for (int r = r0 + half; r < r1; r += 2) acc += __bfloat162float(base[(int64_t)r * sn]);
  __shared__ float s[256];
  s[threadIdx.x] = acc;
  __syncthreads();
  if (half == 0) partial[((int64_t)bh * kMeanChunks + chunk) * 128 + d] = s[d] + s[128 + d];
}

__global__ void kmean_final_kernel(const float* __restrict__ partial, int N, int smooth, __nv_bfloat16* __restrict__ mean) {
  const int bh = blockIdx.x, d = threadIdx.x;
  float acc = 0.f;
  for (int c = 0; c < kMeanChunks; ++c) acc += partial[((int64_t)bh * kMeanChunks + c) * 128 + d];
  mean[(int64_t)bh * 128 + d] = __float2bfloat16_rn(smooth ? acc / (float)N : 0.f);
}

__device__ __forceinline__ int8_t q_half_away(float x, float scale) {
  float y = x / scale;
  y += y >= 0.f ? 0.5f : -0.5f;
  y = fminf(fmaxf(truncf(y), -128.f), 127.f);
  return (int8_t)(int)y;
}

// 16 rows per CTA (256 threads, 16 threads per 128-channel row, 8 channels each).
// kIsK: subtract the bf16 mean (rounding the difference to bf16) and write it as the BF16 copy;
// else multiply by `mul` in fp32, INT8 from the fp32 product and BF16 copy of the product.
// One INT8 scale per ROW (token): scale = max|x| / 127.
template <bool kIsK>
__global__ void __launch_bounds__(256)
row_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sh, int64_t sn, int H, int N,
                 const __nv_bfloat16* __restrict__ mean, float mul,
                 int8_t* __restrict__ xi8, __nv_bfloat16* __restrict__ xbf, float* __restrict__ scale, int scale_pitch) {
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int tid = threadIdx.x;
  const int row = blockIdx.x * 16 + (tid >> 4), c = (tid & 15) * 8;
  const bool ok = row < N;
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (ok) raw = __ldg(reinterpret_cast<const uint4*>(x + b * sb + h * sh + (int64_t)row * sn + c));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
  float amax = 0.f;
  uint4 outbf;
  uint32_t* ob = reinterpret_cast<uint32_t*>(&outbf);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float f0 = __uint_as_float(w[j] << 16), f1 = __uint_as_float(w[j] & 0xFFFF0000u);
    if (kIsK) {
      const float m0 = __bfloat162float(mean[(int64_t)bh * 128 + c + 2 * j]);
      const float m1 = __bfloat162float(mean[(int64_t)bh * 128 + c + 2 * j + 1]);
      f0 = __bfloat162float(__float2bfloat16_rn(f0 - m0));
      f1 = __bfloat162float(__float2bfloat16_rn(f1 - m1));
    } else {
      f0 *= mul; f1 *= mul;
    }
    v[2 * j] = f0; v[2 * j + 1] = f1;
    amax = fmaxf(amax, fmaxf(fabsf(f0), fabsf(f1)));
    __nv_bfloat162 pk = __floats2bfloat162_rn(f0, f1);
    ob[j] = kIsK ? *reinterpret_cast<uint32_t*>(&pk) : w[j];     // the BF16 query copy stays unscaled (exact)
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (!ok) return;
  *reinterpret_cast<uint4*>(xbf + ((int64_t)bh * N + row) * 128 + c) = outbf;
  const float sc = fmaxf(amax, 1e-30f) / 127.f;     // an all-zero row keeps codes 0 instead of NaN
  if ((tid & 15) == 0) scale[(int64_t)bh * scale_pitch + row] = sc;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= ((uint32_t)(uint8_t)q_half_away(v[j], sc)) << (8 * j);
    hi |= ((uint32_t)(uint8_t)q_half_away(v[4 + j], sc)) << (8 * j);
  }
  *reinterpret_cast<uint2*>(xi8 + ((int64_t)bh * N + row) * 128 + c) = make_uint2(lo, hi);
}


// ---- the reference's block quantiser, bit for bit --------------------------------------------------------
// quant_per_block_int8_kernel (src/ops/vendor/sageattention/triton/quant_per_block.py:21-47): one scale per
// block of `blk` token rows x 128 channels, scale = max|x * mul| / 127, code = trunc(x * mul / scale + 0.5 sign).
// Triton lowers both fp32 divisions to div.full.f32 (not IEEE), so this kernel issues the same instruction;
// an all-zero block gives scale 0 and 0 / 0 = NaN, which the float -> int conversion turns into code 0.
__device__ __forceinline__ float div_full(float a, float b) {
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// One CTA per (block, head): 256 threads, 16 threads per row, 8 channels each, rows in steps of 16.
// `mean` (bf16 [BH,128], may be null): subtracted first and the difference rounded to bf16, as k - km is
// formed in the input dtype before the kernel (quant_per_block.py:53-54).
// scale_rows (may be null) receives the block's scale once per token row ([BH, row_pitch]), the layout the
// attention kernel reads; scale_blocks (may be null) is the reference's [BH, ceil(L / blk)].
__global__ void __launch_bounds__(256)
block_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sh, int64_t sn, int H, int L, int blk,
                   const __nv_bfloat16* __restrict__ mean, float mul, int8_t* __restrict__ xi8, int64_t ob, int64_t oh,
                   int64_t on, __nv_bfloat16* __restrict__ xbf, float* __restrict__ scale_blocks, int nblk,
                   float* __restrict__ scale_rows, int row_pitch) {
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, r0 = blockIdx.x * blk;
  const int tid = threadIdx.x, c = (tid & 15) * 8;
  const __nv_bfloat16* src = x + b * sb + h * sh;
  float m[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) m[j] = mean ? __bfloat162float(mean[(int64_t)bh * 128 + c + j]) : 0.f;
  auto load_row = [&](int row, float (&v)[8]) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)row * sn + c));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f0 = __uint_as_float(w[j] << 16), f1 = __uint_as_float(w[j] & 0xFFFF0000u);
      if (mean) {
        f0 = __bfloat162float(__float2bfloat16_rn(f0 - m[2 * j]));
        f1 = __bfloat162float(__float2bfloat16_rn(f1 - m[2 * j + 1]));
      }
      v[2 * j] = f0; v[2 * j + 1] = f1;
    }
  };
  float amax = 0.f;
  for (int row = r0 + (tid >> 4); row < min(L, r0 + blk); row += 16) {
    float v[8];
    load_row(row, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j] * mul));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __shared__ float s_max[8];
  if ((tid & 31) == 0) s_max[tid >> 5] = amax;
  __syncthreads();
  amax = s_max[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_max[w]);
  const float sc = div_full(amax, 127.f);
  if (tid == 0 && scale_blocks) scale_blocks[(int64_t)bh * nblk + blockIdx.x] = sc;
  for (int row = r0 + (tid >> 4); row < min(L, r0 + blk); row += 16) {
    float v[8];
    load_row(row, v);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float y = div_full(v[j] * mul, sc);
      y += y >= 0.f ? 0.5f : -0.5f;
      const int q = (y != y) ? 0 : (int)y;                      // truncation towards zero; NaN -> 0
      (j < 4 ? lo : hi) |= ((uint32_t)(uint8_t)(int8_t)q) << (8 * (j & 3));
    }
    *reinterpret_cast<uint2*>(xi8 + b * ob + h * oh + (int64_t)row * on + c) = make_uint2(lo, hi);
    if (xbf) {
      uint4 o4;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o4);
      if (mean) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { __nv_bfloat162 pk = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]); ow[j] = *reinterpret_cast<uint32_t*>(&pk); }
      } else {
        o4 = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)row * sn + c));
      }
      *reinterpret_cast<uint4*>(xbf + ((int64_t)bh * L + row) * 128 + c) = o4;
    }
    if (scale_rows && (tid & 15) == 0) scale_rows[(int64_t)bh * row_pitch + row] = fmaxf(sc, 1e-30f);
  }
}

}  // namespace hq

extern "C" int hq_prefill_quant_workspace_bytes(int B, int H_KV, int64_t* bytes) {
  using namespace hq;
  HQ_REQUIRE(bytes && B > 0 && H_KV > 0, HQ_ERR_INVALID, "hq_prefill_quant_workspace_bytes: bad sizes");
  *bytes = (int64_t)B * H_KV * kMeanChunks * 128 * 4;
  return HQ_OK;
}

extern "C" int hq_prefill_quant(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_sn,
                                const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn,
                                int B, int H_Q, int H_KV, int N, float sm_scale, int smooth_k,
                                void* q_i8, void* q_bf, float* q_scale,
                                void* k_i8, void* k_bf, float* k_scale, void* k_mean,
                                void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace hq;
  HQ_REQUIRE(B > 0 && H_Q > 0 && H_KV > 0 && N > 0, HQ_ERR_INVALID, "hq_prefill_quant: bad sizes");
  HQ_REQUIRE(q && k && q_i8 && q_bf && q_scale && k_i8 && k_bf && k_scale && k_mean && workspace, HQ_ERR_INVALID,
             "hq_prefill_quant: null pointer");
  int64_t need = 0;
  hq_prefill_quant_workspace_bytes(B, H_KV, &need);
  HQ_REQUIRE(workspace_bytes >= need, HQ_ERR_WORKSPACE, "hq_prefill_quant: workspace of %lld bytes needed", (long long)need);
  HQ_REQUIRE(aligned16(q) && aligned16(k) && q_sb % 8 == 0 && q_sh % 8 == 0 && q_sn % 8 == 0 && k_sb % 8 == 0 &&
                 k_sh % 8 == 0 && k_sn % 8 == 0,
             HQ_ERR_ALIGNMENT, "hq_prefill_quant: q/k rows must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const __nv_bfloat16* kk = (const __nv_bfloat16*)k;
  kmean_partial_kernel<<<dim3(kMeanChunks, B * H_KV), 256, 0, st>>>(kk, k_sb, k_sh, k_sn, H_KV, N, (float*)workspace);
  kmean_final_kernel<<<B * H_KV, 128, 0, st>>>((const float*)workspace, N, smooth_k, (__nv_bfloat16*)k_mean);
  const int nrb = (N + 15) / 16;
  row_quant_kernel<true><<<dim3(nrb, B * H_KV), 256, 0, st>>>(kk, k_sb, k_sh, k_sn, H_KV, N, (const __nv_bfloat16*)k_mean, 1.0f,
                                                             (int8_t*)k_i8, (__nv_bfloat16*)k_bf, k_scale, (N + 63) / 64 * 64);
  row_quant_kernel<false><<<dim3(nrb, B * H_Q), 256, 0, st>>>((const __nv_bfloat16*)q, q_sb, q_sh, q_sn, H_Q, N, nullptr,
                                                             sm_scale * 1.44269504f, (int8_t*)q_i8, (__nv_bfloat16*)q_bf,
                                                             q_scale, (N + 63) / 64 * 64);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

extern "C" int hq_per_block_int8(const void* x, int64_t x_sb, int64_t x_sh, int64_t x_sn, int B, int H, int L, int blk,
                                 float mul, const void* mean, void* x_i8, int64_t o_sb, int64_t o_sh, int64_t o_sn,
                                 float* scale, void* stream) {
  using namespace hq;
  HQ_REQUIRE(x && x_i8 && scale && B > 0 && H > 0 && L > 0 && blk > 0, HQ_ERR_INVALID, "hq_per_block_int8: bad arguments");
  HQ_REQUIRE(aligned16(x) && x_sb % 8 == 0 && x_sh % 8 == 0 && x_sn % 8 == 0 && ((uintptr_t)x_i8 & 7) == 0 && o_sb % 8 == 0 &&
                 o_sh % 8 == 0 && o_sn % 8 == 0, HQ_ERR_ALIGNMENT, "hq_per_block_int8: rows must be 16-byte (input) / 8-byte (codes) aligned");
  const int nblk = (L + blk - 1) / blk;
  block_quant_kernel<<<dim3(nblk, B * H), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, x_sb, x_sh, x_sn, H, L, blk, (const __nv_bfloat16*)mean, mul, (int8_t*)x_i8, o_sb, o_sh, o_sn,
      nullptr, scale, nblk, nullptr, 0);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

extern "C" int hq_prefill_quant_blocks(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_sn,
                                       const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn,
                                       int B, int H_Q, int H_KV, int N, float sm_scale, int smooth_k,
                                       void* q_i8, void* q_bf, float* q_scale,
                                       void* k_i8, void* k_bf, float* k_scale, void* k_mean,
                                       void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace hq;
  HQ_REQUIRE(B > 0 && H_Q > 0 && H_KV > 0 && N > 0, HQ_ERR_INVALID, "hq_prefill_quant_blocks: bad sizes");
  HQ_REQUIRE(q && k && q_i8 && q_bf && q_scale && k_i8 && k_bf && k_scale && k_mean && workspace, HQ_ERR_INVALID,
             "hq_prefill_quant_blocks: null pointer");
  int64_t need = 0;
  hq_prefill_quant_workspace_bytes(B, H_KV, &need);
  HQ_REQUIRE(workspace_bytes >= need, HQ_ERR_WORKSPACE, "hq_prefill_quant_blocks: workspace of %lld bytes needed", (long long)need);
  HQ_REQUIRE(aligned16(q) && aligned16(k) && q_sb % 8 == 0 && q_sh % 8 == 0 && q_sn % 8 == 0 && k_sb % 8 == 0 &&
                 k_sh % 8 == 0 && k_sn % 8 == 0,
             HQ_ERR_ALIGNMENT, "hq_prefill_quant_blocks: q/k rows must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const __nv_bfloat16* kk = (const __nv_bfloat16*)k;
  kmean_partial_kernel<<<dim3(kMeanChunks, B * H_KV), 256, 0, st>>>(kk, k_sb, k_sh, k_sn, H_KV, N, (float*)workspace);
  kmean_final_kernel<<<B * H_KV, 128, 0, st>>>((const float*)workspace, N, smooth_k, (__nv_bfloat16*)k_mean);
  const int pitch = (N + 63) / 64 * 64;
  block_quant_kernel<<<dim3((N + 63) / 64, B * H_KV), 256, 0, st>>>(
      kk, k_sb, k_sh, k_sn, H_KV, N, 64, smooth_k ? (const __nv_bfloat16*)k_mean : nullptr, 1.0f, (int8_t*)k_i8,
      (int64_t)H_KV * N * 128, (int64_t)N * 128, 128, (__nv_bfloat16*)k_bf, nullptr, 0, k_scale, pitch);
  block_quant_kernel<<<dim3((N + 127) / 128, B * H_Q), 256, 0, st>>>(
      (const __nv_bfloat16*)q, q_sb, q_sh, q_sn, H_Q, N, 128, nullptr, sm_scale * 1.44269504f, (int8_t*)q_i8,
      (int64_t)H_Q * N * 128, (int64_t)N * 128, 128, (__nv_bfloat16*)q_bf, nullptr, 0, q_scale, pitch);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}
