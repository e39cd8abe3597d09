// Per-token symmetric quantise + pack, 8 / 4 / 2 bits (flush of the staging buffer
// and the quantisation step of the prefill->decode reorganisation).
//
// HBM-bound: reads 256 B (bf16) per token, writes 64 B codes + 2 B scale.  Eight
// lanes own a token row (16 channels each), so a warp works on four rows at a time;
// a row's loads are one 256-byte line and its stores one 64-byte line.
#include "hq_quant.cuh"

namespace hq {

template <typename T, int BITS>
__global__ void __launch_bounds__(256)
quant_pack_kernel(const T* __restrict__ x, int64_t x_stride_bh, int64_t x_stride_n, int BH, int n,
                  uint8_t* __restrict__ packed, int64_t packed_stride_bh,
                  __half* __restrict__ scale, int64_t scale_stride_bh,
                  int64_t dst_off, int scale_mode) {
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t rows = (int64_t)BH * n;
  for (int64_t r0 = 4 * warp0; r0 < rows; r0 += 4 * nwarps) {
    const int64_t mine = r0 + (lane >> 3);
    const bool live = mine < rows;
    const int64_t r = live ? mine : rows - 1;          // lanes past the end redo the last row and store nothing
    const int bh = rows <= 0x7FFFFFFF ? (int)((uint32_t)r / (uint32_t)n) : (int)(r / n);
    const int tok = (int)(r - (int64_t)bh * n);
    float v[16];
    load16(x + bh * x_stride_bh + tok * x_stride_n + sub * 16, v);
    uint32_t code[BITS / 2];
    const __half s = quant_row16<BITS>(v, scale_mode, code);
    if (live) {
      store_codes16<BITS>(packed + bh * packed_stride_bh + (dst_off + tok) * (16 * BITS), sub, code);
      if (sub == 0) scale[bh * scale_stride_bh + dst_off + tok] = s;
    }
  }
}

// One new token per head into slot `slot` of the staging buffers: k_new/v_new [BH, 128] (row stride
// given) -> staging_k/v [BH, 128 slots, 128].  64 threads per head: 32 move K, 32 move V, 8 bytes each.
__global__ void __launch_bounds__(256)
staging_append_kernel(const uint2* __restrict__ k_new, const uint2* __restrict__ v_new, int64_t k_stride8, int64_t v_stride8,
                      uint2* __restrict__ staging_k, uint2* __restrict__ staging_v, int BH, int slot) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int bh = idx >> 6, part = idx & 63;
  if (bh >= BH) return;
  const int64_t dst = ((int64_t)bh * HQ_GROUP_SIZE + slot) * 32 + (part & 31);
  if (part < 32) staging_k[dst] = __ldg(k_new + bh * k_stride8 + part);
  else staging_v[dst] = __ldg(v_new + bh * v_stride8 + (part - 32));
}

}  // namespace hq

extern "C" int hq_staging_append(const void* k_new, const void* v_new, int64_t k_stride, int64_t v_stride,
                                 void* staging_k, void* staging_v, int BH, int slot, void* stream) {
  using namespace hq;
  HQ_REQUIRE(BH >= 0 && slot >= 0 && slot < HQ_GROUP_SIZE, HQ_ERR_INVALID, "hq_staging_append: slot %d outside 0..127", slot);
  if (BH == 0) return HQ_OK;
  HQ_REQUIRE(k_new && v_new && staging_k && staging_v, HQ_ERR_INVALID, "hq_staging_append: null pointer");
  HQ_REQUIRE(((uintptr_t)k_new % 8) == 0 && ((uintptr_t)v_new % 8) == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 &&
                 ((uintptr_t)staging_k % 8) == 0 && ((uintptr_t)staging_v % 8) == 0,
             HQ_ERR_ALIGNMENT, "hq_staging_append: rows must be 8-byte aligned");
  const int threads = BH * 64;
  staging_append_kernel<<<(threads + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const uint2*)k_new, (const uint2*)v_new, k_stride / 4, v_stride / 4, (uint2*)staging_k, (uint2*)staging_v, BH, slot);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}

namespace hq {
template <int BITS>
static int launch_quant(const void* x, int in_dtype, int64_t x_stride_bh, int64_t x_stride_n, int BH, int n, uint8_t* p,
                        int64_t packed_stride_bh, __half* s, int64_t scale_stride_bh, int64_t dst_off, int scale_mode,
                        dim3 grid, cudaStream_t st) {
  dim3 block(256);
  if (in_dtype == HQ_BF16)
    quant_pack_kernel<__nv_bfloat16, BITS><<<grid, block, 0, st>>>((const __nv_bfloat16*)x, x_stride_bh, x_stride_n, BH, n, p,
                                                                   packed_stride_bh, s, scale_stride_bh, dst_off, scale_mode);
  else if (in_dtype == HQ_F16)
    quant_pack_kernel<__half, BITS><<<grid, block, 0, st>>>((const __half*)x, x_stride_bh, x_stride_n, BH, n, p,
                                                            packed_stride_bh, s, scale_stride_bh, dst_off, scale_mode);
  else if (in_dtype == HQ_F32)
    quant_pack_kernel<float, BITS><<<grid, block, 0, st>>>((const float*)x, x_stride_bh, x_stride_n, BH, n, p,
                                                           packed_stride_bh, s, scale_stride_bh, dst_off, scale_mode);
  else
    HQ_REQUIRE(false, HQ_ERR_UNSUPPORTED, "hq_quant_pack: unknown dtype %d", in_dtype);
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}
}  // namespace hq

extern "C" int hq_quant_pack(const void* x, int in_dtype, int64_t x_stride_bh, int64_t x_stride_n,
                             int BH, int n, int nbits, void* packed, int64_t packed_stride_bh,
                             void* scale, int64_t scale_stride_bh,
                             int64_t dst_token_offset, int scale_mode, void* stream) {
  using namespace hq;
  HQ_REQUIRE(BH >= 0 && n >= 0 && dst_token_offset >= 0, HQ_ERR_INVALID, "hq_quant_pack: negative size");
  HQ_REQUIRE(nbits == 2 || nbits == 4 || nbits == 8, HQ_ERR_UNSUPPORTED, "hq_quant_pack: nbits must be 2, 4 or 8, got %d", nbits);
  if (BH == 0 || n == 0) return HQ_OK;
  HQ_REQUIRE(x && packed && scale, HQ_ERR_INVALID, "hq_quant_pack: null pointer");
  HQ_REQUIRE(scale_mode == 0 || scale_mode == 1, HQ_ERR_INVALID, "hq_quant_pack: scale_mode must be 0 or 1");
  HQ_REQUIRE(((uintptr_t)x % 16) == 0 && (x_stride_bh % 8) == 0 && (x_stride_n % 8) == 0, HQ_ERR_ALIGNMENT,
             "hq_quant_pack: x rows must be 16-byte aligned (strides multiples of 8 elements)");
  const int lane_bytes = 2 * nbits;      // bytes one lane stores
  HQ_REQUIRE(((uintptr_t)packed % lane_bytes) == 0 && (packed_stride_bh % lane_bytes) == 0, HQ_ERR_ALIGNMENT,
             "hq_quant_pack: packed rows must be %d-byte aligned", lane_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows = (int64_t)BH * n;
  const int warps_per_block = 8;
  int64_t blocks = (rows + 4 * warps_per_block - 1) / (4 * warps_per_block);      // a warp takes four rows per trip
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks);
  uint8_t* p = (uint8_t*)packed;
  __half* s = (__half*)scale;
  if (nbits == 8) return launch_quant<8>(x, in_dtype, x_stride_bh, x_stride_n, BH, n, p, packed_stride_bh, s, scale_stride_bh, dst_token_offset, scale_mode, grid, st);
  if (nbits == 4) return launch_quant<4>(x, in_dtype, x_stride_bh, x_stride_n, BH, n, p, packed_stride_bh, s, scale_stride_bh, dst_token_offset, scale_mode, grid, st);
  return launch_quant<2>(x, in_dtype, x_stride_bh, x_stride_n, BH, n, p, packed_stride_bh, s, scale_stride_bh, dst_token_offset, scale_mode, grid, st);
}

extern "C" int hq_quant_pack_int4(const void* x, int in_dtype, int64_t x_stride_bh, int64_t x_stride_n,
                                  int BH, int n, void* packed, int64_t packed_stride_bh,
                                  void* scale, int64_t scale_stride_bh,
                                  int64_t dst_token_offset, int scale_mode, void* stream) {
  return hq_quant_pack(x, in_dtype, x_stride_bh, x_stride_n, BH, n, 4, packed, packed_stride_bh, scale, scale_stride_bh,
                       dst_token_offset, scale_mode, stream);
}
