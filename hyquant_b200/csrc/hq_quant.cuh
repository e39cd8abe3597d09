// Warp-level per-token quantiser (8 / 4 / 2 bits) shared by the flush kernel and the cache
// reorganisation kernel.  Bit-exact contract (reference
// src/ops/decode_d_stage.py:50-77, 104-135), q_max = 2^(bits-1) - 1:
//   absmax = max(max|x|, 1e-5);  scale = half_rn(absmax / q_max)   [IEEE fp32 divide]
//   q = clamp(rint(x / float(scale)), -q_max - 1, q_max)            [IEEE divide, half-to-even]
//   8 bits: one byte per channel;  4 bits: byte = (q[2i] & 0xF) | ((q[2i+1] & 0xF) << 4);
//   2 bits: byte = (q[4i] & 3) | (q[4i+1] & 3) << 2 | (q[4i+2] & 3) << 4 | (q[4i+3] & 3) << 6
// This translation unit must not be built with --use_fast_math.
#pragma once
#include "hq_common.cuh"

namespace hq {

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(u.x << 16);
  v[1] = __uint_as_float(u.x & 0xFFFF0000u);
  v[2] = __uint_as_float(u.y << 16);
  v[3] = __uint_as_float(u.y & 0xFFFF0000u);
}
__device__ __forceinline__ void load4(const __half* p, float (&v)[4]) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  __half2 a = *reinterpret_cast<__half2*>(&u.x), b = *reinterpret_cast<__half2*>(&u.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}

// All 32 lanes call this with their 4 channels of one 128-channel token.  Returns the fp16 scale (same on
// every lane) and this lane's 4 codes in the low bits of `code`: 4 bytes (BITS = 8), 16 bits (4) or one byte (2);
// a token row is 16 * BITS bytes and lane l owns bytes [l * BITS / 2, (l + 1) * BITS / 2).
// NaN inputs: 0/0 cannot happen (the scale is >= half(1e-5 / q_max) > 0); inf / inf gives NaN, which converts to code 0.
template <int BITS>
__device__ __forceinline__ __half quant_row_bits(const float (&v)[4], int scale_mode, uint32_t& code) {
  constexpr float qmax = (float)((1 << (BITS - 1)) - 1), qmin = -(float)(1 << (BITS - 1));
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-5f);
  const float s32 = scale_mode == 0 ? __fdiv_rn(amax, qmax) : __fmul_rn(amax, __fdiv_rn(1.0f, qmax));
  const __half sh = __float2half_rn(s32);
  const float sf = __half2float(sh);
  uint32_t c = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float q = rintf(__fdiv_rn(v[i], sf));
    q = fminf(fmaxf(q, qmin), qmax);
    c |= ((uint32_t)(__float2int_rn(q)) & ((1u << BITS) - 1u)) << (BITS * i);
  }
  code = c;
  return sh;
}

// store the lane's codes of a token row that starts at `prow`
template <int BITS>
__device__ __forceinline__ void store_codes(uint8_t* prow, int lane, uint32_t code) {
  if (BITS == 8) reinterpret_cast<uint32_t*>(prow)[lane] = code;
  else if (BITS == 4) reinterpret_cast<uint16_t*>(prow)[lane] = (uint16_t)code;
  else prow[lane] = (uint8_t)code;
}

// quantise one token row with a run-time bit width and store its codes; returns the scale
__device__ __forceinline__ __half quant_store_row(int bits, const float (&v)[4], int scale_mode, uint8_t* prow, int lane) {
  uint32_t c;
  __half s;
  if (bits == 8) { s = quant_row_bits<8>(v, scale_mode, c); store_codes<8>(prow, lane, c); }
  else if (bits == 4) { s = quant_row_bits<4>(v, scale_mode, c); store_codes<4>(prow, lane, c); }
  else { s = quant_row_bits<2>(v, scale_mode, c); store_codes<2>(prow, lane, c); }
  return s;
}

}  // namespace hq
