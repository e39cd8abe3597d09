// Warp-level per-token INT4 quantiser shared by the flush kernel and the cache
// reorganisation kernel.  Bit-exact contract (reference
// src/ops/decode_d_stage.py:62-68, 104-111):
//   absmax = max(max|x|, 1e-5);  scale = half_rn(absmax / 7)   [IEEE fp32 divide]
//   q = clamp(rint(x / float(scale)), -8, 7)                    [IEEE divide, half-to-even]
//   byte = (q[2i] & 0xF) | ((q[2i+1] & 0xF) << 4)
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

// All 32 lanes call this with their 4 channels of one 128-channel token.
// Returns the fp16 scale (same on every lane) and this lane's 4 codes packed
// into 16 bits (channels 4l,4l+1 in the low byte, 4l+2,4l+3 in the high byte).
__device__ __forceinline__ __half quant_row_int4(const float (&v)[4], int scale_mode, uint16_t& code) {
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-5f);
  const float s32 = scale_mode == 0 ? __fdiv_rn(amax, 7.0f) : __fmul_rn(amax, __fdiv_rn(1.0f, 7.0f));
  const __half sh = __float2half_rn(s32);
  const float sf = __half2float(sh);
  uint32_t c = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float q = rintf(__fdiv_rn(v[i], sf));
    q = fminf(fmaxf(q, -8.0f), 7.0f);
    // NaN (0/0 cannot happen: sf >= half(1e-5/7) > 0; inf/inf gives NaN) -> int conversion yields 0
    c |= ((uint32_t)(__float2int_rn(q)) & 0xFu) << (4 * i);
  }
  code = (uint16_t)c;
  return sh;
}

}  // namespace hq
