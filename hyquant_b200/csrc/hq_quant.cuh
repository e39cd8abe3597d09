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

// Work split: EIGHT lanes per token row, sixteen channels per lane, so a warp works on four rows at a time and the
// per-row overhead (row arithmetic, the maximum's shuffles, the scale) is paid once per four rows.  (With a whole warp
// on one row the kernels were bound by instruction issue at a fifth of the memory bandwidth.)
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
__device__ __forceinline__ void load16(const __half* p, float (&v)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    v[2 * i] = __low2float(h); v[2 * i + 1] = __high2float(h);
  }
}
__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 f = *reinterpret_cast<const float4*>(p + 4 * i);
    v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
  }
}

// Called by all 32 lanes; lanes 8 g .. 8 g + 7 hold one 128-channel token (lane l: channels 16 (l & 7) .. + 15).
// Returns the row's fp16 scale (the same on the row's eight lanes) and this lane's 16 codes packed in channel order
// into `code` (BITS / 2 words: 16 bytes at 8 bits, 8 at 4, 4 at 2); a token row is 16 * BITS bytes and lane l owns
// bytes [2 BITS (l & 7), 2 BITS ((l & 7) + 1)).
// q = rint(x / sf) with the IEEE quotient without sixteen IEEE divisions per lane: the product with the correctly
// rounded reciprocal is within 1.5 * 2^-23 (relative) of the rounded quotient, and |quotient| < 2^BITS, so the two round
// to the same integer unless the product lies within kNearTie of a half-integer - only then the division is done.
// Infinities and NaNs take the same values either way (x * 0 = x / inf = 0 or NaN alike, inf * r = inf / sf).
// NaN inputs: 0/0 cannot happen (the scale is >= half(1e-5 / q_max) > 0); inf / inf gives NaN, which the clamp turns
// into the lowest code.
template <int BITS>
__device__ __forceinline__ __half quant_row16(const float (&v)[16], int scale_mode, uint32_t (&code)[BITS / 2]) {
  constexpr float qmax = (float)((1 << (BITS - 1)) - 1), qmin = -(float)(1 << (BITS - 1));
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-5f);
  const float s32 = scale_mode == 0 ? __fdiv_rn(amax, qmax) : __fmul_rn(amax, __fdiv_rn(1.0f, qmax));
  const __half sh = __float2half_rn(s32);
  const float sf = __half2float(sh);
  const float rcp = __frcp_rn(sf);
  constexpr float kNearTie = BITS == 8 ? 1.5e-4f : 6e-6f;      // > 4 x the largest possible difference of the two
  constexpr int kPerWord = 32 / BITS;
#pragma unroll
  for (int w = 0; w < BITS / 2; ++w) {
    uint32_t c = 0;
#pragma unroll
    for (int i = 0; i < kPerWord; ++i) {
      const float x = v[w * kPerWord + i];
      const float t = __fmul_rn(x, rcp);
      float q = rintf(t);
      if (0.5f - fabsf(t - q) < kNearTie) q = rintf(__fdiv_rn(x, sf));
      q = fminf(fmaxf(q, qmin), qmax);
      c |= ((uint32_t)(__float2int_rn(q)) & ((1u << BITS) - 1u)) << (BITS * i);
    }
    code[w] = c;
  }
  return sh;
}

// store the lane's codes of a token row that starts at `prow` (sub = lane & 7)
template <int BITS>
__device__ __forceinline__ void store_codes16(uint8_t* prow, int sub, const uint32_t (&code)[BITS / 2]) {
  if (BITS == 8) reinterpret_cast<uint4*>(prow)[sub] = make_uint4(code[0], code[1], code[2], code[3]);
  else if (BITS == 4) reinterpret_cast<uint2*>(prow)[sub] = make_uint2(code[0], code[BITS == 4 ? 1 : 0]);
  else reinterpret_cast<uint32_t*>(prow)[sub] = code[0];
}

// quantise one token row (eight lanes) with a run-time bit width and store its codes if `store`; returns the scale
__device__ __forceinline__ __half quant_store_row16(int bits, const float (&v)[16], int scale_mode, uint8_t* prow, int sub, bool store) {
  __half s;
  if (bits == 8) { uint32_t c[4]; s = quant_row16<8>(v, scale_mode, c); if (store) store_codes16<8>(prow, sub, c); }
  else if (bits == 4) { uint32_t c[2]; s = quant_row16<4>(v, scale_mode, c); if (store) store_codes16<4>(prow, sub, c); }
  else { uint32_t c[1]; s = quant_row16<2>(v, scale_mode, c); if (store) store_codes16<2>(prow, sub, c); }
  return s;
}

}  // namespace hq
