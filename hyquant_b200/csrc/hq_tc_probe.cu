// Tensor-pipe peak probe: how fast this GPU's tcgen05 pipe runs kind::i8, kind::f8f6f4 and kind::f16 products
// when nothing else is in the way (operands resident in shared memory, accumulators in tensor memory, no loads, no
// epilogue).  The benchmark divides the prefill kernel's rate by these measured figures instead of by a nominal
// "2 x bf16" for the 8-bit kinds.  It has no counterpart in the reference.
//
// One CTA per SM; one thread issues, per step, the K steps of a 128 x 256 product out of one 128-row A tile and one
// 256-row B tile (128-byte rows, 128-byte swizzle) into two alternating 256-column accumulators, commits every 16
// steps and waits - with a poll limit - before it runs further ahead.
#include "hq_tc05.cuh"

namespace hq {

constexpr int kProbeThreads = 128;

template <int KIND>   // 0 = kind::i8 (s8 x s8 -> s32), 1 = kind::f8f6f4 (e4m3 x e4m3 -> f32), 2 = kind::f16 (bf16 -> f32)
__global__ void __launch_bounds__(kProbeThreads, 1) tc_peak_kernel(int steps, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;                    // 128 rows x 128 B
  uint8_t* sB = smem + 16384;            // 256 rows x 128 B
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 16384 + 32768);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 2);
  const int tid = threadIdx.x;
  // small finite operand values (e4m3 / bf16 bit patterns of modest magnitude, small integers) so that the data paths
  // toggle without overflowing anything
  for (int x = tid; x < (16384 + 32768) / 4; x += kProbeThreads) {
    const uint32_t h = (uint32_t)x * 2654435761u;
    uint32_t w;
    if (KIND == 2) w = 0x3C003C00u ^ (h & 0x007F007Fu);                 // bf16 values near 0.0078
    else if (KIND == 1) w = 0x30303030u ^ (h & 0x07070707u);             // e4m3 values near 0.5
    else w = h & 0x07070707u;                                            // s8 values 0..7
    reinterpret_cast<uint32_t*>(smem)[x] = w;
  }
  if (tid == 0) { mbar_init(bar, 1); *abort_flag = 0; fence_mbar_init(); }
  if (tid < 32) tc::tmem_alloc(tmem_slot, 512);
  fence_proxy_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  if (tid == 0) {
    constexpr uint32_t idesc = KIND == 0 ? tc::make_idesc(2, tc::kFmtS8, tc::kFmtS8, 128, 256)
                               : KIND == 1 ? tc::make_idesc(1, tc::kFmtE4M3, tc::kFmtE4M3, 128, 256)
                                           : tc::make_idesc(1, tc::kFmtBF16, tc::kFmtBF16, 128, 256);
    const uint64_t dA = tc::smem_desc_k128(sA, 0), dB = tc::smem_desc_k128(sB, 0);
    constexpr int kSteps = KIND == 2 ? 4 : 4;             // K steps of 32 bytes across the 128-byte rows
    uint32_t phase = 0;
    bool ok = true;
    for (int s = 0; ok && s < steps; ++s) {
      const uint32_t d = tmem + 256u * (s & 1);
#pragma unroll
      for (int k = 0; k < kSteps; ++k) {
        if (KIND == 0) tc::mma_s8_ss(d, dA + 2 * k, dB + 2 * k, idesc, (s > 1 || k > 0) ? 1u : 0u);
        else if (KIND == 1) {
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                       "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(dA + 2 * k), "l"(dB + 2 * k),
                       "r"(idesc), "r"((s > 1 || k > 0) ? 1u : 0u) : "memory");
        } else tc::mma_bf16_ss(d, dA + 2 * k, dB + 2 * k, idesc, (s > 1 || k > 0) ? 1u : 0u);
      }
      if ((s & 15) == 15 || s + 1 == steps) {
        tc::mma_commit(bar);
        ok = tc::mbar_wait_abortable(bar, phase, abort_flag, 0, 4000000u);
        phase ^= 1u;
      }
    }
    if (!ok) atomicOr(status, 4);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (tid < 32) tc::tmem_dealloc(tmem, 512);
}

}  // namespace hq

// Launches the probe for `kind` (0 = i8, 1 = f8f6f4 e4m3, 2 = f16 bf16) on every SM; the caller times it (CUDA events)
// and computes sms * steps * 2 * 128 * 256 * K / time with K = 128 for the 8-bit kinds and 64 for bf16 (a step runs
// the K range of one 128-byte operand row).  `status` (device word, zeroed by the caller): bit 2 = a bounded wait expired.
extern "C" int hq_tc_peak(int kind, int steps, int* status, int* sms_out, void* stream) {
  using namespace hq;
  HQ_REQUIRE(kind >= 0 && kind <= 2 && steps > 0 && status != nullptr, HQ_ERR_INVALID, "hq_tc_peak: kind 0..2, steps > 0, status required");
  const size_t smem = 16384 + 32768 + 64 + 1024;
  const int sms = sm_count();
  if (sms_out) *sms_out = sms;
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == 0) {
    HQ_CUDA(cudaFuncSetAttribute(tc_peak_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc_peak_kernel<0><<<sms, kProbeThreads, smem, st>>>(steps, status);
  } else if (kind == 1) {
    HQ_CUDA(cudaFuncSetAttribute(tc_peak_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc_peak_kernel<1><<<sms, kProbeThreads, smem, st>>>(steps, status);
  } else {
    HQ_CUDA(cudaFuncSetAttribute(tc_peak_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc_peak_kernel<2><<<sms, kProbeThreads, smem, st>>>(steps, status);
  }
  HQ_CUDA(cudaGetLastError());
  return HQ_OK;
}
