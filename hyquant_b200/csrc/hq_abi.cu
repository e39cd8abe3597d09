// Library identification, thread-local error text and device queries of the C ABI.
#include "hq_common.cuh"

#include <string.h>

namespace hq {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return HQ_ERR_CUDA;
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_sms = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    cached_dev = dev;
    cached_sms = sms;
  }
  return cached_sms;
}

}  // namespace hq

extern "C" const char* hq_version(void) { return "hyquant_b200 0.1 (sm_100a)"; }
extern "C" const char* hq_last_error(void) { return hq::g_err; }
