// Library-wide state of fpq_b200: error text, device queries, version.
#include "common.cuh"

#include <mutex>

namespace fpq {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

const char* get_error() { return g_error; }

int sm_count() {
  static int cached[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace fpq

extern "C" int fpq_version(void) { return 105; }

extern "C" const char* fpq_last_error(void) { return fpq::get_error(); }

extern "C" int fpq_check_device(int device) {
  int major = 0, minor = 0;
  FPQ_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  FPQ_CHECK_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  if (major != 10) {
    fpq::set_error("device %d has compute capability %d.%d; this library is built for sm_100a only", device, major, minor);
    return FPQ_ERR_UNSUPPORTED_DEVICE;
  }
  return FPQ_OK;
}
