// Library-wide state of the C ABI: last-error string, launch counter, device
// status word written by kernels whose bounded waits gave up.
#include "common.cuh"

#include <cstring>

namespace fg {

std::atomic<int64_t> g_launches{0};

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

// 0 = healthy.  A kernel whose mbarrier wait ran out of time stores a non-zero
// code here (see sm100_common.cuh) and returns without finishing its tile.
__device__ int g_device_status = 0;

int* device_status_ptr() {
  static thread_local int cached_dev = -1;
  static thread_local int* ptr = nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev || ptr == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    ptr = (int*)p;
    cached_dev = dev;
  }
  return ptr;
}

}  // namespace fg

namespace fg {
std::atomic<int> g_sm_budget{0};  // 0 = use every SM of the device
int sm_budget() {
  const int n = num_sms();
  const int b = g_sm_budget.load(std::memory_order_relaxed);
  return (b > 0 && b < n) ? b : n;
}
}  // namespace fg

extern "C" int fg_set_num_sms(int sms) {
  if (sms < 0) return fg::fail(FG_ERR_INVALID, "fg_set_num_sms: negative SM count");
  fg::g_sm_budget.store(sms, std::memory_order_relaxed);
  return FG_OK;
}
extern "C" int fg_get_num_sms(void) { return fg::sm_budget(); }

extern "C" int fg_abi_version(void) { return 1; }
extern "C" const char* fg_last_error(void) { return fg::last_error_buf(); }
extern "C" int64_t fg_launch_count(void) { return fg::g_launches.load(std::memory_order_relaxed); }

extern "C" int fg_device_status(int reset) {
  int v = 0;
  int* p = fg::device_status_ptr();
  if (!p) return fg::fail(FG_ERR_CUDA, "device status word unavailable");
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return fg::fail(FG_ERR_CUDA, "reading the device status word failed");
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpy(p, &z, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}
