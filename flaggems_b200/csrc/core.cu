// Library-wide state of the C ABI: last-error string, launch counter, device
// status word written by kernels whose bounded waits gave up.
#include "common.cuh"
#include "sm100_common.cuh"

#include <cstring>
#include <mutex>

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
// code here (see sm100_common.cuh) and returns without finishing its tile; kernels with
// bounded waits that start later read the word first and return at once (the launch drains).
// `host_mirror`, when set, points at this device's word of g_host_status through the
// mapping of the pinned page: the kernel stores the same code there, so the host sees it
// without synchronising and every entry point refuses further launches until the word is
// cleared with fg_device_status(1).
struct alignas(16) DeviceStatus {
  int word;
  int pad;
  int* host_mirror;
};
__device__ DeviceStatus g_device_status = {0, 0, nullptr};

constexpr int kMaxDevices = 64;
constexpr int kMirrorStride = 16;   // ints between two devices' words (one 64-byte line each)
// One word per device in a page of ordinary host memory that is page-locked and mapped into
// the devices' address spaces on first use (no allocation: the storage is this array).
alignas(4096) static volatile int g_host_status[kMaxDevices * kMirrorStride];
static std::mutex g_mirror_mutex;
static int g_mirror_registered = 0;          // 0 = not tried, 1 = page-locked and mapped, -1 = failed
static int g_mirror_ready[kMaxDevices];      // per device: 0 = not set up, 1 = kernel knows the mirror, -1 = failed
static thread_local bool g_mirror_setup_allowed = true;

MirrorSetupGuard::MirrorSetupGuard() : saved_(g_mirror_setup_allowed) { g_mirror_setup_allowed = false; }
MirrorSetupGuard::~MirrorSetupGuard() { g_mirror_setup_allowed = saved_; }

static int current_device_or_zero() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();   // no driver / no device: the host-only queries still work
    dev = 0;
  }
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

// First use of a device: tell its status struct where the host-visible word is.  One
// cudaHostRegister for the process, one pointer lookup and one 8-byte copy per device.
static void setup_mirror(int dev, DeviceStatus* dstatus) {
  std::lock_guard<std::mutex> lock(g_mirror_mutex);
  if (g_mirror_ready[dev] != 0) return;
  if (g_mirror_registered == 0) {
    const cudaError_t e = cudaHostRegister(const_cast<int*>(g_host_status), sizeof(g_host_status),
                                           cudaHostRegisterMapped | cudaHostRegisterPortable);
    g_mirror_registered = (e == cudaSuccess) ? 1 : -1;
    if (e != cudaSuccess) cudaGetLastError();
  }
  g_mirror_ready[dev] = -1;
  if (g_mirror_registered != 1) return;
  void* dptr = nullptr;
  if (cudaHostGetDevicePointer(&dptr, const_cast<int*>(&g_host_status[dev * kMirrorStride]), 0) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  int* mirror = static_cast<int*>(dptr);
  if (cudaMemcpy(&dstatus->host_mirror, &mirror, sizeof(int*), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  g_mirror_ready[dev] = 1;
}

int* device_status_ptr() {
  static thread_local int cached_dev = -1;
  static thread_local int* ptr = nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev || ptr == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    ptr = &static_cast<DeviceStatus*>(p)->word;
    cached_dev = dev;
  }
  if (dev >= 0 && dev < kMaxDevices && g_mirror_ready[dev] == 0 && g_mirror_setup_allowed)
    setup_mirror(dev, reinterpret_cast<DeviceStatus*>(ptr));
  return ptr;
}

int drained_code() { return g_host_status[current_device_or_zero() * kMirrorStride]; }

int fail_drained(const char* what, int code) {
  return fail(FG_ERR_DEVICE,
              "%s: no kernel was launched: a kernel of this library gave up a bounded wait on this device earlier "
              "(status %d) and its output is incomplete; clear the state with fg_device_status(1)",
              what, code);
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

extern "C" int fg_abi_version(void) { return 2; }
extern "C" const char* fg_last_error(void) { return fg::last_error_buf(); }
extern "C" int64_t fg_launch_count(void) { return fg::g_launches.load(std::memory_order_relaxed); }

extern "C" int fg_device_status(int reset) {
  int v = 0;
  const int dev = fg::current_device_or_zero();
  const int mirrored = fg::g_host_status[dev * fg::kMirrorStride];
  int* p = fg::device_status_ptr();
  if (!p) {
    // no usable device: the host-visible word is all there is
    if (reset) fg::g_host_status[dev * fg::kMirrorStride] = 0;
    if (mirrored != 0) return mirrored;
    return fg::fail(FG_ERR_CUDA, "device status word unavailable");
  }
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return fg::fail(FG_ERR_CUDA, "reading the device status word failed");
  if (v == 0) v = mirrored;
  if (reset) {
    if (v != 0) {
      int z = 0;
      cudaMemcpy(p, &z, sizeof(int), cudaMemcpyHostToDevice);
    }
    fg::g_host_status[dev * fg::kMirrorStride] = 0;
  }
  return v;
}

extern "C" int fg_device_status_nosync(void) { return fg::drained_code(); }

// ---- test hooks ---------------------------------------------------------------------
// Store `code` in the status words of the current device as a kernel that gave up would.
extern "C" int fg_debug_set_status(int code) {
  const int dev = fg::current_device_or_zero();
  fg::g_host_status[dev * fg::kMirrorStride] = code;
  int* p = fg::device_status_ptr();
  if (p && cudaMemcpy(p, &code, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) cudaGetLastError();
  return FG_OK;
}

namespace fg {
namespace {
// One thread waits, with the library's bounded wait, on an mbarrier nobody arrives at.
__global__ void wait_timeout_test_kernel(int* status, unsigned long long limit_ns, int* outcome) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sm100::mbar_init(&bar, 1);
    sm100::mbar_fence_init();
    const bool ok = sm100::mbar_wait(&bar, 0, &abort_flag, status, sm100::kStatusTestTimeout, limit_ns);
    *outcome = ok ? 1 : (abort_flag ? 2 : 3);
    sm100::mbar_inval(&bar);
  }
}
}  // namespace
}  // namespace fg

extern "C" int fg_debug_wait_timeout(int64_t limit_ns, int* outcome_dev, void* stream) {
  FG_REQUIRE(limit_ns > 0 && limit_ns <= 100000000LL, "fg_debug_wait_timeout: limit must be within (0, 100 ms]");
  FG_REQUIRE(outcome_dev != nullptr, "fg_debug_wait_timeout: null outcome pointer");
  int* status = fg::device_status_ptr();
  if (!status) return fg::fail(FG_ERR_CUDA, "device status word unavailable");
  fg::wait_timeout_test_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (unsigned long long)limit_ns, outcome_dev);
  FG_CHECK_LAUNCH("wait_timeout_test_kernel");
  return FG_OK;
}

// ---- strided device-to-device copy on the copy engines ---------------------------------
extern "C" int fg_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                          int64_t width_bytes, int64_t rows, void* stream) {
  FG_REQUIRE(width_bytes >= 0 && rows >= 0, "copy_2d: negative size");
  if (width_bytes == 0 || rows == 0) return FG_OK;
  FG_REQUIRE(dst != nullptr && src != nullptr, "copy_2d: null pointer");
  FG_REQUIRE(dst_pitch_bytes >= width_bytes && src_pitch_bytes >= width_bytes, "copy_2d: pitch smaller than the row");
  FG_CUDA_OK(cudaMemcpy2DAsync(dst, (size_t)dst_pitch_bytes, src, (size_t)src_pitch_bytes, (size_t)width_bytes,
                               (size_t)rows, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return FG_OK;
}
