// fg_flash_attn_decode_static: split-KV decode attention that allocates nothing.
//
// The split-KV decode kernel needs scratch for the partial outputs of each KV chunk.
// fg_flash_attn_varlen takes that scratch from the caller.  Some users of this C ABI
// have no allocator to take it from: a serving runtime that reserved all free device
// memory for its KV-cache pool at start-up (a later cudaMalloc may simply fail), a
// C/C++ host that binds this library without torch and its caching allocator, or a
// decode loop that cannot afford the device-wide synchronisation cudaMalloc/cudaFree
// imply.  For them the scratch lives in the library image itself, in the fixed-size
// device array below; every GPU that loads the library holds these bytes until the
// process exits.
#include <mutex>

#include "attn_common.cuh"

namespace fg {
void decode_split_plan(int64_t batch, int64_t num_heads_k, int64_t max_seqlen_k, int forced_splits, int sms,
                       int* chunk_tokens, int* num_splits);
}

#define FG_DECODE_STATIC_SCRATCH_BYTES (64ll << 20)

// Partial (O, log-sum-exp) pairs of the KV chunks, shared by every call on a device.
static __device__ __align__(256) unsigned char g_decode_scratch[FG_DECODE_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// In host code `g_decode_scratch` is only a handle of the symbol; the address the
// kernels must be given is looked up once per device, with that device current.
int scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fg::fail(FG_ERR_CUDA, "flash_attn_decode_static: cannot identify the current device");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fg::fail(FG_ERR_CUDA, "flash_attn_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return FG_OK;
}

}  // namespace

extern "C" int64_t fg_flash_attn_decode_static_capacity(void) { return FG_DECODE_STATIC_SCRATCH_BYTES; }

extern "C" int fg_flash_attn_decode_static(const fg_attn_params* p, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("flash_attn_decode_static");
  FG_REQUIRE(p != nullptr, "flash_attn_decode_static: null params");
  FG_REQUIRE(p->max_seqlen_q == 1 && p->total_q == p->batch,
             "flash_attn_decode_static: exactly one query token per sequence is required");
  FG_REQUIRE(p->num_heads > 0 && p->num_heads_k > 0 && p->head_dim > 0, "flash_attn_decode_static: bad head sizes");
  FG_REQUIRE(fg_flash_attn_path(p) == 2,
             "flash_attn_decode_static: these arguments do not select the split-KV decode kernel "
             "(ALiBi, windows or more than 16 query heads per KV head)");
  // Same chunk plan as fg_flash_attn_varlen makes; the bytes it needs must fit the array.
  int chunk = 0, splits = 1;
  decode_split_plan(p->batch, p->num_heads_k, p->max_seqlen_k, p->num_splits, num_sms(), &chunk, &splits);
  const int64_t need = splits > 1 ? (int64_t)splits * p->total_q * p->num_heads * (p->head_dim + 1) * 4 : 0;
  if (need > FG_DECODE_STATIC_SCRATCH_BYTES)
    return fail(FG_ERR_TOO_LARGE,
                "flash_attn_decode_static: %d KV chunks x %lld tokens x %lld heads need %lld bytes of scratch, the "
                "built-in array holds %lld; use fg_flash_attn_varlen with a caller workspace",
                splits, (long long)p->total_q, (long long)p->num_heads, (long long)need,
                (long long)FG_DECODE_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  const int rc = scratch_address(&scratch);
  if (rc != FG_OK) return rc;
  // This entry point makes no allocating or page-locking call: if no other entry point has
  // set up the host-visible copy of the device status word on this device yet, this call runs
  // without it (a wait that gave up is then reported by fg_device_status only).
  MirrorSetupGuard no_setup;
  fg_attn_params q = *p;
  q.workspace = scratch;
  q.workspace_bytes = FG_DECODE_STATIC_SCRATCH_BYTES;
  return fg_flash_attn_varlen(&q, stream);
}
