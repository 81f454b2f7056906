// reshape_and_cache_flash: scatter new K/V rows into a paged cache (pure copy,
// bit-exact).  Work is flattened over (token, K|V, 16-byte packet) so that small
// decode batches still spread over many CTAs and large prefill batches stream at
// HBM rate; the scalar kernel handles unaligned layouts element by element.
#include "common.cuh"

namespace fg {

struct CacheArgs {
  const char *key, *value;
  char *kc, *vc;
  const int64_t* slots;
  int64_t T;
  int64_t H, D, BS, NB;
  int64_t ks, vs;          // token strides of key / value (elements)
  int64_t cbs, crs, chs;   // cache block / row / head strides (elements)
};

// One packet = 16 bytes inside one head row (D*ES is a multiple of 16).  Index math is
// 32-bit (the host checks that token*packets and the slot range fit).
template <int ES>
__global__ void __launch_bounds__(256) cache_scatter_vec_kernel(CacheArgs a, uint32_t packs_per_head,
                                                                uint32_t packs_per_tok, uint32_t total,
                                                                uint32_t num_slots) {
  for (uint32_t idx = blockIdx.x * 256u + threadIdx.x; idx < total; idx += gridDim.x * 256u) {
    const uint32_t tk = idx / packs_per_tok;  // token * 2 + which
    const uint32_t r = idx - tk * packs_per_tok;
    const uint32_t tok = tk >> 1;
    const bool which = tk & 1;
    const uint32_t h = r / packs_per_head;
    const uint32_t c = r - h * packs_per_head;
    const char* src = (which ? a.value + (int64_t)tok * a.vs * ES : a.key + (int64_t)tok * a.ks * ES) +
                      ((int64_t)h * a.D) * ES + c * 16;
    // the payload does not depend on the slot: fetch both in the same round trip
    const uint4 payload = ldg16_stream(src);
    const int64_t slot64 = a.slots[tok];
    if (slot64 < 0 || slot64 >= (int64_t)num_slots) continue;  // padding, or outside the cache
    const uint32_t slot = (uint32_t)slot64;
    const uint32_t blk = slot / (uint32_t)a.BS, off = slot - blk * (uint32_t)a.BS;
    char* dst = (which ? a.vc : a.kc) + ((int64_t)blk * a.cbs + (int64_t)off * a.crs + (int64_t)h * a.chs) * ES + c * 16;
    stg16(dst, payload);
  }
}

template <typename U>
__global__ void __launch_bounds__(256) cache_scatter_scalar_kernel(CacheArgs a) {
  const int64_t n = a.H * a.D;
  const int64_t total = a.T * n * 2;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t tk = idx / n;
    const int64_t i = idx - tk * n;
    const int64_t tok = tk >> 1;
    const int which = (int)(tk & 1);
    const int64_t slot = a.slots[tok];
    if (slot < 0 || slot >= a.NB * a.BS) continue;  // padding, or outside the cache
    const int64_t h = i / a.D, d = i - h * a.D;
    const int64_t blk = slot / a.BS, off = slot - blk * a.BS;
    const U* src = reinterpret_cast<const U*>(which ? a.value : a.key) + tok * (which ? a.vs : a.ks) + i;
    U* dst = reinterpret_cast<U*>(which ? a.vc : a.kc) + blk * a.cbs + off * a.crs + h * a.chs + d;
    *dst = *src;
  }
}

// ---- vLLM v0 cache layout: K [blocks, heads, D/x, block_size, x], V [blocks, heads, D, block_size]
// (contiguous).  One thread per element of a token row and K|V; the x-element groups of K
// land as contiguous runs, V elements are block_size apart by the layout's definition.
template <typename U>
__global__ void __launch_bounds__(256) cache_scatter_v0_kernel(const U* key, const U* value, U* kc, U* vc,
                                                               const int64_t* slots, int64_t T, int64_t H, int64_t D,
                                                               int64_t BS, int64_t NB, int64_t X, int64_t ks,
                                                               int64_t vs) {
  const int64_t n = H * D;
  const int64_t total = T * n * 2;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t tk = idx / n;
    const int64_t i = idx - tk * n;
    const int64_t tok = tk >> 1;
    const bool which = tk & 1;
    const int64_t slot = slots[tok];
    if (slot < 0 || slot >= NB * BS) continue;  // padding, or outside the cache
    const int64_t h = i / D, d = i - h * D;
    const int64_t blk = slot / BS, off = slot - blk * BS;
    if (!which) {
      const int64_t xi = d / X, xo = d - xi * X;
      kc[(((blk * H + h) * (D / X) + xi) * BS + off) * X + xo] = key[tok * ks + i];
    } else {
      vc[((blk * H + h) * D + d) * BS + off] = value[tok * vs + i];
    }
  }
}

}  // namespace fg

extern "C" int fg_reshape_and_cache_flash(const void* key, const void* value, void* key_cache,
                                          void* value_cache, const int64_t* slot_mapping,
                                          int64_t num_tokens, int64_t num_heads, int64_t head_size,
                                          int64_t block_size, int64_t num_blocks,
                                          int64_t key_stride, int64_t value_stride, int64_t cache_block_stride,
                                          int64_t cache_row_stride, int64_t cache_head_stride,
                                          int elem_size, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("reshape_and_cache_flash");
  FG_REQUIRE(num_tokens >= 0 && num_heads >= 0 && head_size >= 0, "reshape_and_cache_flash: negative size");
  FG_REQUIRE(block_size > 0 && num_blocks >= 0, "reshape_and_cache_flash: block_size must be positive");
  FG_REQUIRE(elem_size == 1 || elem_size == 2 || elem_size == 4,
             "reshape_and_cache_flash: element size %d not in {1,2,4}", elem_size);
  if (num_tokens == 0 || num_heads * head_size == 0) return FG_OK;
  FG_REQUIRE(key && value && key_cache && value_cache && slot_mapping,
             "reshape_and_cache_flash: null pointer");
  CacheArgs a;
  a.key = (const char*)key; a.value = (const char*)value;
  a.kc = (char*)key_cache; a.vc = (char*)value_cache;
  a.slots = slot_mapping; a.T = num_tokens; a.H = num_heads; a.D = head_size; a.BS = block_size; a.NB = num_blocks;
  a.ks = key_stride; a.vs = value_stride;
  a.cbs = cache_block_stride; a.crs = cache_row_stride; a.chs = cache_head_stride;
  cudaStream_t st = (cudaStream_t)stream;
  const int es = elem_size;
  auto b16 = [&](int64_t elems) { return (elems * es) % 16 == 0; };
  const bool vec = b16(head_size) && b16(key_stride) && b16(value_stride) && b16(cache_block_stride) &&
                   b16(cache_row_stride) && b16(cache_head_stride) && aligned16(key) &&
                   aligned16(value) && aligned16(key_cache) && aligned16(value_cache);
  const int64_t cap = (int64_t)num_sms() * 32;
  const int64_t vtotal = num_tokens * num_heads * (head_size * es / 16) * 2;
  if (vec && vtotal < 4000000000LL && num_blocks * block_size < 4000000000LL) {
    const uint32_t pph = (uint32_t)(head_size * es / 16);
    const uint32_t ppt = (uint32_t)num_heads * pph;
    int64_t blocks = (vtotal + 255) / 256;
    if (blocks > cap) blocks = cap;
    const uint32_t nslots = (uint32_t)(num_blocks * block_size);
    switch (es) {
      case 1: cache_scatter_vec_kernel<1><<<(unsigned)blocks, 256, 0, st>>>(a, pph, ppt, (uint32_t)vtotal, nslots); break;
      case 2: cache_scatter_vec_kernel<2><<<(unsigned)blocks, 256, 0, st>>>(a, pph, ppt, (uint32_t)vtotal, nslots); break;
      default: cache_scatter_vec_kernel<4><<<(unsigned)blocks, 256, 0, st>>>(a, pph, ppt, (uint32_t)vtotal, nslots); break;
    }
    FG_CHECK_LAUNCH("cache_scatter_vec_kernel");
  } else {
    const int64_t total = num_tokens * num_heads * head_size * 2;
    int64_t blocks = (total + 255) / 256;
    if (blocks > cap) blocks = cap;
    switch (es) {
      case 1: cache_scatter_scalar_kernel<uint8_t><<<(unsigned)blocks, 256, 0, st>>>(a); break;
      case 2: cache_scatter_scalar_kernel<uint16_t><<<(unsigned)blocks, 256, 0, st>>>(a); break;
      default: cache_scatter_scalar_kernel<uint32_t><<<(unsigned)blocks, 256, 0, st>>>(a); break;
    }
    FG_CHECK_LAUNCH("cache_scatter_scalar_kernel");
  }
  return FG_OK;
}

extern "C" int fg_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                                    const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                                    int64_t head_size, int64_t block_size, int64_t num_blocks, int64_t x,
                                    int64_t key_stride, int64_t value_stride, int elem_size, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("reshape_and_cache");
  FG_REQUIRE(num_tokens >= 0 && num_heads >= 0 && head_size >= 0, "reshape_and_cache: negative size");
  FG_REQUIRE(block_size > 0 && num_blocks >= 0, "reshape_and_cache: block_size must be positive");
  FG_REQUIRE(x > 0 && head_size % x == 0, "reshape_and_cache: head_size %lld is not a multiple of x = %lld",
             (long long)head_size, (long long)x);
  FG_REQUIRE(elem_size == 1 || elem_size == 2 || elem_size == 4, "reshape_and_cache: element size %d not in {1,2,4}",
             elem_size);
  if (num_tokens == 0 || num_heads * head_size == 0) return FG_OK;
  FG_REQUIRE(key && value && key_cache && value_cache && slot_mapping, "reshape_and_cache: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = num_tokens * num_heads * head_size * 2;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)num_sms() * 32;
  if (blocks > cap) blocks = cap;
#define FG_V0(U)                                                                                              \
  cache_scatter_v0_kernel<U><<<(unsigned)blocks, 256, 0, st>>>((const U*)key, (const U*)value, (U*)key_cache,   \
                                                               (U*)value_cache, slot_mapping, num_tokens,     \
                                                               num_heads, head_size, block_size, num_blocks, x, \
                                                               key_stride, value_stride)
  switch (elem_size) {
    case 1: FG_V0(uint8_t); break;
    case 2: FG_V0(uint16_t); break;
    default: FG_V0(uint32_t); break;
  }
#undef FG_V0
  FG_CHECK_LAUNCH("cache_scatter_v0_kernel");
  return FG_OK;
}
