// Placeholder translation unit for the tcgen05 prefill kernel (filled in below).
#include "attn_common.cuh"

namespace fg {

bool attn_prefill_sm100_eligible(const fg_attn_params*) { return false; }

int attn_prefill_sm100(const AttnArgs&, int, cudaStream_t) {
  return fail(FG_ERR_UNSUPPORTED, "flash_attn_varlen: tcgen05 prefill path not available");
}

}  // namespace fg
