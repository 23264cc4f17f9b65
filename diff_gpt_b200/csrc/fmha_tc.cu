// tcgen05 / TMEM prefill attention (bf16, head_dim 64 or 128).
#include "fmha.cuh"

namespace dgpt {

bool fmha_tc_supported(const FmhaArgs&, const dgpt_kv_layout&) { return false; }

int fmha_tc(const FmhaArgs&, const dgpt_kv_layout&, cudaStream_t) {
  set_error("fmha_tc: not built");
  return DGPT_E_UNSUPPORTED;
}

}  // namespace dgpt
