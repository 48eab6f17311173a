// Tensor-core attention over the slot pool (bfloat16 prefill).  Placeholder dispatch: declines every shape, so the plain
// kernel runs.
#include "seq_common.cuh"

namespace pcs {
int launch_attn_tc(const pcs_attn_params&, cudaStream_t, bool* handled) {
  *handled = false;
  return PCS_OK;
}
}  // namespace pcs
