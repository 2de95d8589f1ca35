// Placeholder while the tcgen05 attention kernel is brought up.
#include "attn_params.cuh"
#include "launchers.h"

namespace dsv4 {
bool sm100_attn_supported(int, int) { return false; }
cudaError_t launch_sm100_attn(const AttnParams&, int, int, cudaStream_t) {
  return cudaErrorNotSupported;
}
}  // namespace dsv4
