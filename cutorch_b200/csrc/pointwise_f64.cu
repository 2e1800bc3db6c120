// Pointwise apply kernels instantiated for double.
#include "apply_launch.cuh"

namespace thcb {
int pointwise_f64(thcb200_ctx *ctx, int op, const ApplyPlan &plan, char *const data[4], thcb200_scalar s0,
                 thcb200_scalar s1, cudaStream_t st) {
  return pointwise_typed<double>(ctx, op, plan, data, s0, s1, st);
}
}  // namespace thcb
