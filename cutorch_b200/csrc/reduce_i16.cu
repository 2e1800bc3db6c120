// Reduction kernels instantiated for int16_t.
#include "reduce_launch.cuh"

namespace thcb {
int reduce_all_i16(thcb200_ctx *ctx, int mode, const HostView &in, thcb200_scalar s, void *result, cudaStream_t st) {
  return reduce_all_typed<int16_t>(ctx, mode, in, s, result, st);
}
int reduce_dim_i16(thcb200_ctx *ctx, int mode, const HostView &in, const HostView &out, int dim, thcb200_scalar s,
                  PostOp post, cudaStream_t st) {
  return reduce_dim_typed<int16_t>(ctx, mode, in, out, dim, s, post, st);
}
int reduce_dim_index_i16(thcb200_ctx *ctx, bool is_max, const HostView &in, const HostView &values,
                        const HostView &indices, int dim, cudaStream_t st) {
  return reduce_dim_index_typed<int16_t>(ctx, is_max, in, values, indices, dim, st);
}
}  // namespace thcb
