// The scalar step of renorm: from the per-slice sums of |x|^p to the factor each slice is
// multiplied by.  cutorch does all of renorm in one 32-thread block per slice after copying the
// tensor to a transposed contiguous clone (lib/THC/generic/THCTensorMathReduce.cu:47-74, kernel
// lib/THC/THCTensorMathReduce.cuh:132-183); here the sums come from the dimension reductions and
// the scaling is a broadcast multiply, so this file only holds
//     norm = sum^(1/p);  factor = norm > maxnorm ? maxnorm / (norm + 1e-7) : 1
// with TH's roundings: norm is rounded to the element type, the quotient is formed in double and
// rounded once.
#include "context.h"
#include "core.cuh"
#include "plan.h"

namespace thcb {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) renorm_factor_kernel(T *factors, const T *sums, uint64_t n, double p, T maxnorm) {
  const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const T norm = (T)pow((double)sums[i], 1.0 / p);
  factors[i] = norm > maxnorm ? (T)((double)maxnorm / ((double)norm + 1e-7)) : (T)1;
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" int thcb200_renorm_factor(thcb200_ctx *ctx, const thcb200_tensor *factors, const thcb200_tensor *sums, double p,
                                     double maxnorm, void *stream) {
  if (!ctx) { set_error("renorm_factor: null context"); return THCB200_ERR_ARG; }
  HostView vf, vs;
  int rc = to_host_view(factors, &vf, "renorm_factor output");
  if (!rc) rc = to_host_view(sums, &vs, "renorm_factor input");
  if (rc) return rc;
  if (vf.dtype != vs.dtype || (vf.dtype != THCB200_F32 && vf.dtype != THCB200_F64)) {
    set_error("renorm_factor: operands must both be F32 or both F64");
    return THCB200_ERR_ARG;
  }
  if (vf.numel != vs.numel) { set_error("renorm_factor: operands have different element counts"); return THCB200_ERR_SIZE; }
  if (!(p > 0)) { set_error("renorm_factor: non-positive norm"); return THCB200_ERR_ARG; }
  // both operands must be dense (one element after the other in logical order)
  for (const HostView *v : {&vf, &vs}) {
    int64_t run = 1;
    for (int d = v->ndim - 1; d >= 0; --d) {
      if (v->sizes[d] != 1 && v->strides[d] != run) { set_error("renorm_factor: operands must be contiguous"); return THCB200_ERR_ARG; }
      run *= v->sizes[d];
    }
  }
  if (vf.numel == 0) return THCB200_OK;
  const uint64_t n = (uint64_t)vf.numel;
  const uint64_t blocks = (n + 255) / 256;
  if (blocks >= (1ull << 31)) { set_error("renorm_factor: too many slices"); return THCB200_ERR_DIMS; }
  cudaStream_t st = (cudaStream_t)stream;
  if (vf.dtype == THCB200_F32)
    renorm_factor_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((float *)vf.data, (const float *)vs.data, n, p, (float)maxnorm);
  else
    renorm_factor_kernel<double><<<(unsigned)blocks, 256, 0, st>>>((double *)vf.data, (const double *)vs.data, n, p, maxnorm);
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return THCB200_OK;
}
