// Test helper: user-defined functors run through the C++ template face of the apply
// (include/THC/THCApply.cuh), the way a downstream CUDA library such as cunn uses cutorch.
// Built into cutorch_b200/lib/libthcb200_usertest.so and driven from tests/test_template_api_gpu.py.
#include "THC/THCApply.cuh"

// out = in * k + 1
struct ScaleAddOne {
  float k;
  __device__ __forceinline__ void operator()(float *out, float *in) const { *out = *in * k + 1.0f; }
};

// In place: v += 1
struct AddOne {
  __device__ __forceinline__ void operator()(float *v) const { *v += 1.0f; }
};

// Reaches neighbours through the element pointers (like cutorch's TensorCrossOp): the operands are
// views narrowed to one slot of the 3-vector dim, s* are the strides of that dim.
struct Cross3 {
  long sx, sy, so;
  __device__ __forceinline__ void operator()(float *out, float *x, float *y) const {
    out[0 * so] = x[1 * sx] * y[2 * sy] - x[2 * sx] * y[1 * sy];
    out[1 * so] = x[2 * sx] * y[0 * sy] - x[0 * sx] * y[2 * sy];
    out[2 * so] = x[0 * sx] * y[1 * sy] - x[1 * sx] * y[0 * sy];
  }
};

// Mixed element types: byte mask = a < b
struct LessThan {
  __device__ __forceinline__ void operator()(unsigned char *out, double *a, double *b) const { *out = *a < *b ? 1 : 0; }
};

extern "C" {

__attribute__((visibility("default"))) int usertest_scale(THCState *state, THCudaTensor *out, THCudaTensor *in, float k) {
  ScaleAddOne op;
  op.k = k;
  return THC_pointwiseApply2(state, out, in, op) ? 1 : 0;
}

__attribute__((visibility("default"))) int usertest_add_one(THCState *state, THCudaTensor *t) {
  return THC_pointwiseApply1(state, t, AddOne()) ? 1 : 0;
}

__attribute__((visibility("default"))) int usertest_cross(THCState *state, THCudaTensor *out, THCudaTensor *x, THCudaTensor *y, int dim) {
  Cross3 op;
  op.sx = x->stride[dim];
  op.sy = y->stride[dim];
  op.so = out->stride[dim];
  THCudaTensor *no = THCudaTensor_newNarrow(state, out, dim, 0, 1);
  THCudaTensor *nx = THCudaTensor_newNarrow(state, x, dim, 0, 1);
  THCudaTensor *ny = THCudaTensor_newNarrow(state, y, dim, 0, 1);
  const bool ok = THC_pointwiseApply3(state, no, nx, ny, op);
  THCudaTensor_free(state, no);
  THCudaTensor_free(state, nx);
  THCudaTensor_free(state, ny);
  return ok ? 1 : 0;
}

__attribute__((visibility("default"))) int usertest_less_than(THCState *state, THCudaByteTensor *out, THCudaDoubleTensor *a, THCudaDoubleTensor *b) {
  return THC_pointwiseApply3(state, out, a, b, LessThan()) ? 1 : 0;
}

}  // extern "C"
