// Test helper: user-defined functors run through the C++ template faces of the apply and the
// reductions (include/THC/THCApply.cuh, include/THC/THCReduce.cuh), the way a downstream CUDA library such as cunn uses cutorch.
// Built into cutorch_b200/lib/libthcb200_usertest.so and driven from tests/test_template_api_gpu.py.
#include <thread>
#include <vector>

#include "THC/THCApply.cuh"
#include "THC/THCReduce.cuh"

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

// Reduction functors: modifyOp maps an element, reduceOp folds it into an accumulator, the third
// functor merges two accumulators (the contract of THC_reduceDim / THC_reduceAll).
struct Square { __device__ __forceinline__ float operator()(float x) const { return x * x; } };
struct AbsF { __device__ __forceinline__ float operator()(float x) const { return x < 0 ? -x : x; } };
struct AddF { __device__ __forceinline__ float operator()(float a, float b) const { return a + b; } };
struct MaxF { __device__ __forceinline__ float operator()(float a, float b) const { return a > b ? a : b; } };
struct IsPositive { __device__ __forceinline__ double operator()(double x) const { return x > 0 ? 1.0 : 0.0; } };
struct CountL { __device__ __forceinline__ long operator()(long acc, double flag) const { return acc + (flag != 0.0 ? 1 : 0); } };
struct AddL { __device__ __forceinline__ long operator()(long a, long b) const { return a + b; } };
struct MinMax { int lo, hi; };
struct IdentityI { __device__ __forceinline__ int operator()(int x) const { return x; } };
struct MinMaxStep {
  __device__ __forceinline__ MinMax operator()(MinMax a, int x) const {
    if (x < a.lo) a.lo = x;
    if (x > a.hi) a.hi = x;
    return a;
  }
};
struct MinMaxMerge {
  __device__ __forceinline__ MinMax operator()(MinMax a, MinMax b) const {
    if (b.lo < a.lo) a.lo = b.lo;
    if (b.hi > a.hi) a.hi = b.hi;
    return a;
  }
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

// ---- user functors through THC_reduceDim / THC_reduceAll (include/THC/THCReduce.cuh) ----

// sum of squares along a dim, float accumulator
__attribute__((visibility("default"))) int usertest_sumsq_dim(THCState *state, THCudaTensor *out, THCudaTensor *in, int dim, int keepdim) {
  return THC_reduceDim(state, out, in, Square(), AddF(), AddF(), 0.0f, dim, keepdim) ? 1 : 0;
}

// largest |x| of a tensor, result on the host
__attribute__((visibility("default"))) int usertest_absmax_all(THCState *state, THCudaTensor *in, float *out_host) {
  return THC_reduceAll(state, in, AbsF(), MaxF(), MaxF(), 0.0f, out_host, 0) ? 1 : 0;
}

// number of positive elements of a double tensor as a long, result left on the device
__attribute__((visibility("default"))) int usertest_count_positive_device(THCState *state, THCudaDoubleTensor *in, long *out_dev) {
  return THC_reduceAll(state, in, IsPositive(), CountL(), AddL(), 0L, out_dev, 1) ? 1 : 0;
}

// smallest and largest element in one pass: a struct accumulator
__attribute__((visibility("default"))) int usertest_minmax_all(THCState *state, THCudaIntTensor *in, int *lo, int *hi) {
  MinMax init;
  init.lo = 2147483647;
  init.hi = -2147483647 - 1;
  MinMax r = init;
  const bool ok = THC_reduceAll(state, in, IdentityI(), MinMaxStep(), MinMaxMerge(), init, &r, 0);
  *lo = r.lo;
  *hi = r.hi;
  return ok ? 1 : 0;
}

// Several host threads share one THCState (cutorch: test/test_shutdown.lua:55, one state for all
// Lua threads).  Thread 0 stays on the default stream; every other thread makes a stream of its own
// current (thread-local, lib/THC/THCGeneral.c:516-561) and checks that it alone sees it.  Each then
// runs, `iters` times on its own tensors, the calls that keep partial results in per-stream scratch:
// a full sum, a sum over the outer dim split over many CTAs, a chunked cumulative sum, and a full
// reduction through the template header (result in a per-thread pinned slot).  All values are
// small integers, so every expected result is exact.  Returns the number of wrong results.
__attribute__((visibility("default"))) int usertest_threads(THCState *state, int nthreads, int iters) {
  std::vector<int> bad((size_t)nthreads, 0);
  std::vector<std::thread> pool;
  const cudaStream_t mine_before = THCState_getCurrentStream(state);
  int device = 0;
  cudaGetDevice(&device);
  for (int t = 0; t < nthreads; ++t) {
    pool.emplace_back([state, t, iters, device, &bad]() {
      int wrong = 0;
      cudaSetDevice(device);
      THCStream *stream = nullptr;
      if (THCState_getCurrentStream(state) != 0) ++wrong;          // a new thread starts on the default stream
      if (t > 0) {
        stream = THCStream_new(cudaStreamNonBlocking);
        THCState_setStream(state, stream);
        if (THCState_getCurrentStream(state) != stream->stream) ++wrong;
      }
      const long rows = 4096, cols = 256, n1 = 1 << 22;
      const float v = (float)(t + 1);
      THCudaTensor *m = THCudaTensor_newWithSize2d(state, rows, cols);
      THCudaTensor *colsum = THCudaTensor_newWithSize2d(state, 1, cols);
      THCudaTensor *line = THCudaTensor_newWithSize1d(state, n1);
      THCudaTensor *scan = THCudaTensor_newWithSize1d(state, n1);
      THCudaTensor_fill(state, m, v);
      THCudaTensor_fill(state, line, 1.0f);
      for (int i = 0; i < iters; ++i) {
        if (THCudaTensor_sumall(state, m) != v * (float)(rows * cols)) ++wrong;
        THCudaTensor_sum(state, colsum, m, 0, 1);
        if (THCudaTensor_sumall(state, colsum) != v * (float)(rows * cols)) ++wrong;
        if (THCudaTensor_maxall(state, colsum) != v * (float)rows) ++wrong;
        // the template full reduction writes its host result into a pinned slot of the calling thread
        float biggest = -1.0f;
        if (!THC_reduceAll(state, m, AbsF(), MaxF(), MaxF(), 0.0f, &biggest, 0) || biggest != v) ++wrong;
        THCudaTensor_cumsum(state, scan, line, 0);
        if (THCudaTensor_maxall(state, scan) != (float)n1) ++wrong;
        if (THCudaTensor_sumall(state, scan) != (float)((double)n1 * (double)(n1 + 1) / 2.0)) ++wrong;
      }
      if (THCB200_errorOccurred()) ++wrong;
      THCudaTensor_free(state, m);
      THCudaTensor_free(state, colsum);
      THCudaTensor_free(state, line);
      THCudaTensor_free(state, scan);
      cudaStreamSynchronize(THCState_getCurrentStream(state));
      if (stream) {
        THCState_setStream(state, nullptr);
        THCStream_free(stream);
      }
      bad[(size_t)t] = wrong;
    });
  }
  for (auto &th : pool) th.join();
  int total = 0;
  for (int b : bad) total += b;
  if (THCState_getCurrentStream(state) != mine_before) ++total;   // the caller's own current stream is untouched
  return total;
}

}  // extern "C"
