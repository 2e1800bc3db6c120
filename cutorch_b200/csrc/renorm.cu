// renorm.  cutorch does all of it in one 32-thread block per slice after copying the tensor to a
// transposed contiguous clone (lib/THC/generic/THCTensorMathReduce.cu:47-74, kernel
// lib/THC/THCTensorMathReduce.cuh:132-183).  Two forms here:
//  * thcb200_renorm_rows: when every slice is one dense run of at most 8192 (4-byte) or 4096
//    (8-byte) elements, a warp or a CTA reads the slice once into registers, folds |x|^p,
//    derives the factor and writes the scaled slice: one read and one write of the tensor.
//  * thcb200_renorm_factor: the scalar step alone, for the composed form (sums from the
//    dimension reductions, scaling as a broadcast multiply) that covers every other layout.
// Both use  norm = sum^(1/p);  factor = norm > maxnorm ? maxnorm / (norm + 1e-7) : 1  with TH's
// roundings: the sum (taken in double) and the norm are rounded to the element type, the quotient
// is formed in double and rounded once.
#include "context.h"
#include "core.cuh"
#include "plan.h"

namespace thcb {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) renorm_factor_kernel(T *factors, const T *sums, uint64_t n, double p, T maxnorm) {
  pdl_prologue();
  const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const T norm = (T)pow((double)sums[i], 1.0 / p);
  factors[i] = norm > maxnorm ? (T)((double)maxnorm / ((double)norm + 1e-7)) : (T)1;
}

// R neighbouring slices per group of G threads (a warp, or the whole 256-thread CTA); each thread
// keeps NV 16-byte vectors of every one of them.  The norm of p = 1 is the sum itself and that of
// p = 2 a square root: a double-precision pow per slice in every lane is what held the first form
// of this kernel to 213 us on 2^19 slices of 256 floats.
// PMODE: 1 = sum |x|, 2 = sum x^2, 0 = sum |x|^p.
template <typename T, int NV, int G, int PMODE, int R>
__global__ void __launch_bounds__(256) renorm_rows_kernel(T *out, const T *in, uint64_t nrows, uint32_t nvec,
                                                          int64_t in_pitch, int64_t out_pitch, double p,
                                                          typename TypeTraits<T>::Math maxnorm) {
  pdl_prologue();
  using M = typename TypeTraits<T>::Math;  // half slices are computed as float slices and rounded once
  constexpr int V = 16 / (int)sizeof(T);
  constexpr int GPC = 256 / G;  // groups per CTA
  const uint32_t t = threadIdx.x % G;
  const uint64_t row0 = ((uint64_t)blockIdx.x * GPC + threadIdx.x / G) * R;
  union Vec { Bytes16 b; T e[V]; };
  Vec v[R][NV];
  double sum[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    sum[r] = 0;
    if (row0 + r < nrows) {
      const char *src = reinterpret_cast<const char *>(in + (row0 + r) * in_pitch);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const uint32_t j = t + (uint32_t)k * G;
        if (j < nvec) v[r][k].b = ld16_stream(src + (size_t)j * 16);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (row0 + r < nrows) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const uint32_t j = t + (uint32_t)k * G;
        if (j < nvec) {
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const double x = (double)to_math<T>(v[r][k].e[e]);
            if constexpr (PMODE == 1) sum[r] += fabs(x);
            else if constexpr (PMODE == 2) sum[r] += x * x;
            else sum[r] += pow(fabs(x), p);
          }
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
    for (int r = 0; r < R; ++r) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], o);
  }
  if constexpr (G == 256) {
    __shared__ double part[R][8];
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) part[r][threadIdx.x >> 5] = sum[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r)
      sum[r] = ((part[r][0] + part[r][1]) + (part[r][2] + part[r][3])) + ((part[r][4] + part[r][5]) + (part[r][6] + part[r][7]));
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (row0 + r >= nrows) continue;
    const M total = (M)sum[r];
    M norm;
    if constexpr (PMODE == 1) norm = total;
    else if constexpr (PMODE == 2) norm = (M)sqrt((double)total);
    else norm = (M)pow((double)total, 1.0 / p);
    const bool scale = norm > maxnorm;
    const M factor = scale ? (M)((double)maxnorm / ((double)norm + 1e-7)) : (M)1;
    char *dst = reinterpret_cast<char *>(out + (row0 + r) * out_pitch);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t j = t + (uint32_t)k * G;
      if (j < nvec) {
        if (scale) {
#pragma unroll
          for (int e = 0; e < V; ++e) v[r][k].e[e] = from_math<T>(to_math<T>(v[r][k].e[e]) * factor);
        }
        st16(dst + (size_t)j * 16, v[r][k].b);
      }
    }
  }
}

template <typename T, int NV, int G, int R>
void launch_renorm_rows_r(T *out, const T *in, uint64_t nrows, uint32_t nvec, int64_t ip, int64_t op, double p, double maxnorm,
                          cudaStream_t st) {
  using M = typename TypeTraits<T>::Math;
  constexpr uint64_t rows_per_cta = (uint64_t)(256 / G) * R;
  const unsigned blocks = (unsigned)((nrows + rows_per_cta - 1) / rows_per_cta);
  if (p == 1.0) launch_pdl(renorm_rows_kernel<T, NV, G, 1, R>, blocks, 256, 0, st, out, in, nrows, nvec, ip, op, p, (M)maxnorm);
  else if (p == 2.0) launch_pdl(renorm_rows_kernel<T, NV, G, 2, R>, blocks, 256, 0, st, out, in, nrows, nvec, ip, op, p, (M)maxnorm);
  else launch_pdl(renorm_rows_kernel<T, NV, G, 0, R>, blocks, 256, 0, st, out, in, nrows, nvec, ip, op, p, (M)maxnorm);
}

template <typename T, int NV, int G>
void launch_renorm_rows(T *out, const T *in, uint64_t nrows, uint32_t nvec, int64_t ip, int64_t op, double p, double maxnorm,
                        cudaStream_t st) {
  // two slices per group where that leaves at most eight vectors per thread: measured on 2^19
  // slices of 256 floats, one slice 165 us, two 158 us, four 159 us
  constexpr int R = NV <= 4 ? 2 : 1;
  launch_renorm_rows_r<T, NV, G, R>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
}

template <typename T>
void dispatch_renorm_rows(T *out, const T *in, uint64_t nrows, uint32_t nvec, int64_t ip, int64_t op, double p, double maxnorm,
                          cudaStream_t st) {
  if (nvec <= 32) launch_renorm_rows<T, 1, 32>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
  else if (nvec <= 64) launch_renorm_rows<T, 2, 32>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
  else if (nvec <= 128) launch_renorm_rows<T, 4, 32>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
  else if (nvec <= 256) launch_renorm_rows<T, 8, 32>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
  else if (nvec <= 512) launch_renorm_rows<T, 2, 256>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
  else if (nvec <= 1024) launch_renorm_rows<T, 4, 256>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
  else launch_renorm_rows<T, 8, 256>(out, in, nrows, nvec, ip, op, p, maxnorm, st);
}

constexpr uint32_t kRenormMaxVec = 2048;  // 16-byte vectors of one slice a CTA keeps in registers

// The view with `dim` moved to the front and the other dims collapsed: rows x len with unit inner
// stride, or false.
bool slices_as_rows(const HostView &v, int dim, int64_t *rows, int64_t *len, int64_t *pitch) {
  int64_t sizes[kMaxDims], strides[kMaxDims];
  int nd = 0;
  for (int d = 0; d < v.ndim; ++d) {
    if (d == dim) continue;
    sizes[nd] = v.sizes[d];
    strides[nd] = v.strides[d];
    ++nd;
  }
  if (nd == 0) return false;
  collapse_dims(sizes, strides, &nd, -1);
  if (nd != 1 || (sizes[0] != 1 && strides[0] != 1)) return false;
  *rows = v.sizes[dim];
  *len = sizes[0];
  *pitch = v.strides[dim];
  return true;
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
    launch_pdl(renorm_factor_kernel<float>, (unsigned)blocks, 256, 0, st, (float *)vf.data, (const float *)vs.data, n, p, (float)maxnorm);
  else
    launch_pdl(renorm_factor_kernel<double>, (unsigned)blocks, 256, 0, st, (double *)vf.data, (const double *)vs.data, n, p, maxnorm);
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return THCB200_OK;
}

extern "C" int thcb200_renorm_rows(thcb200_ctx *ctx, const thcb200_tensor *out, const thcb200_tensor *in, int dim, double p,
                                   double maxnorm, void *stream) {
  if (!ctx) { set_error("renorm_rows: null context"); return THCB200_ERR_ARG; }
  HostView vo, vi;
  int rc = to_host_view(out, &vo, "renorm_rows output");
  if (!rc) rc = to_host_view(in, &vi, "renorm_rows input");
  if (rc) return rc;
  if (vo.dtype != vi.dtype || (vo.dtype != THCB200_F32 && vo.dtype != THCB200_F64 && vo.dtype != THCB200_F16)) {
    set_error("renorm_rows: operands must be of one floating-point type");
    return THCB200_ERR_ARG;
  }
  if (vo.ndim != vi.ndim) { set_error("renorm_rows: operands have different shapes"); return THCB200_ERR_SIZE; }
  for (int d = 0; d < vi.ndim; ++d)
    if (vo.sizes[d] != vi.sizes[d]) { set_error("renorm_rows: operands have different shapes"); return THCB200_ERR_SIZE; }
  if (dim < 0 || dim >= vi.ndim) { set_error("renorm_rows: dim %d out of range", dim); return THCB200_ERR_ARG; }
  if (!(p > 0)) { set_error("renorm_rows: non-positive norm"); return THCB200_ERR_ARG; }
  if (vi.numel == 0) return THCB200_OK;
  const int64_t esz = vo.dtype == THCB200_F32 ? 4 : (vo.dtype == THCB200_F64 ? 8 : 2);
  const int64_t V = 16 / esz;
  int64_t rows_i, len_i, pitch_i, rows_o, len_o, pitch_o;
  const bool fits = slices_as_rows(vi, dim, &rows_i, &len_i, &pitch_i) && slices_as_rows(vo, dim, &rows_o, &len_o, &pitch_o) &&
                    len_i % V == 0 && len_i / V <= (int64_t)kRenormMaxVec && pitch_i >= 0 && pitch_o >= 0 &&
                    (rows_i == 1 || (pitch_i % V == 0 && pitch_o % V == 0 && pitch_o >= len_o)) &&
                    (uintptr_t)vi.data % 16 == 0 && (uintptr_t)vo.data % 16 == 0 && (rows_i + 7) / 8 < (1ll << 31);
  if (!fits) {
    set_error("renorm_rows: the slices are not dense 16-byte aligned runs of at most %u vectors", kRenormMaxVec);
    return THCB200_ERR_UNSUPPORTED;
  }
  cudaStream_t st = (cudaStream_t)stream;
  set_plan_name("renorm_rows");
  if (vo.dtype == THCB200_F32)
    dispatch_renorm_rows<float>((float *)vo.data, (const float *)vi.data, (uint64_t)rows_i, (uint32_t)(len_i / V), pitch_i, pitch_o, p,
                                maxnorm, st);
  else if (vo.dtype == THCB200_F16)
    dispatch_renorm_rows<__half>((__half *)vo.data, (const __half *)vi.data, (uint64_t)rows_i, (uint32_t)(len_i / V), pitch_i, pitch_o,
                                 p, maxnorm, st);
  else
    dispatch_renorm_rows<double>((double *)vo.data, (const double *)vi.data, (uint64_t)rows_i, (uint32_t)(len_i / V), pitch_i, pitch_o,
                                 p, maxnorm, st);
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return THCB200_OK;
}
