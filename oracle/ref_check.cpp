// TEST INFRASTRUCTURE -- not part of the product.  Compiles cutorch's own header files, from
// where they lie in the cutorch tree, as host C++ (see refshim/ref_host_shim.h) and exposes
//   * TensorInfo::collapseDims / IndexToOffset      (lib/THC/THCTensorInfo.cuh:74-278)
//   * the pointwise functor bodies                   (lib/THC/THCTensorMathPointwise.cuh:12-772)
//   * THCNumerics<T> math                            (lib/THC/THCNumerics.cuh:12-666)
//   * the comparison functors into Byte and into T   (lib/THC/THCTensorMathCompare.cuh:9-67, THCTensorMathCompareT.cuh:11-51)
//   * the Byte-masked fill / copy / select functors  (lib/THC/THCTensorMasked.cuh:16-56)
// through a C ABI, so that the tests can pin the CPU restatement (th_oracle.cpp) and the
// product's planner against the reference's own code, and so that golden vectors can be
// generated (tests/golden/make_golden.py).  The output goes to oracle/_ref/ and is never
// committed.  No reference source is copied: the headers are only #included.
#include "THCTensorInfo.cuh"
#include "THCNumerics.cuh"
#include "THCTensorMathPointwise.cuh"
#include "THCTensorMathCompare.cuh"
#include "THCTensorMathCompareT.cuh"
#include "THCTensorMasked.cuh"

#include <stdint.h>
#include <string.h>

extern "C" {

// In-place collapseDims on int64 arrays; returns the new index of exclude_dim (or -1).
int ref_collapse_dims(int64_t *sizes, int64_t *strides, int *ndim, int exclude_dim) {
  unsigned long sz[MAX_CUTORCH_DIMS], st[MAX_CUTORCH_DIMS];
  for (int i = 0; i < *ndim; ++i) { sz[i] = (unsigned long)sizes[i]; st[i] = (unsigned long)strides[i]; }
  TensorInfo<float, unsigned long> info((float *)0, *ndim, sz, st);
  int r = info.collapseDims(exclude_dim);
  *ndim = info.dims;
  for (int i = 0; i < info.dims; ++i) { sizes[i] = (int64_t)info.sizes[i]; strides[i] = (int64_t)info.strides[i]; }
  return r;
}

int ref_is_contiguous(const int64_t *sizes, const int64_t *strides, int ndim) {
  unsigned long sz[MAX_CUTORCH_DIMS], st[MAX_CUTORCH_DIMS];
  for (int i = 0; i < ndim; ++i) { sz[i] = (unsigned long)sizes[i]; st[i] = (unsigned long)strides[i]; }
  TensorInfo<float, unsigned long> info((float *)0, ndim, sz, st);
  info.collapseDims();
  return info.isContiguous() ? 1 : 0;
}

// IndexToOffset<T, unsigned long, -1>::get on the view as given (no collapsing).
int64_t ref_index_to_offset(const int64_t *sizes, const int64_t *strides, int ndim, int64_t linear) {
  unsigned long sz[MAX_CUTORCH_DIMS], st[MAX_CUTORCH_DIMS];
  for (int i = 0; i < ndim; ++i) { sz[i] = (unsigned long)sizes[i]; st[i] = (unsigned long)strides[i]; }
  TensorInfo<float, unsigned long> info((float *)0, ndim, sz, st);
  return (int64_t)IndexToOffset<float, unsigned long, -1>::get((unsigned long)linear, info);
}

}  // extern "C"

// Functor ids: a private numbering of this file (the tests map them to library ops by name).
enum {
  F_SIGMOID = 0, F_SIGN, F_ADD, F_CADD, F_SUB, F_MUL, F_POW, F_TPOW, F_CPOW, F_DIV, F_CREMAINDER, F_CFMOD, F_CLAMP,
  F_LERP, F_CMAX, F_CMIN, F_MAXVALUE, F_MINVALUE, F_ADDCMUL, F_ADDCDIV, F_CLSHIFT, F_CRSHIFT, F_BITAND, F_BITOR,
  F_BITXOR,
  // THCNumerics unary math
  F_LOG = 100, F_LGAMMA, F_LOG1P, F_EXP, F_COS, F_SIN, F_SQRT, F_RSQRT, F_CEIL, F_FLOOR, F_TRUNC, F_ACOS, F_COSH,
  F_ASIN, F_SINH, F_TAN, F_ATAN, F_TANH, F_ROUND, F_FRAC, F_CINV, F_NEG, F_ABS
};

namespace {

template <typename T> void pow_dispatch(T *o, T *a, T s0) {
  if (s0 == (T)1) { TensorPowOp<T, 1> f(s0); f(o, a); }
  else if (s0 == (T)2) { TensorPowOp<T, 2> f(s0); f(o, a); }
  else if (s0 == (T)3) { TensorPowOp<T, 3> f(s0); f(o, a); }
  else if (s0 == (T)-1) { TensorPowOp<T, -1> f(s0); f(o, a); }
  else if (s0 == (T)-2) { TensorPowOp<T, -2> f(s0); f(o, a); }
  else { TensorPowOp<T, -3> f(s0); f(o, a); }
}

// Functors defined for every element type.
template <typename T> int run_common(int fid, int64_t n, T *out, T *a, T *b, T *c, T s0, T s1) {
  for (int64_t i = 0; i < n; ++i) {
    T *o = out + i, *x = a ? a + i : 0, *y = b ? b + i : 0, *z = c ? c + i : 0;
    switch (fid) {
      case F_SIGN: { TensorSignOp<T> f; f(o, x); break; }
      case F_ADD: { TensorAddOp<T> f; f(o, x, y); break; }
      case F_CADD: { TensorCAddOp<T> f(s0); f(o, x, y); break; }
      case F_SUB: { TensorSubOp<T> f; f(o, x, y); break; }
      case F_MUL: { TensorMulOp<T> f; f(o, x, y); break; }
      case F_CPOW: { TensorCPowOp<T> f; f(o, x, y); break; }
      case F_DIV: { TensorDivOp<T> f; f(o, x, y); break; }
      case F_CREMAINDER: { TensorCRemainderOp<T> f; f(o, x, y); break; }
      case F_CFMOD: { TensorCFmodOp<T> f; f(o, x, y); break; }
      case F_CLAMP: { TensorClampOp<T> f(s0, s1); f(o, x); break; }
      case F_CMAX: { TensorMaxOp<T> f; f(o, x, y); break; }
      case F_CMIN: { TensorMinOp<T> f; f(o, x, y); break; }
      case F_MAXVALUE: { TensorMaxValueOp<T> f(s0); f(o, x); break; }
      case F_MINVALUE: { TensorMinValueOp<T> f(s0); f(o, x); break; }
      // addcmul/addcdiv update `out` in place: out = out + val * (in1 (*|/) in2); x seeds out
      case F_ADDCMUL: { *o = *x; TensorAddCMulOp<T> f(s0); f(o, y, z); break; }
      case F_ADDCDIV: { *o = *x; TensorAddCDivOp<T> f(s0); f(o, y, z); break; }
      case F_CLSHIFT: { TensorLShiftOp<T> f; f(o, x, y); break; }
      case F_CRSHIFT: { TensorRShiftOp<T> f; f(o, x, y); break; }
      default: return -1;
    }
  }
  return 0;
}

template <typename T> int run_int_only(int fid, int64_t n, T *out, T *a, T *b) {
  for (int64_t i = 0; i < n; ++i) {
    switch (fid) {
      case F_BITAND: { TensorBitAndOp<T> f; f(out + i, a + i, b + i); break; }
      case F_BITOR: { TensorBitOrOp<T> f; f(out + i, a + i, b + i); break; }
      case F_BITXOR: { TensorBitXorOp<T> f; f(out + i, a + i, b + i); break; }
      default: return -1;
    }
  }
  return 0;
}

template <typename T> int run_fp_only(int fid, int64_t n, T *out, T *a, T *b, T s0) {
  typedef THCNumerics<T> N;
  for (int64_t i = 0; i < n; ++i) {
    T *o = out + i, *x = a + i;
    switch (fid) {
      case F_SIGMOID: { TensorSigmoidOp<T> f; f(o, x); break; }
      case F_POW: pow_dispatch<T>(o, x, s0); break;
      case F_TPOW: { TensorTPowOp<T> f(s0); f(o, x); break; }
      case F_LERP: { TensorLerpOp<T> f(s0); f(o, x, b + i); break; }
      case F_LOG: *o = N::log(*x); break;
      case F_LGAMMA: *o = N::lgamma(*x); break;
      case F_LOG1P: *o = N::log1p(*x); break;
      case F_EXP: *o = N::exp(*x); break;
      case F_COS: *o = N::cos(*x); break;
      case F_SIN: *o = N::sin(*x); break;
      case F_SQRT: *o = N::sqrt(*x); break;
      case F_RSQRT: *o = N::rsqrt(*x); break;
      case F_CEIL: *o = N::ceil(*x); break;
      case F_FLOOR: *o = N::floor(*x); break;
      case F_TRUNC: *o = N::trunc(*x); break;
      case F_ACOS: *o = N::acos(*x); break;
      case F_COSH: *o = N::cosh(*x); break;
      case F_ASIN: *o = N::asin(*x); break;
      case F_SINH: *o = N::sinh(*x); break;
      case F_TAN: *o = N::tan(*x); break;
      case F_ATAN: *o = N::atan(*x); break;
      case F_TANH: *o = N::tanh(*x); break;
      case F_ROUND: *o = N::round(*x); break;
      case F_FRAC: *o = N::frac(*x); break;
      case F_CINV: *o = N::cinv(*x); break;
      case F_NEG: *o = N::neg(*x); break;
      case F_ABS: *o = N::abs(*x); break;
      default: return -1;
    }
  }
  return 0;
}

}  // namespace

extern "C" {

// Applies one reference functor element by element to dense arrays of n elements.
// dtype numbering: 0 u8, 1 i8, 2 i16, 3 i32, 4 i64, 6 f32, 7 f64 (no half: the reference's
// half specialisations need CUDA intrinsics).  Scalars arrive as double and int64.
int ref_apply_functor(int fid, int dtype, int64_t n, void *out, void *a, void *b, void *c, double sf0, double sf1,
                      int64_t si0, int64_t si1) {
  int rc = -1;
  switch (dtype) {
    case 0: rc = run_common<unsigned char>(fid, n, (unsigned char *)out, (unsigned char *)a, (unsigned char *)b, (unsigned char *)c, (unsigned char)si0, (unsigned char)si1);
            if (rc) rc = run_int_only<unsigned char>(fid, n, (unsigned char *)out, (unsigned char *)a, (unsigned char *)b); break;
    case 1: rc = run_common<char>(fid, n, (char *)out, (char *)a, (char *)b, (char *)c, (char)si0, (char)si1);
            if (rc) rc = run_int_only<char>(fid, n, (char *)out, (char *)a, (char *)b); break;
    case 2: rc = run_common<short>(fid, n, (short *)out, (short *)a, (short *)b, (short *)c, (short)si0, (short)si1);
            if (rc) rc = run_int_only<short>(fid, n, (short *)out, (short *)a, (short *)b); break;
    case 3: rc = run_common<int>(fid, n, (int *)out, (int *)a, (int *)b, (int *)c, (int)si0, (int)si1);
            if (rc) rc = run_int_only<int>(fid, n, (int *)out, (int *)a, (int *)b); break;
    case 4: rc = run_common<long>(fid, n, (long *)out, (long *)a, (long *)b, (long *)c, (long)si0, (long)si1);
            if (rc) rc = run_int_only<long>(fid, n, (long *)out, (long *)a, (long *)b); break;
    case 6: rc = run_common<float>(fid, n, (float *)out, (float *)a, (float *)b, (float *)c, (float)sf0, (float)sf1);
            if (rc) rc = run_fp_only<float>(fid, n, (float *)out, (float *)a, (float *)b, (float)sf0); break;
    case 7: rc = run_common<double>(fid, n, (double *)out, (double *)a, (double *)b, (double *)c, sf0, sf1);
            if (rc) rc = run_fp_only<double>(fid, n, (double *)out, (double *)a, (double *)b, sf0); break;
  }
  return rc;
}

}  // extern "C"

namespace {

// out[i] = a[i] CMP (b ? b[i] : value), TOut the result type: the ...Value functors of
// THCTensorMathCompare.cuh with a scalar, the tensor functors of THCTensorMathCompareT.cuh otherwise
template <typename T, typename TOut> int run_compare(int cmp, int64_t n, TOut *out, T *a, T *b, T value) {
  for (int64_t i = 0; i < n; ++i) {
    if (b) {
      switch (cmp) {
        case 0: { TensorLTOp<T, TOut> f; f(out + i, a + i, b + i); break; }
        case 1: { TensorGTOp<T, TOut> f; f(out + i, a + i, b + i); break; }
        case 2: { TensorLEOp<T, TOut> f; f(out + i, a + i, b + i); break; }
        case 3: { TensorGEOp<T, TOut> f; f(out + i, a + i, b + i); break; }
        case 4: { TensorEQOp<T, TOut> f; f(out + i, a + i, b + i); break; }
        case 5: { TensorNEOp<T, TOut> f; f(out + i, a + i, b + i); break; }
        default: return -1;
      }
    } else {
      switch (cmp) {
        case 0: { TensorLTValueOp<T, TOut> f(value); f(out + i, a + i); break; }
        case 1: { TensorGTValueOp<T, TOut> f(value); f(out + i, a + i); break; }
        case 2: { TensorLEValueOp<T, TOut> f(value); f(out + i, a + i); break; }
        case 3: { TensorGEValueOp<T, TOut> f(value); f(out + i, a + i); break; }
        case 4: { TensorEQValueOp<T, TOut> f(value); f(out + i, a + i); break; }
        case 5: { TensorNEValueOp<T, TOut> f(value); f(out + i, a + i); break; }
        default: return -1;
      }
    }
  }
  return 0;
}

template <typename T> int run_compare_both(int cmp, int same_type, int64_t n, void *out, T *a, T *b, T value) {
  return same_type ? run_compare<T, T>(cmp, n, (T *)out, a, b, value)
                   : run_compare<T, unsigned char>(cmp, n, (unsigned char *)out, a, b, value);
}

// The masked functors take the exclusive prefix sum of the mask (cutorch computes it with a thrust
// exclusive_scan over a Long copy of the mask, lib/THC/generic/THCTensorMasked.cu:75-93,150-168).
template <typename T> int run_masked(int which, int64_t n, T *t, unsigned char *mask, T *other, T value) {
  long *prefix = (long *)malloc(sizeof(long) * (size_t)(n > 0 ? n : 1));
  long run = 0;
  for (int64_t i = 0; i < n; ++i) { prefix[i] = run; run += mask[i] ? 1 : 0; }
  int rc = 0;
  if (which == 0) { TensorMaskedFillOp<T, unsigned char> f(value); for (int64_t i = 0; i < n; ++i) f(t + i, mask + i); }
  else if (which == 1) { TensorMaskedCopyOp<T, unsigned char, long> f(other); for (int64_t i = 0; i < n; ++i) f(t + i, mask + i, prefix + i); }
  else if (which == 2) { TensorMaskedSelectOp<T, unsigned char, long> f(other); for (int64_t i = 0; i < n; ++i) f(mask + i, prefix + i, t + i); }
  else rc = -1;
  free(prefix);
  return rc;
}

}  // namespace

extern "C" {

// cmp: 0 lt, 1 gt, 2 le, 3 ge, 4 eq, 5 ne.  b == NULL compares with the scalar.  same_type: the
// result has the operands' type (the ...T entry points), else unsigned char.
int ref_compare(int cmp, int same_type, int dtype, int64_t n, void *out, void *a, void *b, double sf, int64_t si) {
  switch (dtype) {
    case 0: return run_compare_both<unsigned char>(cmp, same_type, n, out, (unsigned char *)a, (unsigned char *)b, (unsigned char)si);
    case 1: return run_compare_both<char>(cmp, same_type, n, out, (char *)a, (char *)b, (char)si);
    case 2: return run_compare_both<short>(cmp, same_type, n, out, (short *)a, (short *)b, (short)si);
    case 3: return run_compare_both<int>(cmp, same_type, n, out, (int *)a, (int *)b, (int)si);
    case 4: return run_compare_both<long>(cmp, same_type, n, out, (long *)a, (long *)b, (long)si);
    case 6: return run_compare_both<float>(cmp, same_type, n, out, (float *)a, (float *)b, (float)sf);
    case 7: return run_compare_both<double>(cmp, same_type, n, out, (double *)a, (double *)b, sf);
  }
  return -1;
}

// which: 0 fill t where mask (value), 1 copy: t[i] = other[rank of i] where mask, 2 select: other[rank of i] = t[i] where mask
int ref_masked(int which, int dtype, int64_t n, void *t, unsigned char *mask, void *other, double sf, int64_t si) {
  switch (dtype) {
    case 0: return run_masked<unsigned char>(which, n, (unsigned char *)t, mask, (unsigned char *)other, (unsigned char)si);
    case 1: return run_masked<char>(which, n, (char *)t, mask, (char *)other, (char)si);
    case 2: return run_masked<short>(which, n, (short *)t, mask, (short *)other, (short)si);
    case 3: return run_masked<int>(which, n, (int *)t, mask, (int *)other, (int)si);
    case 4: return run_masked<long>(which, n, (long *)t, mask, (long *)other, (long)si);
    case 6: return run_masked<float>(which, n, (float *)t, mask, (float *)other, (float)sf);
    case 7: return run_masked<double>(which, n, (double *)t, mask, (double *)other, sf);
  }
  return -1;
}

}  // extern "C"
