// TEST INFRASTRUCTURE -- not part of the product.  CPU restatement of the results the THC
// apply / reduce path must reproduce, following torch7's TH CPU tensor semantics (the parity
// target) for the ops whose math is given by cutorch's functor bodies:
//   pointwise expressions   lib/THC/THCTensorMathPointwise.cuh:12-772,
//                           lib/THC/THCTensorMathPairwise.cu:9-476, lib/THC/THCNumerics.cuh
//   entry-point composition lib/THC/generic/THCTensorMathPointwise.cu:5-713,
//                           lib/THC/generic/THCTensorMathReduce.cu:5-436
//   logical iteration order lib/THC/THCTensorInfo.cuh:228-278 (row-major index -> offset)
//   reduction structure     lib/THC/THCReduce.cuh:258-453, lib/THC/THCReduceAll.cuh:234-342
// TH itself (torch/torch7, lib/TH; cutorch's rockspec pins only "torch >= 7.0") is not in the
// cutorch tree, so its rules are restated from its published behaviour: scalar C loops in
// logical order without FMA contraction; float reductions accumulate in double, integer ones
// in 64 bits; max/min along a dim keep the first occurrence and stop at a NaN; half tensors
// are float math on half-rounded inputs rounded back once per call.  PARITY UNPINNED for those
// TH-specific rules (no TH build or golden vectors exist here); the dimension logic and the
// functor bodies are pinned against the reference's own code by oracle/ref_check.
//
// Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load this file's
// shared object.  Build: make -C oracle   (g++ -O2 -ffp-contract=off, no -ffast-math).
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

#define ORACLE_MAX_DIMS 25

typedef struct oracle_tensor {
  void *data;
  int32_t dtype;  // 0 u8, 1 i8, 2 i16, 3 i32, 4 i64, 5 f16, 6 f32, 7 f64
  int32_t ndim;
  int64_t sizes[ORACLE_MAX_DIMS];
  int64_t strides[ORACLE_MAX_DIMS];
} oracle_tensor;

// op numbering is shared with include/thcb200.h (the tests pass the same integers)
enum {
  OP_FILL = 0, OP_COPY, OP_LOG, OP_LGAMMA, OP_LOG1P, OP_EXP, OP_COS, OP_SIN, OP_SQRT, OP_RSQRT, OP_CEIL, OP_FLOOR,
  OP_TRUNC, OP_ACOS, OP_COSH, OP_ASIN, OP_SINH, OP_TAN, OP_ATAN, OP_TANH, OP_ROUND, OP_FRAC, OP_CINV, OP_NEG, OP_ABS,
  OP_SIGN, OP_SIGMOID, OP_CLAMP, OP_POW, OP_TPOW, OP_ADD_S, OP_SUB_S, OP_MUL_S, OP_DIV_S, OP_LSHIFT_S, OP_RSHIFT_S,
  OP_FMOD_S, OP_REMAINDER_S, OP_BITAND_S, OP_BITOR_S, OP_BITXOR_S, OP_MAX_S, OP_MIN_S,
  OP_LT_S, OP_GT_S, OP_LE_S, OP_GE_S, OP_EQ_S, OP_NE_S,
  OP_ADD, OP_SUB, OP_CADD, OP_MUL, OP_DIV, OP_CPOW, OP_CLSHIFT, OP_CRSHIFT, OP_CMAX, OP_CMIN, OP_CFMOD,
  OP_CREMAINDER, OP_CBITAND, OP_CBITOR, OP_CBITXOR, OP_ATAN2, OP_LERP,
  OP_LT, OP_GT, OP_LE, OP_GE, OP_EQ, OP_NE,
  OP_ADDCMUL, OP_ADDCDIV, OP_COUNT
};
enum { RED_SUM = 0, RED_PROD, RED_MIN, RED_MAX, RED_ALL, RED_ANY };
enum { PRE_IDENTITY = 0, PRE_ABS, PRE_SQUARE, PRE_POWABS, PRE_NONZERO, PRE_SQDEV };

}  // extern "C"

namespace {

int g_threads = 1;

typedef _Float16 f16;

// Row-major walk over a strided view: offset of logical index i, advanced one step at a time.
struct Walker {
  int nd;
  int64_t size[ORACLE_MAX_DIMS], stride[ORACLE_MAX_DIMS], idx[ORACLE_MAX_DIMS];
  int64_t off;
  void init(const oracle_tensor &t, int64_t linear) {
    nd = t.ndim;
    off = 0;
    for (int d = nd - 1; d >= 0; --d) {
      size[d] = t.sizes[d];
      stride[d] = t.strides[d];
      idx[d] = size[d] ? linear % size[d] : 0;
      if (size[d]) linear /= size[d];
      off += idx[d] * stride[d];
    }
  }
  inline void next() {
    for (int d = nd - 1; d >= 0; --d) {
      ++idx[d];
      off += stride[d];
      if (idx[d] < size[d]) return;
      off -= idx[d] * stride[d];
      idx[d] = 0;
    }
  }
};

int64_t numel(const oracle_tensor &t) {
  if (t.ndim <= 0) return 0;
  int64_t n = 1;
  for (int d = 0; d < t.ndim; ++d) n *= t.sizes[d];
  return n;
}

// ---- element math ---------------------------------------------------------------------
template <typename T> struct Info;
template <> struct Info<uint8_t> { using M = uint8_t; using P = int; using U = unsigned; static const bool fp = false; };
template <> struct Info<int8_t> { using M = int8_t; using P = int; using U = unsigned; static const bool fp = false; };
template <> struct Info<int16_t> { using M = int16_t; using P = int; using U = unsigned; static const bool fp = false; };
template <> struct Info<int32_t> { using M = int32_t; using P = int; using U = unsigned; static const bool fp = false; };
template <> struct Info<int64_t> { using M = int64_t; using P = int64_t; using U = uint64_t; static const bool fp = false; };
template <> struct Info<f16> { using M = float; static const bool fp = true; };
template <> struct Info<float> { using M = float; static const bool fp = true; };
template <> struct Info<double> { using M = double; static const bool fp = true; };

// Transcendentals of float tensors: evaluate in double and round once (the correctly rounded
// value up to double's own error); the GPU result has to stay within 2 ulp of it.
template <typename M> struct Tr {
  static M f(double (*fn)(double), M x) { return (M)fn((double)x); }
  static M f2(double (*fn)(double, double), M x, M y) { return (M)fn((double)x, (double)y); }
};

template <typename M> M fp_op(int op, M s0, M s1, M a, M b, M c) {
  const M one = (M)1;
  switch (op) {
    case OP_FILL: return s0;
    case OP_COPY: return a;
    case OP_LOG: return Tr<M>::f(log, a);
    case OP_LGAMMA: return Tr<M>::f(lgamma, a);
    case OP_LOG1P: return Tr<M>::f(log1p, a);
    case OP_EXP: return Tr<M>::f(exp, a);
    case OP_COS: return Tr<M>::f(cos, a);
    case OP_SIN: return Tr<M>::f(sin, a);
    case OP_SQRT: return Tr<M>::f(sqrt, a);
    case OP_RSQRT: return one / (M)sqrt((double)a);
    case OP_CEIL: return Tr<M>::f(ceil, a);
    case OP_FLOOR: return Tr<M>::f(floor, a);
    case OP_TRUNC: return Tr<M>::f(trunc, a);
    case OP_ACOS: return Tr<M>::f(acos, a);
    case OP_COSH: return Tr<M>::f(cosh, a);
    case OP_ASIN: return Tr<M>::f(asin, a);
    case OP_SINH: return Tr<M>::f(sinh, a);
    case OP_TAN: return Tr<M>::f(tan, a);
    case OP_ATAN: return Tr<M>::f(atan, a);
    case OP_TANH: return Tr<M>::f(tanh, a);
    case OP_ROUND: return Tr<M>::f(round, a);
    case OP_FRAC: return a - (M)trunc((double)a);
    case OP_CINV: return one / a;
    case OP_NEG: return -a;
    case OP_ABS: return (M)fabs((double)a);
    case OP_SIGN: return (M)((a > 0) - (a < 0));
    case OP_SIGMOID: return (M)(1.0 / (1.0 + exp(-(double)a)));
    case OP_CLAMP: return (a < s0) ? s0 : (a > s1 ? s1 : a);
    case OP_POW:
      if (s0 == (M)1) return a;
      if (s0 == (M)2) return a * a;
      if (s0 == (M)3) return (a * a) * a;
      if (s0 == (M)-1) return one / a;
      if (s0 == (M)-2) return one / (a * a);
      return Tr<M>::f2(pow, a, s0);
    case OP_TPOW: return Tr<M>::f2(pow, s0, a);
    case OP_ADD_S: return a + s0;
    case OP_SUB_S: return a - s0;
    case OP_MUL_S: return a * s0;
    case OP_DIV_S: return a / s0;
    case OP_LSHIFT_S: return a * (M)pow((M)2, s0);
    case OP_RSHIFT_S: return a / (M)pow((M)2, s0);
    case OP_FMOD_S: return (M)fmod((double)a, (double)s0);
    case OP_REMAINDER_S: return a - s0 * (M)floor((double)(a / s0));
    case OP_MAX_S: return (a > s0) ? a : s0;
    case OP_MIN_S: return (a < s0) ? a : s0;
    case OP_LT_S: return (M)(a < s0);
    case OP_GT_S: return (M)(a > s0);
    case OP_LE_S: return (M)(a <= s0);
    case OP_GE_S: return (M)(a >= s0);
    case OP_EQ_S: return (M)(a == s0);
    case OP_NE_S: return (M)(a != s0);
    case OP_ADD: return a + b;
    case OP_SUB: return a - b;
    case OP_CADD: { M t = s0 * b; return a + t; }
    case OP_MUL: return a * b;
    case OP_DIV: return a / b;
    case OP_CPOW: return Tr<M>::f2(pow, a, b);
    case OP_CLSHIFT: return a * Tr<M>::f2(pow, (M)2, b);
    case OP_CRSHIFT: return a / Tr<M>::f2(pow, (M)2, b);
    case OP_CMAX: return (a > b) ? a : b;
    case OP_CMIN: return (a < b) ? a : b;
    case OP_CFMOD: return (M)fmod((double)a, (double)b);
    case OP_CREMAINDER: return (b != (M)0) ? a - b * (M)floor((double)(a / b)) : (M)NAN;
    case OP_ATAN2: return Tr<M>::f2(atan2, a, b);
    case OP_LERP: { M d = b - a; M t = s0 * d; return a + t; }
    case OP_LT: return (M)(a < b);
    case OP_GT: return (M)(a > b);
    case OP_LE: return (M)(a <= b);
    case OP_GE: return (M)(a >= b);
    case OP_EQ: return (M)(a == b);
    case OP_NE: return (M)(a != b);
    // TH writes `r += value * src1 * src2`: the scalar multiplies src1 first
    case OP_ADDCMUL: { M t = s0 * b; t = t * c; return a + t; }
    case OP_ADDCDIV: { M t = s0 * b; t = t / c; return a + t; }
  }
  return a;
}

template <typename I> I int_op(int op, I s0, I s1, I a, I b, I c) {
  using P = typename Info<I>::P;
  using U = typename Info<I>::U;
  const P pa = (P)a, pb = (P)b, pc = (P)c, ps = (P)s0;
  auto add = [](P x, P y) { return (P)((U)x + (U)y); };
  auto sub = [](P x, P y) { return (P)((U)x - (U)y); };
  auto mul = [](P x, P y) { return (P)((U)x * (U)y); };
  const bool is_unsigned = ((I)-1 > (I)0);
  switch (op) {
    case OP_FILL: return s0;
    case OP_COPY: return a;
    case OP_NEG: return (I)sub(0, pa);
    case OP_ABS: return is_unsigned ? a : (I)(pa < 0 ? sub(0, pa) : pa);
    case OP_SIGN: return is_unsigned ? (I)(a != 0) : (I)((a > 0) - (a < 0));
    case OP_CLAMP: return (a < s0) ? s0 : (a > s1 ? s1 : a);
    case OP_ADD_S: return (I)add(pa, ps);
    case OP_SUB_S: return (I)sub(pa, ps);
    case OP_MUL_S: return (I)mul(pa, ps);
    case OP_DIV_S: return (I)(pa / ps);
    case OP_LSHIFT_S: return (I)(P)((U)pa << ps);
    case OP_RSHIFT_S: return (I)(pa >> ps);
    case OP_FMOD_S: return (I)(pa % ps);
    case OP_REMAINDER_S: { P r = pa % ps; if (mul((P)(I)r, ps) < 0) r = add(r, ps); return (I)r; }
    case OP_BITAND_S: return (I)(a & s0);
    case OP_BITOR_S: return (I)(a | s0);
    case OP_BITXOR_S: return (I)(a ^ s0);
    case OP_MAX_S: return (a > s0) ? a : s0;
    case OP_MIN_S: return (a < s0) ? a : s0;
    case OP_LT_S: return (I)(a < s0);
    case OP_GT_S: return (I)(a > s0);
    case OP_LE_S: return (I)(a <= s0);
    case OP_GE_S: return (I)(a >= s0);
    case OP_EQ_S: return (I)(a == s0);
    case OP_NE_S: return (I)(a != s0);
    case OP_ADD: return (I)add(pa, pb);
    case OP_SUB: return (I)sub(pa, pb);
    case OP_CADD: return (I)add(pa, mul(ps, pb));
    case OP_MUL: return (I)mul(pa, pb);
    case OP_DIV: return (I)(pa / pb);
    case OP_CPOW: return (I)pow((double)a, (double)b);
    case OP_CLSHIFT: return (I)(P)((U)pa << pb);
    case OP_CRSHIFT: return (I)(pa >> pb);
    case OP_CMAX: return (a > b) ? a : b;
    case OP_CMIN: return (a < b) ? a : b;
    case OP_CFMOD: return (I)(pa % pb);
    case OP_CREMAINDER: { P r = pa % pb; if (mul((P)(I)r, pb) < 0) r = add(r, pb); return (I)r; }
    case OP_CBITAND: return (I)(a & b);
    case OP_CBITOR: return (I)(a | b);
    case OP_CBITXOR: return (I)(a ^ b);
    case OP_LT: return (I)(a < b);
    case OP_GT: return (I)(a > b);
    case OP_LE: return (I)(a <= b);
    case OP_GE: return (I)(a >= b);
    case OP_EQ: return (I)(a == b);
    case OP_NE: return (I)(a != b);
    case OP_ADDCMUL: return (I)add(pa, mul(mul(ps, pb), pc));
    case OP_ADDCDIV: return (I)add(pa, (P)(mul(ps, pb) / pc));
  }
  return a;
}

template <typename T> struct Elem {
  using M = typename Info<T>::M;
  static M load(const T *p) { return (M)*p; }
  static void store(T *p, M v) { *p = (T)v; }
};

template <typename T>
void pointwise_range(int op, const oracle_tensor &out, const oracle_tensor *in, int nin, double sf0, double sf1, int64_t si0,
                     int64_t si1, int64_t begin, int64_t end) {
  using M = typename Info<T>::M;
  Walker wo, wi[3];
  wo.init(out, begin);
  for (int k = 0; k < nin; ++k) wi[k].init(in[k], begin);
  T *po = (T *)out.data;
  const T *pi[3] = {nin > 0 ? (const T *)in[0].data : nullptr, nin > 1 ? (const T *)in[1].data : nullptr,
                    nin > 2 ? (const T *)in[2].data : nullptr};
  M s0, s1;
  if (Info<T>::fp) { s0 = (M)sf0; s1 = (M)sf1; } else { s0 = (M)si0; s1 = (M)si1; }
  for (int64_t i = begin; i < end; ++i) {
    M a = nin > 0 ? Elem<T>::load(pi[0] + wi[0].off) : M();
    M b = nin > 1 ? Elem<T>::load(pi[1] + wi[1].off) : M();
    M c = nin > 2 ? Elem<T>::load(pi[2] + wi[2].off) : M();
    M r;
    if constexpr (Info<T>::fp) r = fp_op<M>(op, s0, s1, a, b, c);
    else r = int_op<T>(op, s0, s1, a, b, c);
    Elem<T>::store(po + wo.off, r);
    wo.next();
    for (int k = 0; k < nin; ++k) wi[k].next();
  }
}

template <typename T>
void pointwise_t(int op, const oracle_tensor &out, const oracle_tensor *in, int nin, double sf0, double sf1, int64_t si0,
                 int64_t si1) {
  const int64_t n = numel(out);
  const int nt = std::max(1, g_threads);
  if (nt == 1 || n < (1 << 16)) { pointwise_range<T>(op, out, in, nin, sf0, sf1, si0, si1, 0, n); return; }
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < nt; ++t) {
    const int64_t b = n * t / nt, e = n * (t + 1) / nt;
    pointwise_range<T>(op, out, in, nin, sf0, sf1, si0, si1, b, e);
  }
}

// ---- reductions -----------------------------------------------------------------------
template <typename T> struct AccOf { using type = int64_t; };
template <> struct AccOf<f16> { using type = double; };   // FloatTensor math: TH accumulates float in double
template <> struct AccOf<float> { using type = double; };
template <> struct AccOf<double> { using type = double; };

template <typename T, typename A> inline A pre_elem(int pre, double s, T x) {
  A v = (A)(typename Info<T>::M)x;
  switch (pre) {
    case PRE_ABS: return v < 0 ? -v : v;
    case PRE_SQUARE: return v * v;
    case PRE_POWABS: return (A)pow(fabs((double)v), s);
    case PRE_NONZERO: return v != 0 ? (A)1 : (A)0;
    case PRE_SQDEV: return (A)(((double)v - s) * ((double)v - s));
  }
  return v;
}

// Folds one strided run of n elements.  Sum/prod in the accumulate type; min/max with TH's
// scan rule (replace when !(x <= cur) resp. !(x >= cur), stop at a NaN).
template <typename T> struct RunResult { double f; int64_t i; int64_t pos; };

template <typename T>
RunResult<T> fold_run(int rop, int pre, double s, const T *p, int64_t stride, int64_t n) {
  using A = typename AccOf<T>::type;
  using M = typename Info<T>::M;
  RunResult<T> r; r.f = 0; r.i = 0; r.pos = 0;
  if (rop == RED_SUM || rop == RED_PROD) {
    A acc = rop == RED_SUM ? (A)0 : (A)1;
    for (int64_t k = 0; k < n; ++k) {
      A v = pre_elem<T, A>(pre, s, p[k * stride]);
      if (rop == RED_SUM) {
        if constexpr (Info<T>::fp) acc = acc + v; else acc = (A)((uint64_t)acc + (uint64_t)v);
      } else {
        if constexpr (Info<T>::fp) acc = acc * v; else acc = (A)((uint64_t)acc * (uint64_t)v);
      }
    }
    r.f = (double)acc; r.i = (int64_t)acc;
  } else if (rop == RED_MIN || rop == RED_MAX) {
    M cur = (M)p[0];
    int64_t pos = 0;
    if (!(cur != cur)) {
      for (int64_t k = 1; k < n; ++k) {
        M v = (M)p[k * stride];
        const bool take = rop == RED_MAX ? !(v <= cur) : !(v >= cur);
        if (take) { cur = v; pos = k; if (v != v) break; }
      }
    }
    r.f = (double)cur; r.i = (int64_t)cur; r.pos = pos;
  } else {
    int acc = rop == RED_ALL ? 1 : 0;
    for (int64_t k = 0; k < n; ++k) {
      const int v = ((M)p[k * stride] != (M)0);
      acc = rop == RED_ALL ? (acc && v) : (acc || v);
    }
    r.f = acc; r.i = acc;
  }
  return r;
}

template <typename T> T from_result(const RunResult<T> &r) {
  if constexpr (Info<T>::fp) {
    if constexpr (std::is_same<T, f16>::value) return (f16)(float)r.f;  // double -> float -> half, as a FloatTensor result stored to half
    else return (T)r.f;
  } else return (T)r.i;
}

template <typename T>
void reduce_dim_t(int rop, int pre, double s, const oracle_tensor &out, const oracle_tensor *idx, const oracle_tensor &in, int dim) {
  oracle_tensor inb = in;
  inb.sizes[dim] = 1;
  const int64_t nout = numel(out);
  const int64_t K = in.sizes[dim], sk = in.strides[dim];
  const int nt = std::max(1, g_threads);
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1 && nout >= 64)
  for (int t = 0; t < nt; ++t) {
    const int64_t b = nout * t / nt, e = nout * (t + 1) / nt;
    Walker wi, wo, wx;
    wi.init(inb, b);
    wo.init(out, b);
    if (idx) wx.init(*idx, b);
    for (int64_t o = b; o < e; ++o) {
      RunResult<T> r = fold_run<T>(rop, pre, s, (const T *)in.data + wi.off, sk, K);
      ((T *)out.data)[wo.off] = from_result<T>(r);
      if (idx) ((int64_t *)idx->data)[wx.off] = r.pos + 1;
      wi.next(); wo.next();
      if (idx) wx.next();
    }
  }
}

// var / std along a dim with TH's formula: running sum and sum of squares in the accumulate type,
// E[x^2] - E[x]^2 (times n/(n-1) pieces when unbiased), clamped at zero
// (composition of lib/THC/generic/THCTensorMathReduce.cu:76-126 with THCTensorMathReduce.cuh:269-306).
template <typename T>
void var_dim_t(const oracle_tensor &out, const oracle_tensor &in, int dim, int biased, int take_sqrt) {
  oracle_tensor inb = in;
  inb.sizes[dim] = 1;
  const int64_t nout = numel(out);
  const int64_t K = in.sizes[dim], sk = in.strides[dim];
  Walker wi, wo;
  wi.init(inb, 0);
  wo.init(out, 0);
  for (int64_t o = 0; o < nout; ++o) {
    const T *p = (const T *)in.data + wi.off;
    double s = 0, s2 = 0;
    for (int64_t k = 0; k < K; ++k) {
      const double z = (double)(typename Info<T>::M)p[k * sk];
      s += z;
      s2 += z * z;
    }
    const double n = (double)K;
    double mean = s / n, v;
    if (biased) v = s2 / n - mean * mean;
    else v = s2 / (n - 1) - (n / (n - 1)) * mean * mean;
    if (v < 0) v = 0;
    if (take_sqrt) v = sqrt(v);
    RunResult<T> r; r.f = v; r.i = 0; r.pos = 0;
    ((T *)out.data)[wo.off] = from_result<T>(r);
    wi.next(); wo.next();
  }
}

// cumsum / cumprod along a dim: one running accumulator per slice, every output rounded from it
// (the sequential form of THCTensor_kernel_scanOuterDim, lib/THC/THCTensorMathScan.cu:24-45, with
// TH's accumulate type).  Integer accumulation wraps modulo 2^64.
template <typename T>
void scan_dim_t(int prod, const oracle_tensor &out, const oracle_tensor &in, int dim) {
  using A = typename AccOf<T>::type;
  oracle_tensor inb = in, outb = out;
  inb.sizes[dim] = 1;
  outb.sizes[dim] = 1;
  const int64_t nslices = numel(inb);
  const int64_t K = in.sizes[dim], ski = in.strides[dim], sko = out.strides[dim];
  Walker wi, wo;
  wi.init(inb, 0);
  wo.init(outb, 0);
  for (int64_t o = 0; o < nslices; ++o) {
    const T *p = (const T *)in.data + wi.off;
    T *q = (T *)out.data + wo.off;
    RunResult<T> r; r.f = prod ? 1.0 : 0.0; r.i = prod ? 1 : 0; r.pos = 0;
    for (int64_t k = 0; k < K; ++k) {
      if constexpr (Info<T>::fp) {
        const A z = (A)(typename Info<T>::M)p[k * ski];
        r.f = prod ? r.f * z : r.f + z;
      } else {
        const uint64_t z = (uint64_t)(int64_t)p[k * ski];
        r.i = (int64_t)(prod ? (uint64_t)r.i * z : (uint64_t)r.i + z);
      }
      q[k * sko] = from_result<T>(r);
    }
    wi.next(); wo.next();
  }
}

template <typename T>
void reduce_all_t(int rop, int pre, double s, const oracle_tensor &in, double *rf, int64_t *ri) {
  using A = typename AccOf<T>::type;
  using M = typename Info<T>::M;
  const int64_t n = numel(in);
  const int nt = (g_threads > 1 && n >= (1 << 16)) ? g_threads : 1;
  std::vector<double> pf(nt, 0.0);
  std::vector<int64_t> pi(nt, 0);
  std::vector<int> has(nt, 0);
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int t = 0; t < nt; ++t) {
    const int64_t b = n * t / nt, e = n * (t + 1) / nt;
    Walker w;
    w.init(in, b);
    const T *p = (const T *)in.data;
    if (rop == RED_SUM || rop == RED_PROD) {
      A acc = rop == RED_SUM ? (A)0 : (A)1;
      for (int64_t i = b; i < e; ++i) {
        A v = pre_elem<T, A>(pre, s, p[w.off]);
        if (rop == RED_SUM) { if constexpr (Info<T>::fp) acc = acc + v; else acc = (A)((uint64_t)acc + (uint64_t)v); }
        else { if constexpr (Info<T>::fp) acc = acc * v; else acc = (A)((uint64_t)acc * (uint64_t)v); }
        w.next();
      }
      pf[t] = (double)acc; pi[t] = (int64_t)acc; has[t] = 1;
    } else if (rop == RED_MIN || rop == RED_MAX) {
      if (e > b) {
        M cur = (M)p[w.off];
        w.next();
        for (int64_t i = b + 1; i < e && !(cur != cur); ++i) {
          M v = (M)p[w.off];
          const bool take = rop == RED_MAX ? !(v <= cur) : !(v >= cur);
          if (take) cur = v;
          w.next();
        }
        pf[t] = (double)cur; pi[t] = (int64_t)cur; has[t] = 1;
      }
    } else {
      int acc = rop == RED_ALL ? 1 : 0;
      for (int64_t i = b; i < e; ++i) {
        const int v = ((M)p[w.off] != (M)0);
        acc = rop == RED_ALL ? (acc && v) : (acc || v);
        w.next();
      }
      pf[t] = acc; pi[t] = acc; has[t] = 1;
    }
  }
  // combine the per-thread partials in thread order
  double f = 0; int64_t iv = 0; bool first = true;
  for (int t = 0; t < nt; ++t) {
    if (!has[t]) continue;
    if (first) { f = pf[t]; iv = pi[t]; first = false; continue; }
    switch (rop) {
      case RED_SUM: f += pf[t]; iv = (int64_t)((uint64_t)iv + (uint64_t)pi[t]); break;
      case RED_PROD: f *= pf[t]; iv = (int64_t)((uint64_t)iv * (uint64_t)pi[t]); break;
      case RED_MAX: if (!(f != f)) { if (!(pf[t] <= f)) f = pf[t]; } if (pi[t] > iv) iv = pi[t]; break;
      case RED_MIN: if (!(f != f)) { if (!(pf[t] >= f)) f = pf[t]; } if (pi[t] < iv) iv = pi[t]; break;
      case RED_ALL: f = (f != 0 && pf[t] != 0); iv = (iv && pi[t]); break;
      case RED_ANY: f = (f != 0 || pf[t] != 0); iv = (iv || pi[t]); break;
    }
  }
  *rf = f; *ri = iv;
}

template <typename TO, typename TI> void convert_t(const oracle_tensor &out, const oracle_tensor &in) {
  const int64_t n = numel(out);
  Walker wo, wi;
  wo.init(out, 0);
  wi.init(in, 0);
  for (int64_t i = 0; i < n; ++i) {
    const TI v = ((const TI *)in.data)[wi.off];
    TO r;
    if constexpr (std::is_same<TI, f16>::value && !std::is_same<TO, f16>::value) r = (TO)(float)v;
    else if constexpr (std::is_same<TO, f16>::value && !std::is_same<TI, f16>::value) r = (f16)(float)v;
    else r = (TO)v;
    ((TO *)out.data)[wo.off] = r;
    wo.next(); wi.next();
  }
}

template <typename TO> int convert_from(const oracle_tensor &out, const oracle_tensor &in) {
  switch (in.dtype) {
    case 0: convert_t<TO, uint8_t>(out, in); return 0;
    case 1: convert_t<TO, int8_t>(out, in); return 0;
    case 2: convert_t<TO, int16_t>(out, in); return 0;
    case 3: convert_t<TO, int32_t>(out, in); return 0;
    case 4: convert_t<TO, int64_t>(out, in); return 0;
    case 5: convert_t<TO, f16>(out, in); return 0;
    case 6: convert_t<TO, float>(out, in); return 0;
    case 7: convert_t<TO, double>(out, in); return 0;
  }
  return -1;
}

}  // namespace

extern "C" {

void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// out = op(in...), each operand walked in its own row-major order (TH_TENSOR_APPLY order).
int oracle_pointwise(int op, const oracle_tensor *out, const oracle_tensor *in0, const oracle_tensor *in1,
                     const oracle_tensor *in2, int nin, double sf0, double sf1, int64_t si0, int64_t si1) {
  oracle_tensor in[3];
  if (nin > 0) in[0] = *in0;
  if (nin > 1) in[1] = *in1;
  if (nin > 2) in[2] = *in2;
  switch (out->dtype) {
    case 0: pointwise_t<uint8_t>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
    case 1: pointwise_t<int8_t>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
    case 2: pointwise_t<int16_t>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
    case 3: pointwise_t<int32_t>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
    case 4: pointwise_t<int64_t>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
    case 5: pointwise_t<f16>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
    case 6: pointwise_t<float>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
    case 7: pointwise_t<double>(op, *out, in, nin, sf0, sf1, si0, si1); return 0;
  }
  return -1;
}

int oracle_copy_convert(const oracle_tensor *out, const oracle_tensor *in) {
  switch (out->dtype) {
    case 0: return convert_from<uint8_t>(*out, *in);
    case 1: return convert_from<int8_t>(*out, *in);
    case 2: return convert_from<int16_t>(*out, *in);
    case 3: return convert_from<int32_t>(*out, *in);
    case 4: return convert_from<int64_t>(*out, *in);
    case 5: return convert_from<f16>(*out, *in);
    case 6: return convert_from<float>(*out, *in);
    case 7: return convert_from<double>(*out, *in);
  }
  return -1;
}

// out[..., 0, ...] = fold over `dim`; idx (optional, int64) receives 1-based first positions
// for RED_MIN / RED_MAX.
int oracle_reduce_dim(int rop, int pre, double s, const oracle_tensor *out, const oracle_tensor *idx, const oracle_tensor *in,
                      int dim) {
  switch (in->dtype) {
    case 0: reduce_dim_t<uint8_t>(rop, pre, s, *out, idx, *in, dim); return 0;
    case 1: reduce_dim_t<int8_t>(rop, pre, s, *out, idx, *in, dim); return 0;
    case 2: reduce_dim_t<int16_t>(rop, pre, s, *out, idx, *in, dim); return 0;
    case 3: reduce_dim_t<int32_t>(rop, pre, s, *out, idx, *in, dim); return 0;
    case 4: reduce_dim_t<int64_t>(rop, pre, s, *out, idx, *in, dim); return 0;
    case 5: reduce_dim_t<f16>(rop, pre, s, *out, idx, *in, dim); return 0;
    case 6: reduce_dim_t<float>(rop, pre, s, *out, idx, *in, dim); return 0;
    case 7: reduce_dim_t<double>(rop, pre, s, *out, idx, *in, dim); return 0;
  }
  return -1;
}

int oracle_var_dim(const oracle_tensor *out, const oracle_tensor *in, int dim, int biased, int take_sqrt) {
  switch (in->dtype) {
    case 5: var_dim_t<f16>(*out, *in, dim, biased, take_sqrt); return 0;
    case 6: var_dim_t<float>(*out, *in, dim, biased, take_sqrt); return 0;
    case 7: var_dim_t<double>(*out, *in, dim, biased, take_sqrt); return 0;
  }
  return -1;
}

int oracle_scan_dim(int prod, const oracle_tensor *out, const oracle_tensor *in, int dim) {
  switch (in->dtype) {
    case 0: scan_dim_t<uint8_t>(prod, *out, *in, dim); return 0;
    case 1: scan_dim_t<int8_t>(prod, *out, *in, dim); return 0;
    case 2: scan_dim_t<int16_t>(prod, *out, *in, dim); return 0;
    case 3: scan_dim_t<int32_t>(prod, *out, *in, dim); return 0;
    case 4: scan_dim_t<int64_t>(prod, *out, *in, dim); return 0;
    case 5: scan_dim_t<f16>(prod, *out, *in, dim); return 0;
    case 6: scan_dim_t<float>(prod, *out, *in, dim); return 0;
    case 7: scan_dim_t<double>(prod, *out, *in, dim); return 0;
  }
  return -1;
}

// Fold of every element: *rf for floating element types, *ri for integer ones.
int oracle_reduce_all(int rop, int pre, double s, const oracle_tensor *in, double *rf, int64_t *ri) {
  switch (in->dtype) {
    case 0: reduce_all_t<uint8_t>(rop, pre, s, *in, rf, ri); return 0;
    case 1: reduce_all_t<int8_t>(rop, pre, s, *in, rf, ri); return 0;
    case 2: reduce_all_t<int16_t>(rop, pre, s, *in, rf, ri); return 0;
    case 3: reduce_all_t<int32_t>(rop, pre, s, *in, rf, ri); return 0;
    case 4: reduce_all_t<int64_t>(rop, pre, s, *in, rf, ri); return 0;
    case 5: reduce_all_t<f16>(rop, pre, s, *in, rf, ri); return 0;
    case 6: reduce_all_t<float>(rop, pre, s, *in, rf, ri); return 0;
    case 7: reduce_all_t<double>(rop, pre, s, *in, rf, ri); return 0;
  }
  return -1;
}

}  // extern "C"
