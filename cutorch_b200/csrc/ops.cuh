// The pointwise operator table: one value-semantics expression per thcb200_op and
// element type.  The expressions restate the functor bodies of cutorch
// (lib/THC/THCTensorMathPointwise.cuh:12-772, lib/THC/THCTensorMathPairwise.cu:9-476,
// lib/THC/THCNumerics.cuh) with the conventions of TH's CPU tensors, which are the
// parity target: mul+add chains are never contracted to FMAs (the translation unit is
// built with -fmad=false), half computes in float and rounds once per op, integer
// arithmetic wraps, integer fmod is the C `%`.
#pragma once

#include <math.h>

#include "core.cuh"

namespace thcb {

template <typename T>
struct OpParams {
  typename TypeTraits<T>::Math s0, s1;
};

// number of tensor inputs of each op (-1: unknown)
inline int op_arity(int op) {
  if (op == THCB200_OP_FILL) return 0;
  if (op >= THCB200_OP_COPY && op <= THCB200_OP_NE_S) return 1;
  if (op >= THCB200_OP_ADD && op <= THCB200_OP_NE) return 2;
  if (op == THCB200_OP_ADDCMUL || op == THCB200_OP_ADDCDIV) return 3;
  return -1;
}

// Which (op, dtype) pairs exist, following the type guards of
// lib/THC/generic/THCTensorMathPointwise.h:5-42 and the THError branches of
// lib/THC/generic/THCTensorMathPointwise.cu:419-448,631-713 / THCTensorMathPairwise.cu:83-129,261-325.
inline bool op_supported(int op, int dtype) {
  const bool fp = dtype == THCB200_F16 || dtype == THCB200_F32 || dtype == THCB200_F64;
  switch (op) {
    case THCB200_OP_LOG: case THCB200_OP_LGAMMA: case THCB200_OP_LOG1P: case THCB200_OP_EXP:
    case THCB200_OP_COS: case THCB200_OP_SIN: case THCB200_OP_SQRT: case THCB200_OP_RSQRT:
    case THCB200_OP_CEIL: case THCB200_OP_FLOOR: case THCB200_OP_TRUNC: case THCB200_OP_ACOS:
    case THCB200_OP_COSH: case THCB200_OP_ASIN: case THCB200_OP_SINH: case THCB200_OP_TAN:
    case THCB200_OP_ATAN: case THCB200_OP_TANH: case THCB200_OP_ROUND: case THCB200_OP_FRAC:
    case THCB200_OP_CINV: case THCB200_OP_SIGMOID: case THCB200_OP_POW: case THCB200_OP_TPOW:
    case THCB200_OP_ATAN2: case THCB200_OP_LERP:
      return fp;
    case THCB200_OP_NEG:
      return dtype != THCB200_U8 && dtype != THCB200_I8;
    case THCB200_OP_LSHIFT_S: case THCB200_OP_RSHIFT_S: case THCB200_OP_CLSHIFT: case THCB200_OP_CRSHIFT:
      return dtype != THCB200_F16;
    case THCB200_OP_BITAND_S: case THCB200_OP_BITOR_S: case THCB200_OP_BITXOR_S:
    case THCB200_OP_CBITAND: case THCB200_OP_CBITOR: case THCB200_OP_CBITXOR:
      return !fp;
    default:
      return op >= 0 && op < THCB200_OP_COUNT;
  }
}

// ---- scalar math in the Math type ---------------------------------------------------
// float transcendentals whose CUDA single-precision version may be more than 2 ulp from a
// correctly rounded result are evaluated in double and rounded once.
__device__ __forceinline__ float m_pow(float a, float b) { return (float)pow((double)a, (double)b); }
__device__ __forceinline__ double m_pow(double a, double b) { return pow(a, b); }
__device__ __forceinline__ float m_lgamma(float a) { return (float)lgamma((double)a); }
__device__ __forceinline__ double m_lgamma(double a) { return lgamma(a); }
__device__ __forceinline__ float m_tan(float a) { return (float)tan((double)a); }
__device__ __forceinline__ double m_tan(double a) { return tan(a); }
__device__ __forceinline__ float m_sinh(float a) { return (float)sinh((double)a); }
__device__ __forceinline__ double m_sinh(double a) { return sinh(a); }
__device__ __forceinline__ float m_cosh(float a) { return (float)cosh((double)a); }
__device__ __forceinline__ double m_cosh(double a) { return cosh(a); }
__device__ __forceinline__ float m_fmod(float a, float b) { return fmodf(a, b); }
__device__ __forceinline__ double m_fmod(double a, double b) { return fmod(a, b); }
__device__ __forceinline__ float m_floor(float a) { return floorf(a); }
__device__ __forceinline__ double m_floor(double a) { return floor(a); }
__device__ __forceinline__ float m_abs(float a) { return fabsf(a); }
__device__ __forceinline__ double m_abs(double a) { return fabs(a); }
__device__ __forceinline__ float m_nan(float) { return __int_as_float(0x7fc00000); }
__device__ __forceinline__ double m_nan(double) { return __longlong_as_double(0x7ff8000000000000LL); }

#define THCB_UNARY_FD(name, ff, fd)                                         \
  __device__ __forceinline__ float m_##name(float a) { return ff(a); }      \
  __device__ __forceinline__ double m_##name(double a) { return fd(a); }
THCB_UNARY_FD(log, logf, log)
THCB_UNARY_FD(log1p, log1pf, log1p)
THCB_UNARY_FD(exp, expf, exp)
THCB_UNARY_FD(cos, cosf, cos)
THCB_UNARY_FD(sin, sinf, sin)
THCB_UNARY_FD(sqrt, sqrtf, sqrt)
THCB_UNARY_FD(ceil, ceilf, ceil)
THCB_UNARY_FD(trunc, truncf, trunc)
THCB_UNARY_FD(acos, acosf, acos)
THCB_UNARY_FD(asin, asinf, asin)
THCB_UNARY_FD(atan, atanf, atan)
THCB_UNARY_FD(tanh, tanhf, tanh)
THCB_UNARY_FD(round, roundf, round)
#undef THCB_UNARY_FD
__device__ __forceinline__ float m_atan2(float a, float b) { return atan2f(a, b); }
__device__ __forceinline__ double m_atan2(double a, double b) { return atan2(a, b); }

// wrap-around integer arithmetic (C semantics after promotion, without signed-overflow UB)
template <typename I> struct WideU { using type = uint32_t; };
template <> struct WideU<int64_t> { using type = uint64_t; };
template <typename I> __device__ __forceinline__ I w_add(I a, I b) { using U = typename WideU<I>::type; return (I)((U)a + (U)b); }
template <typename I> __device__ __forceinline__ I w_sub(I a, I b) { using U = typename WideU<I>::type; return (I)((U)a - (U)b); }
template <typename I> __device__ __forceinline__ I w_mul(I a, I b) { using U = typename WideU<I>::type; return (I)((U)a * (U)b); }
// the type C promotes I to before arithmetic
template <typename I> struct Promoted { using type = int; };
template <> struct Promoted<int64_t> { using type = int64_t; };

// ---- floating-point element types (Math = float or double) ---------------------------
template <int OP, typename M>
__device__ __forceinline__ M fp_apply(M s0, M s1, M a, M b, M c) {
  const M one = (M)1;
  if constexpr (OP == THCB200_OP_FILL) return s0;
  else if constexpr (OP == THCB200_OP_COPY) return a;
  else if constexpr (OP == THCB200_OP_LOG) return m_log(a);
  else if constexpr (OP == THCB200_OP_LGAMMA) return m_lgamma(a);
  else if constexpr (OP == THCB200_OP_LOG1P) return m_log1p(a);
  else if constexpr (OP == THCB200_OP_EXP) return m_exp(a);
  else if constexpr (OP == THCB200_OP_COS) return m_cos(a);
  else if constexpr (OP == THCB200_OP_SIN) return m_sin(a);
  else if constexpr (OP == THCB200_OP_SQRT) return m_sqrt(a);
  else if constexpr (OP == THCB200_OP_RSQRT) return one / m_sqrt(a);
  else if constexpr (OP == THCB200_OP_CEIL) return m_ceil(a);
  else if constexpr (OP == THCB200_OP_FLOOR) return m_floor(a);
  else if constexpr (OP == THCB200_OP_TRUNC) return m_trunc(a);
  else if constexpr (OP == THCB200_OP_ACOS) return m_acos(a);
  else if constexpr (OP == THCB200_OP_COSH) return m_cosh(a);
  else if constexpr (OP == THCB200_OP_ASIN) return m_asin(a);
  else if constexpr (OP == THCB200_OP_SINH) return m_sinh(a);
  else if constexpr (OP == THCB200_OP_TAN) return m_tan(a);
  else if constexpr (OP == THCB200_OP_ATAN) return m_atan(a);
  else if constexpr (OP == THCB200_OP_TANH) return m_tanh(a);
  else if constexpr (OP == THCB200_OP_ROUND) return m_round(a);
  else if constexpr (OP == THCB200_OP_FRAC) return a - m_trunc(a);
  else if constexpr (OP == THCB200_OP_CINV) return one / a;
  else if constexpr (OP == THCB200_OP_NEG) return -a;
  else if constexpr (OP == THCB200_OP_ABS) return m_abs(a);
  else if constexpr (OP == THCB200_OP_SIGN) return (M)((a > 0) - (a < 0));
  else if constexpr (OP == THCB200_OP_SIGMOID) return one / (one + m_exp(-a));
  else if constexpr (OP == THCB200_OP_CLAMP) return (a < s0) ? s0 : (a > s1 ? s1 : a);  // TH's form: a NaN passes through
  else if constexpr (OP == THCB200_OP_POW) {
    // lib/THC/THCTensorMathPointwise.cuh:267-306: exact forms for 1, 2, 3, -1, -2
    if (s0 == (M)1) return a;
    if (s0 == (M)2) return a * a;
    if (s0 == (M)3) return (a * a) * a;
    if (s0 == (M)-1) return one / a;
    if (s0 == (M)-2) return one / (a * a);
    return m_pow(a, s0);
  }
  else if constexpr (OP == THCB200_OP_TPOW) return m_pow(s0, a);
  else if constexpr (OP == THCB200_OP_ADD_S) return a + s0;
  else if constexpr (OP == THCB200_OP_SUB_S) return a - s0;
  else if constexpr (OP == THCB200_OP_MUL_S) return a * s0;
  else if constexpr (OP == THCB200_OP_DIV_S) return a / s0;      // TH divides; cutorch's x*(1/v) differs by <= 1 ulp
  else if constexpr (OP == THCB200_OP_LSHIFT_S) return a * s0;   // s0 = 2^v from the host
  else if constexpr (OP == THCB200_OP_RSHIFT_S) return a / s0;   // s0 = 2^v from the host
  else if constexpr (OP == THCB200_OP_FMOD_S) return m_fmod(a, s0);
  else if constexpr (OP == THCB200_OP_REMAINDER_S) return a - s0 * m_floor(a / s0);
  else if constexpr (OP == THCB200_OP_MAX_S) return (a > s0) ? a : s0;
  else if constexpr (OP == THCB200_OP_MIN_S) return (a < s0) ? a : s0;
  else if constexpr (OP == THCB200_OP_ADD) return a + b;
  else if constexpr (OP == THCB200_OP_SUB) return a - b;
  else if constexpr (OP == THCB200_OP_CADD) return a + s0 * b;
  else if constexpr (OP == THCB200_OP_MUL) return a * b;
  else if constexpr (OP == THCB200_OP_DIV) return a / b;
  else if constexpr (OP == THCB200_OP_CPOW) return m_pow(a, b);
  else if constexpr (OP == THCB200_OP_CLSHIFT) return a * m_pow((M)2, b);
  else if constexpr (OP == THCB200_OP_CRSHIFT) return a / m_pow((M)2, b);
  else if constexpr (OP == THCB200_OP_CMAX) return (a > b) ? a : b;
  else if constexpr (OP == THCB200_OP_CMIN) return (a < b) ? a : b;
  else if constexpr (OP == THCB200_OP_CFMOD) return m_fmod(a, b);
  else if constexpr (OP == THCB200_OP_CREMAINDER) return (b != (M)0) ? a - b * m_floor(a / b) : m_nan(a);
  else if constexpr (OP == THCB200_OP_ATAN2) return m_atan2(a, b);
  else if constexpr (OP == THCB200_OP_LERP) return a + s0 * (b - a);
  // TH writes r += value * src1 * src2: the scalar multiplies src1 first (cutorch: value * (src1 * src2))
  else if constexpr (OP == THCB200_OP_ADDCMUL) return a + (s0 * b) * c;
  else if constexpr (OP == THCB200_OP_LT_S) return (M)(a < s0);
  else if constexpr (OP == THCB200_OP_GT_S) return (M)(a > s0);
  else if constexpr (OP == THCB200_OP_LE_S) return (M)(a <= s0);
  else if constexpr (OP == THCB200_OP_GE_S) return (M)(a >= s0);
  else if constexpr (OP == THCB200_OP_EQ_S) return (M)(a == s0);
  else if constexpr (OP == THCB200_OP_NE_S) return (M)(a != s0);
  else if constexpr (OP == THCB200_OP_LT) return (M)(a < b);
  else if constexpr (OP == THCB200_OP_GT) return (M)(a > b);
  else if constexpr (OP == THCB200_OP_LE) return (M)(a <= b);
  else if constexpr (OP == THCB200_OP_GE) return (M)(a >= b);
  else if constexpr (OP == THCB200_OP_EQ) return (M)(a == b);
  else if constexpr (OP == THCB200_OP_NE) return (M)(a != b);
  else if constexpr (OP == THCB200_OP_ADDCDIV) return a + (s0 * b) / c;
  else return a;
}

// ---- integer element types ------------------------------------------------------------
// a ** b on integers.  TH evaluates pow() in double and converts back, which is exact for every
// result a double holds; repeated squaring gives those same values without depending on the
// last bits of a device pow().  Negative exponents follow 1 / a**|b| truncated toward zero.
template <typename I> __device__ __forceinline__ I int_pow(I a, I b) {
  using P = typename Promoted<I>::type;
  using U = typename WideU<P>::type;
  if (b < 0) {
    if (a == (I)1) return (I)1;
    if ((I)-1 < (I)0 && a == (I)-1) return (b & 1) ? (I)-1 : (I)1;
    return (I)0;
  }
  U base = (U)(P)a, r = 1;
  uint64_t e = (uint64_t)b;
  while (e) {
    if (e & 1) r *= base;
    base *= base;
    e >>= 1;
  }
  return (I)(P)r;
}

template <int OP, typename I>
__device__ __forceinline__ I int_apply(I s0, I s1, I a, I b, I c) {
  using P = typename Promoted<I>::type;  // arithmetic happens in P, the store truncates to I
  if constexpr (OP == THCB200_OP_FILL) return s0;
  else if constexpr (OP == THCB200_OP_COPY) return a;
  else if constexpr (OP == THCB200_OP_NEG) return (I)w_sub<P>((P)0, (P)a);
  else if constexpr (OP == THCB200_OP_ABS) {
    if constexpr (sizeof(I) == 1 && ((I)-1 > (I)0)) return a;  // byte: identity
    else return (I)((P)a < 0 ? w_sub<P>((P)0, (P)a) : (P)a);
  }
  else if constexpr (OP == THCB200_OP_SIGN) {
    if constexpr ((I)-1 > (I)0) return (I)(a == 0 ? 0 : 1);
    else return (I)((a > 0) - (a < 0));
  }
  else if constexpr (OP == THCB200_OP_CLAMP) return (a < s0) ? s0 : (a > s1 ? s1 : a);
  else if constexpr (OP == THCB200_OP_ADD_S) return (I)w_add<P>((P)a, (P)s0);
  else if constexpr (OP == THCB200_OP_SUB_S) return (I)w_sub<P>((P)a, (P)s0);
  else if constexpr (OP == THCB200_OP_MUL_S) return (I)w_mul<P>((P)a, (P)s0);
  else if constexpr (OP == THCB200_OP_DIV_S) return (I)((P)a / (P)s0);
  else if constexpr (OP == THCB200_OP_LSHIFT_S) return (I)((P)a << (P)s0);
  else if constexpr (OP == THCB200_OP_RSHIFT_S) return (I)((P)a >> (P)s0);
  else if constexpr (OP == THCB200_OP_FMOD_S) return (I)((P)a % (P)s0);
  else if constexpr (OP == THCB200_OP_REMAINDER_S) {
    P r = (P)a % (P)s0;
    if (w_mul<P>((P)(I)r, (P)s0) < 0) r = w_add<P>(r, (P)s0);
    return (I)r;
  }
  else if constexpr (OP == THCB200_OP_BITAND_S) return (I)(a & s0);
  else if constexpr (OP == THCB200_OP_BITOR_S) return (I)(a | s0);
  else if constexpr (OP == THCB200_OP_BITXOR_S) return (I)(a ^ s0);
  else if constexpr (OP == THCB200_OP_MAX_S) return (a > s0) ? a : s0;
  else if constexpr (OP == THCB200_OP_MIN_S) return (a < s0) ? a : s0;
  else if constexpr (OP == THCB200_OP_ADD) return (I)w_add<P>((P)a, (P)b);
  else if constexpr (OP == THCB200_OP_SUB) return (I)w_sub<P>((P)a, (P)b);
  else if constexpr (OP == THCB200_OP_CADD) return (I)w_add<P>((P)a, w_mul<P>((P)s0, (P)b));
  else if constexpr (OP == THCB200_OP_MUL) return (I)w_mul<P>((P)a, (P)b);
  else if constexpr (OP == THCB200_OP_DIV) return (I)((P)a / (P)b);
  else if constexpr (OP == THCB200_OP_CPOW) return int_pow<I>(a, b);
  else if constexpr (OP == THCB200_OP_CLSHIFT) return (I)((P)a << (P)b);
  else if constexpr (OP == THCB200_OP_CRSHIFT) return (I)((P)a >> (P)b);
  else if constexpr (OP == THCB200_OP_CMAX) return (a > b) ? a : b;
  else if constexpr (OP == THCB200_OP_CMIN) return (a < b) ? a : b;
  else if constexpr (OP == THCB200_OP_CFMOD) return (I)((P)a % (P)b);
  else if constexpr (OP == THCB200_OP_CREMAINDER) {
    P r = (P)a % (P)b;
    if (w_mul<P>((P)(I)r, (P)b) < 0) r = w_add<P>(r, (P)b);
    return (I)r;
  }
  else if constexpr (OP == THCB200_OP_CBITAND) return (I)(a & b);
  else if constexpr (OP == THCB200_OP_CBITOR) return (I)(a | b);
  else if constexpr (OP == THCB200_OP_CBITXOR) return (I)(a ^ b);
  else if constexpr (OP == THCB200_OP_ADDCMUL) return (I)w_add<P>((P)a, w_mul<P>((P)s0, w_mul<P>((P)b, (P)c)));
  else if constexpr (OP == THCB200_OP_LT_S) return (I)(a < s0);
  else if constexpr (OP == THCB200_OP_GT_S) return (I)(a > s0);
  else if constexpr (OP == THCB200_OP_LE_S) return (I)(a <= s0);
  else if constexpr (OP == THCB200_OP_GE_S) return (I)(a >= s0);
  else if constexpr (OP == THCB200_OP_EQ_S) return (I)(a == s0);
  else if constexpr (OP == THCB200_OP_NE_S) return (I)(a != s0);
  else if constexpr (OP == THCB200_OP_LT) return (I)(a < b);
  else if constexpr (OP == THCB200_OP_GT) return (I)(a > b);
  else if constexpr (OP == THCB200_OP_LE) return (I)(a <= b);
  else if constexpr (OP == THCB200_OP_GE) return (I)(a >= b);
  else if constexpr (OP == THCB200_OP_EQ) return (I)(a == b);
  else if constexpr (OP == THCB200_OP_NE) return (I)(a != b);
  else if constexpr (OP == THCB200_OP_ADDCDIV) return (I)w_add<P>((P)a, (P)(w_mul<P>((P)s0, (P)b) / (P)c));
  else return a;
}

// Half sigmoid.  The stored result keeps 11 significand bits, so the float evaluation can use the
// special-function unit's ex2 and rcp directly (each within 2 float ulp, i.e. 2^-22 relative): the
// rounded half equals the one obtained from expf and an IEEE division except where the float value
// lies within 2^-21 of a half rounding boundary, and differs by one half ulp there.  The exact
// forms cost about 20 issue slots per element, which holds a 2-byte stream below the HBM rate.
// Limits: ex2(+inf) = inf -> rcp = 0; ex2(-inf) = 0 -> 1; NaN stays NaN.
__device__ __forceinline__ float sigmoid_for_half(float a) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}

template <int OP, typename T>
__device__ __forceinline__ T pw_apply(const OpParams<T> &p, T a, T b, T c) {
  if constexpr (OP == THCB200_OP_SIGMOID && sizeof(T) == 2 && TypeTraits<T>::is_fp) {
    return from_math<T>(sigmoid_for_half(to_math<T>(a)));
  } else if constexpr (TypeTraits<T>::is_fp) {
    using M = typename TypeTraits<T>::Math;
    return from_math<T>(fp_apply<OP, M>(p.s0, p.s1, to_math<T>(a), to_math<T>(b), to_math<T>(c)));
  } else {
    return int_apply<OP, T>(p.s0, p.s1, a, b, c);
  }
}

}  // namespace thcb
