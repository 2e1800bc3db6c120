// Typed launch code of the pointwise apply: turns an ApplyPlan into a kernel launch for one
// element type.  One translation unit per element type instantiates pointwise_typed<T>.
#pragma once

#include "apply.cuh"
#include "context.h"
#include "plan.h"

namespace thcb {

template <typename T>
inline OpParams<T> make_params(int op, thcb200_scalar s0, thcb200_scalar s1) {
  using M = typename TypeTraits<T>::Math;
  OpParams<T> p;
  if constexpr (TypeTraits<T>::is_fp) {
    p.s0 = (M)s0.f;
    p.s1 = (M)s1.f;
    // x << v and x >> v on floating tensors scale by 2^v
    // (lib/THC/generic/THCTensorMathPairwise.cu:83-129); the power is taken once here.
    if (op == THCB200_OP_LSHIFT_S || op == THCB200_OP_RSHIFT_S) p.s0 = (M)pow((M)2, (M)s0.f);
  } else {
    p.s0 = (M)s0.i;
    p.s1 = (M)s1.i;
  }
  return p;
}

template <int OP, typename T, int NIN>
int launch_apply(thcb200_ctx *ctx, const ApplyPlan &plan, char *const data[4], OpParams<T> p,
                 cudaStream_t st) {
  T *out = reinterpret_cast<T *>(data[0]);
  const T *a = reinterpret_cast<const T *>(data[1]);
  const T *b = reinterpret_cast<const T *>(data[2]);
  const T *c = reinterpret_cast<const T *>(data[3]);
  const uint64_t n = plan.numel;
  switch (plan.kind) {
    case kApplyContigVec: {
      bool wide = true;   // 256-bit accesses need 32-byte alignment of every operand
      for (int o = 0; o <= NIN; ++o) if (((uintptr_t)data[o]) % 32 != 0) wide = false;
      const uint64_t tile = wide ? contig_tile<T, 32>() : contig_tile<T, 16>();
      const uint64_t blocks = (n + tile - 1) / tile;
      if (blocks >= (1ULL << 31)) { set_error("pointwise: tensor too large"); return THCB200_ERR_DIMS; }
      if (wide) {
        set_plan_name("contig_vec");
        launch_pdl(apply_contig_vec_kernel<OP, T, NIN, 32>, (unsigned)blocks, kApplyThreads, 0, st, out, a, b, c, n, p);
      } else {
        set_plan_name("contig_vec16");
        launch_pdl(apply_contig_vec_kernel<OP, T, NIN, 16>, (unsigned)blocks, kApplyThreads, 0, st, out, a, b, c, n, p);
      }
      break;
    }
    case kApplyTiled: {
      const TiledPlan &t = plan.tiled;
      uint64_t blocks = (uint64_t)t.tilesC * t.tilesJ;
      for (int i = 0; i < t.nouter; ++i) blocks *= t.outerSizes[i].d;
      const size_t smem = tiled_smem_bytes<T>(plan.tiled_slots);
      static thread_local int smem_set_for_device = -1;
      if (smem > 48 * 1024 && smem_set_for_device != ctx->device) {
        THCB_CUDA_TRY(cudaFuncSetAttribute(apply_tiled_kernel<OP, T, NIN>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)tiled_smem_bytes<T>(4)));
        smem_set_for_device = ctx->device;
      }
      set_plan_name("tiled");
      launch_pdl(apply_tiled_kernel<OP, T, NIN>, (unsigned)blocks, kTiledThreads, smem, st, out, a, b, c, t, p, plan.tiled_slots);
      break;
    }
    case kApplyRows: {
      const RowsPlan &r = plan.rows;
      const uint64_t rows_per_cta = (uint64_t)(kApplyThreads >> r.log2_tx) * kRowsUnroll;
      const uint64_t blocks = (uint64_t)r.tiles_c * (((uint64_t)r.R + rows_per_cta - 1) / rows_per_cta);
      if (r.vec) {
        set_plan_name("rows");
        launch_pdl(apply_rows_kernel<OP, T, NIN, 16 / (int)sizeof(T)>, (unsigned)blocks, kApplyThreads, 0, st, out, a, b, c, r, p);
      } else {
        set_plan_name("rows_scalar");
        launch_pdl(apply_rows_kernel<OP, T, NIN, 1>, (unsigned)blocks, kApplyThreads, 0, st, out, a, b, c, r, p);
      }
      break;
    }
    case kApplyGeneric: {
      const uint64_t tile = (uint64_t)kApplyThreads * kApplyUnroll;
      const uint64_t blocks = (n + tile - 1) / tile;
      if (blocks >= (1ULL << 31)) { set_error("pointwise: tensor too large"); return THCB200_ERR_DIMS; }
      if (!plan.index64) {
        set_plan_name("generic32");
        launch_pdl(apply_generic_kernel<OP, T, NIN, uint32_t>, (unsigned)blocks, kApplyThreads, 0, st, 
            out, to_strided_view<uint32_t>(plan, 0), a, to_strided_view<uint32_t>(plan, 1), b,
            to_strided_view<uint32_t>(plan, 2), c, to_strided_view<uint32_t>(plan, 3), (uint32_t)n, p);
      } else {
        set_plan_name("generic64");
        launch_pdl(apply_generic_kernel<OP, T, NIN, uint64_t>, (unsigned)blocks, kApplyThreads, 0, st, 
            out, to_strided_view<uint64_t>(plan, 0), a, to_strided_view<uint64_t>(plan, 1), b,
            to_strided_view<uint64_t>(plan, 2), c, to_strided_view<uint64_t>(plan, 3), (uint64_t)n, p);
      }
      break;
    }
    default:
      set_error("pointwise: internal error, unexpected plan kind");
      return THCB200_ERR_ARG;
  }
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

#define THCB_CASE(OPNAME, NIN) \
  case OPNAME: return launch_apply<OPNAME, T, NIN>(ctx, plan, data, p, st);

template <typename T>
int pointwise_typed(thcb200_ctx *ctx, int op, const ApplyPlan &plan, char *const data[4],
                    thcb200_scalar s0, thcb200_scalar s1, cudaStream_t st) {
  OpParams<T> p = make_params<T>(op, s0, s1);
  constexpr bool fp = TypeTraits<T>::is_fp;
  constexpr bool is_half = TypeTraits<T>::dtype == THCB200_F16;
  constexpr bool has_neg = TypeTraits<T>::dtype != THCB200_U8 && TypeTraits<T>::dtype != THCB200_I8;
  switch (op) {
    THCB_CASE(THCB200_OP_FILL, 0)
    THCB_CASE(THCB200_OP_COPY, 1)
    THCB_CASE(THCB200_OP_ABS, 1)
    THCB_CASE(THCB200_OP_SIGN, 1)
    THCB_CASE(THCB200_OP_CLAMP, 1)
    THCB_CASE(THCB200_OP_ADD_S, 1)
    THCB_CASE(THCB200_OP_SUB_S, 1)
    THCB_CASE(THCB200_OP_MUL_S, 1)
    THCB_CASE(THCB200_OP_DIV_S, 1)
    THCB_CASE(THCB200_OP_FMOD_S, 1)
    THCB_CASE(THCB200_OP_REMAINDER_S, 1)
    THCB_CASE(THCB200_OP_MAX_S, 1)
    THCB_CASE(THCB200_OP_MIN_S, 1)
    THCB_CASE(THCB200_OP_LT_S, 1)
    THCB_CASE(THCB200_OP_GT_S, 1)
    THCB_CASE(THCB200_OP_LE_S, 1)
    THCB_CASE(THCB200_OP_GE_S, 1)
    THCB_CASE(THCB200_OP_EQ_S, 1)
    THCB_CASE(THCB200_OP_NE_S, 1)
    THCB_CASE(THCB200_OP_LT, 2)
    THCB_CASE(THCB200_OP_GT, 2)
    THCB_CASE(THCB200_OP_LE, 2)
    THCB_CASE(THCB200_OP_GE, 2)
    THCB_CASE(THCB200_OP_EQ, 2)
    THCB_CASE(THCB200_OP_NE, 2)
    THCB_CASE(THCB200_OP_ADD, 2)
    THCB_CASE(THCB200_OP_SUB, 2)
    THCB_CASE(THCB200_OP_CADD, 2)
    THCB_CASE(THCB200_OP_MUL, 2)
    THCB_CASE(THCB200_OP_DIV, 2)
    THCB_CASE(THCB200_OP_CPOW, 2)
    THCB_CASE(THCB200_OP_CMAX, 2)
    THCB_CASE(THCB200_OP_CMIN, 2)
    THCB_CASE(THCB200_OP_CFMOD, 2)
    THCB_CASE(THCB200_OP_CREMAINDER, 2)
    THCB_CASE(THCB200_OP_ADDCMUL, 3)
    THCB_CASE(THCB200_OP_ADDCDIV, 3)
    default: break;
  }
  if constexpr (has_neg) {
    switch (op) {
      THCB_CASE(THCB200_OP_NEG, 1)
      default: break;
    }
  }
  if constexpr (!is_half) {
    switch (op) {
      THCB_CASE(THCB200_OP_LSHIFT_S, 1)
      THCB_CASE(THCB200_OP_RSHIFT_S, 1)
      THCB_CASE(THCB200_OP_CLSHIFT, 2)
      THCB_CASE(THCB200_OP_CRSHIFT, 2)
      default: break;
    }
  }
  if constexpr (!fp) {
    switch (op) {
      THCB_CASE(THCB200_OP_BITAND_S, 1)
      THCB_CASE(THCB200_OP_BITOR_S, 1)
      THCB_CASE(THCB200_OP_BITXOR_S, 1)
      THCB_CASE(THCB200_OP_CBITAND, 2)
      THCB_CASE(THCB200_OP_CBITOR, 2)
      THCB_CASE(THCB200_OP_CBITXOR, 2)
      default: break;
    }
  } else {
    switch (op) {
      THCB_CASE(THCB200_OP_LOG, 1)
      THCB_CASE(THCB200_OP_LGAMMA, 1)
      THCB_CASE(THCB200_OP_LOG1P, 1)
      THCB_CASE(THCB200_OP_EXP, 1)
      THCB_CASE(THCB200_OP_COS, 1)
      THCB_CASE(THCB200_OP_SIN, 1)
      THCB_CASE(THCB200_OP_SQRT, 1)
      THCB_CASE(THCB200_OP_RSQRT, 1)
      THCB_CASE(THCB200_OP_CEIL, 1)
      THCB_CASE(THCB200_OP_FLOOR, 1)
      THCB_CASE(THCB200_OP_TRUNC, 1)
      THCB_CASE(THCB200_OP_ACOS, 1)
      THCB_CASE(THCB200_OP_COSH, 1)
      THCB_CASE(THCB200_OP_ASIN, 1)
      THCB_CASE(THCB200_OP_SINH, 1)
      THCB_CASE(THCB200_OP_TAN, 1)
      THCB_CASE(THCB200_OP_ATAN, 1)
      THCB_CASE(THCB200_OP_TANH, 1)
      THCB_CASE(THCB200_OP_ROUND, 1)
      THCB_CASE(THCB200_OP_FRAC, 1)
      THCB_CASE(THCB200_OP_CINV, 1)
      THCB_CASE(THCB200_OP_SIGMOID, 1)
      THCB_CASE(THCB200_OP_POW, 1)
      THCB_CASE(THCB200_OP_TPOW, 1)
      THCB_CASE(THCB200_OP_ATAN2, 2)
      THCB_CASE(THCB200_OP_LERP, 2)
      default: break;
    }
  }
  set_error("pointwise: op %d is not defined for dtype %d", op, TypeTraits<T>::dtype);
  return THCB200_ERR_UNSUPPORTED;
}
#undef THCB_CASE

// one definition per element type, each in its own translation unit
int pointwise_u8(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
int pointwise_i8(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
int pointwise_i16(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
int pointwise_i32(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
int pointwise_i64(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
int pointwise_f16(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
int pointwise_f32(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
int pointwise_f64(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);

}  // namespace thcb
