/*
 * thcb200.h -- descriptor-level C ABI of the B200 strided-tensor apply / reduce core.
 *
 * This is the thin boundary between host code (C, C++, Lua FFI, ctypes ...) and the
 * hand-written sm_100a kernels.  Every entry point takes plain pointers and sizes; no
 * C++ or framework types cross it.  The THC-compatible C API (include/THC/THC.h:
 * THCudaTensor_cadd, THCudaTensor_sumall, ...) is implemented on top of these calls.
 *
 * Reference interfaces replaced (paths inside the cutorch tree):
 *   thcb200_pointwise        <- THC_pointwiseApply1/2/3      lib/THC/THCApply.cuh:124-640
 *   thcb200_reduce_dim       <- THC_reduceDim                lib/THC/THCReduce.cuh:258-453
 *   thcb200_reduce_dim_index <- THC_reduceDimIndex           lib/THC/THCTensorMathReduce.cuh:619-661
 *   thcb200_reduce_all       <- THC_reduceAll                lib/THC/THCReduceAll.cuh:234-342
 *   thcb200_collapse_dims    <- TensorInfo::collapseDims     lib/THC/THCTensorInfo.cuh:74-224
 *   thcb200_overlapping      <- TensorUtils::overlappingIndices  lib/THC/THCTensorTypeUtils.cu:163-218
 *   thcb200_can_use_32bit    <- TensorUtils::canUse32BitIndexMath lib/THC/THCTensorTypeUtils.cu:220-245
 *
 * All functions return 0 on success or a negative thcb200_status; the message of the
 * last failure on the calling thread is available from thcb200_last_error().
 * Kernels are launched asynchronously on the given stream unless stated otherwise.
 */
#ifndef THCB200_H
#define THCB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define THCB200_API __attribute__((visibility("default")))
#else
#define THCB200_API
#endif

#define THCB200_MAX_DIMS 25 /* MAX_CUTORCH_DIMS, lib/THC/THCTensorInfo.cuh:10 */

typedef enum thcb200_status {
  THCB200_OK = 0,
  THCB200_ERR_ARG = -1,        /* bad argument (dtype/op combination, null pointer ...) */
  THCB200_ERR_DIMS = -2,       /* more than THCB200_MAX_DIMS dimensions */
  THCB200_ERR_SIZE = -3,       /* element counts of the operands differ */
  THCB200_ERR_CUDA = -4,       /* a CUDA runtime call failed */
  THCB200_ERR_UNSUPPORTED = -5,/* op is not defined for this dtype (e.g. bit ops on float) */
  THCB200_ERR_NOMEM = -6,      /* workspace allocation failed */
  THCB200_ERR_LIMIT = -7       /* size beyond a documented fixed limit */
} thcb200_status;

/* Element types, in the order of cutorch's eight tensor types. */
typedef enum thcb200_dtype {
  THCB200_U8 = 0,  /* THCudaByteTensor   */
  THCB200_I8 = 1,  /* THCudaCharTensor   */
  THCB200_I16 = 2, /* THCudaShortTensor  */
  THCB200_I32 = 3, /* THCudaIntTensor    */
  THCB200_I64 = 4, /* THCudaLongTensor   */
  THCB200_F16 = 5, /* THCudaHalfTensor   */
  THCB200_F32 = 6, /* THCudaTensor       */
  THCB200_F64 = 7  /* THCudaDoubleTensor */
} thcb200_dtype;

/* A strided view: `data` already includes the storage offset; strides are in elements. */
typedef struct thcb200_tensor {
  void *data;
  int32_t dtype;
  int32_t ndim;
  int64_t sizes[THCB200_MAX_DIMS];
  int64_t strides[THCB200_MAX_DIMS];
} thcb200_tensor;

/* A scalar argument: the caller fills both views of the value (f is used by the
 * floating-point element types, i by the integer ones). */
typedef struct thcb200_scalar {
  double f;
  int64_t i;
} thcb200_scalar;

/* Pointwise operations.  out = f(in0[, in1[, in2]]; s0, s1).  In-place use passes the
 * same view as `out` and `in0`. */
typedef enum thcb200_op {
  /* no input */
  THCB200_OP_FILL = 0,       /* out = s0 */
  /* one input, no scalar */
  THCB200_OP_COPY,           /* out = in0 (same dtype) */
  THCB200_OP_LOG, THCB200_OP_LGAMMA, THCB200_OP_LOG1P, THCB200_OP_EXP, THCB200_OP_COS,
  THCB200_OP_SIN, THCB200_OP_SQRT, THCB200_OP_RSQRT, THCB200_OP_CEIL, THCB200_OP_FLOOR,
  THCB200_OP_TRUNC, THCB200_OP_ACOS, THCB200_OP_COSH, THCB200_OP_ASIN, THCB200_OP_SINH,
  THCB200_OP_TAN, THCB200_OP_ATAN, THCB200_OP_TANH, THCB200_OP_ROUND, THCB200_OP_FRAC,
  THCB200_OP_CINV, THCB200_OP_NEG, THCB200_OP_ABS, THCB200_OP_SIGN, THCB200_OP_SIGMOID,
  /* one input, scalar(s) */
  THCB200_OP_CLAMP,          /* s0 = min, s1 = max */
  THCB200_OP_POW,            /* in0 ** s0 (special cases 1, 2, 3, -1, -2) */
  THCB200_OP_TPOW,           /* s0 ** in0 */
  THCB200_OP_ADD_S, THCB200_OP_SUB_S, THCB200_OP_MUL_S,
  THCB200_OP_DIV_S,          /* in0 / s0: a true division as in TH (cutorch multiplies by 1/s0) */
  THCB200_OP_LSHIFT_S, THCB200_OP_RSHIFT_S, THCB200_OP_FMOD_S, THCB200_OP_REMAINDER_S,
  THCB200_OP_BITAND_S, THCB200_OP_BITOR_S, THCB200_OP_BITXOR_S,
  THCB200_OP_MAX_S, THCB200_OP_MIN_S,
  /* comparisons with s0, result 1 or 0 in the element type (lib/THC/THCTensorMathCompare.cuh) */
  THCB200_OP_LT_S, THCB200_OP_GT_S, THCB200_OP_LE_S, THCB200_OP_GE_S, THCB200_OP_EQ_S, THCB200_OP_NE_S,
  /* two inputs */
  THCB200_OP_ADD,            /* in0 + in1 */
  THCB200_OP_SUB,            /* in0 - in1 */
  THCB200_OP_CADD,           /* in0 + s0 * in1 (not contracted to an FMA) */
  THCB200_OP_MUL, THCB200_OP_DIV, THCB200_OP_CPOW, THCB200_OP_CLSHIFT, THCB200_OP_CRSHIFT,
  THCB200_OP_CMAX, THCB200_OP_CMIN, THCB200_OP_CFMOD, THCB200_OP_CREMAINDER,
  THCB200_OP_CBITAND, THCB200_OP_CBITOR, THCB200_OP_CBITXOR, THCB200_OP_ATAN2,
  THCB200_OP_LERP,           /* in0 + s0 * (in1 - in0) */
  /* element-wise comparisons, result 1 or 0 in the element type (lib/THC/THCTensorMathCompareT.cuh) */
  THCB200_OP_LT, THCB200_OP_GT, THCB200_OP_LE, THCB200_OP_GE, THCB200_OP_EQ, THCB200_OP_NE,
  /* three inputs */
  THCB200_OP_ADDCMUL,        /* in0 + (s0 * in1) * in2, TH's association */
  THCB200_OP_ADDCDIV,        /* in0 + (s0 * in1) / in2 */
  THCB200_OP_COUNT
} thcb200_op;

/* Fold operators of the reductions. */
typedef enum thcb200_reduce_op {
  THCB200_RED_SUM = 0,
  THCB200_RED_PROD = 1,
  THCB200_RED_MIN = 2,  /* TH rule: a NaN element wins */
  THCB200_RED_MAX = 3,
  THCB200_RED_ALL = 4,  /* logical and of (x != 0), result 0/1 */
  THCB200_RED_ANY = 5,
  THCB200_RED_COUNT
} thcb200_reduce_op;

/* Per-element transform applied before the fold (modifyOp of THC_reduceDim). */
typedef enum thcb200_pre_op {
  THCB200_PRE_IDENTITY = 0,
  THCB200_PRE_ABS = 1,      /* norm p = 1 */
  THCB200_PRE_SQUARE = 2,   /* norm p = 2 */
  THCB200_PRE_POWABS = 3,   /* |x| ** s   (norm p) */
  THCB200_PRE_NONZERO = 4,  /* x != 0 ? 1 : 0 (norm p = 0) */
  THCB200_PRE_SQDEV = 5,    /* (x - s) ** 2 (varall) */
  THCB200_PRE_MOMENTS = 6,  /* running sums of x and x*x; only with a THCB200_POST_VAR_* / _STD_* step */
  THCB200_PRE_COUNT
} thcb200_pre_op;

/* Opaque context of one device: the reduction workspace (per-block partials, tickets),
 * a pinned, mapped host slot that kernels store host-bound results into, and cached device
 * properties.  It replaces the scratch-space services of THCState, which are kept per device and
 * per stream there (lib/THC/THCGeneral.c:563-590, 677-712).
 *   Streams: the scratch is reused from call to call, which is safe in the order of one stream;
 *   give every stream whose work may overlap another's a context of its own (the THC layer keeps
 *   one per device and stream that has been current).
 *   Threads: several host threads may call into one context; the calls that use its scratch are
 *   serialised by a lock inside it, including the wait for a result returned to the host. */
typedef struct thcb200_ctx thcb200_ctx;

THCB200_API int thcb200_ctx_create(thcb200_ctx **out, int device);
THCB200_API void thcb200_ctx_destroy(thcb200_ctx *ctx);
/* The context's scratch buffer on its device, grown to at least `min_bytes` (256-byte aligned;
 * *bytes receives its size).  The reductions use it for their partials, so its contents are
 * only stable between calls on the context; NULL when it cannot be allocated.  It stands for
 * THCState_getCurrentDeviceScratchSpace (lib/THC/THCGeneral.c:677-712). */
THCB200_API void *thcb200_ctx_workspace(thcb200_ctx *ctx, size_t min_bytes, size_t *bytes);
THCB200_API const char *thcb200_last_error(void);
/* Failure injection for tests: the nth device allocation the library makes for itself from now on
 * (workspace growth, mask offsets, dense temporaries, gather buffers) fails as if the GPU were out
 * of memory, without any CUDA call; 0 disarms.  The call that hits it returns THCB200_ERR_NOMEM and
 * leaves its context usable.  cutorch reports a failed allocation through THCudaCheck / THError
 * (lib/THC/THCGeneral.c:714-726, 842-854); nothing in its tree injects one. */
THCB200_API void thcb200_debug_fail_allocation(int nth);
/* Number of kernels this library has launched in this process (all contexts). */
THCB200_API int64_t thcb200_launch_count(void);
/* Name of the kernel family picked by the most recent pointwise / reduce call of this
 * thread ("contig_vec", "tiled", "generic", "row_warp", "col_tile", ...). */
THCB200_API const char *thcb200_last_plan(void);

/* Plain synchronous copies between host and device memory (cudaMemcpyAsync on `stream`
 * followed by a stream synchronize); for hosts that have no CUDA binding of their own. */
THCB200_API int thcb200_memcpy_h2d(void *dst_dev, const void *src_host, size_t bytes, void *stream);
THCB200_API int thcb200_memcpy_d2h(void *dst_host, const void *src_dev, size_t bytes, void *stream);
THCB200_API int thcb200_stream_synchronize(void *stream);

/* ---- host-side layout helpers (no GPU work) -------------------------------------- */

/* In-place TensorInfo::collapseDims.  Returns the new index of exclude_dim (or -1). */
THCB200_API int thcb200_collapse_dims(int64_t *sizes, int64_t *strides, int *ndim, int exclude_dim);
/* 1 if two distinct index tuples of the view address the same element. */
THCB200_API int thcb200_overlapping(const thcb200_tensor *t);
/* 1 if element count and largest offset both fit 32-bit unsigned arithmetic. */
/* The smallest and largest element offset (relative to `data`) that the view can reach: the sums
 * of (size - 1) * stride over the dims with negative and with positive strides, as
 * TensorUtils::canUse32BitIndexMath computes the largest (lib/THC/THCTensorTypeUtils.cu:220-245).
 * Returns 1 and fills the outputs, 0 for a view without elements, a negative status for a bad
 * descriptor.  thcb200_check_extent refuses (THCB200_ERR_SIZE) a view that reaches more than
 * `elements_before` elements in front of `data` or more than `elements_after` behind it: the check
 * a caller who knows the allocation runs before handing the view to a kernel (the THC layer runs
 * it against the storage's size on every call; cutorch asserts inside its kernels instead,
 * lib/THC/THCTensorInfo.cuh:228-278). */
THCB200_API int thcb200_view_extent(const thcb200_tensor *t, int64_t *min_offset, int64_t *max_offset);
THCB200_API int thcb200_check_extent(const thcb200_tensor *t, int64_t elements_before, int64_t elements_after);
THCB200_API int thcb200_can_use_32bit(const thcb200_tensor *t);
/* Element offset of logical (row-major) index `linear` in the view. */
THCB200_API int64_t thcb200_index_to_offset(const thcb200_tensor *t, int64_t linear);

/* Name of the kernel family thcb200_pointwise would pick for these views ("contig_vec",
 * "contig_vec16", "tiled", "rows", "rows_scalar", "generic32", "generic64", "deep"), without
 * launching anything: the planner is host code.  NULL (and thcb200_last_error) on bad views. */
THCB200_API const char *thcb200_pointwise_plan(const thcb200_tensor *out, const thcb200_tensor *in0,
                                   const thcb200_tensor *in1, const thcb200_tensor *in2, int nin);

/* ---- device work ----------------------------------------------------------------- */

/* out = op(in...).  Operands need equal element counts, not equal shapes; each is
 * walked in its own row-major order.  nin must match the op's arity. */
THCB200_API int thcb200_pointwise(thcb200_ctx *ctx, int op, const thcb200_tensor *out,
                      const thcb200_tensor *in0, const thcb200_tensor *in1,
                      const thcb200_tensor *in2, int nin, thcb200_scalar s0,
                      thcb200_scalar s1, void *stream);

/* Same with flags.  THCB200_FLAG_IGNORE_OVERLAP writes through an output view whose index
 * tuples alias without the dense temporary (copyIgnoringOverlaps,
 * lib/THC/THCTensorCopy.cu:24-205). */
#define THCB200_FLAG_IGNORE_OVERLAP 1
THCB200_API int thcb200_pointwise_ex(thcb200_ctx *ctx, int op, const thcb200_tensor *out,
                         const thcb200_tensor *in0, const thcb200_tensor *in1,
                         const thcb200_tensor *in2, int nin, thcb200_scalar s0,
                         thcb200_scalar s1, void *stream, int flags);

/* out = convert(in): element-wise copy between any two dtypes (C cast semantics; half
 * goes through float).  lib/THC/THCTensorCopy.cu:12-21,114-121. */
THCB200_API int thcb200_copy_convert(thcb200_ctx *ctx, const thcb200_tensor *out,
                         const thcb200_tensor *in, void *stream);

/* Fold `in` along `dim`.  `out` has in's sizes with sizes[dim] == 1 and in's dtype;
 * accumulation is in double (f32, f64), float (f16) or int64 (integers). */
THCB200_API int thcb200_reduce_dim(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s,
                       const thcb200_tensor *out, const thcb200_tensor *in, int dim,
                       void *stream);

/* thcb200_reduce_dim followed, inside the same kernel, by the second call cutorch composes
 * some entry points from: mean = sum then div by the length of the dim
 * (lib/THC/generic/THCTensorMathReduce.cu:37-43), norm = fold then pow (:160-187).  The fold is
 * rounded to the element type first, then the step is applied in the element's math type and
 * rounded again, so the values are those of the two-call form. */
typedef enum thcb200_post_op {
  THCB200_POST_NONE = 0,
  THCB200_POST_DIV = 1,   /* out = fold / post_value */
  THCB200_POST_POW = 2,   /* out = fold ** post_value (floating types) */
  /* var / std along the dim from the sums of x and x*x (pre = THCB200_PRE_MOMENTS), in the
   * accumulate type: E[x^2] - E[x]^2, with the n/(n-1) correction when unbiased, clamped at 0
   * (lib/THC/THCTensorMathReduce.cuh:269-306, generic/THCTensorMathReduce.cu:76-126) */
  THCB200_POST_VAR_BIASED = 3, THCB200_POST_VAR_UNBIASED = 4,
  THCB200_POST_STD_BIASED = 5, THCB200_POST_STD_UNBIASED = 6
} thcb200_post_op;
THCB200_API int thcb200_reduce_dim_post(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s,
                            int post_kind, thcb200_scalar post_value, const thcb200_tensor *out,
                            const thcb200_tensor *in, int dim, void *stream);

/* thcb200_reduce_dim for callers that cannot allocate device memory when they call it (their
 * memory pool owns the whole device, their plug-in contract forbids allocations after start-up,
 * or they cannot take the synchronisation an allocation may imply).  It has no counterpart in
 * cutorch.  Same arguments minus the context, same kernels and results; the partials of split
 * reductions live in a static device array of THCB200_STATIC_SCRATCH_BYTES that every GPU
 * holding this library keeps until the process exits, and the call performs no cudaMalloc,
 * cudaFree or other allocating call.  A reduction whose partials exceed the array returns
 * THCB200_ERR_LIMIT.  The first call on each device resolves the array's device address: make
 * it outside any stream capture.  All calls on a device share the array: do not let two of them
 * overlap on the GPU. */
#define THCB200_STATIC_SCRATCH_BYTES (2u << 20)
THCB200_API int thcb200_reduce_dim_static(int rop, int pre, thcb200_scalar s,
                              const thcb200_tensor *out, const thcb200_tensor *in, int dim,
                              void *stream);

/* max / min along `dim` with 1-based int64 positions of the first occurrence (a NaN
 * counts as the extreme value).  `indices` is an I64 view shaped like `values`. */
THCB200_API int thcb200_reduce_dim_index(thcb200_ctx *ctx, int rop, const thcb200_tensor *values,
                             const thcb200_tensor *indices, const thcb200_tensor *in,
                             int dim, void *stream);

/* Fold every element of `in`.  The result is written to `result_dev` (8-byte aligned
 * device memory, 8 bytes) as a double for the floating element types and as an int64 for
 * the integer ones, whatever the fold.  Accumulation is in double (f32, f64), float (f16)
 * or int64.  One launch, fixed combine order, no atomics on data: repeatable bit for bit. */
THCB200_API int thcb200_reduce_all(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s,
                       const thcb200_tensor *in, void *result_dev, void *stream);

/* Same, then waits for the stream and stores the accumulator in *result_host (8 bytes,
 * same typing as above). */
THCB200_API int thcb200_reduce_all_host(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s,
                            const thcb200_tensor *in, void *result_host, void *stream);

/* Inclusive scan along `dim`: out[.., k, ..] = in[.., 0, ..] (+|*) ... (+|*) in[.., k, ..]
 * with rop = THCB200_RED_SUM (cumsum) or THCB200_RED_PROD (cumprod).  `out` has in's shape and
 * dtype (any strides; out == in scans in place).  The running value is kept in the accumulate
 * type of the reductions and rounded to the element type for every output.
 * THCTensor_(scanDim): lib/THC/generic/THCTensorMathScan.cu:76-118, kernels
 * lib/THC/THCTensorMathScan.cu:24-126. */
THCB200_API int thcb200_scan_dim(thcb200_ctx *ctx, int rop, const thcb200_tensor *out,
                     const thcb200_tensor *in, int dim, void *stream);

/* Lower (upper = 0: keep c - r <= k) or upper (upper = 1: keep c - r >= k) triangle of a 2-D
 * view; the other elements of `out` become 0.  out == in works in place.
 * lib/THC/generic/THCTensorMathPairwise.cu:169-233, TensorTriOp lib/THC/THCTensorMathPairwise.cu:373-406. */
THCB200_API int thcb200_tri(thcb200_ctx *ctx, int upper, int64_t k, const thcb200_tensor *out,
                const thcb200_tensor *in, void *stream);

/* factors[i] = n > maxnorm ? maxnorm / (n + 1e-7) : 1 with n = sums[i] ** (1/p): the scalar step
 * of renorm between the per-slice sums of |x|^p (thcb200_reduce_dim with THCB200_PRE_POWABS ...)
 * and the broadcast multiply.  Dense F32 or F64 operands.
 * lib/THC/THCTensorMathReduce.cuh:160-183 (THCTensor_kernel_renorm, clip step). */
THCB200_API int thcb200_renorm_factor(thcb200_ctx *ctx, const thcb200_tensor *factors,
                          const thcb200_tensor *sums, double p, double maxnorm, void *stream);

/* renorm in one pass: every slice in.select(dim, j) whose p-norm exceeds maxnorm is written to
 * out scaled by maxnorm / (norm + 1e-7), every other slice is copied.  Taken only when each slice
 * of both views is one dense, 16-byte aligned run of at most 2048 16-byte vectors (a warp or a
 * CTA holds it in registers between the fold and the scaling); any other layout returns
 * THCB200_ERR_UNSUPPORTED before anything is launched, and the caller composes renorm from
 * thcb200_reduce_dim, thcb200_renorm_factor and a broadcast multiply.  F16 (computed as float,
 * rounded once), F32, F64; out == in works in place.
 * lib/THC/generic/THCTensorMathReduce.cu:47-74, lib/THC/THCTensorMathReduce.cuh:132-183. */
THCB200_API int thcb200_renorm_rows(thcb200_ctx *ctx, const thcb200_tensor *out, const thcb200_tensor *in,
                        int dim, double p, double maxnorm, void *stream);

/* Copies between a view in HOST memory (`src_host` / `dst_host`: the data pointer is a host
 * address, pageable or pinned; no negative strides) and a view in device memory, converting the
 * element type like thcb200_copy_convert and walking both sides in logical order.  A dense host
 * side crosses the bus as it is; otherwise its runs are packed on the host first.  Striding on the
 * device side and the conversion run on the GPU.  Both return when the copy is complete.
 * THCTensor_(copy<Type>) / TH<Type>Tensor_copyCuda<Real>: lib/THC/generic/THCTensorCopy.c:7-164. */
THCB200_API int thcb200_copy_from_host(thcb200_ctx *ctx, const thcb200_tensor *dst,
                           const thcb200_tensor *src_host, void *stream);
THCB200_API int thcb200_copy_to_host(thcb200_ctx *ctx, const thcb200_tensor *dst_host,
                         const thcb200_tensor *src, void *stream);

/* ---- indexed moves along one dim ------------------------------------------------------- */

/* For every coordinate tuple c of the iteration space, p = index value (1-based), and c' = c with
 * c'[dim] = p - 1:
 *   GATHER        dst[c]  = src[c']      iteration space: dst's shape
 *   SCATTER       dst[c'] = src[c]       iteration space: src's shape
 *   SCATTER_ADD   dst[c'] += src[c]      (atomic; duplicates accumulate in no fixed order)
 *   SCATTER_FILL  dst[c'] = value        iteration space: the index's shape (index_is_vector: dst's
 *                                        shape with the indexed dim as long as the vector)
 * `index` is an I64 view of the iteration space's shape, read at c; with index_is_vector it is a
 * 1-D view read at c[dim].  That covers gather / scatter / scatterAdd / scatterFill
 * (lib/THC/generic/THCTensorScatterGather.cu:8-351) and, with a vector, indexSelect (GATHER),
 * indexCopy (SCATTER), indexAdd (SCATTER_ADD) and indexFill (SCATTER_FILL)
 * (lib/THC/generic/THCTensorIndex.cu:14-589).  Positions outside 1..size[dim] are skipped and
 * counted (see thcb200_take_index_errors) instead of asserting on the device. */
typedef enum thcb200_index_mode {
  THCB200_INDEX_GATHER = 0,
  THCB200_INDEX_SCATTER = 1,
  THCB200_INDEX_SCATTER_ADD = 2,
  THCB200_INDEX_SCATTER_FILL = 3
} thcb200_index_mode;
THCB200_API int thcb200_indexed(thcb200_ctx *ctx, int mode, const thcb200_tensor *dst,
                    const thcb200_tensor *src, const thcb200_tensor *index, int dim,
                    int index_is_vector, thcb200_scalar value, void *stream);
/* Number of out-of-range positions skipped by thcb200_indexed on this context since the last
 * call of this function; waits for the stream. */
THCB200_API int thcb200_take_index_errors(thcb200_ctx *ctx, int64_t *count_host, void *stream);

/* ---- operands of two element types: comparisons into Byte, Byte masks ------------------ */

/* out[i] = (a[i] CMP b[i]) ? 1 : 0 with `out` a U8 view; `cmp` is one of THCB200_OP_LT..NE.
 * With b == NULL the right-hand side is the scalar `s` (THCB200_OP_LT_S..NE_S are accepted
 * too).  Equal element counts, each operand walked in its own row-major order.
 * THC_logicalValue / THC_logicalTensor with a ByteTensor result:
 * lib/THC/THCTensorMathCompare.cuh:5-85, THCTensorMathCompareT.cuh:5-72,
 * generic/THCTensorMathCompare.cu:5-99 (ltValue ...), generic/THCTensorMathCompareT.cu:5-111. */
THCB200_API int thcb200_compare(thcb200_ctx *ctx, int cmp, const thcb200_tensor *out_u8,
                    const thcb200_tensor *a, const thcb200_tensor *b, thcb200_scalar s,
                    void *stream);

/* t[i] = value where mask[i] != 0 (mask: U8, same element count).
 * lib/THC/generic/THCTensorMasked.cu:5-19, THCTensorMasked.cuh:16-26. */
THCB200_API int thcb200_masked_fill(thcb200_ctx *ctx, const thcb200_tensor *t,
                        const thcb200_tensor *mask_u8, thcb200_scalar value, void *stream);

/* Number of non-zero mask elements, written as int64 to *count_host after a stream
 * synchronize (the count the reference takes with sumall before maskedCopy / maskedSelect,
 * lib/THC/generic/THCTensorMasked.cu:52,128).  The per-tile positions computed on the way stay
 * in the context; a following masked_copy / masked_select on the same mask view and stream may
 * reuse them by passing THCB200_FLAG_MASK_COUNTED, which asserts that the mask's contents have
 * not changed in between.  On such a reuse the count is known on the host, and a packed side
 * (the output of masked_select / mask_coords, the source of masked_copy) that is too short for it
 * is refused with THCB200_ERR_SIZE; without the reuse sizing that operand is the caller's job. */
#define THCB200_FLAG_MASK_COUNTED 2
THCB200_API int thcb200_masked_count(thcb200_ctx *ctx, const thcb200_tensor *mask_u8,
                         int64_t *count_host, void *stream);

/* t[i] = src[k] where mask[i] != 0, k = number of non-zero mask elements before logical
 * position i; src is walked in its own row-major order and must hold at least that many
 * elements (checked by the caller through thcb200_masked_count).
 * lib/THC/generic/THCTensorMasked.cu:35-104, THCTensorMasked.cuh:28-42. */
THCB200_API int thcb200_masked_copy(thcb200_ctx *ctx, const thcb200_tensor *t,
                        const thcb200_tensor *mask_u8, const thcb200_tensor *src, void *stream,
                        int flags);

/* out[k] = src[i] for every i with mask[i] != 0, in logical order; `out` is walked in its own
 * row-major order and must hold at least thcb200_masked_count elements.
 * lib/THC/generic/THCTensorMasked.cu:119-177, THCTensorMasked.cuh:44-56. */
THCB200_API int thcb200_masked_select(thcb200_ctx *ctx, const thcb200_tensor *out,
                          const thcb200_tensor *src, const thcb200_tensor *mask_u8, void *stream,
                          int flags);

/* For every set element of a dense mask, in order, its 1-based coordinates in a tensor of the given
 * sizes (their product is the mask's element count): row r of the dense I64 output [count, nd]
 * holds the coordinates of the r-th set element.  The count comes from thcb200_masked_count; with
 * THCB200_FLAG_MASK_COUNTED the tile offsets of that call are reused.  This is the second half of
 * nonzero (lib/THC/generic/THCTensorMath.cu:262-356); the first half is a comparison with zero. */
THCB200_API int thcb200_mask_coords(thcb200_ctx *ctx, const thcb200_tensor *out_i64,
                        const thcb200_tensor *mask_u8, const int64_t *sizes, int nd,
                        void *stream, int flags);

/* ---- sharded reductions: one rank per GPU of a box, NCCL over NVLink ---------------------
 *
 * cutorch drives several GPUs from one process and has no collective layer
 * (lib/THC/THCGeneral.h.in:57-123); these calls are what a tensor split by rows over several
 * GPUs needs on top of the per-device ones.  A communicator is NCCL's: one rank calls
 * thcb200_comm_unique_id and hands the THCB200_COMM_ID_BYTES to the others by any means (MPI, a
 * file, torch.distributed ...), then every rank, with its own device current, calls
 * thcb200_comm_create (collective: it returns when all ranks have joined).  NCCL is looked up at
 * run time (libnccl.so.2, or the path in the environment variable THCB200_NCCL_LIB); without it
 * these calls return THCB200_ERR_UNSUPPORTED and the rest of the library works as before.
 * Every rank must make the same sequence of sharded calls.  All work is asynchronous on `stream`. */
typedef struct thcb200_comm thcb200_comm;
#define THCB200_COMM_ID_BYTES 128
THCB200_API int thcb200_comm_unique_id(void *id, size_t bytes);
THCB200_API int thcb200_comm_create(thcb200_comm **out, int nranks, int rank, const void *id, size_t bytes);
THCB200_API void thcb200_comm_destroy(thcb200_comm *comm);
THCB200_API int thcb200_comm_info(const thcb200_comm *comm, int *nranks, int *rank, int *nccl_version);
/* ncclAllReduce in place over `count` elements (rop: THCB200_RED_SUM / PROD / MIN / MAX); dtypes NCCL has. */
THCB200_API int thcb200_comm_all_reduce(thcb200_comm *comm, void *buf_dev, int64_t count, int dtype, int rop, void *stream);
/* ncclAllGather of `bytes_per_rank` bytes from every rank into recv_dev[rank * bytes_per_rank ...]. */
THCB200_API int thcb200_comm_all_gather(thcb200_comm *comm, const void *send_dev, void *recv_dev, int64_t bytes_per_rank, void *stream);

/* thcb200_reduce_all over a tensor whose rows are split over the ranks: each rank folds its block,
 * the accumulators (double / int64, in the 8-byte slot `result_dev` on each rank) are combined, and
 * every rank ends with the global result in its slot.  Sums, products and integer min / max are one
 * ncclAllReduce on the slot; floating min / max gather the slots and fold them in rank order with
 * the library's kernel, so that a NaN wins as in the unsharded call. */
THCB200_API int thcb200_sharded_reduce_all(thcb200_ctx *ctx, thcb200_comm *comm, int rop, int pre, thcb200_scalar s,
                               const thcb200_tensor *in, void *result_dev, void *stream);
/* Overlapped mode (off by default).  With it on, the ncclAllReduce of thcb200_sharded_reduce_all runs on
 * a stream the communicator owns, ordered after the local fold by an event, so the kernels the caller
 * enqueues next do not wait for the collective; the slot holds the GLOBAL result only once that
 * all-reduce is done.  thcb200_comm_wait makes `stream` wait for it: call it before anything reads the
 * slot (the next thcb200_sharded_reduce_all waits by itself before it reuses a slot).  The folds that
 * gather and combine (floating min / max) always run in the caller's stream order. */
THCB200_API int thcb200_comm_set_overlap(thcb200_comm *comm, int on);
THCB200_API int thcb200_comm_wait(thcb200_comm *comm, void *stream);
/* Exchange through peer memory instead of NCCL, for thcb200_sharded_reduce_all: the CTA that finishes a
 * rank's reduction stores the rank's accumulator into a small block in every rank's device memory (peer
 * stores over NVLink), waits until its own block holds every rank's, and folds them in rank order -- the
 * reduction and its all-reduce are one kernel and every rank gets the same bits.  The wait is bounded:
 * after `max_polls` polls per awaited rank (0 keeps the default of about a second) the kernel stores the
 * rank's own accumulator, sets a status word and returns; thcb200_comm_peer_status synchronises `stream`
 * and reports (and clears) that word.  At most 16 ranks; every rank must make the same calls.
 *   between processes: every rank calls _peer_export (a cudaIpc handle of THCB200_PEER_HANDLE_BYTES), the
 *     handles are gathered by any means into one array in rank order, every rank calls _peer_attach;
 *   inside one process that drives several devices, as cutorch programs do (peer access enabled by the
 *     caller): allocate _peer_block_bytes() zeroed bytes per rank with cudaMalloc and hand every
 *     communicator the same array of pointers with _peer_attach_local; such communicators need no NCCL
 *     (thcb200_comm_create_local).
 * Then thcb200_comm_set_peer_exchange(comm, 1, 0) on every rank. */
#define THCB200_PEER_HANDLE_BYTES 64
THCB200_API int thcb200_comm_create_local(thcb200_comm **out, int nranks, int rank);
THCB200_API size_t thcb200_comm_peer_block_bytes(void);
THCB200_API int thcb200_comm_peer_export(thcb200_comm *comm, void *handle, size_t bytes);
THCB200_API int thcb200_comm_peer_attach(thcb200_comm *comm, const void *handles, size_t bytes_each);
THCB200_API int thcb200_comm_peer_attach_local(thcb200_comm *comm, void *const *blocks);
THCB200_API int thcb200_comm_set_peer_exchange(thcb200_comm *comm, int on, unsigned int max_polls);
THCB200_API int thcb200_comm_peer_status(thcb200_comm *comm, int *timed_out, void *stream);
/* thcb200_reduce_dim along the dim the tensor is split on: each rank reduces its rows into `out`
 * (dense), then the ranks' outputs are folded and every rank holds the result in `out`.  float /
 * double / int32 / int64 sums and products and integer min / max use ncclAllReduce on the element
 * type (each rank's partial is rounded to the element type first); every other case gathers the
 * ranks' vectors and folds them in rank order with thcb200_reduce_dim. */
THCB200_API int thcb200_sharded_reduce_dim(thcb200_ctx *ctx, thcb200_comm *comm, int rop, int pre, thcb200_scalar s,
                               const thcb200_tensor *out, const thcb200_tensor *in, int dim, void *stream);
/* thcb200_reduce_dim_index along the split dim: `shard_start` is the number of rows in front of
 * this rank's block.  (value, global position) pairs are all-gathered and combined with the rule of
 * the unsharded call: the largest (smallest) value, a NaN first, the lowest global position among
 * equals.  `values` and `indices` (1-based, global) are dense and end up identical on every rank. */
THCB200_API int thcb200_sharded_reduce_dim_index(thcb200_ctx *ctx, thcb200_comm *comm, int rop,
                                     const thcb200_tensor *values, const thcb200_tensor *indices,
                                     const thcb200_tensor *in, int dim, int64_t shard_start, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* THCB200_H */
