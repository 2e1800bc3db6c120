// C-ABI entry points declared in include/thcb200.h: argument validation, the per-device
// context, dispatch on element type.  All device work happens in the typed translation units.
#include <stdio.h>
#include <string.h>

#include "apply_launch.cuh"
#include "context.h"
#include "plan.h"
#include "reduce_launch.cuh"

namespace thcb {
int64_t launch_count();
void arm_allocation_failure(int nth);

void *ctx_workspace(thcb200_ctx *ctx, size_t bytes) {
  if (bytes <= ctx->ws_bytes) return ctx->ws;
  // grow: wait for work that may still read the old buffer
  if (cudaDeviceSynchronize() != cudaSuccess) { set_error("workspace: device synchronize failed"); return nullptr; }
  if (ctx->ws) cudaFree(ctx->ws);
  ctx->ws = nullptr;
  ctx->ws_bytes = 0;
  size_t want = 1 << 20;
  while (want < bytes) want <<= 1;
  void *p = nullptr;
  if (device_alloc(&p, want) != cudaSuccess) {
    cudaGetLastError();
    set_error("workspace: cannot allocate %zu bytes", want);
    return nullptr;
  }
  ctx->ws = p;
  ctx->ws_bytes = want;
  return p;
}

namespace {

// Gather/scatter between a view of up to 25 dims and a dense buffer, for operands whose
// collapsed form is deeper than the generic kernels hold inline.  Element size in bytes.
struct DeepView {
  int n;
  uint64_t size[kMaxDims];
  int64_t stride[kMaxDims];
};
template <int B> struct ElemOf;
template <> struct ElemOf<1> { using type = uint8_t; };
template <> struct ElemOf<2> { using type = uint16_t; };
template <> struct ElemOf<4> { using type = uint32_t; };
template <> struct ElemOf<8> { using type = uint64_t; };

template <int B, bool GATHER>
__global__ void __launch_bounds__(256) deep_copy_kernel(void *dense_raw, void *strided_raw, DeepView v, uint64_t n) {
  pdl_prologue();
  using E = typename ElemOf<B>::type;
  E *dense = reinterpret_cast<E *>(dense_raw);
  E *strided = reinterpret_cast<E *>(strided_raw);
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (uint64_t)gridDim.x * 256) {
    uint64_t lin = i;
    int64_t off = 0;
    for (int d = v.n - 1; d >= 0; --d) {
      const uint64_t q = lin / v.size[d];
      off += (int64_t)(lin - q * v.size[d]) * v.stride[d];
      lin = q;
    }
    if (GATHER) dense[i] = strided[off]; else strided[off] = dense[i];
  }
}

int deep_copy(bool gather, void *dense, const HostView &v, size_t esz, cudaStream_t st) {
  DeepView dv;
  dv.n = v.ndim;
  for (int i = 0; i < v.ndim; ++i) { dv.size[i] = (uint64_t)v.sizes[i]; dv.stride[i] = v.strides[i]; }
  const uint64_t n = (uint64_t)v.numel;
  uint64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
#define THCB_DC(B)                                                                                   \
  if (gather) launch_pdl(deep_copy_kernel<B, true>, (unsigned)blocks, 256, 0, st, dense, v.data, dv, n);     \
  else launch_pdl(deep_copy_kernel<B, false>, (unsigned)blocks, 256, 0, st, dense, v.data, dv, n);
  switch (esz) {
    case 1: THCB_DC(1) break;
    case 2: THCB_DC(2) break;
    case 4: THCB_DC(4) break;
    default: THCB_DC(8) break;
  }
#undef THCB_DC
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

HostView dense_view(void *data, const HostView &like) {
  HostView v;
  v.data = (char *)data;
  v.dtype = like.dtype;
  v.ndim = 1;
  v.sizes[0] = like.numel;
  v.strides[0] = 1;
  v.numel = like.numel;
  return v;
}

typedef int (*PointwiseFn)(thcb200_ctx *, int, const ApplyPlan &, char *const[4], thcb200_scalar, thcb200_scalar, cudaStream_t);
const PointwiseFn kPointwise[8] = {pointwise_u8, pointwise_i8, pointwise_i16, pointwise_i32,
                                   pointwise_i64, pointwise_f16, pointwise_f32, pointwise_f64};
typedef int (*ReduceAllFn)(thcb200_ctx *, int, const HostView &, thcb200_scalar, void *, cudaStream_t);
const ReduceAllFn kReduceAll[8] = {reduce_all_u8, reduce_all_i8, reduce_all_i16, reduce_all_i32,
                                   reduce_all_i64, reduce_all_f16, reduce_all_f32, reduce_all_f64};
typedef int (*ReduceDimFn)(thcb200_ctx *, int, const HostView &, const HostView &, int, thcb200_scalar, PostOp, cudaStream_t);
const ReduceDimFn kReduceDim[8] = {reduce_dim_u8, reduce_dim_i8, reduce_dim_i16, reduce_dim_i32,
                                   reduce_dim_i64, reduce_dim_f16, reduce_dim_f32, reduce_dim_f64};
typedef int (*ReduceDimIndexFn)(thcb200_ctx *, bool, const HostView &, const HostView &, const HostView &, int, cudaStream_t);
const ReduceDimIndexFn kReduceDimIndex[8] = {reduce_dim_index_u8, reduce_dim_index_i8, reduce_dim_index_i16,
                                             reduce_dim_index_i32, reduce_dim_index_i64, reduce_dim_index_f16,
                                             reduce_dim_index_f32, reduce_dim_index_f64};

// Runs one pointwise op on validated views (no overlap handling).
int run_pointwise(thcb200_ctx *ctx, int op, HostView *v, int nops, thcb200_scalar s0, thcb200_scalar s1,
                  cudaStream_t st) {
  const size_t esz = dtype_size(v[0].dtype);
  ApplyPlan plan;
  make_apply_plan(v, nops, esz, &plan);
  void *temps[4] = {nullptr, nullptr, nullptr, nullptr};
  HostView orig_out = v[0];
  bool out_deep = false;
  int rc = 0;
  if (plan.kind == kApplyDeep) {
    // Views that stay deeper than kGenericDims after collapsing go through dense copies.
    for (int o = 0; o < nops && rc == 0; ++o) {
      if (plan.gdims[o] <= kGenericDims) continue;
      if (device_alloc_async(&temps[o], (size_t)v[o].numel * esz, st) != cudaSuccess) {
        cudaGetLastError();
        set_error("pointwise: cannot allocate a dense temporary");
        rc = THCB200_ERR_NOMEM;
        break;
      }
      if (o > 0) rc = deep_copy(true, temps[o], v[o], esz, st);
      if (o == 0) out_deep = true;
      v[o] = dense_view(temps[o], v[o]);
    }
    if (rc == 0) make_apply_plan(v, nops, esz, &plan);
  }
  if (rc == 0) {
    char *data[4] = {nullptr, nullptr, nullptr, nullptr};
    for (int o = 0; o < nops; ++o) data[o] = v[o].data;
    rc = kPointwise[v[0].dtype](ctx, op, plan, data, s0, s1, st);
  }
  if (rc == 0 && out_deep) rc = deep_copy(false, temps[0], orig_out, esz, st);
  for (int o = 0; o < 4; ++o)
    if (temps[o]) cudaFreeAsync(temps[o], st);
  return rc;
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" {

int thcb200_ctx_create(thcb200_ctx **out, int device) {
  if (!out) { set_error("ctx_create: null output pointer"); return THCB200_ERR_ARG; }
  int prev = 0;
  THCB_CUDA_TRY(cudaGetDevice(&prev));
  THCB_CUDA_TRY(cudaSetDevice(device));
  thcb200_ctx *c = new thcb200_ctx();
  c->device = device;
  cudaError_t e = cudaDeviceGetAttribute(&c->num_sms, cudaDevAttrMultiProcessorCount, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&c->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  if (e == cudaSuccess) e = cudaMalloc((void **)&c->tickets, kNumTickets * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(c->tickets, 0, kNumTickets * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMalloc((void **)&c->status, 64);
  if (e == cudaSuccess) e = cudaMemset(c->status, 0, 64);
  if (e == cudaSuccess) e = cudaMalloc(&c->dev_slot, 64);
  if (e == cudaSuccess) e = cudaHostAlloc(&c->host_slot, 64, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e == cudaSuccess) e = cudaHostGetDevicePointer(&c->host_slot_dev, c->host_slot, 0);
  if (e == cudaSuccess) e = cudaMalloc(&c->ws, 1 << 20);
  if (e == cudaSuccess) c->ws_bytes = 1 << 20;
  cudaSetDevice(prev);
  if (e != cudaSuccess) {
    set_error("ctx_create: %s", cudaGetErrorString(e));
    thcb200_ctx_destroy(c);
    return THCB200_ERR_CUDA;
  }
  *out = c;
  return THCB200_OK;
}

void thcb200_ctx_destroy(thcb200_ctx *c) {
  if (!c) return;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(c->device);
  if (c->tickets) cudaFree(c->tickets);
  if (c->status) cudaFree(c->status);
  if (c->dev_slot) cudaFree(c->dev_slot);
  if (c->host_slot) cudaFreeHost(c->host_slot);
  if (c->ws) cudaFree(c->ws);
  if (c->mask_ws) cudaFree(c->mask_ws);
  cudaSetDevice(prev);
  delete c;
}

void *thcb200_ctx_workspace(thcb200_ctx *ctx, size_t min_bytes, size_t *bytes) {
  if (!ctx) { set_error("ctx_workspace: null context"); return nullptr; }
  THCB_CTX_LOCK(ctx);
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  void *p = ctx_workspace(ctx, min_bytes);
  if (prev != ctx->device) cudaSetDevice(prev);
  if (bytes) *bytes = p ? ctx->ws_bytes : 0;
  return p;
}

void thcb200_debug_fail_allocation(int nth) { arm_allocation_failure(nth); }
const char *thcb200_last_error(void) { return get_error(); }
int64_t thcb200_launch_count(void) { return launch_count(); }
const char *thcb200_last_plan(void) { return get_plan_name(); }

int thcb200_memcpy_h2d(void *dst_dev, const void *src_host, size_t bytes, void *stream) {
  THCB_CUDA_TRY(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  THCB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  return THCB200_OK;
}
int thcb200_memcpy_d2h(void *dst_host, const void *src_dev, size_t bytes, void *stream) {
  THCB_CUDA_TRY(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  THCB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  return THCB200_OK;
}
int thcb200_stream_synchronize(void *stream) {
  THCB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  return THCB200_OK;
}

int thcb200_collapse_dims(int64_t *sizes, int64_t *strides, int *ndim, int exclude_dim) {
  return collapse_dims(sizes, strides, ndim, exclude_dim);
}

int thcb200_overlapping(const thcb200_tensor *t) {
  HostView v;
  if (to_host_view(t, &v, "overlapping")) return 0;
  return overlapping_indices(v) ? 1 : 0;
}

int thcb200_can_use_32bit(const thcb200_tensor *t) {
  HostView v;
  if (to_host_view(t, &v, "can_use_32bit")) return 0;
  return can_use_32bit(v) ? 1 : 0;
}

int thcb200_view_extent(const thcb200_tensor *t, int64_t *min_offset, int64_t *max_offset) {
  HostView v;
  if (to_host_view(t, &v, "view_extent")) return THCB200_ERR_ARG;
  if (v.numel == 0) return 0;
  int64_t lo = 0, hi = 0;
  offset_range(v, &lo, &hi);
  if (min_offset) *min_offset = lo;
  if (max_offset) *max_offset = hi;
  return 1;
}

int thcb200_check_extent(const thcb200_tensor *t, int64_t elements_before, int64_t elements_after) {
  int64_t lo = 0, hi = 0;
  const int rc = thcb200_view_extent(t, &lo, &hi);
  if (rc <= 0) return rc;
  if (lo < -elements_before || hi > elements_after) {
    set_error("the view reaches offsets %lld..%lld; the allocation allows %lld..%lld", (long long)lo, (long long)hi,
              (long long)-elements_before, (long long)elements_after);
    return THCB200_ERR_SIZE;
  }
  return THCB200_OK;
}

int64_t thcb200_index_to_offset(const thcb200_tensor *t, int64_t linear) {
  int64_t off = 0;
  for (int d = t->ndim - 1; d >= 0; --d) {
    const int64_t q = linear / t->sizes[d];
    off += (linear - q * t->sizes[d]) * t->strides[d];
    linear = q;
  }
  return off;
}

const char *thcb200_pointwise_plan(const thcb200_tensor *out, const thcb200_tensor *in0, const thcb200_tensor *in1,
                                   const thcb200_tensor *in2, int nin) {
  if (nin < 0 || nin > 3) { set_error("pointwise_plan: nin out of range"); return nullptr; }
  const thcb200_tensor *t[4] = {out, in0, in1, in2};
  HostView v[4];
  for (int o = 0; o <= nin; ++o) {
    if (to_host_view(t[o], &v[o], "pointwise_plan operand")) return nullptr;
    if (v[o].dtype != v[0].dtype) { set_error("pointwise_plan: operands have different dtypes"); return nullptr; }
    if (v[o].numel != v[0].numel) { set_error("pointwise_plan: operands have different element counts"); return nullptr; }
  }
  ApplyPlan plan;
  make_apply_plan(v, nin + 1, dtype_size(v[0].dtype), &plan);
  switch (plan.kind) {
    case kApplyContigVec: {
      bool wide = true;
      for (int o = 0; o <= nin; ++o) if (((uintptr_t)v[o].data) % 32 != 0) wide = false;
      return wide ? "contig_vec" : "contig_vec16";
    }
    case kApplyTiled: return "tiled";
    case kApplyRows: return plan.rows.vec ? "rows" : "rows_scalar";
    case kApplyGeneric: return plan.index64 ? "generic64" : "generic32";
    default: return "deep";
  }
}

int thcb200_pointwise(thcb200_ctx *ctx, int op, const thcb200_tensor *out, const thcb200_tensor *in0,
                      const thcb200_tensor *in1, const thcb200_tensor *in2, int nin, thcb200_scalar s0,
                      thcb200_scalar s1, void *stream) {
  return thcb200_pointwise_ex(ctx, op, out, in0, in1, in2, nin, s0, s1, stream, 0);
}

int thcb200_pointwise_ex(thcb200_ctx *ctx, int op, const thcb200_tensor *out, const thcb200_tensor *in0,
                         const thcb200_tensor *in1, const thcb200_tensor *in2, int nin, thcb200_scalar s0,
                         thcb200_scalar s1, void *stream, int flags) {
  if (!ctx) { set_error("pointwise: null context"); return THCB200_ERR_ARG; }
  if (op_arity(op) < 0) { set_error("pointwise: unknown op %d", op); return THCB200_ERR_ARG; }
  if (op_arity(op) != nin) { set_error("pointwise: op %d takes %d inputs, got %d", op, op_arity(op), nin); return THCB200_ERR_ARG; }
  const thcb200_tensor *t[4] = {out, in0, in1, in2};
  static const char *names[4] = {"pointwise output", "pointwise input 0", "pointwise input 1", "pointwise input 2"};
  HostView v[4];
  for (int o = 0; o <= nin; ++o) {
    int rc = to_host_view(t[o], &v[o], names[o]);
    if (rc) return rc;
    if (v[o].dtype != v[0].dtype) { set_error("pointwise: operands have different dtypes"); return THCB200_ERR_ARG; }
    if (v[o].numel != v[0].numel) { set_error("pointwise: operands have different element counts"); return THCB200_ERR_SIZE; }
  }
  if (!op_supported(op, v[0].dtype)) { set_error("pointwise: op %d is not defined for dtype %d", op, v[0].dtype); return THCB200_ERR_UNSUPPORTED; }
  if (v[0].numel == 0) return THCB200_OK;  // THC_pointwiseApply: empty tensors are a no-op
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = dtype_size(v[0].dtype);
  if (!(flags & THCB200_FLAG_IGNORE_OVERLAP) && overlapping_indices(v[0])) {
    // An output whose index tuples alias (e.g. an expanded view) is computed into a dense
    // temporary and written back element by element; which duplicate lands last is not
    // defined (lib/THC/THCApply.cuh:288-302,401-417).
    void *tmp = nullptr;
    if (device_alloc_async(&tmp, (size_t)v[0].numel * esz, st) != cudaSuccess) {
      cudaGetLastError();
      set_error("pointwise: cannot allocate a dense temporary");
      return THCB200_ERR_NOMEM;
    }
    HostView real_out = v[0];
    // dense temporary walked in the output's logical order
    HostView dense = v[0];
    dense.data = (char *)tmp;
    int64_t st_run = 1;
    for (int d = dense.ndim - 1; d >= 0; --d) { dense.strides[d] = st_run; st_run *= dense.sizes[d]; }
    v[0] = dense;
    int rc = run_pointwise(ctx, op, v, nin + 1, s0, s1, st);
    if (rc == 0) {
      HostView cp[2] = {real_out, dense};
      thcb200_scalar z = {0.0, 0};
      rc = run_pointwise(ctx, THCB200_OP_COPY, cp, 2, z, z, st);
    }
    cudaFreeAsync(tmp, st);
    return rc;
  }
  return run_pointwise(ctx, op, v, nin + 1, s0, s1, st);
}

static int check_reduce_common(thcb200_ctx *ctx, const thcb200_tensor *in, HostView *vin, const char *what) {
  if (!ctx) { set_error("%s: null context", what); return THCB200_ERR_ARG; }
  return to_host_view(in, vin, what);
}

// bytes [16, 24) of the pinned slot receive the result of thcb200_reduce_all_host; the first bytes
// stay the staging area of the small host <-> device copies
static constexpr size_t kHostResultOffset = 16;

int thcb200_reduce_all(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s, const thcb200_tensor *in,
                       void *result_dev, void *stream) {
  HostView vin;
  int rc = check_reduce_common(ctx, in, &vin, "reduce_all");
  if (rc) return rc;
  const int mode = reduce_mode(rop, pre);
  if (mode < 0) { set_error("reduce_all: unknown reduce op %d / pre op %d", rop, pre); return THCB200_ERR_ARG; }
  if (!result_dev) { set_error("reduce_all: null result pointer"); return THCB200_ERR_ARG; }
  cudaStream_t st = (cudaStream_t)stream;
  THCB_CTX_LOCK(ctx);
  if (vin.numel == 0) {
    // THC_reduceAll on an empty tensor yields the initial value (lib/THC/THCReduceAll.cuh:253-257)
    if (mode == kMin || mode == kMax) { set_error("reduce_all: min/max of an empty tensor"); return THCB200_ERR_ARG; }
    const bool fp = vin.dtype >= THCB200_F16;
    const bool one = (mode == kProd || mode == kAll);
    union { double d; int64_t i; } u;
    if (fp) u.d = one ? 1.0 : 0.0; else u.i = one ? 1 : 0;
    if (result_dev == (char *)ctx->host_slot_dev + kHostResultOffset) {   // thcb200_reduce_all_host
      THCB_CUDA_TRY(cudaStreamSynchronize(st));
      memcpy((char *)ctx->host_slot + kHostResultOffset, &u, 8);
      return THCB200_OK;
    }
    memcpy(ctx->host_slot, &u, 8);
    THCB_CUDA_TRY(cudaMemcpyAsync(result_dev, ctx->host_slot, 8, cudaMemcpyHostToDevice, st));
    return THCB200_OK;
  }
  return kReduceAll[vin.dtype](ctx, mode, vin, s, result_dev, st);
}

int thcb200_reduce_all_host(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s, const thcb200_tensor *in,
                            void *result_host, void *stream) {
  if (!result_host) { set_error("reduce_all_host: null result pointer"); return THCB200_ERR_ARG; }
  if (!ctx) { set_error("reduce_all_host: null context"); return THCB200_ERR_ARG; }
  // The kernel that finishes the fold stores the result straight into the pinned, mapped host
  // slot: no device-to-host copy is enqueued behind it, the stream synchronisation is all.
  THCB_CTX_LOCK(ctx);
  int rc = thcb200_reduce_all(ctx, rop, pre, s, in, (char *)ctx->host_slot_dev + kHostResultOffset, stream);
  if (rc) return rc;
  THCB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  memcpy(result_host, (char *)ctx->host_slot + kHostResultOffset, 8);
  return THCB200_OK;
}

static int check_reduce_dim(const HostView &vin, const HostView &vout, int dim, const char *what) {
  if (dim < 0 || dim >= vin.ndim) { set_error("%s: dimension %d out of range", what, dim); return THCB200_ERR_ARG; }
  if (vout.ndim != vin.ndim) { set_error("%s: output must have the input's dimension count", what); return THCB200_ERR_ARG; }
  for (int i = 0; i < vin.ndim; ++i) {
    const int64_t want = (i == dim) ? 1 : vin.sizes[i];
    if (vout.sizes[i] != want) { set_error("%s: output size mismatch in dim %d", what, i); return THCB200_ERR_SIZE; }
  }
  if (vin.sizes[dim] == 0) { set_error("%s: reduced dimension is empty", what); return THCB200_ERR_ARG; }
  return 0;
}

int thcb200_reduce_dim(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s, const thcb200_tensor *out,
                       const thcb200_tensor *in, int dim, void *stream) {
  thcb200_scalar none = {0.0, 0};
  return thcb200_reduce_dim_post(ctx, rop, pre, s, THCB200_POST_NONE, none, out, in, dim, stream);
}

int thcb200_reduce_dim_post(thcb200_ctx *ctx, int rop, int pre, thcb200_scalar s, int post_kind, thcb200_scalar post_value,
                            const thcb200_tensor *out, const thcb200_tensor *in, int dim, void *stream) {
  HostView vin, vout;
  if (post_kind < THCB200_POST_NONE || post_kind > THCB200_POST_STD_UNBIASED) { set_error("reduce_dim: unknown post op %d", post_kind); return THCB200_ERR_ARG; }
  if ((pre == THCB200_PRE_MOMENTS) != (post_kind >= THCB200_POST_VAR_BIASED)) {
    set_error("reduce_dim: THCB200_PRE_MOMENTS and the var/std post steps go together");
    return THCB200_ERR_ARG;
  }
  if (post_kind == THCB200_POST_DIV && post_value.f == 0.0 && post_value.i == 0) { set_error("reduce_dim: division by zero"); return THCB200_ERR_ARG; }
  PostOp post = {post_kind, post_value.f, post_value.i};
  int rc = check_reduce_common(ctx, in, &vin, "reduce_dim input");
  if (rc) return rc;
  rc = to_host_view(out, &vout, "reduce_dim output");
  if (rc) return rc;
  if (vin.dtype != vout.dtype) { set_error("reduce_dim: input and output dtypes differ"); return THCB200_ERR_ARG; }
  const int mode = reduce_mode(rop, pre);
  if (mode < 0) { set_error("reduce_dim: unknown reduce op %d / pre op %d", rop, pre); return THCB200_ERR_ARG; }
  rc = check_reduce_dim(vin, vout, dim, "reduce_dim");
  if (rc) return rc;
  if (vout.numel == 0) return THCB200_OK;
  if (post_kind >= THCB200_POST_VAR_BIASED) post.f = (double)vin.sizes[dim];  // n of the var/std formulas
  THCB_CTX_LOCK(ctx);
  return kReduceDim[vin.dtype](ctx, mode, vin, vout, dim, s, post, (cudaStream_t)stream);
}

int thcb200_reduce_dim_index(thcb200_ctx *ctx, int rop, const thcb200_tensor *values, const thcb200_tensor *indices,
                             const thcb200_tensor *in, int dim, void *stream) {
  HostView vin, vval, vidx;
  int rc = check_reduce_common(ctx, in, &vin, "reduce_dim_index input");
  if (rc) return rc;
  rc = to_host_view(values, &vval, "reduce_dim_index values");
  if (rc) return rc;
  rc = to_host_view(indices, &vidx, "reduce_dim_index indices");
  if (rc) return rc;
  if (rop != THCB200_RED_MAX && rop != THCB200_RED_MIN) { set_error("reduce_dim_index: only max and min carry positions"); return THCB200_ERR_ARG; }
  if (vin.dtype != vval.dtype) { set_error("reduce_dim_index: input and values dtypes differ"); return THCB200_ERR_ARG; }
  if (vidx.dtype != THCB200_I64) { set_error("reduce_dim_index: indices must be int64"); return THCB200_ERR_ARG; }
  rc = check_reduce_dim(vin, vval, dim, "reduce_dim_index");
  if (rc) return rc;
  rc = check_reduce_dim(vin, vidx, dim, "reduce_dim_index (indices)");
  if (rc) return rc;
  if (vval.numel == 0) return THCB200_OK;
  THCB_CTX_LOCK(ctx);
  return kReduceDimIndex[vin.dtype](ctx, rop == THCB200_RED_MAX, vin, vval, vidx, dim, (cudaStream_t)stream);
}

}  // extern "C"
