// Indexed moves along one dim: indexSelect / indexCopy / indexAdd / indexFill
// (lib/THC/THCTensorIndex.cu:22-387, generic/THCTensorIndex.cu) and gather / scatter / scatterAdd /
// scatterFill (lib/THC/THCTensorScatterGather.cu:78-159, generic/THCTensorScatterGather.cu).
//
// All eight are one walk: for every coordinate tuple c of an iteration space, read a 1-based
// position from the index tensor (at c for gather/scatter, at c[dim] for the index* calls: a
// vector is an index tensor with stride 0 in every other dim), and move one element between the
// plain side, addressed by c, and the redirected side, addressed by c with c[dim] replaced by the
// position.  gather-like calls redirect the source, scatter-like calls the destination.
//
// The reference instantiates separate small/large-index kernels per dims; here one kernel takes
// jointly collapsed dims (neighbouring dims that form one run in all three tensors merge) and
// walks them with multiply-high division, four elements in flight per thread.  Positions outside
// 1..size are not dereferenced (the reference asserts on the device): the element is skipped and
// counted in the context's status word, which thcb200_take_index_errors reads and clears.
// Adds use atomics, as in the reference: with duplicate positions the order of floating-point
// additions is not fixed.
#include <cuda_fp16.h>
#include <string.h>

#include <type_traits>

#include "context.h"
#include "core.cuh"
#include "plan.h"

namespace thcb {
namespace {

constexpr int kIdxThreads = 256;
constexpr int kIdxUnroll = 4;

enum IdxMode { kIdxCopy = 0, kIdxAdd = 1, kIdxFill = 2 };

struct alignas(16) Word16 { uint32_t w[4]; };

template <typename IndexT>
struct IdxPlan {
  int nd;
  DivHelper<IndexT> size[kGenericDims];
  int64_t plain[kGenericDims];   // strides of the side addressed by c
  int64_t redir[kGenericDims];   // strides of the redirected side (0 in the indexed dim)
  int64_t index[kGenericDims];   // strides of the index tensor
  int64_t redirect_stride;       // stride of the indexed dim on the redirected side
  int64_t limit;                 // positions 1..limit are valid
};

template <typename T> __device__ __forceinline__ void atomic_add_elem(T *p, T v) { atomicAdd(p, v); }
template <> __device__ __forceinline__ void atomic_add_elem<Word16>(Word16 *, Word16) {}   // never used: adds are per element
template <> __device__ __forceinline__ void atomic_add_elem<int64_t>(int64_t *p, int64_t v) {
  atomicAdd(reinterpret_cast<unsigned long long *>(p), (unsigned long long)v);
}
// 8- and 16-bit integers: compare-and-swap on the aligned 32-bit word that holds the element
template <typename T> __device__ __forceinline__ void atomic_add_narrow(T *p, T v) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  unsigned int *word = reinterpret_cast<unsigned int *>(a & ~(uintptr_t)3);
  const unsigned shift = (unsigned)(a & 3) * 8;
  const unsigned int mask = (sizeof(T) == 1 ? 0xFFu : 0xFFFFu) << shift;
  unsigned int old = *word, assumed;
  do {
    assumed = old;
    const unsigned int cur = (assumed & mask) >> shift;
    const unsigned int sum = ((unsigned int)(T)((T)cur + v) << shift) & mask;
    old = atomicCAS(word, assumed, (assumed & ~mask) | sum);
  } while (old != assumed);
}
template <> __device__ __forceinline__ void atomic_add_elem<uint8_t>(uint8_t *p, uint8_t v) { atomic_add_narrow(p, v); }
template <> __device__ __forceinline__ void atomic_add_elem<int8_t>(int8_t *p, int8_t v) { atomic_add_narrow(p, v); }
template <> __device__ __forceinline__ void atomic_add_elem<int16_t>(int16_t *p, int16_t v) { atomic_add_narrow(p, v); }

// REDIRECT_DST: destination is the redirected side (scatter-like); else the source is (gather-like)
template <typename T, int MODE, bool REDIRECT_DST, typename IndexT>
__global__ void __launch_bounds__(kIdxThreads)
indexed_kernel(T *dst, const T *src, const int64_t *index, IdxPlan<IndexT> p, IndexT n, T value, unsigned int *errors) {
  pdl_prologue();
  // Offsets are kept in IndexT: with 32-bit indices every tensor's largest offset fits 32 bits, so
  // sums taken modulo 2^32 are exact.
  const IndexT base = (IndexT)blockIdx.x * (IndexT)(kIdxThreads * kIdxUnroll) + threadIdx.x;
  IndexT off_plain[kIdxUnroll], off_redir[kIdxUnroll];
  int64_t pos[kIdxUnroll];
  bool live[kIdxUnroll];
#pragma unroll
  for (int u = 0; u < kIdxUnroll; ++u) {
    IndexT lin = base + (IndexT)u * kIdxThreads;
    live[u] = lin < n;
    IndexT op = 0, orr = 0, oi = 0;
    if (live[u]) {
      // only the dims in use are walked (the plan sits in constant memory, indexed at run time)
#pragma unroll 1
      for (int d = p.nd - 1; d >= 0; --d) {
        IndexT q, r;
        p.size[d].divmod(lin, q, r);
        op += r * (IndexT)p.plain[d];
        orr += r * (IndexT)p.redir[d];
        oi += r * (IndexT)p.index[d];
        lin = q;
      }
      pos[u] = index[oi] - 1;   // positions are 1-based (TH_INDEX_BASE)
    }
    off_plain[u] = op;
    off_redir[u] = orr;
  }
  unsigned int bad = 0;
#pragma unroll
  for (int u = 0; u < kIdxUnroll; ++u) {
    if (!live[u]) continue;
    if ((uint64_t)pos[u] >= (uint64_t)p.limit) { live[u] = false; ++bad; continue; }
    off_redir[u] += (IndexT)pos[u] * (IndexT)p.redirect_stride;
  }
  if (bad) atomicAdd(errors, bad);
  T x[kIdxUnroll];
  if (MODE != kIdxFill) {
#pragma unroll
    for (int u = 0; u < kIdxUnroll; ++u)
      if (live[u]) x[u] = src[REDIRECT_DST ? off_plain[u] : off_redir[u]];
  }
#pragma unroll
  for (int u = 0; u < kIdxUnroll; ++u) {
    if (!live[u]) continue;
    T *q = dst + (REDIRECT_DST ? off_redir[u] : off_plain[u]);
    if constexpr (MODE == kIdxCopy) *q = x[u];
    else if constexpr (MODE == kIdxFill) *q = value;
    else atomic_add_elem<T>(q, x[u]);
  }
}

// Four neighbours of the innermost dim per thread, for the layouts where that dim has unit stride
// on the plain side and in the index tensor (gather / scatter on contiguous tensors): one decode of
// the linear position, one 32-byte load of four index entries and one vector access on the plain
// side per four elements; only the redirected side is touched element by element.  p.size[nd-1]
// counts groups of four.
template <typename T> struct alignas(4 * sizeof(T)) Quad { T e[4]; };

template <typename T, int MODE, bool REDIRECT_DST, typename IndexT>
__global__ void __launch_bounds__(kIdxThreads)
indexed_quad_kernel(T *dst, const T *src, const int64_t *index, IdxPlan<IndexT> p, IndexT nquads, T value, unsigned int *errors) {
  pdl_prologue();
  const IndexT quad = (IndexT)blockIdx.x * (IndexT)kIdxThreads + threadIdx.x;
  if (quad >= nquads) return;
  const int L = p.nd - 1;
  IndexT lin, r, op, orr, oi;
  p.size[L].divmod(quad, lin, r);
  r *= 4;
  op = r;
  oi = r;
  orr = r * (IndexT)p.redir[L];
#pragma unroll 1
  for (int d = L - 1; d >= 0; --d) {
    IndexT q;
    p.size[d].divmod(lin, q, r);
    op += r * (IndexT)p.plain[d];
    orr += r * (IndexT)p.redir[d];
    oi += r * (IndexT)p.index[d];
    lin = q;
  }
  union { Bytes32 b; int64_t e[4]; } ix;
  ix.b = ld32_stream(index + oi);
  IndexT off[4];
  bool ok[4];
  unsigned int bad = 0;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t pos = ix.e[u] - 1;   // positions are 1-based (TH_INDEX_BASE)
    ok[u] = (uint64_t)pos < (uint64_t)p.limit;
    bad += ok[u] ? 0u : 1u;
    off[u] = orr + (IndexT)u * (IndexT)p.redir[L] + (IndexT)pos * (IndexT)p.redirect_stride;
  }
  if (bad) atomicAdd(errors, bad);
  if constexpr (REDIRECT_DST) {
    Quad<T> x;
    if constexpr (MODE != kIdxFill) x = *reinterpret_cast<const Quad<T> *>(src + op);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!ok[u]) continue;
      if constexpr (MODE == kIdxCopy) dst[off[u]] = x.e[u];
      else if constexpr (MODE == kIdxFill) dst[off[u]] = value;
      else atomic_add_elem<T>(dst + off[u], x.e[u]);
    }
  } else {
    Quad<T> x;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (ok[u]) x.e[u] = src[off[u]];
    if (bad == 0) {
      *reinterpret_cast<Quad<T> *>(dst + op) = x;
    } else {   // elements with a position out of range stay as they are
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (ok[u]) dst[op + u] = x.e[u];
    }
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
struct HostIdxPlan {
  int nd;
  int64_t size[kMaxDims], plain[kMaxDims], redir[kMaxDims], index[kMaxDims];
  int64_t redirect_stride, limit;
  uint64_t n;
  bool fits32;   // element counts and largest offsets of all three tensors fit 32 bits
  bool quads;    // size[nd-1] and n count groups of four neighbours (indexed_quad_kernel)
};

template <typename IndexT>
IdxPlan<IndexT> to_device_plan(const HostIdxPlan &h) {
  IdxPlan<IndexT> p;
  p.nd = h.nd;
  for (int d = 0; d < kGenericDims; ++d) {
    const bool used = d < h.nd;
    p.size[d] = DivHelper<IndexT>(used ? (uint64_t)h.size[d] : 1);
    p.plain[d] = used ? h.plain[d] : 0;
    p.redir[d] = used ? h.redir[d] : 0;
    p.index[d] = used ? h.index[d] : 0;
  }
  p.redirect_stride = h.redirect_stride;
  p.limit = h.limit;
  return p;
}

template <typename T, int MODE, bool REDIRECT_DST>
int launch_indexed(thcb200_ctx *ctx, const HostIdxPlan &h, void *dst, const void *src, const void *index, T value,
                   cudaStream_t st) {
  const uint64_t per_cta = (uint64_t)kIdxThreads * kIdxUnroll;
  const uint64_t blocks = (h.n + per_cta - 1) / per_cta;
  if (blocks >= (1ull << 31)) { set_error("indexed: tensor too large"); return THCB200_ERR_DIMS; }
  unsigned int *errors = reinterpret_cast<unsigned int *>(ctx->status) + 1;
  if constexpr (!std::is_same<T, Word16>::value) {
    if (h.quads) {
      const uint64_t qblocks = (h.n + kIdxThreads - 1) / kIdxThreads;
      if (h.fits32) {
        set_plan_name("indexed_quad32");
        launch_pdl(indexed_quad_kernel<T, MODE, REDIRECT_DST, uint32_t>, (unsigned)qblocks, kIdxThreads, 0, st, 
            (T *)dst, (const T *)src, (const int64_t *)index, to_device_plan<uint32_t>(h), (uint32_t)h.n, value, errors);
      } else {
        set_plan_name("indexed_quad64");
        launch_pdl(indexed_quad_kernel<T, MODE, REDIRECT_DST, uint64_t>, (unsigned)qblocks, kIdxThreads, 0, st, 
            (T *)dst, (const T *)src, (const int64_t *)index, to_device_plan<uint64_t>(h), (uint64_t)h.n, value, errors);
      }
      count_launch();
      THCB_CUDA_TRY(cudaGetLastError());
      return 0;
    }
  }
  if (h.fits32 && h.n < (1ull << 32) - per_cta) {
    set_plan_name("indexed32");
    launch_pdl(indexed_kernel<T, MODE, REDIRECT_DST, uint32_t>, (unsigned)blocks, kIdxThreads, 0, st, 
        (T *)dst, (const T *)src, (const int64_t *)index, to_device_plan<uint32_t>(h), (uint32_t)h.n, value, errors);
  } else {
    set_plan_name("indexed64");
    launch_pdl(indexed_kernel<T, MODE, REDIRECT_DST, uint64_t>, (unsigned)blocks, kIdxThreads, 0, st, 
        (T *)dst, (const T *)src, (const int64_t *)index, to_device_plan<uint64_t>(h), (uint64_t)h.n, value, errors);
  }
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

template <typename W, int MODE>
int launch_move_sized(thcb200_ctx *ctx, bool redirect_dst, const HostIdxPlan &h, void *dst, const void *src, const void *index,
                      uint64_t bits, cudaStream_t st) {
  const W value = (W)bits;
  return redirect_dst ? launch_indexed<W, MODE, true>(ctx, h, dst, src, index, value, st)
                      : launch_indexed<W, MODE, false>(ctx, h, dst, src, index, value, st);
}

uint64_t value_bits(int dt, thcb200_scalar s) {
  uint64_t bits = 0;
  switch (dt) {
    case THCB200_U8: { uint8_t v = (uint8_t)s.i; memcpy(&bits, &v, 1); break; }
    case THCB200_I8: { int8_t v = (int8_t)s.i; memcpy(&bits, &v, 1); break; }
    case THCB200_I16: { int16_t v = (int16_t)s.i; memcpy(&bits, &v, 2); break; }
    case THCB200_I32: { int32_t v = (int32_t)s.i; memcpy(&bits, &v, 4); break; }
    case THCB200_I64: { int64_t v = s.i; memcpy(&bits, &v, 8); break; }
    case THCB200_F16: { __half v = __float2half_rn((float)s.f); memcpy(&bits, &v, 2); break; }
    case THCB200_F32: { float v = (float)s.f; memcpy(&bits, &v, 4); break; }
    default: { double v = s.f; memcpy(&bits, &v, 8); break; }
  }
  return bits;
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" {

int thcb200_indexed(thcb200_ctx *ctx, int mode, const thcb200_tensor *dst, const thcb200_tensor *src,
                    const thcb200_tensor *index, int dim, int index_is_vector, thcb200_scalar value, void *stream) {
  if (!ctx) { set_error("indexed: null context"); return THCB200_ERR_ARG; }
  if (mode < THCB200_INDEX_GATHER || mode > THCB200_INDEX_SCATTER_FILL) { set_error("indexed: unknown mode %d", mode); return THCB200_ERR_ARG; }
  const bool fill = mode == THCB200_INDEX_SCATTER_FILL;
  const bool redirect_dst = mode != THCB200_INDEX_GATHER;
  HostView vd, vs, vi;
  int rc = to_host_view(dst, &vd, "indexed destination");
  if (!rc && !fill) rc = to_host_view(src, &vs, "indexed source");
  if (!rc) rc = to_host_view(index, &vi, "indexed index");
  if (rc) return rc;
  if (vi.dtype != THCB200_I64) { set_error("indexed: the index must be an I64 view"); return THCB200_ERR_ARG; }
  if (!fill && vs.dtype != vd.dtype) { set_error("indexed: source and destination have different dtypes"); return THCB200_ERR_ARG; }
  const HostView &redir = redirect_dst ? vd : vs;
  const int nd = redir.ndim;
  if (dim < 0 || dim >= nd) { set_error("indexed: dim %d out of range", dim); return THCB200_ERR_ARG; }
  if (!fill && vs.ndim != vd.ndim) { set_error("indexed: source and destination have different numbers of dims"); return THCB200_ERR_ARG; }
  if (index_is_vector ? vi.ndim != 1 : vi.ndim != nd) { set_error("indexed: the index has the wrong number of dims"); return THCB200_ERR_ARG; }
  // iteration space
  int64_t it[kMaxDims];
  const HostView *plain = fill ? nullptr : (redirect_dst ? &vs : &vd);
  for (int d = 0; d < nd; ++d) {
    if (plain) it[d] = plain->sizes[d];
    else it[d] = index_is_vector ? (d == dim ? vi.sizes[0] : vd.sizes[d]) : vi.sizes[d];
  }
  if (index_is_vector) {
    if (vi.sizes[0] != it[dim]) { set_error("indexed: the index vector has %lld entries, the indexed dim %lld", (long long)vi.sizes[0], (long long)it[dim]); return THCB200_ERR_SIZE; }
  } else {
    for (int d = 0; d < nd; ++d)
      if (vi.sizes[d] != it[d]) { set_error("indexed: the index does not have the shape of the tensor it walks with"); return THCB200_ERR_SIZE; }
  }
  for (int d = 0; d < nd; ++d)
    if (d != dim && redir.sizes[d] < it[d]) { set_error("indexed: size mismatch in dim %d", d); return THCB200_ERR_SIZE; }
  uint64_t n = 1;
  for (int d = 0; d < nd; ++d) n *= (uint64_t)it[d];
  if (n == 0) return THCB200_OK;

  // per-dim strides, then drop size-1 dims and merge neighbours that are one run everywhere
  HostIdxPlan h;
  h.nd = 0;
  h.n = n;
  h.quads = false;
  h.fits32 = can_use_32bit(vd) && can_use_32bit(vi) && (fill || can_use_32bit(vs));
  h.redirect_stride = redir.strides[dim];
  h.limit = redir.sizes[dim];
  bool prev_mergeable = false;
  int h_dim = -1;   // entry of the indexed dim among the collapsed ones
  for (int d = 0; d < nd; ++d) {
    if (it[d] == 1) continue;
    const int64_t sp = plain ? plain->strides[d] : 0;
    const int64_t sr = d == dim ? 0 : redir.strides[d];
    const int64_t sx = index_is_vector ? (d == dim ? vi.strides[0] : 0) : vi.strides[d];
    const bool mergeable = d != dim;
    if (mergeable && prev_mergeable && h.nd > 0 && h.plain[h.nd - 1] == it[d] * sp && h.redir[h.nd - 1] == it[d] * sr &&
        h.index[h.nd - 1] == it[d] * sx) {
      h.size[h.nd - 1] *= it[d];
      h.plain[h.nd - 1] = sp;
      h.redir[h.nd - 1] = sr;
      h.index[h.nd - 1] = sx;
    } else {
      if (d == dim) h_dim = h.nd;
      h.size[h.nd] = it[d];
      h.plain[h.nd] = sp;
      h.redir[h.nd] = sr;
      h.index[h.nd] = sx;
      ++h.nd;
    }
    prev_mergeable = mergeable;
  }
  if (h.nd > kGenericDims) { set_error("indexed: more than %d dims remain after collapsing", kGenericDims); return THCB200_ERR_DIMS; }
  cudaStream_t st = (cudaStream_t)stream;
  void *dp = vd.data;
  const void *sp = fill ? nullptr : vs.data;
  const void *xp = vi.data;
  // Groups of four neighbours: the innermost dim has unit stride on the plain side and in the
  // index tensor, and every other stride of those two keeps the vectors aligned.
  auto try_quads = [&]() {
    const int esz = (int)dtype_size(vd.dtype);
    const int L = h.nd - 1;
    if (L < 0 || h.index[L] != 1 || (plain && h.plain[L] != 1) || h.size[L] % 4 != 0) return;
    if ((uintptr_t)xp % 32 != 0 || (plain && (uintptr_t)plain->data % (uintptr_t)(4 * esz) != 0)) return;
    for (int d = 0; d < L; ++d)
      if (h.index[d] % 4 != 0 || h.plain[d] % 4 != 0) return;
    h.size[L] /= 4;
    h.n /= 4;
    h.quads = true;
  };
  if (mode == THCB200_INDEX_SCATTER_ADD) try_quads();
  if (mode == THCB200_INDEX_SCATTER_ADD) {
    switch (vd.dtype) {
      case THCB200_U8: return launch_indexed<uint8_t, kIdxAdd, true>(ctx, h, dp, sp, xp, 0, st);
      case THCB200_I8: return launch_indexed<int8_t, kIdxAdd, true>(ctx, h, dp, sp, xp, 0, st);
      case THCB200_I16: return launch_indexed<int16_t, kIdxAdd, true>(ctx, h, dp, sp, xp, 0, st);
      case THCB200_I32: return launch_indexed<int32_t, kIdxAdd, true>(ctx, h, dp, sp, xp, 0, st);
      case THCB200_I64: return launch_indexed<int64_t, kIdxAdd, true>(ctx, h, dp, sp, xp, 0, st);
      case THCB200_F16: return launch_indexed<__half, kIdxAdd, true>(ctx, h, dp, sp, xp, __half(), st);
      case THCB200_F32: return launch_indexed<float, kIdxAdd, true>(ctx, h, dp, sp, xp, 0.f, st);
      default: return launch_indexed<double, kIdxAdd, true>(ctx, h, dp, sp, xp, 0.0, st);
    }
  }
  const uint64_t bits = fill ? value_bits(vd.dtype, value) : 0;
  // Whole 16-byte words move when the innermost run is dense on both sides, every position of it
  // shares one index entry, and all other strides keep 16-byte alignment (the index* calls on
  // rows of a matrix): same kernel, element = 16 bytes.
  {
    const int esz = (int)dtype_size(vd.dtype);
    const int V = 16 / esz;
    const int L = h.nd - 1;
    bool vec = V > 1 && L >= 0 && L != h_dim && h.redir[L] == 1 && (fill || h.plain[L] == 1) && h.index[L] == 0 &&
               h.size[L] % V == 0 && h.redirect_stride % V == 0 && (uintptr_t)dp % 16 == 0 && (fill || (uintptr_t)sp % 16 == 0);
    for (int d = 0; vec && d < L; ++d)
      if (h.plain[d] % V != 0 || h.redir[d] % V != 0) vec = false;
    if (vec) {
      h.size[L] /= V;
      for (int d = 0; d < L; ++d) { h.plain[d] /= V; h.redir[d] /= V; }
      h.redirect_stride /= V;
      h.n /= (uint64_t)V;
      Word16 w;
      for (int b = 0; b < 16; b += esz) memcpy(reinterpret_cast<char *>(&w) + b, &bits, (size_t)esz);
      if (fill) return launch_indexed<Word16, kIdxFill, true>(ctx, h, dp, sp, xp, w, st);
      return redirect_dst ? launch_indexed<Word16, kIdxCopy, true>(ctx, h, dp, sp, xp, w, st)
                          : launch_indexed<Word16, kIdxCopy, false>(ctx, h, dp, sp, xp, w, st);
    }
  }
  try_quads();
#define THCB_IDX_SIZED(W) (fill ? launch_move_sized<W, kIdxFill>(ctx, true, h, dp, sp, xp, bits, st) \
                                : launch_move_sized<W, kIdxCopy>(ctx, redirect_dst, h, dp, sp, xp, bits, st))
  switch (dtype_size(vd.dtype)) {
    case 1: return THCB_IDX_SIZED(uint8_t);
    case 2: return THCB_IDX_SIZED(uint16_t);
    case 4: return THCB_IDX_SIZED(uint32_t);
    default: return THCB_IDX_SIZED(uint64_t);
  }
#undef THCB_IDX_SIZED
}

int thcb200_take_index_errors(thcb200_ctx *ctx, int64_t *count_host, void *stream) {
  if (!ctx || !count_host) { set_error("take_index_errors: null argument"); return THCB200_ERR_ARG; }
  THCB_CTX_LOCK(ctx);
  cudaStream_t st = (cudaStream_t)stream;
  unsigned int *errors = reinterpret_cast<unsigned int *>(ctx->status) + 1;
  THCB_CUDA_TRY(cudaMemcpyAsync(ctx->host_slot, errors, sizeof(unsigned int), cudaMemcpyDeviceToHost, st));
  THCB_CUDA_TRY(cudaMemsetAsync(errors, 0, sizeof(unsigned int), st));
  THCB_CUDA_TRY(cudaStreamSynchronize(st));
  unsigned int c = 0;
  memcpy(&c, ctx->host_slot, sizeof(c));
  *count_host = (int64_t)c;
  return THCB200_OK;
}

}  // extern "C"
