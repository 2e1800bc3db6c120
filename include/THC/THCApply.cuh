/*
 * THCApply.cuh -- the C++ template face of the pointwise apply for user-defined functors.
 *
 * cutorch installs THC_pointwiseApply1/2/3 as templates (lib/THC/THCApply.cuh:124-129, 247-255,
 * 422-433) so that downstream CUDA code (cunn and friends) can run its own functors over
 * arbitrarily strided tensors.  A functor receives element POINTERS and may reach neighbours
 * through them (TensorCrossOp, TensorTriOp), so this path cannot use the value-semantics fast
 * kernels of the built-in op table; it keeps the reference's contract instead:
 *
 *   template <typename TensorTypeA, typename Op>
 *   bool THC_pointwiseApply1(THCState*, TensorTypeA* a, const Op& op, TensorArgType aType = ReadWrite);
 *   ... THC_pointwiseApply2 / THC_pointwiseApply3 likewise, b and c defaulting to ReadOnly.
 *
 * Semantics kept: operands need equal element counts, not equal shapes, and each is walked in its
 * own row-major order; more than 25 dims or a count mismatch returns false; a tensor without
 * dimensions is a no-op returning true; a ReadWrite / WriteOnly operand whose index tuples alias is
 * replaced by a contiguous copy and copied back (copyIgnoringOverlaps); the launch goes to the
 * THCState's current stream.  Layout planning (collapseDims, overlap test, 32- vs 64-bit indices)
 * is done by the host functions exported from libthcb200 (thcb200.h).  Three walks:
 *   dense    every operand one stride-1 run on a 16-byte boundary, storages apart: a thread takes
 *            runs of 16 bytes of consecutive elements, which the compiler merges into 16-byte
 *            accesses through the functor's pointers;
 *   patch    some operand is a transposed matrix: threads are assigned to elements patch by patch
 *            (32 x 32) instead of in index order, so that operands dense along either direction
 *            are touched in short runs whose lines the CTA finishes out of the L1 (a pointer-taking
 *            functor cannot be staged through shared memory, but which thread runs it is free);
 *   plain    anything else: index order, four elements per thread, offsets decoded together.
 * Views of at most two collapsed dims use a form with one multiply-high division at most (none in
 * the patch walk); deeper ones decode dim by dim.  The kernels are compiled with non-aliasing
 * pointers when the operands sit in storages that do not overlap, so that the loads of a thread's
 * elements can be in flight together.
 *
 * Include this header from a .cu file compiled for sm_100a and link libthcb200.
 */
#ifndef THCB200_THC_APPLY_CUH
#define THCB200_THC_APPLY_CUH

#include <cuda_runtime.h>
#include <stdint.h>

#include "../thcb200.h"
#include "THC.h"

enum TensorArgType { ReadWrite, ReadOnly };

namespace thcb_user {

// Element type and struct access for the eight THC tensor types.
template <typename TensorType> struct TensorAccess;
#define THCB_USER_ACCESS(TENSOR, REAL, DTYPE)                                                                  \
  template <> struct TensorAccess<TENSOR> {                                                                    \
    typedef REAL DataType;                                                                                     \
    static const int dtype = DTYPE;                                                                            \
    static TENSOR *newContiguous(THCState *s, TENSOR *t) { return TENSOR##_newContiguous(s, t); }             \
    static void copyIgnoringOverlaps(THCState *s, TENSOR *d, TENSOR *t) { TENSOR##_copyIgnoringOverlaps(s, d, t); } \
    static void free(THCState *s, TENSOR *t) { TENSOR##_free(s, t); }                                          \
  };
THCB_USER_ACCESS(THCudaByteTensor, unsigned char, THCB200_U8)
THCB_USER_ACCESS(THCudaCharTensor, char, THCB200_I8)
THCB_USER_ACCESS(THCudaShortTensor, short, THCB200_I16)
THCB_USER_ACCESS(THCudaIntTensor, int, THCB200_I32)
THCB_USER_ACCESS(THCudaLongTensor, long, THCB200_I64)
THCB_USER_ACCESS(THCudaHalfTensor, half, THCB200_F16)
THCB_USER_ACCESS(THCudaTensor, float, THCB200_F32)
THCB_USER_ACCESS(THCudaDoubleTensor, double, THCB200_F64)
#undef THCB_USER_ACCESS

// Collapsed view of one operand as the kernel sees it.  With 32-bit indices the per-dim division
// is a multiply-high by a constant worked out on the host (n / d = (umulhi(n, mul) + n) >> shift for
// n < 2^32, round-up method of Granlund and Montgomery) instead of a hardware divide.
template <typename IndexT> struct Divisor;
template <> struct Divisor<uint32_t> {
  uint32_t d, mul, shift;
  void set(uint64_t div) {
    d = (uint32_t)div;
    for (shift = 0; shift < 32; ++shift)
      if ((1ULL << shift) >= div) break;
    mul = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << shift) - div)) / div + 1);
  }
  __device__ __forceinline__ uint32_t quotient(uint32_t n) const { return (uint32_t)(((uint64_t)__umulhi(n, mul) + n) >> shift); }
};
template <> struct Divisor<uint64_t> {
  uint64_t d;
  void set(uint64_t div) { d = div; }
  __device__ __forceinline__ uint64_t quotient(uint64_t n) const { return n / d; }
};

template <typename IndexT>
struct View {
  int dims;
  Divisor<IndexT> sizes[THCB200_MAX_DIMS];
  IndexT strides[THCB200_MAX_DIMS];
  __device__ __forceinline__ IndexT offset(IndexT linear) const {
    if (dims == 1) return linear * strides[0];
    IndexT off = 0;
    for (int d = dims - 1; d > 0; --d) {
      const IndexT q = sizes[d].quotient(linear);
      off += (linear - q * sizes[d].d) * strides[d];
      linear = q;
    }
    return off + linear * strides[0];
  }
  __device__ __forceinline__ IndexT offset(IndexT linear, IndexT, IndexT) const { return offset(linear); }
};

// A view of at most two collapsed dims, its sizes known when the kernel is compiled: one division
// at most, and none when the walk already knows the element's (row, column) in this view's own
// shape (`by_row_col`: a patch walk whose N is this view's inner size, or any 1-D view).
template <typename IndexT>
struct View2 {
  Divisor<IndexT> inner;   // size of the inner dim (of the whole view if it has one dim)
  IndexT s0, s1;           // strides of the outer and the inner dim
  bool by_row_col;
  __device__ __forceinline__ IndexT offset(IndexT linear, IndexT row, IndexT col) const {
    if (by_row_col) return row * s0 + col * s1;
    const IndexT q = inner.quotient(linear);
    return q * s0 + (linear - q * inner.d) * s1;
  }
};

template <typename TensorType>
inline thcb200_tensor describe(TensorType *t) {
  thcb200_tensor d;
  d.dtype = TensorAccess<TensorType>::dtype;
  d.ndim = t->nDimension;
  for (int i = 0; i < t->nDimension && i < THCB200_MAX_DIMS; ++i) { d.sizes[i] = t->size[i]; d.strides[i] = t->stride[i]; }
  d.data = t->storage ? (void *)(t->storage->data + t->storageOffset) : 0;
  return d;
}

template <typename IndexT>
inline View<IndexT> collapse(const thcb200_tensor &d) {
  int64_t sz[THCB200_MAX_DIMS], st[THCB200_MAX_DIMS];
  int nd = d.ndim;
  for (int i = 0; i < nd; ++i) { sz[i] = d.sizes[i]; st[i] = d.strides[i]; }
  thcb200_collapse_dims(sz, st, &nd, -1);
  View<IndexT> v;
  v.dims = nd;
  for (int i = 0; i < nd; ++i) { v.sizes[i].set((uint64_t)sz[i]); v.strides[i] = (IndexT)st[i]; }
  return v;
}

inline int64_t numel(const thcb200_tensor &d) {
  if (d.ndim <= 0) return 0;
  int64_t n = 1;
  for (int i = 0; i < d.ndim; ++i) n *= d.sizes[i];
  return n;
}

constexpr int kThreads = 256;
constexpr int kPerThread = 4;   // elements per thread and step: their offsets are decoded together
constexpr int kSlotsPerBlock = kThreads * kPerThread;

// Which element a thread takes.  Plain walk: block `blk` covers kSlotsPerBlock consecutive logical
// indices, neighbouring lanes on neighbouring elements.  Patch walk (N != 0), chosen on the host
// when some operand is a transposed matrix (its innermost collapsed dim is strided and the next one
// is dense): the logical index space is seen as rows x N, a block covers a 32 x 32 patch of it, a
// warp four rows of it and a warp instruction a piece of 4 rows x 8 columns, so that every operand
// is touched in runs of 16 or 32 bytes and the rest of each line is used by the same CTA out of the
// L1.  Only the assignment of elements to threads changes: the functor still gets the element's
// own pointers.  (Measured on a 16384 x 8192 fp32 transposed source: pieces of 8 x 4 or 2 x 16
// instead of 4 x 8, patches numbered in 8 x 8 clusters instead of row by row, and eight elements per
// thread were each slower.  With a dim-by-dim offset decode the kernel was bound by instruction
// issue, hence the short index arithmetic here and in View2.)
template <typename IndexT>
struct Walk {
  IndexT n, nblk;
  IndexT N, rows;
  Divisor<IndexT> patches_per_row;
  template <int PT>
  __device__ __forceinline__ bool slot(IndexT blk, int u, IndexT &i, IndexT &row, IndexT &col) const {
    if (N == 0) {
      i = blk * (IndexT)(kThreads * PT) + (IndexT)(u * kThreads) + threadIdx.x;
      row = 0;
      col = i;
      return i < n;
    }
    const IndexT pr = patches_per_row.quotient(blk), pc = blk - pr * patches_per_row.d;
    row = pr * 32 + (threadIdx.x >> 3);                        // warp w: rows 4w .. 4w+3 of the patch
    col = pc * (IndexT)(8 * PT) + (IndexT)(u * 8) + (threadIdx.x & 7);
    i = row * N + col;
    return row < rows && col < N;
  }
};
static_assert(kThreads == 256, "a block of the patch walk is 32 rows (8 warps x 4) x 8 columns per element of a thread");
constexpr int kPerThreadPatch = 4;   // elements per thread in the patch walk: patches of 32 rows x 32 columns (8 per thread: 215 -> 268 us)
static_assert(kPerThreadPatch == kPerThread, "views of more than two dims take the patch walk in the kernels built for kPerThread");

// N of the patch walk this operand asks for, or 0
template <typename IndexT>
inline uint64_t wants_patches(const View<IndexT> &v) {
  if (v.dims < 2 || v.strides[v.dims - 1] == 1 || v.strides[v.dims - 2] != 1) return 0;
  return v.sizes[v.dims - 1].d >= 16 ? (uint64_t)v.sizes[v.dims - 1].d : 0;
}
// A patch walk (w.N != 0) is for the kernels with kPerThreadPatch elements per thread, a plain one
// for those with kPerThread.
template <typename IndexT>
inline Walk<IndexT> make_walk(uint64_t n, uint64_t patchN) {
  Walk<IndexT> w;
  w.n = (IndexT)n;
  w.N = 0;
  w.rows = 0;
  w.patches_per_row.set(1);
  const uint64_t width = 8ull * kPerThreadPatch;
  w.nblk = (IndexT)((n + kSlotsPerBlock - 1) / kSlotsPerBlock);
  if (patchN && n / patchN >= 16) {
    const uint64_t rows = n / patchN, ppr = (patchN + width - 1) / width, blocks = (rows + 31) / 32 * ppr;
    if (blocks < (1ull << 31)) {
      w.N = (IndexT)patchN;
      w.rows = (IndexT)rows;
      w.patches_per_row.set(ppr);
      w.nblk = (IndexT)blocks;
    }
  }
  return w;
}
// the two-dim form of a collapsed view of at most two dims, for this walk
template <typename IndexT>
inline View2<IndexT> two_dims(const View<uint64_t> &v, const Walk<IndexT> &w, uint64_t n) {
  View2<IndexT> r;
  if (v.dims <= 1) {
    // one run of stride s: element (row, col) of any rows x N reading of the index space sits at (row * N + col) * s
    const uint64_t st = v.dims == 1 ? v.strides[0] : 0;
    r.inner.set(n ? n : 1);
    r.s0 = (IndexT)((w.N ? (uint64_t)w.N : 0) * st);
    r.s1 = (IndexT)st;
    r.by_row_col = true;        // plain walk: row = 0, col = the index
  } else {
    r.inner.set(v.sizes[1].d);
    r.s0 = (IndexT)v.strides[0];
    r.s1 = (IndexT)v.strides[1];
    r.by_row_col = w.N != 0 && (uint64_t)w.N == v.sizes[1].d;
  }
  return r;
}
// the 32-bit kernels count slots up to the next multiple of kSlotsPerBlock
inline bool slots_fit_32bit(int64_t n) { return (uint64_t)n + kSlotsPerBlock < (1ull << 32); }

// A thread takes kPerThread elements, decodes all their offsets first and then runs the functor on
// each.  NOALIAS (picked on the host when the operands' memory ranges are disjoint) lets the
// compiler start the loads of all four before the first store; otherwise a store through one
// pointer orders every later load.
#define THCB_USER_PTR(T, NOALIAS) typename PtrOf<T, NOALIAS>::type
template <typename T, bool NOALIAS> struct PtrOf { typedef T *type; };
template <typename T> struct PtrOf<T, true> { typedef T *__restrict__ type; };

template <typename Op, typename Ta, typename IndexT, typename ViewT, int PT>
__global__ void __launch_bounds__(kThreads) apply1_kernel(Ta *a, ViewT va, Walk<IndexT> w, Op op) {
  for (IndexT blk = blockIdx.x; blk < w.nblk; blk += gridDim.x) {
    IndexT oa[PT];
    bool ok[PT];
#pragma unroll
    for (int u = 0; u < PT; ++u) {
      IndexT i, row, col;
      ok[u] = w.template slot<PT>(blk, u, i, row, col);
      oa[u] = va.offset(i, row, col);
    }
#pragma unroll
    for (int u = 0; u < PT; ++u)
      if (ok[u]) op(&a[oa[u]]);
  }
}
template <typename Op, typename Ta, typename Tb, typename IndexT, bool NOALIAS, typename ViewT, int PT>
__global__ void __launch_bounds__(kThreads)
apply2_kernel(THCB_USER_PTR(Ta, NOALIAS) a, ViewT va, THCB_USER_PTR(Tb, NOALIAS) b, ViewT vb, Walk<IndexT> w, Op op) {
  for (IndexT blk = blockIdx.x; blk < w.nblk; blk += gridDim.x) {
    IndexT oa[PT], ob[PT];
    bool ok[PT];
#pragma unroll
    for (int u = 0; u < PT; ++u) {
      IndexT i, row, col;
      ok[u] = w.template slot<PT>(blk, u, i, row, col);
      oa[u] = va.offset(i, row, col);
      ob[u] = vb.offset(i, row, col);
    }
#pragma unroll
    for (int u = 0; u < PT; ++u)
      if (ok[u]) op(&a[oa[u]], &b[ob[u]]);
  }
}
template <typename Op, typename Ta, typename Tb, typename Tc, typename IndexT, bool NOALIAS, typename ViewT, int PT>
__global__ void __launch_bounds__(kThreads)
apply3_kernel(THCB_USER_PTR(Ta, NOALIAS) a, ViewT va, THCB_USER_PTR(Tb, NOALIAS) b, ViewT vb,
              THCB_USER_PTR(Tc, NOALIAS) c, ViewT vc, Walk<IndexT> w, Op op) {
  for (IndexT blk = blockIdx.x; blk < w.nblk; blk += gridDim.x) {
    IndexT oa[PT], ob[PT], oc[PT];
    bool ok[PT];
#pragma unroll
    for (int u = 0; u < PT; ++u) {
      IndexT i, row, col;
      ok[u] = w.template slot<PT>(blk, u, i, row, col);
      oa[u] = va.offset(i, row, col);
      ob[u] = vb.offset(i, row, col);
      oc[u] = vc.offset(i, row, col);
    }
#pragma unroll
    for (int u = 0; u < PT; ++u)
      if (ok[u]) op(&a[oa[u]], &b[ob[u]], &c[oc[u]]);
  }
}

// Dense operands (every one a single stride-1 run, 16-byte aligned, in storages that do not overlap):
// a thread takes runs of kRun consecutive elements, so that the compiler can merge the functor's
// element accesses into 16-byte ones; two runs per step.
template <int A, int B, int C> struct MinSize { static const int value = A < B ? (A < C ? A : C) : (B < C ? B : C); };
template <typename Op, typename Ta, int RUN>
__global__ void __launch_bounds__(kThreads) apply1_dense_kernel(Ta *__restrict__ a, uint64_t n, Op op) {
  const uint64_t nruns = (n + RUN - 1) / RUN;
  for (uint64_t r = (uint64_t)blockIdx.x * kThreads + threadIdx.x; r < nruns; r += (uint64_t)gridDim.x * kThreads) {
    Ta *pa = (Ta *)__builtin_assume_aligned(a + r * RUN, 16);
    if ((r + 1) * RUN <= n) {
#pragma unroll
      for (int j = 0; j < RUN; ++j) op(pa + j);
    } else {
      for (uint64_t j = 0; r * RUN + j < n; ++j) op(pa + j);
    }
  }
}
template <typename Op, typename Ta, typename Tb, int RUN>
__global__ void __launch_bounds__(kThreads) apply2_dense_kernel(Ta *__restrict__ a, Tb *__restrict__ b, uint64_t n, Op op) {
  const uint64_t nruns = (n + RUN - 1) / RUN;
  for (uint64_t r = (uint64_t)blockIdx.x * kThreads + threadIdx.x; r < nruns; r += (uint64_t)gridDim.x * kThreads) {
    Ta *pa = (Ta *)__builtin_assume_aligned(a + r * RUN, 16);
    Tb *pb = (Tb *)__builtin_assume_aligned(b + r * RUN, 16);
    if ((r + 1) * RUN <= n) {
#pragma unroll
      for (int j = 0; j < RUN; ++j) op(pa + j, pb + j);
    } else {
      for (uint64_t j = 0; r * RUN + j < n; ++j) op(pa + j, pb + j);
    }
  }
}
template <typename Op, typename Ta, typename Tb, typename Tc, int RUN>
__global__ void __launch_bounds__(kThreads)
apply3_dense_kernel(Ta *__restrict__ a, Tb *__restrict__ b, Tc *__restrict__ c, uint64_t n, Op op) {
  const uint64_t nruns = (n + RUN - 1) / RUN;
  for (uint64_t r = (uint64_t)blockIdx.x * kThreads + threadIdx.x; r < nruns; r += (uint64_t)gridDim.x * kThreads) {
    Ta *pa = (Ta *)__builtin_assume_aligned(a + r * RUN, 16);
    Tb *pb = (Tb *)__builtin_assume_aligned(b + r * RUN, 16);
    Tc *pc = (Tc *)__builtin_assume_aligned(c + r * RUN, 16);
    if ((r + 1) * RUN <= n) {
#pragma unroll
      for (int j = 0; j < RUN; ++j) op(pa + j, pb + j, pc + j);
    } else {
      for (uint64_t j = 0; r * RUN + j < n; ++j) op(pa + j, pb + j, pc + j);
    }
  }
}
#undef THCB_USER_PTR

inline unsigned grid_for_blocks(uint64_t blocks) {
  // enough CTAs to fill a B200 several times over; the kernels stride over the rest
  const uint64_t cap = 148 * 16;
  return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}
// one stride-1 run starting on a 16-byte boundary
template <typename IndexT>
inline bool dense_aligned(const View<IndexT> &v, const void *data) {
  return v.dims == 1 && v.strides[0] == 1 && ((uintptr_t)data & 15) == 0;
}

// True when the two tensors live in storages whose memory does not overlap: the kernels may then
// be told that their pointers do not alias.  Storages, not views: a functor may reach neighbours of
// its element through the pointer, but never leaves the tensor's storage.
template <typename TensorTypeA, typename TensorTypeB>
inline bool storages_apart(TensorTypeA *a, TensorTypeB *b) {
  if (!a->storage || !b->storage || !a->storage->data || !b->storage->data) return false;
  const uintptr_t al = (uintptr_t)a->storage->data, bl = (uintptr_t)b->storage->data;
  const uintptr_t ah = al + (size_t)a->storage->size * sizeof(typename TensorAccess<TensorTypeA>::DataType);
  const uintptr_t bh = bl + (size_t)b->storage->size * sizeof(typename TensorAccess<TensorTypeB>::DataType);
  return ah <= bl || bh <= al;
}

// Replaces an aliasing ReadWrite operand by a contiguous copy; `orig` remembers the original.
template <typename TensorType>
inline void fix_overlap(THCState *state, TensorType *&t, TensorType *&orig, TensorArgType type) {
  orig = 0;
  thcb200_tensor d = describe(t);
  if (type == ReadWrite && thcb200_overlapping(&d)) {
    orig = t;
    t = TensorAccess<TensorType>::newContiguous(state, t);
  }
}
template <typename TensorType>
inline void restore_overlap(THCState *state, TensorType *t, TensorType *orig) {
  if (orig) {
    TensorAccess<TensorType>::copyIgnoringOverlaps(state, orig, t);
    TensorAccess<TensorType>::free(state, t);
  }
}

}  // namespace thcb_user

template <typename TensorTypeA, typename Op>
bool THC_pointwiseApply1(THCState *state, TensorTypeA *a, const Op &op, TensorArgType aType = ReadWrite) {
  using namespace thcb_user;
  if (a->nDimension > THCB200_MAX_DIMS) return false;
  if (a->nDimension == 0) return true;
  TensorTypeA *oa;
  fix_overlap(state, a, oa, aType);
  thcb200_tensor da = describe(a);
  const int64_t n = numel(da);
  cudaStream_t st = THCState_getCurrentStream(state);
  typedef typename TensorAccess<TensorTypeA>::DataType Ta;
  if (n > 0) {
    const View<uint64_t> va = collapse<uint64_t>(da);
    constexpr int RUN = 16 / (int)sizeof(Ta);
    if (dense_aligned(va, da.data)) {
      apply1_dense_kernel<Op, Ta, RUN><<<grid_for_blocks(((uint64_t)n + RUN * kThreads - 1) / (RUN * kThreads)), kThreads, 0, st>>>((Ta *)da.data, (uint64_t)n, op);
    } else if (thcb200_can_use_32bit(&da) && slots_fit_32bit(n)) {
      const uint64_t patchN = va.dims <= 2 ? wants_patches(va) : 0;
      const Walk<uint32_t> w = make_walk<uint32_t>((uint64_t)n, patchN);
      if (w.N)
        apply1_kernel<Op, Ta, uint32_t, View2<uint32_t>, kPerThreadPatch><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>((Ta *)da.data, two_dims(va, w, (uint64_t)n), w, op);
      else if (va.dims <= 2)
        apply1_kernel<Op, Ta, uint32_t, View2<uint32_t>, kPerThread><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>((Ta *)da.data, two_dims(va, w, (uint64_t)n), w, op);
      else
        apply1_kernel<Op, Ta, uint32_t, View<uint32_t>, kPerThread><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>((Ta *)da.data, collapse<uint32_t>(da), w, op);
    } else {
      const Walk<uint64_t> w = make_walk<uint64_t>((uint64_t)n, 0);
      apply1_kernel<Op, Ta, uint64_t, View<uint64_t>, kPerThread><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>((Ta *)da.data, va, w, op);
    }
  }
  restore_overlap(state, a, oa);
  return true;
}

template <typename TensorTypeA, typename TensorTypeB, typename Op>
bool THC_pointwiseApply2(THCState *state, TensorTypeA *a, TensorTypeB *b, const Op &op, TensorArgType aType = ReadWrite,
                         TensorArgType bType = ReadOnly) {
  using namespace thcb_user;
  if (a->nDimension > THCB200_MAX_DIMS || b->nDimension > THCB200_MAX_DIMS) return false;
  thcb200_tensor ta = describe(a), tb = describe(b);
  if (numel(ta) != numel(tb)) return false;
  if (a->nDimension == 0) return true;
  TensorTypeA *oa;
  TensorTypeB *ob;
  fix_overlap(state, a, oa, aType);
  fix_overlap(state, b, ob, bType);
  thcb200_tensor da = describe(a), db = describe(b);
  const int64_t n = numel(da);
  cudaStream_t st = THCState_getCurrentStream(state);
  typedef typename TensorAccess<TensorTypeA>::DataType Ta;
  typedef typename TensorAccess<TensorTypeB>::DataType Tb;
  if (n > 0) {
    const bool apart = storages_apart(a, b);
    const bool i32 = thcb200_can_use_32bit(&da) && thcb200_can_use_32bit(&db) && slots_fit_32bit(n);
    const View<uint64_t> va = collapse<uint64_t>(da), vb = collapse<uint64_t>(db);
    uint64_t patchN = wants_patches(va);
    if (!patchN) patchN = wants_patches(vb);
    constexpr int RUN = 16 / MinSize<(int)sizeof(Ta), (int)sizeof(Tb), 16>::value;
#define THCB_USER_LAUNCH2(IDX, NA)                                                                                   \
  do {                                                                                                               \
    const bool two = sizeof(IDX) == 4 && va.dims <= 2 && vb.dims <= 2;                                               \
    const Walk<IDX> w = make_walk<IDX>((uint64_t)n, patchN);                                                     \
    if (two && w.N)                                                                                                  \
      apply2_kernel<Op, Ta, Tb, IDX, NA, View2<IDX>, kPerThreadPatch><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>( \
          (Ta *)da.data, two_dims(va, w, (uint64_t)n), (Tb *)db.data, two_dims(vb, w, (uint64_t)n), w, op);         \
    else if (two)                                                                                                    \
      apply2_kernel<Op, Ta, Tb, IDX, NA, View2<IDX>, kPerThread><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>(      \
          (Ta *)da.data, two_dims(va, w, (uint64_t)n), (Tb *)db.data, two_dims(vb, w, (uint64_t)n), w, op);         \
    else                                                                                                             \
      apply2_kernel<Op, Ta, Tb, IDX, NA, View<IDX>, kPerThread><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>(       \
          (Ta *)da.data, collapse<IDX>(da), (Tb *)db.data, collapse<IDX>(db), w, op);                               \
  } while (0)
    if (apart && dense_aligned(va, da.data) && dense_aligned(vb, db.data))
      apply2_dense_kernel<Op, Ta, Tb, RUN><<<grid_for_blocks(((uint64_t)n + 2 * RUN * kThreads - 1) / (2 * RUN * kThreads)), kThreads, 0, st>>>(
          (Ta *)da.data, (Tb *)db.data, (uint64_t)n, op);
    else if (i32) { if (apart) THCB_USER_LAUNCH2(uint32_t, true); else THCB_USER_LAUNCH2(uint32_t, false); }
    else { if (apart) THCB_USER_LAUNCH2(uint64_t, true); else THCB_USER_LAUNCH2(uint64_t, false); }
#undef THCB_USER_LAUNCH2
  }
  restore_overlap(state, a, oa);
  restore_overlap(state, b, ob);
  return true;
}

template <typename TensorTypeA, typename TensorTypeB, typename TensorTypeC, typename Op>
bool THC_pointwiseApply3(THCState *state, TensorTypeA *a, TensorTypeB *b, TensorTypeC *c, const Op &op,
                         TensorArgType aType = ReadWrite, TensorArgType bType = ReadOnly, TensorArgType cType = ReadOnly) {
  using namespace thcb_user;
  if (a->nDimension > THCB200_MAX_DIMS || b->nDimension > THCB200_MAX_DIMS || c->nDimension > THCB200_MAX_DIMS) return false;
  thcb200_tensor ta = describe(a), tb = describe(b), tc = describe(c);
  if (numel(ta) != numel(tb) || numel(ta) != numel(tc)) return false;
  if (a->nDimension == 0) return true;
  TensorTypeA *oa;
  TensorTypeB *ob;
  TensorTypeC *oc;
  fix_overlap(state, a, oa, aType);
  fix_overlap(state, b, ob, bType);
  fix_overlap(state, c, oc, cType);
  thcb200_tensor da = describe(a), db = describe(b), dc = describe(c);
  const int64_t n = numel(da);
  cudaStream_t st = THCState_getCurrentStream(state);
  typedef typename TensorAccess<TensorTypeA>::DataType Ta;
  typedef typename TensorAccess<TensorTypeB>::DataType Tb;
  typedef typename TensorAccess<TensorTypeC>::DataType Tc;
  if (n > 0) {
    const bool apart = storages_apart(a, b) && storages_apart(a, c) && storages_apart(b, c);
    const bool i32 = thcb200_can_use_32bit(&da) && thcb200_can_use_32bit(&db) && thcb200_can_use_32bit(&dc) && slots_fit_32bit(n);
    const View<uint64_t> va = collapse<uint64_t>(da), vb = collapse<uint64_t>(db), vc = collapse<uint64_t>(dc);
    uint64_t patchN = wants_patches(va);
    if (!patchN) patchN = wants_patches(vb);
    if (!patchN) patchN = wants_patches(vc);
    constexpr int RUN = 16 / MinSize<(int)sizeof(Ta), (int)sizeof(Tb), (int)sizeof(Tc)>::value;
#define THCB_USER_LAUNCH3(IDX, NA)                                                                                       \
  do {                                                                                                                   \
    const bool two = sizeof(IDX) == 4 && va.dims <= 2 && vb.dims <= 2 && vc.dims <= 2;                                   \
    const Walk<IDX> w = make_walk<IDX>((uint64_t)n, patchN);                                                         \
    if (two && w.N)                                                                                                      \
      apply3_kernel<Op, Ta, Tb, Tc, IDX, NA, View2<IDX>, kPerThreadPatch><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>( \
          (Ta *)da.data, two_dims(va, w, (uint64_t)n), (Tb *)db.data, two_dims(vb, w, (uint64_t)n), (Tc *)dc.data,      \
          two_dims(vc, w, (uint64_t)n), w, op);                                                                          \
    else if (two)                                                                                                        \
      apply3_kernel<Op, Ta, Tb, Tc, IDX, NA, View2<IDX>, kPerThread><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>(      \
          (Ta *)da.data, two_dims(va, w, (uint64_t)n), (Tb *)db.data, two_dims(vb, w, (uint64_t)n), (Tc *)dc.data,      \
          two_dims(vc, w, (uint64_t)n), w, op);                                                                          \
    else                                                                                                                 \
      apply3_kernel<Op, Ta, Tb, Tc, IDX, NA, View<IDX>, kPerThread><<<grid_for_blocks(w.nblk), kThreads, 0, st>>>(       \
          (Ta *)da.data, collapse<IDX>(da), (Tb *)db.data, collapse<IDX>(db), (Tc *)dc.data, collapse<IDX>(dc), w, op);  \
  } while (0)
    if (apart && dense_aligned(va, da.data) && dense_aligned(vb, db.data) && dense_aligned(vc, dc.data))
      apply3_dense_kernel<Op, Ta, Tb, Tc, RUN><<<grid_for_blocks(((uint64_t)n + 2 * RUN * kThreads - 1) / (2 * RUN * kThreads)), kThreads, 0, st>>>(
          (Ta *)da.data, (Tb *)db.data, (Tc *)dc.data, (uint64_t)n, op);
    else if (i32) { if (apart) THCB_USER_LAUNCH3(uint32_t, true); else THCB_USER_LAUNCH3(uint32_t, false); }
    else { if (apart) THCB_USER_LAUNCH3(uint64_t, true); else THCB_USER_LAUNCH3(uint64_t, false); }
#undef THCB_USER_LAUNCH3
  }
  restore_overlap(state, a, oa);
  restore_overlap(state, b, ob);
  restore_overlap(state, c, oc);
  return true;
}

#endif /* THCB200_THC_APPLY_CUH */
