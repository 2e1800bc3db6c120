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
 * is done by the host functions exported from libthcb200 (thcb200.h).  The kernels decode offsets
 * with multiply-high divisions, take four elements per thread, and are compiled with non-aliasing
 * pointers when the operands sit in storages that do not overlap (so the loads of the four
 * elements can be in flight together); the memory pattern itself is the functor's: a transposed
 * operand is read the way its strides say, since pointer-taking functors cannot be staged through
 * shared memory.
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

// A thread takes kPerThread elements, kThreads apart (neighbouring lanes on neighbouring elements),
// decodes all their offsets first and then runs the functor on each.  NOALIAS (picked on the host
// when the operands' memory ranges are disjoint) lets the compiler start the loads of all four
// before the first store; otherwise a store through one pointer orders every later load.
#define THCB_USER_PTR(T, NOALIAS) typename PtrOf<T, NOALIAS>::type
template <typename T, bool NOALIAS> struct PtrOf { typedef T *type; };
template <typename T> struct PtrOf<T, true> { typedef T *__restrict__ type; };

template <typename Op, typename Ta, typename IndexT>
__global__ void __launch_bounds__(kThreads) apply1_kernel(Ta *a, View<IndexT> va, IndexT n, Op op) {
  const IndexT step = (IndexT)gridDim.x * (kThreads * kPerThread);
  for (IndexT base = (IndexT)blockIdx.x * (kThreads * kPerThread) + threadIdx.x; base < n; base += step) {
    IndexT oa[kPerThread];
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      const IndexT i = base + (IndexT)u * kThreads;
      oa[u] = (i < n && i >= base) ? va.offset(i) : 0;
    }
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      const IndexT i = base + (IndexT)u * kThreads;
      if (i < n && i >= base) op(&a[oa[u]]);
    }
    if (base + step < base) break;   // the index type would wrap
  }
}
template <typename Op, typename Ta, typename Tb, typename IndexT, bool NOALIAS>
__global__ void __launch_bounds__(kThreads)
apply2_kernel(THCB_USER_PTR(Ta, NOALIAS) a, View<IndexT> va, THCB_USER_PTR(Tb, NOALIAS) b, View<IndexT> vb, IndexT n, Op op) {
  const IndexT step = (IndexT)gridDim.x * (kThreads * kPerThread);
  for (IndexT base = (IndexT)blockIdx.x * (kThreads * kPerThread) + threadIdx.x; base < n; base += step) {
    IndexT oa[kPerThread], ob[kPerThread];
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      const IndexT i = base + (IndexT)u * kThreads;
      const bool ok = i < n && i >= base;
      oa[u] = ok ? va.offset(i) : 0;
      ob[u] = ok ? vb.offset(i) : 0;
    }
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      const IndexT i = base + (IndexT)u * kThreads;
      if (i < n && i >= base) op(&a[oa[u]], &b[ob[u]]);
    }
    if (base + step < base) break;
  }
}
template <typename Op, typename Ta, typename Tb, typename Tc, typename IndexT, bool NOALIAS>
__global__ void __launch_bounds__(kThreads)
apply3_kernel(THCB_USER_PTR(Ta, NOALIAS) a, View<IndexT> va, THCB_USER_PTR(Tb, NOALIAS) b, View<IndexT> vb,
              THCB_USER_PTR(Tc, NOALIAS) c, View<IndexT> vc, IndexT n, Op op) {
  const IndexT step = (IndexT)gridDim.x * (kThreads * kPerThread);
  for (IndexT base = (IndexT)blockIdx.x * (kThreads * kPerThread) + threadIdx.x; base < n; base += step) {
    IndexT oa[kPerThread], ob[kPerThread], oc[kPerThread];
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      const IndexT i = base + (IndexT)u * kThreads;
      const bool ok = i < n && i >= base;
      oa[u] = ok ? va.offset(i) : 0;
      ob[u] = ok ? vb.offset(i) : 0;
      oc[u] = ok ? vc.offset(i) : 0;
    }
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      const IndexT i = base + (IndexT)u * kThreads;
      if (i < n && i >= base) op(&a[oa[u]], &b[ob[u]], &c[oc[u]]);
    }
    if (base + step < base) break;
  }
}
#undef THCB_USER_PTR

inline unsigned grid_for(int64_t n) {
  // enough CTAs to fill a B200 several times over; the kernels stride over the rest
  int64_t blocks = (n + kThreads * kPerThread - 1) / (kThreads * kPerThread);
  const int64_t cap = 148 * 16;  // keeps the loop's step inside 32 bits for every n the 32-bit path accepts
  return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
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
    if (thcb200_can_use_32bit(&da))
      apply1_kernel<Op, Ta, uint32_t><<<grid_for(n), kThreads, 0, st>>>((Ta *)da.data, collapse<uint32_t>(da), (uint32_t)n, op);
    else
      apply1_kernel<Op, Ta, uint64_t><<<grid_for(n), kThreads, 0, st>>>((Ta *)da.data, collapse<uint64_t>(da), (uint64_t)n, op);
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
    const bool i32 = thcb200_can_use_32bit(&da) && thcb200_can_use_32bit(&db);
#define THCB_USER_LAUNCH2(IDX, NA)                                                                                   \
  apply2_kernel<Op, Ta, Tb, IDX, NA><<<grid_for(n), kThreads, 0, st>>>((Ta *)da.data, collapse<IDX>(da), (Tb *)db.data, \
                                                                       collapse<IDX>(db), (IDX)n, op)
    if (i32) { if (apart) THCB_USER_LAUNCH2(uint32_t, true); else THCB_USER_LAUNCH2(uint32_t, false); }
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
    const bool i32 = thcb200_can_use_32bit(&da) && thcb200_can_use_32bit(&db) && thcb200_can_use_32bit(&dc);
#define THCB_USER_LAUNCH3(IDX, NA)                                                                                       \
  apply3_kernel<Op, Ta, Tb, Tc, IDX, NA><<<grid_for(n), kThreads, 0, st>>>((Ta *)da.data, collapse<IDX>(da), (Tb *)db.data, \
                                                                           collapse<IDX>(db), (Tc *)dc.data, collapse<IDX>(dc), (IDX)n, op)
    if (i32) { if (apart) THCB_USER_LAUNCH3(uint32_t, true); else THCB_USER_LAUNCH3(uint32_t, false); }
    else { if (apart) THCB_USER_LAUNCH3(uint64_t, true); else THCB_USER_LAUNCH3(uint64_t, false); }
#undef THCB_USER_LAUNCH3
  }
  restore_overlap(state, a, oa);
  restore_overlap(state, b, ob);
  restore_overlap(state, c, oc);
  return true;
}

#endif /* THCB200_THC_APPLY_CUH */
