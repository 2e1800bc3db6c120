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
 * is done by the host functions exported from libthcb200 (thcb200.h).
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

// Collapsed view of one operand as the kernel sees it.
template <typename IndexT>
struct View {
  int dims;
  IndexT sizes[THCB200_MAX_DIMS];
  IndexT strides[THCB200_MAX_DIMS];
  __device__ __forceinline__ IndexT offset(IndexT linear) const {
    if (dims == 1) return linear * strides[0];
    IndexT off = 0;
    for (int d = dims - 1; d > 0; --d) {
      const IndexT q = linear / sizes[d];
      off += (linear - q * sizes[d]) * strides[d];
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
  for (int i = 0; i < nd; ++i) { v.sizes[i] = (IndexT)sz[i]; v.strides[i] = (IndexT)st[i]; }
  return v;
}

inline int64_t numel(const thcb200_tensor &d) {
  if (d.ndim <= 0) return 0;
  int64_t n = 1;
  for (int i = 0; i < d.ndim; ++i) n *= d.sizes[i];
  return n;
}

constexpr int kThreads = 256;

template <typename Op, typename Ta, typename IndexT>
__global__ void __launch_bounds__(kThreads) apply1_kernel(Ta *a, View<IndexT> va, IndexT n, Op op) {
  for (IndexT i = (IndexT)blockIdx.x * kThreads + threadIdx.x; i < n; i += (IndexT)gridDim.x * kThreads)
    op(&a[va.offset(i)]);
}
template <typename Op, typename Ta, typename Tb, typename IndexT>
__global__ void __launch_bounds__(kThreads) apply2_kernel(Ta *a, View<IndexT> va, Tb *b, View<IndexT> vb, IndexT n, Op op) {
  for (IndexT i = (IndexT)blockIdx.x * kThreads + threadIdx.x; i < n; i += (IndexT)gridDim.x * kThreads)
    op(&a[va.offset(i)], &b[vb.offset(i)]);
}
template <typename Op, typename Ta, typename Tb, typename Tc, typename IndexT>
__global__ void __launch_bounds__(kThreads)
apply3_kernel(Ta *a, View<IndexT> va, Tb *b, View<IndexT> vb, Tc *c, View<IndexT> vc, IndexT n, Op op) {
  for (IndexT i = (IndexT)blockIdx.x * kThreads + threadIdx.x; i < n; i += (IndexT)gridDim.x * kThreads)
    op(&a[va.offset(i)], &b[vb.offset(i)], &c[vc.offset(i)]);
}

inline unsigned grid_for(int64_t n) {
  // enough CTAs to fill a B200 several times over; the kernels stride over the rest
  int64_t blocks = (n + kThreads - 1) / kThreads;
  const int64_t cap = 148 * 16;  // keeps i + gridDim.x * kThreads inside 32 bits for every n the 32-bit path accepts
  return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
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
    if (thcb200_can_use_32bit(&da) && thcb200_can_use_32bit(&db))
      apply2_kernel<Op, Ta, Tb, uint32_t><<<grid_for(n), kThreads, 0, st>>>((Ta *)da.data, collapse<uint32_t>(da), (Tb *)db.data,
                                                                          collapse<uint32_t>(db), (uint32_t)n, op);
    else
      apply2_kernel<Op, Ta, Tb, uint64_t><<<grid_for(n), kThreads, 0, st>>>((Ta *)da.data, collapse<uint64_t>(da), (Tb *)db.data,
                                                                          collapse<uint64_t>(db), (uint64_t)n, op);
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
    if (thcb200_can_use_32bit(&da) && thcb200_can_use_32bit(&db) && thcb200_can_use_32bit(&dc))
      apply3_kernel<Op, Ta, Tb, Tc, uint32_t><<<grid_for(n), kThreads, 0, st>>>(
          (Ta *)da.data, collapse<uint32_t>(da), (Tb *)db.data, collapse<uint32_t>(db), (Tc *)dc.data, collapse<uint32_t>(dc),
          (uint32_t)n, op);
    else
      apply3_kernel<Op, Ta, Tb, Tc, uint64_t><<<grid_for(n), kThreads, 0, st>>>(
          (Ta *)da.data, collapse<uint64_t>(da), (Tb *)db.data, collapse<uint64_t>(db), (Tc *)dc.data, collapse<uint64_t>(dc),
          (uint64_t)n, op);
  }
  restore_overlap(state, a, oa);
  restore_overlap(state, b, ob);
  restore_overlap(state, c, oc);
  return true;
}

#endif /* THCB200_THC_APPLY_CUH */
