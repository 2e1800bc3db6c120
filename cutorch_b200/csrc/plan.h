// Host-side layout analysis: TensorInfo-style dimension collapsing, overlap and index-width
// predicates, and the per-call plan that selects a pointwise kernel family.
#pragma once

#include <string>

#include "apply.cuh"
#include "core.cuh"

namespace thcb {

// thread-local error text / plan name reported through thcb200_last_error/_last_plan
void set_error(const char *fmt, ...);
const char *get_error();
void set_plan_name(const char *name);
const char *get_plan_name();
void count_launch(int n = 1);

int64_t view_numel(const thcb200_tensor *t);
// Validates a descriptor and converts it (dims <= 25, non-negative sizes).  0 on success.
int to_host_view(const thcb200_tensor *t, HostView *v, const char *what);

// TensorInfo::collapseDims (lib/THC/THCTensorInfo.cuh:74-224) on plain arrays.
int collapse_dims(int64_t *sizes, int64_t *strides, int *ndim, int exclude_dim);
// TensorUtils::overlappingIndices (lib/THC/THCTensorTypeUtils.cu:163-218).
bool overlapping_indices(const HostView &v);
// Largest and smallest element offset touched by the view.
void offset_range(const HostView &v, int64_t *lo, int64_t *hi);
// TensorUtils::canUse32BitIndexMath (lib/THC/THCTensorTypeUtils.cu:220-245).
bool can_use_32bit(const HostView &v);

enum ApplyKind { kApplyContigVec = 0, kApplyTiled = 1, kApplyGeneric = 2, kApplyDeep = 3, kApplyRows = 4 };

struct ApplyPlan {
  ApplyKind kind;
  bool index64;
  int nops;                        // operands including the output (index 0)
  uint64_t numel;
  // generic: one collapsed view per operand (sizes/strides as plain arrays; the typed
  // launcher converts them to StridedView<IndexT>)
  int gdims[4];
  int64_t gsizes[4][kMaxDims];
  int64_t gstrides[4][kMaxDims];
  // tiled
  TiledPlan tiled;
  int tiled_slots;                 // number of operands staged through shared memory
  // rows
  RowsPlan rows;
};

// ops[0] is the output.  All views hold the same number of elements.
void make_apply_plan(const HostView *ops, int nops, size_t elem_size, ApplyPlan *plan);

template <typename IndexT>
inline StridedView<IndexT> to_strided_view(const ApplyPlan &p, int o) {
  StridedView<IndexT> v;
  if (o >= p.nops) {  // operand not used by this op: a trivial view (the plan holds nothing for it)
    v.dims = 1;
    for (int i = 0; i < kGenericDims; ++i) { v.sizes[i] = DivHelper<IndexT>(1); v.strides[i] = 0; }
    return v;
  }
  v.dims = p.gdims[o];
  for (int i = 0; i < kGenericDims; ++i) {
    if (i < v.dims) {
      v.sizes[i] = DivHelper<IndexT>((uint64_t)p.gsizes[o][i]);
      v.strides[i] = (IndexT)p.gstrides[o][i];
    } else {
      v.sizes[i] = DivHelper<IndexT>(1);
      v.strides[i] = 0;
    }
  }
  return v;
}

}  // namespace thcb
