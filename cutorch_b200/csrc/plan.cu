// Host-side layout analysis for the apply / reduce planners (no device code).
#include "plan.h"
#include "context.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>

namespace thcb {

static thread_local char g_error[512] = "";
static thread_local const char *g_plan = "";
static std::atomic<int64_t> g_launches{0};

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char *get_error() { return g_error; }
void set_plan_name(const char *name) { g_plan = name; }
const char *get_plan_name() { return g_plan; }
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// countdown to an injected allocation failure: 0 = off, n = the n-th allocation from now fails
static std::atomic<int> g_fail_alloc_in{0};
static bool injected_failure() {
  int n = g_fail_alloc_in.load(std::memory_order_relaxed);
  while (n > 0) {
    if (g_fail_alloc_in.compare_exchange_weak(n, n - 1, std::memory_order_relaxed)) return n == 1;
  }
  return false;
}
void arm_allocation_failure(int nth) { g_fail_alloc_in.store(nth > 0 ? nth : 0, std::memory_order_relaxed); }
cudaError_t device_alloc(void **p, size_t bytes) {
  if (injected_failure()) { *p = nullptr; return cudaErrorMemoryAllocation; }
  return cudaMalloc(p, bytes);
}
cudaError_t device_alloc_async(void **p, size_t bytes, cudaStream_t st) {
  if (injected_failure()) { *p = nullptr; return cudaErrorMemoryAllocation; }
  return cudaMallocAsync(p, bytes, st);
}

bool pdl_enabled() {
  static const bool on = [] {
    const char *e = getenv("THCB200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

int64_t view_numel(const thcb200_tensor *t) {
  if (t->ndim <= 0) return 0;
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->sizes[i];
  return n;
}

int to_host_view(const thcb200_tensor *t, HostView *v, const char *what) {
  if (!t) { set_error("%s: null tensor descriptor", what); return THCB200_ERR_ARG; }
  if (t->ndim > kMaxDims) {
    set_error("%s: tensor too large or too many (>%d) dimensions", what, kMaxDims);
    return THCB200_ERR_DIMS;
  }
  if (t->ndim < 0) { set_error("%s: negative dimension count", what); return THCB200_ERR_ARG; }
  if (t->dtype < 0 || t->dtype > THCB200_F64) { set_error("%s: unknown dtype %d", what, t->dtype); return THCB200_ERR_ARG; }
  v->data = (char *)t->data;
  v->dtype = t->dtype;
  v->ndim = t->ndim;
  int64_t n = t->ndim > 0 ? 1 : 0;
  for (int i = 0; i < t->ndim; ++i) {
    if (t->sizes[i] < 0) { set_error("%s: negative size", what); return THCB200_ERR_ARG; }
    v->sizes[i] = t->sizes[i];
    v->strides[i] = t->strides[i];
    n *= t->sizes[i];
  }
  v->numel = n;
  if (n > 0 && !t->data) { set_error("%s: null data pointer", what); return THCB200_ERR_ARG; }
  return 0;
}

int collapse_dims(int64_t *sizes, int64_t *strides, int *ndim, int exclude_dim) {
  const int nd = *ndim;
  // innermost dimension that has to survive: the excluded one or the first of size != 1
  int inner = -1;
  for (int i = nd - 1; i >= 0; --i) {
    if (i == exclude_dim || sizes[i] != 1) { inner = i; break; }
  }
  if (inner < 0) {  // a single point
    *ndim = 1;
    sizes[0] = 1;
    strides[0] = 1;
    return 0;
  }
  // Build the surviving runs innermost-first.
  int64_t rs[kMaxDims], rt[kMaxDims];
  int n = 0, kept_at = -1;
  rs[0] = sizes[inner];
  rt[0] = strides[inner];
  if (inner == exclude_dim) kept_at = 0;
  n = 1;
  for (int i = inner - 1; i >= 0; --i) {
    const bool may_merge = (i != exclude_dim) && (i + 1 != exclude_dim);
    if (may_merge) {
      if (sizes[i] == 1) continue;                       // addressing point only
      if (strides[i] == rs[n - 1] * rt[n - 1]) {         // extends the current run
        rs[n - 1] *= sizes[i];
        continue;
      }
    }
    rs[n] = sizes[i];
    rt[n] = strides[i];
    if (i == exclude_dim) kept_at = n;
    ++n;
  }
  for (int i = 0; i < n; ++i) {
    sizes[i] = rs[n - 1 - i];
    strides[i] = rt[n - 1 - i];
  }
  *ndim = n;
  return kept_at < 0 ? -1 : n - 1 - kept_at;
}

bool overlapping_indices(const HostView &v) {
  struct SS { int64_t size, stride; };
  SS d[kMaxDims];
  int n = 0;
  for (int i = 0; i < v.ndim; ++i)
    if (v.sizes[i] > 1) d[n++] = SS{v.sizes[i], v.strides[i]};
  if (n == 0) return false;
  std::sort(d, d + n, [](const SS &a, const SS &b) { return a.stride < b.stride; });
  if (d[0].stride < 1) return true;
  for (int i = 1; i < n; ++i)
    if (d[i].stride < d[i - 1].size * d[i - 1].stride) return true;
  return false;
}

void offset_range(const HostView &v, int64_t *lo, int64_t *hi) {
  int64_t l = 0, h = 0;
  for (int i = 0; i < v.ndim; ++i) {
    if (v.sizes[i] <= 1) continue;
    const int64_t span = (v.sizes[i] - 1) * v.strides[i];
    if (span > 0) h += span; else l += span;
  }
  *lo = l;
  *hi = h;
}

bool can_use_32bit(const HostView &v) {
  if (v.numel >= 0xFFF00000LL) return false;
  int64_t lo, hi;
  offset_range(v, &lo, &hi);
  return lo >= 0 && hi < 0xFFFFFFFFLL;
}

// -----------------------------------------------------------------------------------
// Apply planner
// -----------------------------------------------------------------------------------
namespace {

struct Dims {
  int n;
  int64_t size[kMaxDims];
  int64_t stride[4][kMaxDims];
};

// true if every operand has the same shape once size-1 dims are dropped
bool same_squeezed_shape(const HostView *ops, int nops, Dims *out) {
  out->n = 0;
  for (int i = 0; i < ops[0].ndim; ++i) {
    if (ops[0].sizes[i] != 1) {
      out->size[out->n] = ops[0].sizes[i];
      out->stride[0][out->n] = ops[0].strides[i];
      ++out->n;
    }
  }
  for (int o = 1; o < nops; ++o) {
    int k = 0;
    for (int i = 0; i < ops[o].ndim; ++i) {
      if (ops[o].sizes[i] == 1) continue;
      if (k >= out->n || ops[o].sizes[i] != out->size[k]) return false;
      out->stride[o][k] = ops[o].strides[i];
      ++k;
    }
    if (k != out->n) return false;
  }
  return true;
}

bool try_tiled(const Dims &d, int nops, size_t elem_size, ApplyPlan *plan) {
  const int k = d.n;
  if (k < 2) return false;
  const int tc = tiled_tc_for(elem_size);
  // classify operands: direct = smallest |stride| sits in the last dim
  int p = -1;
  bool staged[4] = {false, false, false, false};
  int nstaged = 0;
  for (int o = 0; o < nops; ++o) {
    int unit = -1;
    for (int i = 0; i < k; ++i)
      if (d.stride[o][i] == 1) unit = i;
    if (unit >= 0 && unit != k - 1 && d.stride[o][k - 1] * (int64_t)elem_size >= 32) {
      if (p >= 0 && p != unit) return false;  // two different transpositions: generic
      p = unit;
      staged[o] = true;
      ++nstaged;
    }
  }
  if (nstaged == 0 || nstaged == nops) return false;
  const int njd = k - 1 - p;
  if (njd > kTiledJDims || p > kTiledOuterDims) return false;
  int64_t sizeJ = 1;
  for (int i = p + 1; i < k; ++i) sizeJ *= d.size[i];
  const int64_t sizeC = d.size[p];
  if (sizeJ < 16 || sizeC < tc / 2 || sizeJ >= (1LL << 31) || sizeC >= (1LL << 31)) return false;
  // the J group has to be one run for every direct operand
  for (int o = 0; o < nops; ++o) {
    if (staged[o]) continue;
    for (int i = p + 1; i + 1 < k; ++i)
      if (d.stride[o][i] != d.size[i + 1] * d.stride[o][i + 1]) return false;
  }
  TiledPlan &t = plan->tiled;
  memset(&t, 0, sizeof(t));
  t.nouter = p;
  t.njd = njd;
  t.c_fastest = 1;  // measured on B200: either CTA order gives the same bandwidth
  t.sizeC = (uint32_t)sizeC;
  t.sizeJ = (uint32_t)sizeJ;
  t.tilesC = (uint32_t)((sizeC + tc - 1) / tc);
  t.tilesJ = (uint32_t)((sizeJ + kTJ - 1) / kTJ);
  t.tilesCdiv = FastDiv32(t.tilesC);
  t.tilesJdiv = FastDiv32(t.tilesJ);
  uint64_t blocks = (uint64_t)t.tilesC * t.tilesJ;
  for (int i = 0; i < kTiledOuterDims; ++i) t.outerSizes[i] = FastDiv32(1);
  for (int i = 0; i < p; ++i) {
    if (d.size[i] >= (1LL << 31)) return false;
    t.outerSizes[i] = FastDiv32((uint32_t)d.size[i]);
    blocks *= (uint64_t)d.size[i];
    if (blocks >= (1ULL << 31)) return false;
  }
  for (int i = 0; i < kTiledJDims; ++i) t.jSizes[i] = FastDiv32(1);
  for (int i = 0; i < njd; ++i) t.jSizes[i] = FastDiv32((uint32_t)d.size[p + 1 + i]);
  int slot = 0;
  for (int o = 0; o < nops; ++o) {
    TiledOperand &to = t.op[o];
    to.staged = staged[o] ? 1 : 0;
    to.slot = staged[o] ? slot++ : 0;
    to.strideC = d.stride[o][p];
    to.strideJ = d.stride[o][k - 1];
    for (int i = 0; i < njd; ++i) to.jstrides[i] = d.stride[o][p + 1 + i];
    for (int i = 0; i < p; ++i) to.ostrides[i] = d.stride[o][i];
  }
  plan->tiled_slots = slot;
  return true;
}

// Two collapsed dims, every operand dense or constant along the inner one (see apply_rows_kernel).
// Rows move as 16-byte vectors when every dense operand keeps that alignment from row to row,
// else element by element.
bool try_rows(const Dims &d, int nops, const HostView *ops, size_t elem_size, ApplyPlan *plan) {
  if (d.n < 2 || d.n - 1 > kRowsOuterDims || elem_size == 0) return false;
  const int nouter = d.n - 1;
  const int64_t V = (int64_t)(16 / elem_size);
  const int64_t C = d.size[nouter];
  int64_t R = 1;
  for (int i = 0; i < nouter; ++i) {
    if (d.size[i] >= (1LL << 31)) return false;
    R *= d.size[i];
    if (R >= (1LL << 31)) return false;
  }
  if (C >= (1LL << 31)) return false;
  if (d.stride[0][nouter] != 1) return false;   // the output has to be dense along C
  RowsPlan &rp = plan->rows;
  bool vec = C % V == 0;
  rp.nouter = nouter;
  for (int i = 0; i < kRowsOuterDims; ++i) {
    rp.outer_size[i] = FastDiv32(i < nouter ? (uint32_t)d.size[i] : 1u);
    for (int o = 0; o < 4; ++o) rp.outer_stride[o][i] = 0;
  }
  for (int o = 0; o < 4; ++o) rp.constant[o] = 0;
  for (int o = 0; o < nops; ++o) {
    const int64_t sc = d.stride[o][nouter];
    if (sc != 0 && sc != 1) return false;
    if (sc == 1 && ((uintptr_t)ops[o].data) % 16 != 0) vec = false;
    for (int i = 0; i < nouter; ++i) {
      rp.outer_stride[o][i] = d.stride[o][i];
      if (sc == 1 && d.stride[o][i] % V != 0) vec = false;
    }
    rp.constant[o] = sc == 0 ? 1 : 0;
  }
  rp.vec = vec ? 1 : 0;
  rp.R = (uint32_t)R;
  rp.Cvec = (uint32_t)(vec ? C / V : C);
  const uint32_t per_thread = vec ? 1 : kRowsScalarCols;
  const uint32_t slots = (rp.Cvec + per_thread - 1) / per_thread;   // threads wanted along C
  int lg = 0;
  while ((1u << lg) < slots && lg < 8) ++lg;
  rp.log2_tx = lg;
  const uint32_t per_cta = (1u << lg) * per_thread;
  rp.tiles_c = (rp.Cvec + per_cta - 1) / per_cta;
  const uint64_t rows_per_cta = (uint64_t)(256 >> lg) * kRowsUnroll;
  const uint64_t blocks = (uint64_t)rp.tiles_c * (((uint64_t)R + rows_per_cta - 1) / rows_per_cta);
  return blocks < (1ULL << 31);
}

}  // namespace

void make_apply_plan(const HostView *ops, int nops, size_t elem_size, ApplyPlan *plan) {
  plan->nops = nops;
  plan->numel = (uint64_t)ops[0].numel;
  plan->tiled_slots = 0;

  Dims d;
  const bool same_shape = same_squeezed_shape(ops, nops, &d);
  if (same_shape && d.n > 0) {
    // Pointwise work is order-free when the shapes agree: walk the dims from the
    // output's largest stride to its smallest so that stores are as dense as possible.
    int order[kMaxDims];
    for (int i = 0; i < d.n; ++i) order[i] = i;
    std::stable_sort(order, order + d.n, [&](int a, int b) {
      int64_t sa = d.stride[0][a] < 0 ? -d.stride[0][a] : d.stride[0][a];
      int64_t sb = d.stride[0][b] < 0 ? -d.stride[0][b] : d.stride[0][b];
      return sa > sb;
    });
    Dims s;
    s.n = d.n;
    for (int i = 0; i < d.n; ++i) {
      s.size[i] = d.size[order[i]];
      for (int o = 0; o < nops; ++o) s.stride[o][i] = d.stride[o][order[i]];
    }
    // joint collapse: merge dim i into i+1 when that is a run for every operand
    Dims j;
    j.n = 0;
    for (int i = s.n - 1; i >= 0; --i) {
      bool merge = j.n > 0;
      if (merge)
        for (int o = 0; o < nops; ++o)
          if (s.stride[o][i] != j.size[j.n - 1] * j.stride[o][j.n - 1]) { merge = false; break; }
      if (merge) {
        j.size[j.n - 1] *= s.size[i];
      } else {
        j.size[j.n] = s.size[i];
        for (int o = 0; o < nops; ++o) j.stride[o][j.n] = s.stride[o][i];
        ++j.n;
      }
    }
    // j is innermost-first; flip to outermost-first
    Dims f;
    f.n = j.n;
    for (int i = 0; i < j.n; ++i) {
      f.size[i] = j.size[j.n - 1 - i];
      for (int o = 0; o < nops; ++o) f.stride[o][i] = j.stride[o][j.n - 1 - i];
    }
    for (int o = 0; o < nops; ++o) {
      plan->gdims[o] = f.n;
      for (int i = 0; i < f.n; ++i) {
        plan->gsizes[o][i] = f.size[i];
        plan->gstrides[o][i] = f.stride[o][i];
      }
      // operands whose own dims still merge (e.g. contiguous ones) get a shorter walk
      collapse_dims(plan->gsizes[o], plan->gstrides[o], &plan->gdims[o], -1);
    }
    bool all_unit = true;
    for (int o = 0; o < nops; ++o) {
      if (!(plan->gdims[o] == 1 && plan->gstrides[o][0] == 1)) all_unit = false;
      if (((uintptr_t)ops[o].data) % 16 != 0) all_unit = false;
    }
    if (all_unit && elem_size) { plan->kind = kApplyContigVec; plan->index64 = true; return; }
    if (elem_size && try_tiled(f, nops, elem_size, plan)) { plan->kind = kApplyTiled; plan->index64 = false; return; }
    if (elem_size && try_rows(f, nops, ops, elem_size, plan)) { plan->kind = kApplyRows; plan->index64 = false; return; }
  } else {
    // Shapes differ (only the element counts agree): every operand is walked in its own
    // row-major order, as THC_pointwiseApply does.
    for (int o = 0; o < nops; ++o) {
      plan->gdims[o] = ops[o].ndim;
      for (int i = 0; i < ops[o].ndim; ++i) {
        plan->gsizes[o][i] = ops[o].sizes[i];
        plan->gstrides[o][i] = ops[o].strides[i];
      }
      collapse_dims(plan->gsizes[o], plan->gstrides[o], &plan->gdims[o], -1);
    }
    bool all_unit = true;
    for (int o = 0; o < nops; ++o) {
      if (!(plan->gdims[o] == 1 && plan->gstrides[o][0] == 1)) all_unit = false;
      if (((uintptr_t)ops[o].data) % 16 != 0) all_unit = false;
    }
    if (all_unit && elem_size) { plan->kind = kApplyContigVec; plan->index64 = true; return; }
  }
  bool deep = false, i32 = true;
  for (int o = 0; o < nops; ++o) {
    if (plan->gdims[o] > kGenericDims) deep = true;
    HostView c;
    c.ndim = plan->gdims[o];
    c.numel = ops[o].numel;
    for (int i = 0; i < c.ndim; ++i) { c.sizes[i] = plan->gsizes[o][i]; c.strides[i] = plan->gstrides[o][i]; }
    if (!can_use_32bit(c)) i32 = false;
  }
  plan->index64 = !i32;
  plan->kind = deep ? kApplyDeep : kApplyGeneric;
}

}  // namespace thcb
