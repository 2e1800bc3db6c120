// Typed launch code and layout planning of the reductions.  One translation unit per element
// type instantiates reduce_all_typed<T>, reduce_dim_typed<T> and reduce_dim_index_typed<T>.
#pragma once

#include <string.h>

#include <algorithm>

#include "context.h"
#include "plan.h"
#include "reduce.cuh"

namespace thcb {

// ------------------------------------------------------------------------------------
// reduce_all
// ------------------------------------------------------------------------------------
template <typename T, int MODE>
int launch_reduce_all(thcb200_ctx *ctx, const HostView &in, thcb200_scalar s, void *result, cudaStream_t st) {
  using F = Folder<T, MODE>;
  typename F::Params prm;
  if constexpr (TypeTraits<T>::is_fp) prm.s = (typename F::Scalar)s.f; else prm.s = (typename F::Scalar)s.i;
  // A full reduction does not depend on the order of the elements: the dims are walked from the
  // largest stride to the smallest, so a permuted (transposed) tensor collapses like its base.
  int64_t sizes[kMaxDims], strides[kMaxDims];
  int nd = 0;
  {
    int order[kMaxDims], m = 0;
    for (int i = 0; i < in.ndim; ++i) if (in.sizes[i] != 1) order[m++] = i;
    std::stable_sort(order, order + m, [&](int a, int b) {
      const int64_t sa = in.strides[a] < 0 ? -in.strides[a] : in.strides[a];
      const int64_t sb = in.strides[b] < 0 ? -in.strides[b] : in.strides[b];
      return sa > sb;
    });
    for (int i = 0; i < m; ++i) { sizes[i] = in.sizes[order[i]]; strides[i] = in.strides[order[i]]; }
    nd = m;
    if (nd == 0) { nd = 1; sizes[0] = 1; strides[0] = 1; }
  }
  collapse_dims(sizes, strides, &nd, -1);
  if (nd > kGenericDims) { set_error("reduce_all: more than %d non-collapsible dimensions", kGenericDims); return THCB200_ERR_DIMS; }
  const uint64_t n = (uint64_t)in.numel;
  // a sharded call hands its exchange description over through the context (which it holds locked)
  PeerExchange px;
  if (ctx->px) px = *ctx->px; else memset(&px, 0, sizeof(px));
  const bool unit = nd == 1 && strides[0] == 1;
  const T *p = reinterpret_cast<const T *>(in.data);
  const uint64_t max_grid = (uint64_t)ctx->num_sms * 4;

  // dense rows under strided outer dims (padded rows, windows): the row walk
  if (!unit && nd >= 2 && nd - 1 <= kRedRowsOuterDims && strides[nd - 1] == 1) {
    constexpr int VF = 16 / (int)sizeof(T);
    const int nouter = nd - 1;
    uint64_t R = 1;
    bool fits = sizes[nouter] < (1LL << 31);
    for (int i = 0; i < nouter; ++i) {
      R *= (uint64_t)sizes[i];
      if (sizes[i] >= (1LL << 31) || R >= (1ull << 31)) fits = false;
    }
    if (fits) {
      RedRowsView rv;
      rv.nouter = nouter;
      for (int i = 0; i < kRedRowsOuterDims; ++i) {
        rv.outer_size[i] = FastDiv32(i < nouter ? (uint32_t)sizes[i] : 1u);
        rv.outer_stride[i] = i < nouter ? strides[i] : 0;
      }
      rv.R = (uint32_t)R;
      rv.Cunits = (uint32_t)sizes[nouter];
      // threads along the row: each takes kRedRowsSlots vectors; at least the up to 2 (V - 1) edge elements
      uint32_t slots = (uint32_t)((sizes[nouter] / VF + kRedRowsSlots - 1) / kRedRowsSlots);
      if (slots < 2u * (VF - 1)) slots = 2u * (VF - 1);
      if (slots < 1) slots = 1;
      int lg = 0;
      while ((1u << lg) < slots && lg < 8) ++lg;
      rv.log2_tx = lg;
      const uint64_t vec_per_tile = (uint64_t)kRedRowsSlots << lg;
      rv.tiles_c = (uint32_t)((sizes[nouter] / VF + vec_per_tile - 1) / vec_per_tile);
      if (rv.tiles_c < 1) rv.tiles_c = 1;
      rv.tiles_c_div = FastDiv32(rv.tiles_c);
      const uint64_t rows_per_tile = (uint64_t)(kRedThreads >> lg);
      const uint64_t ntiles = (uint64_t)rv.tiles_c * ((R + rows_per_tile - 1) / rows_per_tile);
      if (ntiles < (1ull << 31)) {
        const uint64_t per_cta = (ntiles + max_grid - 1) / max_grid;
        const uint64_t grid = (ntiles + per_cta - 1) / per_cta;
        void *partials = ctx_workspace(ctx, grid * 16);
        if (!partials) return THCB200_ERR_NOMEM;
        set_plan_name("reduce_all_rows");
        launch_pdl(reduce_all_rows_kernel<T, MODE>, (unsigned)grid, kRedThreads, 0, st, p, rv, (uint32_t)ntiles, prm, partials, ctx->tickets, result, px);
        count_launch();
        THCB_CUDA_TRY(cudaGetLastError());
        return 0;
      }
    }
  }

  // A dense run is read as 256-bit vectors from its first 32-byte boundary on; the few elements in
  // front of it go to the first threads of CTA 0.  Anything else takes the per-element walk.
  const T *body = p;
  uint64_t nbody = n;
  uint32_t nedge = 0;
  int vb = 0;
  if (unit) {
    constexpr uint64_t V32 = 32 / sizeof(T);
    const uint64_t mis = ((uintptr_t)in.data / sizeof(T)) % V32;
    uint64_t head = mis ? V32 - mis : 0;
    if (head > n) head = n;
    nedge = (uint32_t)head;
    body = p + head;
    nbody = n - head;
    vb = 32;
  }
  const uint64_t tile = (uint64_t)kRedThreads * kRedUnroll * (vb ? vb / sizeof(T) : 1);
  uint64_t ntiles = (nbody + tile - 1) / tile;
  if (ntiles < 1) ntiles = 1;
  // 4 CTAs per SM, all resident at once (measured on B200: more CTAs in flight lower the read
  // bandwidth), walking the tiles block-cyclically: every CTA gets the same number of tiles to
  // within one and, with the CTAs dealt round the SMs, so does every SM (a grid cut down to whole
  // tiles per CTA left some SMs with 16 tiles and others with 12 on a 64 MiB tensor).  A function
  // of n and the SM count only.
  uint64_t grid = ntiles < max_grid ? ntiles : max_grid;
  if (grid < 1) grid = 1;
  void *partials = ctx_workspace(ctx, grid * 16);
  if (!partials) return THCB200_ERR_NOMEM;
  StridedView<uint64_t> view;
  view.dims = nd;
  for (int i = 0; i < kGenericDims; ++i) {
    view.sizes[i] = DivHelper<uint64_t>(i < nd ? (uint64_t)sizes[i] : 1);
    view.strides[i] = i < nd ? (uint64_t)strides[i] : 0;
  }
  if (vb == 32) {
    set_plan_name(nedge ? "reduce_all_vec_peeled" : "reduce_all_vec");
    launch_pdl(reduce_all_kernel<T, MODE, 32>, (unsigned)grid, kRedThreads, 0, st, body, view, nbody, prm, partials, ctx->tickets, result, p, nedge, px);
  } else {
    set_plan_name("reduce_all_strided");
    launch_pdl(reduce_all_kernel<T, MODE, 0>, (unsigned)grid, kRedThreads, 0, st, p, view, n, prm, partials, ctx->tickets, result, p, 0u, px);
  }
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

template <typename T>
int reduce_all_typed(thcb200_ctx *ctx, int mode, const HostView &in, thcb200_scalar s, void *result, cudaStream_t st) {
  switch (mode) {
    case kSum: return launch_reduce_all<T, kSum>(ctx, in, s, result, st);
    case kProd: return launch_reduce_all<T, kProd>(ctx, in, s, result, st);
    case kMin: return launch_reduce_all<T, kMin>(ctx, in, s, result, st);
    case kMax: return launch_reduce_all<T, kMax>(ctx, in, s, result, st);
    default: break;
  }
  if constexpr (TypeTraits<T>::is_fp) {
    switch (mode) {
      case kSumAbs: return launch_reduce_all<T, kSumAbs>(ctx, in, s, result, st);
      case kSumSquare: return launch_reduce_all<T, kSumSquare>(ctx, in, s, result, st);
      case kSumPowAbs: return launch_reduce_all<T, kSumPowAbs>(ctx, in, s, result, st);
      case kSumNonZero: return launch_reduce_all<T, kSumNonZero>(ctx, in, s, result, st);
      case kSumSqDev: return launch_reduce_all<T, kSumSqDev>(ctx, in, s, result, st);
      default: break;
    }
  } else {
    switch (mode) {
      case kAll: return launch_reduce_all<T, kAll>(ctx, in, s, result, st);
      case kAny: return launch_reduce_all<T, kAny>(ctx, in, s, result, st);
      default: break;
    }
  }
  set_error("reduce_all: fold mode %d is not defined for dtype %d", mode, TypeTraits<T>::dtype);
  return THCB200_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------
// reduce_dim planning (shared by the value and the value+index forms)
// ------------------------------------------------------------------------------------
// workspace bytes per partial accumulator (the largest is two doubles and a flag)
constexpr size_t kPartialSlotBytes = 32;
constexpr int kRedColScalarUnroll = 16;

enum RedDimKind { kRedRowWarp, kRedRowBlock, kRedCol, kRedStrided };

struct RedDimPlan {
  RedDimKind kind;
  bool vec;
  SliceMap map;
  uint64_t nslices;       // outputs for ROW/STRIDED, nouter for COL
  uint64_t K;
  int64_t strideK;
  uint64_t I;             // COL: inner extent
  int64_t out_inner_stride, idx_inner_stride;
  uint32_t nsplit;
  uint64_t split_len;
  uint32_t tiles_i;
};

// in/out/idx: same dims; `dim` is reduced (out/idx have size 1 there).  idx may be null.
inline int plan_reduce_dim(thcb200_ctx *ctx, const HostView &in, const HostView &out, const HostView *idx,
                           int dim, size_t elem_size, int vec_elems, int col_vec, RedDimPlan *pl) {
  pl->K = (uint64_t)in.sizes[dim];
  pl->strideK = in.strides[dim];
  // non-reduced dims of size > 1
  int nd = 0;
  int64_t size[kMaxDims], is[kMaxDims], os[kMaxDims], xs[kMaxDims];
  for (int i = 0; i < in.ndim; ++i) {
    if (i == dim || in.sizes[i] == 1) continue;
    size[nd] = in.sizes[i]; is[nd] = in.strides[i]; os[nd] = out.strides[i]; xs[nd] = idx ? idx->strides[i] : 0;
    ++nd;
  }
  uint64_t nout = 1;
  for (int i = 0; i < nd; ++i) nout *= (uint64_t)size[i];
  const bool ptr_aligned = ((uintptr_t)in.data % 16) == 0;
  const uint64_t target_ctas = (uint64_t)ctx->num_sms * 4;

  int inner = -1;
  // the row / column kernels track positions as 32-bit offsets inside a unit of work
  const bool huge_k = pl->K > 0xFFFFFFF0ull;
  const bool row = (pl->strideK == 1 || pl->K <= 1) && !huge_k;
  if (!row && !huge_k) {
    for (int i = nd - 1; i >= 0; --i)
      if (is[i] == 1 && size[i] >= 32) { inner = i; break; }
  }
  // slice map over the remaining dims, merging neighbours that form a run in every tensor
  SliceMap &m = pl->map;
  m.n = 0;
  int prev = -1;
  for (int i = 0; i < nd; ++i) {
    if (i == inner) { prev = -1; continue; }
    if (prev >= 0 && is[prev] == size[i] * is[i] && os[prev] == size[i] * os[i] && xs[prev] == size[i] * xs[i] &&
        m.n > 0) {
      // dim i extends the previous entry inward
      m.size[m.n - 1] *= (uint64_t)size[i];
      m.in_stride[m.n - 1] = is[i];
      m.out_stride[m.n - 1] = os[i];
      m.idx_stride[m.n - 1] = xs[i];
    } else {
      m.size[m.n] = (uint64_t)size[i];
      m.in_stride[m.n] = is[i];
      m.out_stride[m.n] = os[i];
      m.idx_stride[m.n] = xs[i];
      ++m.n;
    }
    prev = i;
  }
  pl->nsplit = 1;
  pl->split_len = pl->K;
  pl->I = 1;
  pl->out_inner_stride = pl->idx_inner_stride = 0;
  pl->tiles_i = 1;
  pl->vec = false;

  if (row) {
    pl->nslices = nout;
    if (pl->K < 64) { pl->kind = kRedStrided; return 0; }
    // the row kernel peels each unit up to a 16-byte boundary itself: no alignment needed
    const bool vec = true;
    pl->vec = vec;
    const uint64_t warp_step = 32ull * vec_elems * kRedUnroll;       // elements per warp iteration
    const uint64_t block_step = (uint64_t)kRedThreads * vec_elems * kRedUnroll;
    if (nout * 32 >= target_ctas * kRedThreads / 2 || pl->K <= 2 * warp_step) {
      pl->kind = kRedRowWarp;
    } else {
      pl->kind = kRedRowBlock;
      if (nout < target_ctas / 2 && pl->K >= 4 * block_step) {
        uint64_t want = target_ctas / nout;  // all units resident at once (one wave, 4 CTAs per SM)
        uint64_t maxs = pl->K / (2 * block_step);
        if (want > maxs) want = maxs;
        if (want > 1) {
          uint64_t len = (pl->K + want - 1) / want;
          len = (len + block_step - 1) / block_step * block_step;
          pl->split_len = len;
          pl->nsplit = (uint32_t)((pl->K + len - 1) / len);
        }
      }
    }
    return 0;
  }
  if (inner >= 0) {
    pl->kind = kRedCol;
    pl->I = (uint64_t)size[inner];
    pl->out_inner_stride = os[inner];
    pl->idx_inner_stride = xs[inner];
    uint64_t nouter = 1;
    for (int i = 0; i < m.n; ++i) nouter *= m.size[i];
    pl->nslices = nouter;
    bool vec = ptr_aligned && (pl->I % col_vec == 0) && (pl->strideK % col_vec == 0);
    for (int i = 0; i < m.n; ++i) if (m.in_stride[i] % col_vec != 0) vec = false;
    pl->vec = vec;
    const int v = vec ? col_vec : 1;
    pl->tiles_i = (uint32_t)((pl->I + 32ull * v - 1) / (32ull * v));
    const uint64_t ctas = nouter * pl->tiles_i;
    const uint64_t step = (uint64_t)kRedWarps * kRedUnroll;  // rows per CTA iteration
    if (ctas < target_ctas && pl->K >= 4 * step) {
      uint64_t want = target_ctas / ctas;  // all CTAs resident at once (one wave, 4 CTAs per SM)
      uint64_t maxs = pl->K / (2 * step);
      if (want > maxs) want = maxs;
      if (want > 1) {
        // equal splits, each warp the same number of rows: rounding the length up to a whole number
        // of iterations instead left 8192 rows as 17 splits of 480 and one of 32
        uint64_t len = (pl->K + want - 1) / want;
        len = (len + kRedWarps - 1) / kRedWarps * kRedWarps;
        pl->split_len = len;
        pl->nsplit = (uint32_t)((pl->K + len - 1) / len);
      }
    }
    if ((uint64_t)ctas * pl->nsplit >= (1ull << 31)) { pl->kind = kRedStrided; pl->nslices = nout; }
    else return 0;
  }
  // fallback: rebuild the map over all non-reduced dims
  m.n = 0;
  for (int i = 0; i < nd; ++i) {
    m.size[m.n] = (uint64_t)size[i]; m.in_stride[m.n] = is[i]; m.out_stride[m.n] = os[i]; m.idx_stride[m.n] = xs[i];
    ++m.n;
  }
  pl->kind = kRedStrided;
  pl->nslices = nout;
  pl->nsplit = 1;
  pl->split_len = pl->K;
  return 0;
}

template <typename T, int MODE, bool INDEX, bool IS_MAX>
int launch_reduce_dim(thcb200_ctx *ctx, const HostView &in, const HostView &out, const HostView *idx, int dim,
                      thcb200_scalar s, PostOp post, cudaStream_t st) {
  using F = Folder<T, MODE>;
  typename F::Params prm;
  if constexpr (TypeTraits<T>::is_fp) prm.s = (typename F::Scalar)s.f; else prm.s = (typename F::Scalar)s.i;
  constexpr int V = 16 / sizeof(T);
  constexpr int CV = col_vec_elems<T>();
  RedDimPlan pl;
  int rc = plan_reduce_dim(ctx, in, out, idx, dim, sizeof(T), V, CV, &pl);
  if (rc) return rc;
  const T *ip = reinterpret_cast<const T *>(in.data);
  T *op = reinterpret_cast<T *>(out.data);
  int64_t *xp = idx ? reinterpret_cast<int64_t *>(idx->data) : nullptr;
  void *partials = nullptr;
  const uint64_t noutputs = (pl.kind == kRedCol) ? pl.nslices * pl.I : pl.nslices;
  if (pl.nsplit > 1) {
    partials = ctx_workspace(ctx, noutputs * pl.nsplit * kPartialSlotBytes);
    if (!partials) return THCB200_ERR_NOMEM;
  }
  // With few enough tiles the CTA that completes a tile folds its partials itself (ticket per
  // tile); otherwise, or without ticket counters, a second small launch does.
  unsigned int *tickets = nullptr;
  if (pl.nsplit > 1 && ctx->tickets) {
    const uint64_t ntiles = (pl.kind == kRedCol) ? pl.nslices * pl.tiles_i : pl.nslices;
    if (ntiles <= (uint64_t)kNumTickets) tickets = ctx->tickets;
  }
  int launches = 1;
  switch (pl.kind) {
    case kRedRowWarp: {
      const uint64_t blocks = (pl.nslices + kRedWarps - 1) / kRedWarps;
      if (blocks >= (1ull << 31)) { set_error("reduce_dim: too many slices"); return THCB200_ERR_DIMS; }
      set_plan_name(pl.vec ? "row_warp_vec" : "row_warp");
      if (pl.vec) launch_pdl(reduce_row_kernel<T, MODE, INDEX, IS_MAX, true, true>, (unsigned)blocks, kRedThreads, 0, st, ip, op, xp, pl.map, pl.nslices, pl.K, 1, pl.K, prm, nullptr, nullptr, post);
      else launch_pdl(reduce_row_kernel<T, MODE, INDEX, IS_MAX, false, true>, (unsigned)blocks, kRedThreads, 0, st, ip, op, xp, pl.map, pl.nslices, pl.K, 1, pl.K, prm, nullptr, nullptr, post);
      break;
    }
    case kRedRowBlock: {
      const uint64_t blocks = pl.nslices * pl.nsplit;
      if (blocks >= (1ull << 31)) { set_error("reduce_dim: too many slices"); return THCB200_ERR_DIMS; }
      set_plan_name(pl.nsplit > 1 ? "row_block_split" : "row_block");
      if (pl.vec) launch_pdl(reduce_row_kernel<T, MODE, INDEX, IS_MAX, true, false>, (unsigned)blocks, kRedThreads, 0, st, ip, op, xp, pl.map, pl.nslices, pl.K, pl.nsplit, pl.split_len, prm, partials, tickets, post);
      else launch_pdl(reduce_row_kernel<T, MODE, INDEX, IS_MAX, false, false>, (unsigned)blocks, kRedThreads, 0, st, ip, op, xp, pl.map, pl.nslices, pl.K, pl.nsplit, pl.split_len, prm, partials, tickets, post);
      break;
    }
    case kRedCol: {
      const uint64_t blocks = pl.nslices * pl.tiles_i * pl.nsplit;
      set_plan_name(pl.nsplit > 1 ? "col_tile_split" : "col_tile");
      if (pl.vec) launch_pdl(reduce_col_kernel<T, MODE, INDEX, IS_MAX, CV, kRedUnroll>, (unsigned)blocks, kRedThreads, 0, st, ip, op, xp, pl.map, pl.nslices, pl.K, pl.strideK, pl.I, pl.out_inner_stride, pl.idx_inner_stride, pl.nsplit, pl.split_len, pl.tiles_i, prm, partials, tickets, post);
      // one column per lane moves 4 bytes a load: more row loads in flight per thread make up for it
      else launch_pdl(reduce_col_kernel<T, MODE, INDEX, IS_MAX, 1, kRedColScalarUnroll>, (unsigned)blocks, kRedThreads, 0, st, ip, op, xp, pl.map, pl.nslices, pl.K, pl.strideK, pl.I, pl.out_inner_stride, pl.idx_inner_stride, pl.nsplit, pl.split_len, pl.tiles_i, prm, partials, tickets, post);
      break;
    }
    case kRedStrided: {
      const uint64_t blocks = (pl.nslices + kRedThreads - 1) / kRedThreads;
      if (blocks >= (1ull << 31)) { set_error("reduce_dim: too many slices"); return THCB200_ERR_DIMS; }
      set_plan_name("strided");
      launch_pdl(reduce_strided_kernel<T, MODE, INDEX, IS_MAX>, (unsigned)blocks, kRedThreads, 0, st, ip, op, xp, pl.map, pl.nslices, pl.K, pl.strideK, prm, post);
      break;
    }
  }
  THCB_CUDA_TRY(cudaGetLastError());
  if (pl.nsplit > 1 && !tickets) {
    const uint64_t blocks = (noutputs + kRedThreads - 1) / kRedThreads;
    const uint64_t I = pl.kind == kRedCol ? pl.I : 1;
    launch_pdl(reduce_finish_kernel<T, MODE, INDEX, IS_MAX>, (unsigned)blocks, kRedThreads, 0, st, 
        op, xp, pl.map, pl.nslices, I, pl.out_inner_stride, pl.idx_inner_stride, pl.nsplit, partials, post);
    THCB_CUDA_TRY(cudaGetLastError());
    ++launches;
  }
  count_launch(launches);
  return 0;
}

template <typename T>
int reduce_dim_typed(thcb200_ctx *ctx, int mode, const HostView &in, const HostView &out, int dim, thcb200_scalar s,
                     PostOp post, cudaStream_t st) {
  switch (mode) {
    case kSum: return launch_reduce_dim<T, kSum, false, false>(ctx, in, out, nullptr, dim, s, post, st);
    case kProd: return launch_reduce_dim<T, kProd, false, false>(ctx, in, out, nullptr, dim, s, post, st);
    case kMin: return launch_reduce_dim<T, kMin, false, false>(ctx, in, out, nullptr, dim, s, post, st);
    case kMax: return launch_reduce_dim<T, kMax, false, false>(ctx, in, out, nullptr, dim, s, post, st);
    default: break;
  }
  if constexpr (TypeTraits<T>::is_fp) {
    switch (mode) {
      case kSumAbs: return launch_reduce_dim<T, kSumAbs, false, false>(ctx, in, out, nullptr, dim, s, post, st);
      case kSumSquare: return launch_reduce_dim<T, kSumSquare, false, false>(ctx, in, out, nullptr, dim, s, post, st);
      case kSumPowAbs: return launch_reduce_dim<T, kSumPowAbs, false, false>(ctx, in, out, nullptr, dim, s, post, st);
      case kSumNonZero: return launch_reduce_dim<T, kSumNonZero, false, false>(ctx, in, out, nullptr, dim, s, post, st);
      case kSumMoments: return launch_reduce_dim<T, kSumMoments, false, false>(ctx, in, out, nullptr, dim, s, post, st);
      default: break;
    }
  }
  set_error("reduce_dim: fold mode %d is not defined for dtype %d", mode, TypeTraits<T>::dtype);
  return THCB200_ERR_UNSUPPORTED;
}

template <typename T>
int reduce_dim_index_typed(thcb200_ctx *ctx, bool is_max, const HostView &in, const HostView &values,
                           const HostView &indices, int dim, cudaStream_t st) {
  thcb200_scalar s = {0.0, 0};
  if (is_max) return launch_reduce_dim<T, kMax, true, true>(ctx, in, values, &indices, dim, s, PostOp{kPostNone, 0.0, 0}, st);
  return launch_reduce_dim<T, kMin, true, false>(ctx, in, values, &indices, dim, s, PostOp{kPostNone, 0.0, 0}, st);
}

#define THCB_DECLARE_REDUCE(SUFFIX)                                                                                    \
  int reduce_all_##SUFFIX(thcb200_ctx *, int, const HostView &, thcb200_scalar, void *, cudaStream_t);                  \
  int reduce_dim_##SUFFIX(thcb200_ctx *, int, const HostView &, const HostView &, int, thcb200_scalar, PostOp, cudaStream_t);   \
  int reduce_dim_index_##SUFFIX(thcb200_ctx *, bool, const HostView &, const HostView &, const HostView &, int, cudaStream_t);
THCB_DECLARE_REDUCE(u8)
THCB_DECLARE_REDUCE(i8)
THCB_DECLARE_REDUCE(i16)
THCB_DECLARE_REDUCE(i32)
THCB_DECLARE_REDUCE(i64)
THCB_DECLARE_REDUCE(f16)
THCB_DECLARE_REDUCE(f32)
THCB_DECLARE_REDUCE(f64)
#undef THCB_DECLARE_REDUCE

}  // namespace thcb
