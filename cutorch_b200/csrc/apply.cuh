// Pointwise apply kernels for sm_100a and the per-call planner that picks one of them.
//
//   contig_vec : every operand collapses to one unit-stride run and is 16-byte aligned.
//                Each thread keeps 64 bytes per operand in flight as 32-byte (256-bit) or
//                16-byte vectors, all loads issued before the first use; one tile per CTA,
//                the tail handled by scalars.
//   tiled      : some operands have their unit stride in a different dimension than the
//                others (a transposed view).  A CTA stages a [TC x TJ] tile of those
//                operands through shared memory so that both the global reads (along the
//                operand's own unit-stride dim) and the global writes (along the output's)
//                move whole 32-byte sectors.
//   generic    : anything else: each operand individually collapsed
//                (TensorInfo::collapseDims rule), linear index -> offset by multiply-high
//                division, four independent elements in flight per thread.
//
// Replaces kernelPointwiseApply1/2/3 and THC_pointwiseApply1/2/3
// (lib/THC/THCApply.cuh:19-98,124-640).
#pragma once

#include "core.cuh"
#include "ops.cuh"

namespace thcb {

constexpr int kApplyThreads = 256;
constexpr int kApplyUnroll = 4;

// ----------------------------------------------------------------------------------
// contig_vec
// ----------------------------------------------------------------------------------
// VB = bytes per vector: 32 (256-bit ld/st.global of sm_100) when every operand is 32-byte aligned,
// else 16.  Each thread keeps 64 bytes per operand in flight either way.
template <int VB> constexpr int contig_unroll() { return 64 / VB; }
template <typename T, int VB> constexpr uint64_t contig_tile() { return (uint64_t)kApplyThreads * contig_unroll<VB>() * (VB / sizeof(T)); }

template <int OP, typename T, int NIN, int VB>
__global__ void __launch_bounds__(kApplyThreads)
apply_contig_vec_kernel(T *out, const T *a, const T *b, const T *c, uint64_t n,
                        OpParams<T> p) {
  pdl_prologue();
  constexpr int V = VB / sizeof(T);                       // elements per vector
  constexpr int U = contig_unroll<VB>();
  constexpr uint64_t kTile = contig_tile<T, VB>();
  using Vec = typename VecBytes<VB>::type;
  const uint64_t base = (uint64_t)blockIdx.x * kTile;
  if (base + kTile <= n) {
    Vec va[U], vb[U], vc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t i = base + ((uint64_t)u * kApplyThreads + threadIdx.x) * V;
      if constexpr (NIN >= 1) va[u] = ldv_stream<VB>(a + i);
      if constexpr (NIN >= 2) vb[u] = ldv_stream<VB>(b + i);
      if constexpr (NIN >= 3) vc[u] = ldv_stream<VB>(c + i);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t i = base + ((uint64_t)u * kApplyThreads + threadIdx.x) * V;
      Vec vo;
      T *eo = reinterpret_cast<T *>(&vo);
      const T *ea = reinterpret_cast<const T *>(&va[u]);
      const T *eb = reinterpret_cast<const T *>(&vb[u]);
      const T *ec = reinterpret_cast<const T *>(&vc[u]);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        T x = NIN >= 1 ? ea[k] : T();
        T y = NIN >= 2 ? eb[k] : T();
        T z = NIN >= 3 ? ec[k] : T();
        eo[k] = pw_apply<OP, T>(p, x, y, z);
      }
      stv<VB>(out + i, vo);
    }
  } else {
    for (uint64_t i = base + threadIdx.x; i < n; i += kApplyThreads) {
      T x = T(), y = T(), z = T();
      if constexpr (NIN >= 1) x = a[i];
      if constexpr (NIN >= 2) y = b[i];
      if constexpr (NIN >= 3) z = c[i];
      out[i] = pw_apply<OP, T>(p, x, y, z);
    }
  }
}

// ----------------------------------------------------------------------------------
// rows: along the innermost collapsed dim C every operand is either dense (stride 1) or constant
// (stride 0: one value per row, e.g. an expanded per-row factor); the outer dims (up to
// kRowsOuterDims of them, R rows in all) may have any strides, 0 included (an expanded bias
// vector), and need not collapse (a window cut out of a larger tensor).  Rows with padding
// between them land here too.  A row's offsets are decoded once per thread and row; a thread
// moves 16-byte vectors of the dense operands and reads the constant ones as scalars; the CTA
// is shaped [ty rows x tx vectors] with tx = the power of two covering C.
// ----------------------------------------------------------------------------------
constexpr int kRowsUnroll = 4;      // rows per thread
constexpr int kRowsScalarCols = 4;  // column slots per thread when elements move one by one
constexpr int kRowsOuterDims = 7;
struct RowsPlan {
  uint32_t R, Cvec;        // rows; units per row (16-byte vectors, or single elements when !vec)
  uint32_t tiles_c;        // CTAs along C
  int log2_tx;             // threads along C = 1 << log2_tx (<= 256)
  int vec;                 // 1: 16-byte vectors (rows aligned), 0: single elements (any pitch)
  int nouter;              // outer dims (>= 1); row number = row-major index over them
  FastDiv32 outer_size[kRowsOuterDims];
  int64_t outer_stride[4][kRowsOuterDims];   // elements, per operand
  int constant[4];         // 1: stride 0 along C
  // element offsets of row r in the four operands
  __device__ __forceinline__ void row_offsets(uint32_t r, int64_t (&off)[4]) const {
    off[0] = off[1] = off[2] = off[3] = 0;
    uint32_t rem = r;
#pragma unroll 1
    for (int i = nouter - 1; i >= 1; --i) {
      uint32_t q, m;
      outer_size[i].divmod(rem, q, m);
#pragma unroll
      for (int o = 0; o < 4; ++o) off[o] += (int64_t)m * outer_stride[o][i];
      rem = q;
    }
#pragma unroll
    for (int o = 0; o < 4; ++o) off[o] += (int64_t)rem * outer_stride[o][0];
  }
};

// V = elements per unit: 16 / sizeof(T), or 1 for rows whose pitch or base breaks the alignment.
template <int OP, typename T, int NIN, int V>
__global__ void __launch_bounds__(kApplyThreads)
apply_rows_kernel(T *out, const T *a, const T *b, const T *c, RowsPlan pl, OpParams<T> p) {
  pdl_prologue();
  constexpr int U = kRowsUnroll;
  constexpr int UC = V == 1 ? kRowsScalarCols : 1;
  struct alignas(V * sizeof(T)) Unit { T v[V]; };
  const unsigned tx = 1u << pl.log2_tx, ty = kApplyThreads >> pl.log2_tx;
  const unsigned x = threadIdx.x & (tx - 1), y = threadIdx.x >> pl.log2_tx;
  const uint32_t ctile = blockIdx.x % pl.tiles_c, rtile = blockIdx.x / pl.tiles_c;
  const T *in[3] = {a, b, c};
  Unit v[3][U][UC];
  int64_t out_off[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint32_t r = (rtile * U + u) * ty + y;
    int64_t off[4] = {0, 0, 0, 0};
    if (r < pl.R) pl.row_offsets(r, off);
    out_off[u] = off[0];
#pragma unroll
    for (int k = 0; k < UC; ++k) {
      const uint32_t cv = (ctile * UC + k) * tx + x;
      if (r < pl.R && cv < pl.Cvec) {
#pragma unroll
        for (int o = 0; o < NIN; ++o) {
          const T *row = in[o] + off[o + 1];
          if (pl.constant[o + 1]) {
            const T s = *row;
#pragma unroll
            for (int j = 0; j < V; ++j) v[o][u][k].v[j] = s;
          } else {
            v[o][u][k] = *reinterpret_cast<const Unit *>(row + (uint64_t)cv * V);
          }
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint32_t r = (rtile * U + u) * ty + y;
#pragma unroll
    for (int k = 0; k < UC; ++k) {
      const uint32_t cv = (ctile * UC + k) * tx + x;
      if (r < pl.R && cv < pl.Cvec) {
        Unit vo;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          T xx = NIN >= 1 ? v[0][u][k].v[j] : T();
          T yy = NIN >= 2 ? v[1][u][k].v[j] : T();
          T zz = NIN >= 3 ? v[2][u][k].v[j] : T();
          vo.v[j] = pw_apply<OP, T>(p, xx, yy, zz);
        }
        *reinterpret_cast<Unit *>(out + out_off[u] + (uint64_t)cv * V) = vo;
      }
    }
  }
}

// ----------------------------------------------------------------------------------
// generic
// ----------------------------------------------------------------------------------
template <int OP, typename T, int NIN, typename IndexT>
__global__ void __launch_bounds__(kApplyThreads)
apply_generic_kernel(T *out, StridedView<IndexT> vo, const T *a, StridedView<IndexT> va,
                     const T *b, StridedView<IndexT> vb, const T *c, StridedView<IndexT> vc,
                     IndexT n, OpParams<T> p) {
  pdl_prologue();
  constexpr int U = kApplyUnroll;
  const IndexT tile = (IndexT)kApplyThreads * U;
  // grid is sized so that blockIdx.x * tile never wraps; one tile per CTA
  const IndexT base = (IndexT)blockIdx.x * tile + threadIdx.x;
  T x[U], y[U], z[U];
  IndexT oo[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const IndexT i = base + (IndexT)u * kApplyThreads;
    x[u] = T(); y[u] = T(); z[u] = T();
    if (i < n) {
      oo[u] = vo.offset(i);
      if constexpr (NIN >= 1) x[u] = a[va.offset(i)];
      if constexpr (NIN >= 2) y[u] = b[vb.offset(i)];
      if constexpr (NIN >= 3) z[u] = c[vc.offset(i)];
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const IndexT i = base + (IndexT)u * kApplyThreads;
    if (i < n) out[oo[u]] = pw_apply<OP, T>(p, x[u], y[u], z[u]);
  }
}

// ----------------------------------------------------------------------------------
// tiled (transposed operands)
//
// Iteration space as seen by the kernel: [outer] x [C] x [J] in the output's logical
// order restricted to the dims that matter:
//   J  the trailing group of logical dims (row-major linear index j within the group),
//   C  one earlier logical dim in which the "staged" operands have stride 1,
//   outer: all remaining dims, decoded from blockIdx.
// "Direct" operands are addressed as base(outer) + c*strideC + j*strideJ (the J group
// collapses for them).  "Staged" operands are addressed as base(outer) + c + offJ(j),
// where offJ walks the (at most kTiledJDims) dims of the group with the operand's own
// strides.  A CTA handles TC consecutive c and TJ consecutive j.
//
// Phase 1 brings the staged tiles in with lanes along C: a warp instruction reads 256
// contiguous bytes of the staged operand, and each thread issues all of its row loads
// before the first shared-memory store.  Phase 2 runs with lanes along J: direct operands
// and the output move in contiguous runs, the staged values come transposed out of padded
// shared memory (conflict-free both ways), all global loads of a thread again first.
// ----------------------------------------------------------------------------------
constexpr int kTiledJDims = 3;
constexpr int kTiledOuterDims = 6;
constexpr int kTiledThreads = 256;
constexpr int kTJ = 64;            // j extent of a tile
constexpr int kTiledRunBytes = 256; // bytes of the staged operand's unit-stride run per tile row

struct TiledOperand {
  int staged;                        // 1: unit stride along C, goes through shared memory
  int slot;                          // shared-memory slot of a staged operand
  int64_t strideC;                   // element stride along C (1 when staged)
  int64_t strideJ;                   // direct operands: stride of the collapsed J group
  int64_t jstrides[kTiledJDims];     // staged operands: per-dim strides inside the J group
  int64_t ostrides[kTiledOuterDims]; // strides of the outer dims
};

struct TiledPlan {
  int nouter;
  int njd;                           // dims in the J group (staged-operand walk)
  int c_fastest;                     // 1: consecutive CTAs walk C first (neighbours share the staged operand's lines)
  uint32_t sizeC, sizeJ;
  uint32_t tilesC, tilesJ;
  FastDiv32 outerSizes[kTiledOuterDims];
  FastDiv32 jSizes[kTiledJDims];
  FastDiv32 tilesCdiv, tilesJdiv;
  TiledOperand op[4];                // 0 = out, 1..3 = inputs
};

inline int tiled_tc_for(size_t elem_size) { return (int)(kTiledRunBytes / elem_size); }
template <typename T> constexpr int tiled_tc() { return kTiledRunBytes / (int)sizeof(T); }
// padding that makes the row pitch an odd number of 32-bit words (64-bit words for 8-byte types)
template <typename T> constexpr int tiled_pad() { return sizeof(T) >= 4 ? 1 : (sizeof(T) == 2 ? 2 : 4); }
template <typename T> constexpr size_t tiled_slot_bytes() { return (size_t)kTJ * (tiled_tc<T>() + tiled_pad<T>()) * sizeof(T); }
// dynamic shared memory: the staged tiles, then one row-offset table per slot
template <typename T> constexpr size_t tiled_smem_bytes(int slots) {
  return (((size_t)slots * tiled_slot_bytes<T>() + 15) / 16) * 16 + (size_t)slots * kTJ * sizeof(int64_t);
}

template <int OP, typename T, int NIN>
__global__ void __launch_bounds__(kTiledThreads)
apply_tiled_kernel(T *out, const T *a, const T *b, const T *c, TiledPlan P, OpParams<T> p, int slots) {
  pdl_prologue();
  constexpr int TC = tiled_tc<T>();
  constexpr int LD = TC + tiled_pad<T>();    // padded row length in shared memory
  constexpr int NW = kTiledThreads / 32;
  constexpr int RPW = kTJ / NW;              // phase 1: rows (j) per warp
  constexpr int CPL = TC / 32;               // phase 1: c per lane
  constexpr int CPW = TC / NW;               // phase 2: c per warp
  constexpr int JPL = kTJ / 32;              // phase 2: j per lane
  constexpr int CPP = (CPW > 4) ? 4 : CPW;   // c per pass of phase 2 (bounds the registers)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T *tile = reinterpret_cast<T *>(smem_raw);  // [slots][kTJ][LD]
  constexpr int kSlot = kTJ * LD;
  int64_t *joffs = reinterpret_cast<int64_t *>(smem_raw + (((size_t)slots * tiled_slot_bytes<T>() + 15) / 16) * 16);

  // decode blockIdx -> (outer, tile_c, tile_j)
  uint32_t bid = blockIdx.x, tj, tc, rest;
  if (P.c_fastest) {
    P.tilesCdiv.divmod(bid, rest, tc);
    P.tilesJdiv.divmod(rest, rest, tj);
  } else {
    P.tilesJdiv.divmod(bid, rest, tj);
    P.tilesCdiv.divmod(rest, rest, tc);
  }
  int64_t base[4] = {0, 0, 0, 0};
#pragma unroll
  for (int d = kTiledOuterDims - 1; d >= 0; --d) {
    if (d < P.nouter) {
      uint32_t q, r;
      P.outerSizes[d].divmod(rest, q, r);
      rest = q;
#pragma unroll
      for (int o = 0; o <= NIN; ++o) base[o] += (int64_t)r * P.op[o].ostrides[d];
    }
  }
  const uint32_t c0 = tc * TC, j0 = tj * kTJ;
  const uint32_t nc = min((uint32_t)TC, P.sizeC - c0), nj = min((uint32_t)kTJ, P.sizeJ - j0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T *in[4] = {nullptr, a, b, c};
  const bool full = (nc == (uint32_t)TC) && (nj == (uint32_t)kTJ);
  const bool out_staged = P.op[0].staged;

  // ---- prologue: one thread per tile row walks the J group once for every staged operand
  if (threadIdx.x < kTJ && threadIdx.x < nj) {
    uint32_t q = j0 + threadIdx.x, r;
    uint32_t idx[kTiledJDims] = {0, 0, 0};
#pragma unroll
    for (int d = kTiledJDims - 1; d >= 0; --d) {
      if (d < P.njd) { P.jSizes[d].divmod(q, q, r); idx[d] = r; }
    }
#pragma unroll
    for (int o = 0; o <= NIN; ++o) {
      if (P.op[o].staged) {
        int64_t off = 0;
#pragma unroll
        for (int d = 0; d < kTiledJDims; ++d) off += (int64_t)idx[d] * P.op[o].jstrides[d];
        joffs[P.op[o].slot * kTJ + threadIdx.x] = off;
      }
    }
  }
  __syncthreads();

  // ---- phase 1: staged inputs -> shared memory, lanes along C
#pragma unroll
  for (int o = 1; o <= NIN; ++o) {
    if (!P.op[o].staged) continue;
    T *slot = tile + P.op[o].slot * kSlot;
    const int64_t *jo = joffs + P.op[o].slot * kTJ;
    const T *src = in[o] + base[o] + c0;
    if (full) {
      T v[RPW][CPL];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const T *row = src + jo[warp + r * NW] + lane;
#pragma unroll
        for (int q = 0; q < CPL; ++q) v[r][q] = row[32 * q];
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int q = 0; q < CPL; ++q) slot[(warp + r * NW) * LD + lane + 32 * q] = v[r][q];
    } else {
      for (uint32_t jj = warp; jj < nj; jj += NW) {
        const T *row = src + jo[jj];
        for (uint32_t cc = lane; cc < nc; cc += 32) slot[jj * LD + cc] = row[cc];
      }
    }
  }
  __syncthreads();

  // ---- phase 2: compute with lanes along J
  if (full) {
    // per-operand pointer of this thread's first element; later ones are whole multiples of incC / incJ away
    const T *ptr[4] = {nullptr, nullptr, nullptr, nullptr};
    int64_t incC[4] = {0, 0, 0, 0}, incJ[4] = {0, 0, 0, 0};
#pragma unroll
    for (int o = 1; o <= NIN; ++o) {
      if (!P.op[o].staged) {
        ptr[o] = in[o] + base[o] + (int64_t)(c0 + warp) * P.op[o].strideC + (int64_t)(j0 + lane) * P.op[o].strideJ;
        incC[o] = (int64_t)NW * P.op[o].strideC;
        incJ[o] = 32 * P.op[o].strideJ;
      }
    }
    T *optr = out + base[0] + (int64_t)(c0 + warp) * P.op[0].strideC + (int64_t)(j0 + lane) * P.op[0].strideJ;
    const int64_t oincC = (int64_t)NW * P.op[0].strideC, oincJ = 32 * P.op[0].strideJ;
#pragma unroll 1
    for (int r0 = 0; r0 < CPW; r0 += CPP) {
      T v[CPP][JPL][4];
#pragma unroll
      for (int o = 1; o <= NIN; ++o) {
        if (P.op[o].staged) {
          const T *slot = tile + P.op[o].slot * kSlot + lane * LD + warp + r0 * NW;
#pragma unroll
          for (int r = 0; r < CPP; ++r)
#pragma unroll
            for (int h = 0; h < JPL; ++h) v[r][h][o] = slot[h * 32 * LD + r * NW];
        } else {
          const T *pr = ptr[o] + (int64_t)r0 * P.op[o].strideC * NW;
#pragma unroll
          for (int r = 0; r < CPP; ++r) {
#pragma unroll
            for (int h = 0; h < JPL; ++h) v[r][h][o] = pr[h * incJ[o]];
            pr += incC[o];
          }
        }
      }
      T *po = optr + (int64_t)r0 * oincC;
#pragma unroll
      for (int r = 0; r < CPP; ++r) {
#pragma unroll
        for (int h = 0; h < JPL; ++h) {
          const T res = pw_apply<OP, T>(p, NIN >= 1 ? v[r][h][1] : T(), NIN >= 2 ? v[r][h][2] : T(), NIN >= 3 ? v[r][h][3] : T());
          if (out_staged) tile[P.op[0].slot * kSlot + (lane + 32 * h) * LD + warp + (r0 + r) * NW] = res;
          else po[h * oincJ] = res;
        }
        po += oincC;
      }
    }
  } else {
    for (uint32_t cc = warp; cc < nc; cc += NW) {
      for (uint32_t jj = lane; jj < nj; jj += 32) {
        T v[4];
#pragma unroll
        for (int o = 1; o <= NIN; ++o) {
          if (P.op[o].staged) v[o] = tile[P.op[o].slot * kSlot + jj * LD + cc];
          else v[o] = in[o][base[o] + (int64_t)(c0 + cc) * P.op[o].strideC + (int64_t)(j0 + jj) * P.op[o].strideJ];
        }
        const T res = pw_apply<OP, T>(p, NIN >= 1 ? v[1] : T(), NIN >= 2 ? v[2] : T(), NIN >= 3 ? v[3] : T());
        if (out_staged) tile[P.op[0].slot * kSlot + jj * LD + cc] = res;
        else out[base[0] + (int64_t)(c0 + cc) * P.op[0].strideC + (int64_t)(j0 + jj) * P.op[0].strideJ] = res;
      }
    }
  }

  // ---- phase 3: a staged output leaves through shared memory, lanes along C again
  if (out_staged) {
    __syncthreads();
    const T *slot = tile + P.op[0].slot * kSlot;
    const int64_t *jo = joffs + P.op[0].slot * kTJ;
    T *dst = out + base[0] + c0;
    for (uint32_t jj = warp; jj < nj; jj += NW) {
      T *row = dst + jo[jj];
      for (uint32_t cc = lane; cc < nc; cc += 32) row[cc] = slot[jj * LD + cc];
    }
  }
}

}  // namespace thcb
