// Calls whose operands have two element types: comparisons that write a Byte tensor and the
// Byte-masked fill / copy / select.  In cutorch these are THC_pointwiseApply2/3 instances with
// mixed types (lib/THC/THCTensorMathCompare.cuh, THCTensorMathCompareT.cuh, THCTensorMasked.cuh)
// plus a thrust prefix sum over a Long copy of the mask (lib/THC/generic/THCTensorMasked.cu:35-177).
// Here: vector kernels when every operand is one unit-stride run, strided kernels otherwise, and
// for copy / select a per-tile count + scan of tile counts + move, with the mask read as bytes.
#include <string.h>

#include "context.h"
#include "core.cuh"
#include "plan.h"

namespace thcb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

enum Cmp { kLT = 0, kGT = 1, kLE = 2, kGE = 3, kEQ = 4, kNE = 5 };

template <typename M>
__device__ __forceinline__ uint32_t cmp_eval(int cmp, M a, M b) {
  switch (cmp) {
    case kLT: return a < b;
    case kGT: return a > b;
    case kLE: return a <= b;
    case kGE: return a >= b;
    case kEQ: return a == b;
    default: return a != b;
  }
}

template <int B> struct Word;
template <> struct Word<1> { using type = uint8_t; };
template <> struct Word<2> { using type = uint16_t; };
template <> struct Word<4> { using type = uint32_t; };
template <> struct Word<8> { using type = uint64_t; };
template <> struct Word<16> { using type = Bytes16; };

// ---------------------------------------------------------------------------------
// compare, unit-stride operands: one 16-byte vector of `a` (and `b`) per step gives
// EV = 16 / sizeof(T) results, stored as one EV-byte word.  Lanes take adjacent vectors.
// ---------------------------------------------------------------------------------
template <typename T, bool HAS_B>
__global__ void __launch_bounds__(kThreads)
compare_contig_kernel(uint8_t *out, const T *a, const T *b, uint64_t n, int cmp, typename TypeTraits<T>::Math s) {
  pdl_prologue();
  using M = typename TypeTraits<T>::Math;
  constexpr int EV = 16 / (int)sizeof(T);
  using OutW = typename Word<EV>::type;
  const uint64_t nvec = n / EV;
  const uint64_t vbase = (uint64_t)blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
  Bytes16 va[kUnroll], vb[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint64_t v = vbase + (uint64_t)u * kThreads;
    if (v < nvec) {
      va[u] = ld16_stream(reinterpret_cast<const Bytes16 *>(a) + v);
      if constexpr (HAS_B) vb[u] = ld16_stream(reinterpret_cast<const Bytes16 *>(b) + v);
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint64_t v = vbase + (uint64_t)u * kThreads;
    if (v < nvec) {
      const T *xa = reinterpret_cast<const T *>(&va[u]);
      const T *xb = reinterpret_cast<const T *>(&vb[u]);
      alignas(16) uint8_t r[EV];
#pragma unroll
      for (int e = 0; e < EV; ++e) {
        const M y = HAS_B ? to_math<T>(xb[e]) : s;
        r[e] = (uint8_t)cmp_eval<M>(cmp, to_math<T>(xa[e]), y);
      }
      reinterpret_cast<OutW *>(out)[v] = *reinterpret_cast<const OutW *>(r);
    }
  }
  // elements past the last whole vector
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - nvec * EV)) {
    const uint64_t i = nvec * EV + threadIdx.x;
    const M y = HAS_B ? to_math<T>(b[i]) : s;
    out[i] = (uint8_t)cmp_eval<M>(cmp, to_math<T>(a[i]), y);
  }
}

template <typename T, bool HAS_B, typename IndexT>
__global__ void __launch_bounds__(kThreads)
compare_strided_kernel(uint8_t *out, StridedView<IndexT> vo, const T *a, StridedView<IndexT> va, const T *b,
                       StridedView<IndexT> vb, IndexT n, int cmp, typename TypeTraits<T>::Math s) {
  pdl_prologue();
  using M = typename TypeTraits<T>::Math;
  const IndexT base = (IndexT)blockIdx.x * (IndexT)(kThreads * kUnroll) + threadIdx.x;
  T x[kUnroll], y[kUnroll];
  IndexT oo[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const IndexT i = base + (IndexT)u * kThreads;
    x[u] = T(); y[u] = T(); oo[u] = 0;
    if (i < n) {
      oo[u] = vo.offset(i);
      x[u] = a[va.offset(i)];
      if constexpr (HAS_B) y[u] = b[vb.offset(i)];
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const IndexT i = base + (IndexT)u * kThreads;
    if (i < n) out[oo[u]] = (uint8_t)cmp_eval<M>(cmp, to_math<T>(x[u]), HAS_B ? to_math<T>(y[u]) : s);
  }
}

// ---------------------------------------------------------------------------------
// masked fill.  Elements are moved as raw words of their size (W = uintN_t).
// Unit-stride: per 16-byte vector of t the EV mask bytes are one word; a vector whose mask
// word is zero is neither read nor written, one whose mask bytes are all set is not read.
// ---------------------------------------------------------------------------------
template <typename W>
__global__ void __launch_bounds__(kThreads)
masked_fill_contig_kernel(W *t, const uint8_t *mask, uint64_t n, W value) {
  pdl_prologue();
  constexpr int EV = 16 / (int)sizeof(W);
  using MaskW = typename Word<EV>::type;
  const uint64_t nvec = n / EV;
  const uint64_t vbase = (uint64_t)blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
  MaskW mw[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint64_t v = vbase + (uint64_t)u * kThreads;
    mw[u] = MaskW();
    if (v < nvec) mw[u] = reinterpret_cast<const MaskW *>(mask)[v];
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint64_t v = vbase + (uint64_t)u * kThreads;
    if (v >= nvec) continue;
    const uint8_t *mb = reinterpret_cast<const uint8_t *>(&mw[u]);
    int nset = 0;
#pragma unroll
    for (int e = 0; e < EV; ++e) nset += mb[e] != 0;
    if (nset == 0) continue;
    Bytes16 x;
    if (nset < EV) x = ld16(reinterpret_cast<const Bytes16 *>(t) + v);
    W *xe = reinterpret_cast<W *>(&x);
#pragma unroll
    for (int e = 0; e < EV; ++e)
      if (mb[e]) xe[e] = value;
    st16(reinterpret_cast<Bytes16 *>(t) + v, x);
  }
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - nvec * EV)) {
    const uint64_t i = nvec * EV + threadIdx.x;
    if (mask[i]) t[i] = value;
  }
}

template <typename W, typename IndexT>
__global__ void __launch_bounds__(kThreads)
masked_fill_strided_kernel(W *t, StridedView<IndexT> vt, const uint8_t *mask, StridedView<IndexT> vm, IndexT n, W value) {
  pdl_prologue();
  const IndexT base = (IndexT)blockIdx.x * (IndexT)(kThreads * kUnroll) + threadIdx.x;
  uint8_t m[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const IndexT i = base + (IndexT)u * kThreads;
    m[u] = 0;
    if (i < n) m[u] = mask[vm.offset(i)];
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const IndexT i = base + (IndexT)u * kThreads;
    if (i < n && m[u]) t[vt.offset(i)] = value;
  }
}

// ---------------------------------------------------------------------------------
// masked copy / select.  The logical index space is cut into tiles of kTile elements; a CTA
// of 8 warps owns one tile, warp w the 512 consecutive elements [w*512, w*512+512) of it, and
// in step k lane l looks at element k*32 + l of those: a ballot per step is the mask of 32
// consecutive elements, so positions inside a warp come from popcounts and need no scan.
//   1. mask_tile_count_kernel: non-zero mask elements per tile.
//   2. tile_scan_kernel (one CTA): exclusive prefix of the tile counts, and the total.
//   3. masked_move_kernel: recomputes the ballots of its tile and moves the elements.
// ---------------------------------------------------------------------------------
// a / b with the 32-bit divide when both fit
__device__ __forceinline__ uint64_t div_by_u32_or_64(uint64_t a, uint64_t b) {
  if (((a | b) >> 32) == 0) return (uint32_t)a / (uint32_t)b;
  return a / b;
}
constexpr int kSteps = 16;
constexpr int kWarpSpan = 32 * kSteps;            // 512
constexpr int kTile = (kThreads / 32) * kWarpSpan;  // 4096

// ballots[k] = mask bits of elements wbase + k*32 .. + 31.  With `vec` (unit-stride, 16-byte
// aligned mask) a lane reads its 16 consecutive mask bytes in one load and the per-step words
// are put together from two lanes' 16-bit masks.
template <typename IndexT>
__device__ __forceinline__ uint32_t warp_mask_ballots(const uint8_t *mask, const StridedView<IndexT> &vm, uint64_t wbase,
                                                      uint64_t n, bool vec, uint32_t (&ballots)[kSteps]) {
  const unsigned lane = threadIdx.x & 31;
  uint32_t total = 0;
  if (vec && wbase + kWarpSpan <= n) {
    const Bytes16 v = ld16_stream(mask + wbase + (uint64_t)lane * 16);
    uint32_t bits = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int b = 0; b < 4; ++b) bits |= (((v.w[w] >> (8 * b)) & 0xFFu) != 0 ? 1u : 0u) << (4 * w + b);
    }
#pragma unroll
    for (int k = 0; k < kSteps; ++k) {
      const uint32_t lo = __shfl_sync(0xffffffffu, bits, 2 * k);
      const uint32_t hi = __shfl_sync(0xffffffffu, bits, 2 * k + 1);
      ballots[k] = lo | (hi << 16);
      total += __popc(ballots[k]);
    }
    return total;
  }
  uint8_t m[kSteps];
#pragma unroll
  for (int k = 0; k < kSteps; ++k) {
    const uint64_t i = wbase + (uint64_t)k * 32 + lane;
    m[k] = 0;
    if (i < n) m[k] = mask[vm.offset((IndexT)i)];
  }
#pragma unroll
  for (int k = 0; k < kSteps; ++k) {
    ballots[k] = __ballot_sync(0xffffffffu, m[k] != 0);
    total += __popc(ballots[k]);
  }
  return total;
}

// 0x80 in every byte of w that is not zero
__device__ __forceinline__ uint32_t nonzero_bytes(uint32_t w) {
  return (((w & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | w) & 0x80808080u;
}
// one bit per byte of a 16-byte mask vector: bit j set when byte j is not zero
__device__ __forceinline__ uint32_t nonzero_bits16(const Bytes16 &v) {
  uint32_t bits = 0;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    // the four flags sit at bits 7, 15, 23, 31; the multiply lines them up at bits 21..24
    const uint32_t nib = (((nonzero_bytes(v.w[w]) >> 7) * 0x00204081u) >> 21) & 0xFu;
    bits |= nib << (4 * w);
  }
  return bits;
}

// Unit-stride, 16-byte aligned mask, whole tiles only: a thread counts its 16 bytes of a tile with
// bit arithmetic; a CTA takes kCountTiles consecutive tiles, all loads first.
constexpr int kCountTiles = 4;
// It also leaves one bit per mask byte behind (16 bits per thread, 512 bytes per tile): the select
// and copy kernels that follow read those instead of the mask bytes again (an eighth of the traffic).
__global__ void __launch_bounds__(kThreads) mask_tile_count_vec_kernel(const uint8_t *mask, uint64_t full_tiles, uint32_t *counts,
                                                                       uint16_t *tile_bits) {
  pdl_prologue();
  __shared__ uint32_t wsum[kCountTiles][kThreads / 32];
  const uint64_t tile0 = (uint64_t)blockIdx.x * kCountTiles;
  Bytes16 v[kCountTiles];
#pragma unroll
  for (int t = 0; t < kCountTiles; ++t) {
    v[t] = Bytes16();
    if (tile0 + t < full_tiles) v[t] = ld16_stream(mask + (tile0 + t) * kTile + (uint64_t)threadIdx.x * 16);
  }
#pragma unroll
  for (int t = 0; t < kCountTiles; ++t) {
    const uint32_t b16 = nonzero_bits16(v[t]);
    if (tile0 + t < full_tiles) tile_bits[(tile0 + t) * (uint64_t)kThreads + threadIdx.x] = (uint16_t)b16;
    uint32_t c = __popc(b16);
    c = __reduce_add_sync(0xffffffffu, c);
    if ((threadIdx.x & 31) == 0) wsum[t][threadIdx.x >> 5] = c;
  }
  __syncthreads();
  if (threadIdx.x < kCountTiles && tile0 + threadIdx.x < full_tiles) {
    uint32_t s = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) s += wsum[threadIdx.x][w];
    counts[tile0 + threadIdx.x] = s;
  }
}

// maskedSelect with a unit-stride aligned mask and a unit-stride aligned source, whole tiles only.
// A lane owns 16 consecutive elements: one 16-byte mask load and the 16 * sizeof(W) bytes of data
// in 32-byte loads when the source allows (WIDE), so that every sector is fetched by exactly one
// instruction: with 16-byte loads and no L1 allocation two instructions fetch each sector from the
// L2.  The selected elements of a warp are packed into its slice of shared memory and leave as
// coalesced stores (the packed side keeps its own strides).
template <typename W, typename IndexT, bool WIDE>
__global__ void __launch_bounds__(kThreads)
masked_select_vec_kernel(const W *src, W *packed, StridedView<IndexT> vp, const uint16_t *tile_bits, const uint64_t *offsets) {
  pdl_prologue();
  __shared__ uint32_t wsum[kThreads / 32];
  __shared__ W stage[kThreads / 32][kWarpSpan];
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t ebase = (uint64_t)blockIdx.x * kTile + (uint64_t)warp * kWarpSpan + (uint64_t)lane * 16;
  uint64_t pos = offsets[blockIdx.x];   // needed last: in flight together with the mask bits and the data
  // the bits the counting pass left for this thread's 16 mask bytes
  const uint32_t bits = tile_bits[(uint64_t)blockIdx.x * kThreads + threadIdx.x];
  alignas(32) W e[16];
  constexpr int NV = (int)sizeof(W);   // 16-byte vectors holding 16 elements
  if constexpr (WIDE && NV >= 2) {
#pragma unroll
    for (int v = 0; v < NV / 2; ++v)
      *reinterpret_cast<Bytes32 *>(reinterpret_cast<char *>(e) + 32 * v) =
          ld32_stream(reinterpret_cast<const char *>(src + ebase) + 32 * v);
  } else {
#pragma unroll
    for (int v = 0; v < NV; ++v)
      *reinterpret_cast<Bytes16 *>(reinterpret_cast<char *>(e) + 16 * v) =
          ld16_stream(reinterpret_cast<const char *>(src + ebase) + 16 * v);
  }
  const uint32_t cnt = __popc(bits);
  uint32_t incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl += y;
  }
  const uint32_t wtotal = __shfl_sync(0xffffffffu, incl, 31);
  if (lane == 0) wsum[warp] = wtotal;
  uint32_t r = incl - cnt;
#pragma unroll
  for (int j = 0; j < 16; ++j)
    if ((bits >> j) & 1u) stage[warp][r++] = e[j];
  __syncthreads();
  for (unsigned w = 0; w < warp; ++w) pos += wsum[w];
  for (uint32_t i = lane; i < wtotal; i += 32) packed[vp.offset((IndexT)(pos + i))] = stage[warp][i];
}

template <typename IndexT>
__global__ void __launch_bounds__(kThreads)
mask_tile_count_kernel(const uint8_t *mask, StridedView<IndexT> vm, uint64_t n, bool vec, uint32_t *counts, uint32_t tile0) {
  pdl_prologue();
  __shared__ uint32_t wsum[kThreads / 32];
  const unsigned warp = threadIdx.x >> 5;
  const uint64_t tile = (uint64_t)blockIdx.x + tile0;
  const uint64_t wbase = tile * kTile + (uint64_t)warp * kWarpSpan;
  uint32_t ballots[kSteps];
  const uint32_t total = warp_mask_ballots<IndexT>(mask, vm, wbase, n, vec, ballots);
  if ((threadIdx.x & 31) == 0) wsum[warp] = total;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t s = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) s += wsum[w];
    counts[tile] = s;
  }
}

// offsets[i] = counts[0] + ... + counts[i-1]; *total = sum of all.  One CTA of 1024 threads: warp w
// owns a consecutive span of tiles and walks it 32 tiles at a time with coalesced loads (first to
// add its span up, then, once the 32 span totals are scanned, to write the offsets).
__global__ void __launch_bounds__(1024) tile_scan_kernel(const uint32_t *counts, uint64_t *offsets, uint64_t ntiles,
                                                         int64_t *total, int64_t *total_host) {
  pdl_prologue();
  __shared__ uint64_t span_total[32];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t steps = (ntiles + 1023) / 1024;          // 32-tile steps per warp
  const uint64_t lo = (uint64_t)warp * steps * 32;
  constexpr int B = 8;   // loads in flight per lane: a step is one dependent round trip to the L2
  uint64_t s = 0;
  for (uint64_t j = 0; j < steps; j += B) {
    uint32_t v[B];
#pragma unroll
    for (int u = 0; u < B; ++u) {
      const uint64_t i = lo + (j + u) * 32 + lane;
      v[u] = (j + u < steps && i < ntiles) ? counts[i] : 0u;
    }
#pragma unroll
    for (int u = 0; u < B; ++u) s += v[u];
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  if (lane == 0) span_total[warp] = s;
  __syncthreads();
  uint64_t run = 0;
  for (unsigned w = 0; w < warp; ++w) run += span_total[w];
  if (threadIdx.x == 1023) {
    *total = (int64_t)(run + s);
    *total_host = (int64_t)(run + s);   // mapped pinned memory: the caller reads it after a stream synchronisation
  }
  for (uint64_t j = 0; j < steps; j += B) {
    uint32_t v[B], incl[B];
#pragma unroll
    for (int u = 0; u < B; ++u) {
      const uint64_t i = lo + (j + u) * 32 + lane;
      v[u] = (j + u < steps && i < ntiles) ? counts[i] : 0u;
    }
#pragma unroll
    for (int u = 0; u < B; ++u) {
      incl[u] = v[u];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, incl[u], d);
        if (lane >= (unsigned)d) incl[u] += y;
      }
    }
#pragma unroll
    for (int u = 0; u < B; ++u) {
      const uint64_t i = lo + (j + u) * 32 + lane;
      if (j + u < steps && i < ntiles) offsets[i] = run + (incl[u] - v[u]);
      run += __shfl_sync(0xffffffffu, incl[u], 31);
    }
  }
}

// The same over several CTAs, for up to 2^18 tiles: CTA b owns tiles [1024 b, 1024 b + 1024), one
// per thread.  It first adds up every count before its span (at most 1 MiB of counts, resident in
// the L2, read with coalesced loads), then scans its own 1024 counts.  The single CTA above spends
// 17 us issuing instructions for 32768 tiles; spread over 32 SMs the scan takes a few.
__global__ void __launch_bounds__(1024) tile_scan_spread_kernel(const uint32_t *counts, uint64_t *offsets, uint32_t ntiles,
                                                                int64_t *total, int64_t *total_host) {
  pdl_prologue();
  __shared__ uint64_t before_part[32];
  __shared__ uint32_t warp_total[32];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t base = blockIdx.x * 1024u;
  const uint32_t i = base + threadIdx.x;
  const uint32_t mine = i < ntiles ? counts[i] : 0u;
  uint64_t before = 0;
  for (uint32_t j = threadIdx.x; j < base; j += 4096u) {
    uint32_t v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = j + (uint32_t)u * 1024u < base ? counts[j + (uint32_t)u * 1024u] : 0u;
#pragma unroll
    for (int u = 0; u < 4; ++u) before += v[u];
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) before += __shfl_xor_sync(0xffffffffu, before, d);
  uint32_t incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl += y;
  }
  if (lane == 0) before_part[warp] = before;
  if (lane == 31) warp_total[warp] = incl;
  __syncthreads();
  uint64_t run = 0;
#pragma unroll
  for (int w = 0; w < 32; ++w) run += before_part[w];
  for (unsigned w = 0; w < warp; ++w) run += warp_total[w];
  if (i < ntiles) offsets[i] = run + (incl - mine);
  if (i == ntiles - 1) {
    *total = (int64_t)(run + incl);
    *total_host = (int64_t)(run + incl);   // mapped pinned memory: the caller reads it after a stream synchronisation
  }
}

// SELECT: packed[pos] = strided[i];  otherwise (copy): strided[i] = packed[pos]; for set mask
// elements, pos = rank of i among them.  `packed` is walked through its own view too.
template <typename W, typename IndexT, bool SELECT>
__global__ void __launch_bounds__(kThreads)
masked_move_kernel(W *strided, StridedView<IndexT> vs, W *packed, StridedView<IndexT> vp, const uint8_t *mask,
                   StridedView<IndexT> vm, uint64_t n, bool vec, const uint64_t *offsets, uint32_t tile0) {
  pdl_prologue();
  __shared__ uint32_t wsum[kThreads / 32];
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t tile = (uint64_t)blockIdx.x + tile0;
  const uint64_t wbase = tile * kTile + (uint64_t)warp * kWarpSpan;
  uint32_t ballots[kSteps];
  const uint32_t total = warp_mask_ballots<IndexT>(mask, vm, wbase, n, vec, ballots);
  if (lane == 0) wsum[warp] = total;
  __syncthreads();
  uint64_t pos = offsets[tile];
  for (unsigned w = 0; w < warp; ++w) pos += wsum[w];
  const uint32_t below = (1u << lane) - 1u;
  if (SELECT) {
    W x[kSteps];
#pragma unroll
    for (int k = 0; k < kSteps; ++k)
      if ((ballots[k] >> lane) & 1u) x[k] = strided[vs.offset((IndexT)(wbase + (uint64_t)k * 32 + lane))];
#pragma unroll
    for (int k = 0; k < kSteps; ++k) {
      if ((ballots[k] >> lane) & 1u) packed[vp.offset((IndexT)(pos + __popc(ballots[k] & below)))] = x[k];
      pos += __popc(ballots[k]);
    }
  } else {
    W x[kSteps];
    uint64_t p = pos;
#pragma unroll
    for (int k = 0; k < kSteps; ++k) {
      if ((ballots[k] >> lane) & 1u) x[k] = packed[vp.offset((IndexT)(p + __popc(ballots[k] & below)))];
      p += __popc(ballots[k]);
    }
#pragma unroll
    for (int k = 0; k < kSteps; ++k)
      if ((ballots[k] >> lane) & 1u) strided[vs.offset((IndexT)(wbase + (uint64_t)k * 32 + lane))] = x[k];
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
struct Collapsed {
  int dims;
  int64_t sizes[kMaxDims];
  int64_t strides[kMaxDims];
  bool unit;      // one run of stride 1
  bool fits32;
};

// Collapses one operand on its own (TensorInfo::collapseDims).  False when more than
// kGenericDims dims remain.
bool collapse_view(const HostView &v, Collapsed *c) {
  c->dims = v.ndim;
  for (int i = 0; i < v.ndim; ++i) { c->sizes[i] = v.sizes[i]; c->strides[i] = v.strides[i]; }
  if (c->dims == 0) { c->dims = 1; c->sizes[0] = 1; c->strides[0] = 1; }
  collapse_dims(c->sizes, c->strides, &c->dims, -1);
  c->unit = c->dims == 1 && c->strides[0] == 1;
  c->fits32 = can_use_32bit(v);
  return c->dims <= kGenericDims;
}

template <typename IndexT>
StridedView<IndexT> make_view(const Collapsed &c) {
  StridedView<IndexT> v;
  v.dims = c.dims;
  for (int i = 0; i < kGenericDims; ++i) {
    if (i < c.dims) {
      v.sizes[i] = DivHelper<IndexT>((uint64_t)c.sizes[i]);
      v.strides[i] = (IndexT)c.strides[i];
    } else {
      v.sizes[i] = DivHelper<IndexT>(1);
      v.strides[i] = 0;
    }
  }
  return v;
}

inline bool aligned16(const void *p) { return ((uintptr_t)p) % 16 == 0; }

int grid_for(uint64_t units, uint64_t per_cta, unsigned *grid, const char *what) {
  const uint64_t blocks = (units + per_cta - 1) / per_cta;
  if (blocks >= (1ULL << 31)) { set_error("%s: tensor too large", what); return THCB200_ERR_DIMS; }
  *grid = (unsigned)(blocks ? blocks : 1);
  return 0;
}

template <typename T>
int compare_typed(int cmp, bool has_b, const HostView &vo, const HostView &va, const HostView &vb,
                  thcb200_scalar s, cudaStream_t st) {
  using M = typename TypeTraits<T>::Math;
  M sv;
  if constexpr (TypeTraits<T>::is_fp) sv = (M)s.f; else sv = (M)s.i;
  Collapsed co, ca, cb;
  bool ok = collapse_view(vo, &co) && collapse_view(va, &ca);
  if (has_b) ok = ok && collapse_view(vb, &cb); else cb = ca;
  if (!ok) { set_error("compare: a view keeps more than %d dims after collapsing", kGenericDims); return THCB200_ERR_DIMS; }
  const uint64_t n = (uint64_t)vo.numel;
  uint8_t *out = reinterpret_cast<uint8_t *>(vo.data);
  const T *a = reinterpret_cast<const T *>(va.data);
  const T *b = has_b ? reinterpret_cast<const T *>(vb.data) : nullptr;
  unsigned grid;
  if (co.unit && ca.unit && (!has_b || cb.unit) && aligned16(out) && aligned16(a) && aligned16(b)) {
    constexpr int EV = 16 / (int)sizeof(T);
    int rc = grid_for(n / EV, (uint64_t)kThreads * kUnroll, &grid, "compare");
    if (rc) return rc;
    set_plan_name("compare_contig_vec");
    if (has_b) launch_pdl(compare_contig_kernel<T, true>, grid, kThreads, 0, st, out, a, b, n, cmp, sv);
    else launch_pdl(compare_contig_kernel<T, false>, grid, kThreads, 0, st, out, a, b, n, cmp, sv);
  } else {
    int rc = grid_for(n, (uint64_t)kThreads * kUnroll, &grid, "compare");
    if (rc) return rc;
    const bool i32 = co.fits32 && ca.fits32 && (!has_b || cb.fits32);
    set_plan_name(i32 ? "compare_strided32" : "compare_strided64");
#define THCB_CMP_LAUNCH(HB, IDX)                                                                          \
  launch_pdl(compare_strided_kernel<T, HB, IDX>, grid, kThreads, 0, st, out, make_view<IDX>(co), a, make_view<IDX>(ca), b, \
                                                                make_view<IDX>(cb), (IDX)n, cmp, sv)
    if (i32) { if (has_b) THCB_CMP_LAUNCH(true, uint32_t); else THCB_CMP_LAUNCH(false, uint32_t); }
    else { if (has_b) THCB_CMP_LAUNCH(true, uint64_t); else THCB_CMP_LAUNCH(false, uint64_t); }
#undef THCB_CMP_LAUNCH
  }
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

// the scalar as the raw bits of an element of dtype `dt`
uint64_t scalar_bits(int dt, thcb200_scalar s) {
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

template <typename W>
int masked_fill_sized(const HostView &vt, const HostView &vm, uint64_t bits, cudaStream_t st) {
  Collapsed ct, cm;
  if (!collapse_view(vt, &ct) || !collapse_view(vm, &cm)) {
    set_error("masked_fill: a view keeps more than %d dims after collapsing", kGenericDims);
    return THCB200_ERR_DIMS;
  }
  const uint64_t n = (uint64_t)vt.numel;
  W *t = reinterpret_cast<W *>(vt.data);
  const uint8_t *mask = reinterpret_cast<const uint8_t *>(vm.data);
  const W value = (W)bits;
  unsigned grid;
  if (ct.unit && cm.unit && aligned16(t) && aligned16(mask)) {
    constexpr int EV = 16 / (int)sizeof(W);
    int rc = grid_for(n / EV, (uint64_t)kThreads * kUnroll, &grid, "masked_fill");
    if (rc) return rc;
    set_plan_name("masked_fill_contig_vec");
    launch_pdl(masked_fill_contig_kernel<W>, grid, kThreads, 0, st, t, mask, n, value);
  } else {
    int rc = grid_for(n, (uint64_t)kThreads * kUnroll, &grid, "masked_fill");
    if (rc) return rc;
    if (ct.fits32 && cm.fits32) {
      set_plan_name("masked_fill_strided32");
      launch_pdl(masked_fill_strided_kernel<W, uint32_t>, grid, kThreads, 0, st, t, make_view<uint32_t>(ct), mask,
                                                                         make_view<uint32_t>(cm), (uint32_t)n, value);
    } else {
      set_plan_name("masked_fill_strided64");
      launch_pdl(masked_fill_strided_kernel<W, uint64_t>, grid, kThreads, 0, st, t, make_view<uint64_t>(ct), mask,
                                                                         make_view<uint64_t>(cm), (uint64_t)n, value);
    }
  }
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

// ---- mask counting shared by masked_count / masked_copy / masked_select ----
uint64_t layout_hash(const HostView &v) {
  uint64_t h = 1469598103934665603ULL;
  auto mix = [&h](uint64_t x) { h = (h ^ x) * 1099511628211ULL; };
  mix((uint64_t)v.ndim);
  for (int i = 0; i < v.ndim; ++i) { mix((uint64_t)v.sizes[i]); mix((uint64_t)v.strides[i]); }
  return h;
}

// bytes [24, 32) of the context's pinned, mapped slot receive the number of set mask elements
constexpr size_t kHostCountOffset = 24;

struct MaskPrep {
  uint64_t ntiles;
  uint64_t *offsets;   // device, ntiles entries
  int64_t *total;      // device
  uint16_t *tile_bits; // device: one bit per mask byte for the whole tiles of a dense aligned mask (else unused)
  Collapsed cm;
  bool hit;            // the offsets were found in the context and thcb200_masked_count has read their total
};

// When the tile offsets of a mask are found in the context, thcb200_masked_count ran on it before and
// the number of set elements sits in the pinned slot (that call synchronised to read it).  True, with *rc set, when an output of `have` elements cannot hold
// count * per_element of them.
bool counted_on_host(thcb200_ctx *ctx, int *rc, int64_t have, int64_t per_element, const char *what) {
  int64_t count = 0;
  memcpy(&count, (char *)ctx->host_slot + kHostCountOffset, 8);
  if (count < 0 || have >= count * per_element) return false;
  set_error("%s: the output holds %lld elements, the mask selects %lld x %lld", what, (long long)have, (long long)count,
            (long long)per_element);
  *rc = THCB200_ERR_SIZE;
  return true;
}


// Fills the context's tile offsets for this mask view (or finds them there when `reuse`).
int prepare_mask(thcb200_ctx *ctx, const HostView &vm, bool reuse, cudaStream_t st, MaskPrep *mp) {
  if (!collapse_view(vm, &mp->cm)) {
    set_error("masked: the mask keeps more than %d dims after collapsing", kGenericDims);
    return THCB200_ERR_DIMS;
  }
  const uint64_t n = (uint64_t)vm.numel;
  mp->ntiles = (n + kTile - 1) / kTile;
  if (mp->ntiles >= (1ULL << 31)) { set_error("masked: tensor too large"); return THCB200_ERR_DIMS; }
  // layout: [total: 8 B, padded to 256][offsets: 8 B x ntiles][counts: 4 B x ntiles][bits: 512 B x ntiles]
  // (the bits only for a dense 16-byte aligned mask: n / 8 bytes)
  const bool dense_aligned = mp->cm.unit && aligned16(vm.data);
  const size_t bits_at = (256 + mp->ntiles * 12 + 255) & ~(size_t)255;
  const size_t need = bits_at + (dense_aligned ? mp->ntiles * (size_t)kThreads * 2 : 0);
  const uint64_t lh = layout_hash(vm);
  const bool hit = reuse && ctx->prep_valid && ctx->prep_mask == (const void *)vm.data && ctx->prep_numel == vm.numel &&
                   ctx->prep_layout == lh && ctx->prep_stream == (void *)st && ctx->mask_ws_bytes >= need;
  if (!hit && ctx->mask_ws_bytes < need) {
    ctx->prep_valid = 0;
    if (ctx->mask_ws) {
      THCB_CUDA_TRY(cudaDeviceSynchronize());
      cudaFree(ctx->mask_ws);
      ctx->mask_ws = nullptr;
      ctx->mask_ws_bytes = 0;
    }
    size_t want = 1 << 20;
    while (want < need) want <<= 1;
    if (device_alloc(&ctx->mask_ws, want) != cudaSuccess) {
      cudaGetLastError();
      ctx->mask_ws = nullptr;
      set_error("masked: cannot allocate %zu bytes of tile offsets", want);
      return THCB200_ERR_NOMEM;
    }
    ctx->mask_ws_bytes = want;
  }
  char *base = reinterpret_cast<char *>(ctx->mask_ws);
  mp->total = reinterpret_cast<int64_t *>(base);
  mp->offsets = reinterpret_cast<uint64_t *>(base + 256);
  uint32_t *counts = reinterpret_cast<uint32_t *>(base + 256 + mp->ntiles * 8);
  mp->tile_bits = reinterpret_cast<uint16_t *>(base + bits_at);
  mp->hit = hit && ctx->prep_count_known;
  if (hit) return 0;
  ctx->prep_valid = 0;
  ctx->prep_count_known = 0;
  const uint8_t *mask = reinterpret_cast<const uint8_t *>(vm.data);
  const bool mask_vec = mp->cm.unit && aligned16(mask);
  // whole tiles of a unit-stride aligned mask go through the vector count; the rest (a ragged last
  // tile, or any other layout) through the strided one
  const uint64_t full = mask_vec ? n / kTile : 0;
  int launches = 1;
  if (full > 0) {
    launch_pdl(mask_tile_count_vec_kernel, (unsigned)((full + kCountTiles - 1) / kCountTiles), kThreads, 0, st, mask, full, counts, mp->tile_bits);
    ++launches;
  }
  if (full < mp->ntiles) {
    const unsigned rest = (unsigned)(mp->ntiles - full);
    if (mp->cm.fits32)
      launch_pdl(mask_tile_count_kernel<uint32_t>, rest, kThreads, 0, st, mask, make_view<uint32_t>(mp->cm), n, mask_vec, counts, (uint32_t)full);
    else
      launch_pdl(mask_tile_count_kernel<uint64_t>, rest, kThreads, 0, st, mask, make_view<uint64_t>(mp->cm), n, mask_vec, counts, (uint32_t)full);
    ++launches;
  }
  int64_t *total_host = reinterpret_cast<int64_t *>((char *)ctx->host_slot_dev + kHostCountOffset);
  if (mp->ntiles > 1024 && mp->ntiles <= (1u << 18))
    launch_pdl(tile_scan_spread_kernel, (unsigned)((mp->ntiles + 1023) / 1024), 1024, 0, st, counts, mp->offsets, (uint32_t)mp->ntiles, mp->total, total_host);
  else
    launch_pdl(tile_scan_kernel, 1, 1024, 0, st, counts, mp->offsets, mp->ntiles, mp->total, total_host);
  count_launch(launches);
  THCB_CUDA_TRY(cudaGetLastError());
  ctx->prep_mask = vm.data;
  ctx->prep_numel = vm.numel;
  ctx->prep_layout = lh;
  ctx->prep_stream = (void *)st;
  ctx->prep_valid = 1;
  return 0;
}

// nonzero: for every set element of a dense mask, in order, the 1-based coordinates it has in a
// tensor of the given sizes, one row of `nd` int64 per element.  Same tiles, ranks and tile offsets
// as the select kernel; a lane owns 16 consecutive mask bytes.
struct CoordShape {
  int nd;
  uint64_t size[kMaxDims];
};
__global__ void __launch_bounds__(kThreads)
mask_coords_kernel(const uint8_t *mask, uint64_t n, bool vec /* mask base is 16-byte aligned */, const uint64_t *offsets,
                   CoordShape shape, int64_t *out) {
  pdl_prologue();
  __shared__ uint32_t wsum[kThreads / 32];
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t ebase = (uint64_t)blockIdx.x * kTile + (uint64_t)warp * kWarpSpan + (uint64_t)lane * 16;
  uint64_t pos = offsets[blockIdx.x];
  uint32_t bits = 0;
  if (vec && ebase + 16 <= n) {
    bits = nonzero_bits16(ld16_stream(mask + ebase));
  } else {
    // a ragged end, or a dense mask that starts off a 16-byte boundary (a narrowed ByteTensor)
    for (int j = 0; j < 16; ++j)
      if (ebase + j < n && mask[ebase + j]) bits |= 1u << j;
  }
  const uint32_t cnt = __popc(bits);
  uint32_t incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl += y;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  for (unsigned w = 0; w < warp; ++w) pos += wsum[w];
  pos += incl - cnt;
  for (int j = 0; j < 16; ++j) {
    if (!((bits >> j) & 1u)) continue;
    uint64_t rem = ebase + j;
    int64_t *row = out + pos * (uint64_t)shape.nd;
    for (int d = shape.nd - 1; d >= 0; --d) {
      const uint64_t q = d == 0 ? 0 : div_by_u32_or_64(rem, shape.size[d]);
      row[d] = (int64_t)(rem - q * shape.size[d]) + 1;
      rem = q;
    }
    ++pos;
  }
}

template <typename W, bool SELECT>
int masked_move_sized(thcb200_ctx *ctx, const HostView &vstrided, const HostView &vpacked, const HostView &vm,
                      bool reuse, cudaStream_t st) {
  MaskPrep mp;
  int rc = prepare_mask(ctx, vm, reuse, st, &mp);
  if (rc) return rc;
  // with the count already on the host a packed side that is too short is refused instead of overrun
  if (mp.hit && counted_on_host(ctx, &rc, vpacked.numel, 1, SELECT ? "masked_select" : "masked_copy")) return rc;
  Collapsed cs, cp;
  if (!collapse_view(vstrided, &cs) || !collapse_view(vpacked, &cp)) {
    set_error("masked: a view keeps more than %d dims after collapsing", kGenericDims);
    return THCB200_ERR_DIMS;
  }
  W *strided = reinterpret_cast<W *>(vstrided.data);
  W *packed = reinterpret_cast<W *>(vpacked.data);
  const uint8_t *mask = reinterpret_cast<const uint8_t *>(vm.data);
  const uint64_t n = (uint64_t)vm.numel;
  const bool mask_vec = mp.cm.unit && aligned16(mask);
  const bool i32 = cs.fits32 && cp.fits32 && mp.cm.fits32;
  // select from a dense aligned source under a dense aligned mask: whole tiles take the vector kernel
  uint64_t full = 0;
  int launches = 0;
  if (SELECT && mask_vec && cs.unit && aligned16(strided)) {
    full = n / kTile;
    if (full > 0) {
      set_plan_name(i32 ? "masked_select_vec32" : "masked_select_vec64");
      const bool wide = ((uintptr_t)strided) % 32 == 0;
      if (i32 && wide) launch_pdl(masked_select_vec_kernel<W, uint32_t, true>, (unsigned)full, kThreads, 0, st, strided, packed, make_view<uint32_t>(cp), mp.tile_bits, mp.offsets);
      else if (i32) launch_pdl(masked_select_vec_kernel<W, uint32_t, false>, (unsigned)full, kThreads, 0, st, strided, packed, make_view<uint32_t>(cp), mp.tile_bits, mp.offsets);
      else if (wide) launch_pdl(masked_select_vec_kernel<W, uint64_t, true>, (unsigned)full, kThreads, 0, st, strided, packed, make_view<uint64_t>(cp), mp.tile_bits, mp.offsets);
      else launch_pdl(masked_select_vec_kernel<W, uint64_t, false>, (unsigned)full, kThreads, 0, st, strided, packed, make_view<uint64_t>(cp), mp.tile_bits, mp.offsets);
      ++launches;
    }
  }
  if (full < mp.ntiles) {
    const unsigned rest = (unsigned)(mp.ntiles - full);
    if (full == 0) set_plan_name(SELECT ? (i32 ? "masked_select32" : "masked_select64") : (i32 ? "masked_copy32" : "masked_copy64"));
    if (i32)
      launch_pdl(masked_move_kernel<W, uint32_t, SELECT>, rest, kThreads, 0, st, strided, make_view<uint32_t>(cs), packed, make_view<uint32_t>(cp), mask,
                                                                       make_view<uint32_t>(mp.cm), n, mask_vec, mp.offsets, (uint32_t)full);
    else
      launch_pdl(masked_move_kernel<W, uint64_t, SELECT>, rest, kThreads, 0, st, strided, make_view<uint64_t>(cs), packed, make_view<uint64_t>(cp), mask,
                                                                       make_view<uint64_t>(mp.cm), n, mask_vec, mp.offsets, (uint32_t)full);
    ++launches;
  }
  count_launch(launches);
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

int check_mask(const thcb200_tensor *mask, HostView *vm, const char *what) {
  int rc = to_host_view(mask, vm, what);
  if (rc) return rc;
  if (vm->dtype != THCB200_U8) { set_error("%s: the mask must be a U8 view", what); return THCB200_ERR_ARG; }
  return 0;
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" {

int thcb200_compare(thcb200_ctx *ctx, int cmp, const thcb200_tensor *out_u8, const thcb200_tensor *a,
                    const thcb200_tensor *b, thcb200_scalar s, void *stream) {
  if (!ctx) { set_error("compare: null context"); return THCB200_ERR_ARG; }
  int code;
  if (cmp >= THCB200_OP_LT && cmp <= THCB200_OP_NE) code = cmp - THCB200_OP_LT;
  else if (cmp >= THCB200_OP_LT_S && cmp <= THCB200_OP_NE_S) code = cmp - THCB200_OP_LT_S;
  else { set_error("compare: op %d is not a comparison", cmp); return THCB200_ERR_ARG; }
  HostView vo, va, vb;
  int rc = to_host_view(out_u8, &vo, "compare output");
  if (!rc) rc = to_host_view(a, &va, "compare input 0");
  if (!rc && b) rc = to_host_view(b, &vb, "compare input 1");
  if (rc) return rc;
  if (vo.dtype != THCB200_U8) { set_error("compare: the output must be a U8 view"); return THCB200_ERR_ARG; }
  if (b && vb.dtype != va.dtype) { set_error("compare: inputs have different dtypes"); return THCB200_ERR_ARG; }
  if (vo.numel != va.numel || (b && vb.numel != va.numel)) {
    set_error("compare: operands have different element counts");
    return THCB200_ERR_SIZE;
  }
  if (vo.numel == 0) return THCB200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool hb = b != nullptr;
  switch (va.dtype) {
    case THCB200_U8: return compare_typed<uint8_t>(code, hb, vo, va, vb, s, st);
    case THCB200_I8: return compare_typed<int8_t>(code, hb, vo, va, vb, s, st);
    case THCB200_I16: return compare_typed<int16_t>(code, hb, vo, va, vb, s, st);
    case THCB200_I32: return compare_typed<int32_t>(code, hb, vo, va, vb, s, st);
    case THCB200_I64: return compare_typed<int64_t>(code, hb, vo, va, vb, s, st);
    case THCB200_F16: return compare_typed<__half>(code, hb, vo, va, vb, s, st);
    case THCB200_F32: return compare_typed<float>(code, hb, vo, va, vb, s, st);
    default: return compare_typed<double>(code, hb, vo, va, vb, s, st);
  }
}

int thcb200_masked_fill(thcb200_ctx *ctx, const thcb200_tensor *t, const thcb200_tensor *mask_u8, thcb200_scalar value,
                        void *stream) {
  if (!ctx) { set_error("masked_fill: null context"); return THCB200_ERR_ARG; }
  HostView vt, vm;
  int rc = to_host_view(t, &vt, "masked_fill tensor");
  if (!rc) rc = check_mask(mask_u8, &vm, "masked_fill");
  if (rc) return rc;
  if (vt.numel != vm.numel) { set_error("masked_fill: tensor and mask have different element counts"); return THCB200_ERR_SIZE; }
  if (vt.numel == 0) return THCB200_OK;
  const uint64_t bits = scalar_bits(vt.dtype, value);
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype_size(vt.dtype)) {
    case 1: return masked_fill_sized<uint8_t>(vt, vm, bits, st);
    case 2: return masked_fill_sized<uint16_t>(vt, vm, bits, st);
    case 4: return masked_fill_sized<uint32_t>(vt, vm, bits, st);
    default: return masked_fill_sized<uint64_t>(vt, vm, bits, st);
  }
}

int thcb200_masked_count(thcb200_ctx *ctx, const thcb200_tensor *mask_u8, int64_t *count_host, void *stream) {
  if (!ctx || !count_host) { set_error("masked_count: null argument"); return THCB200_ERR_ARG; }
  HostView vm;
  int rc = check_mask(mask_u8, &vm, "masked_count");
  if (rc) return rc;
  if (vm.numel == 0) { *count_host = 0; return THCB200_OK; }
  THCB_CTX_LOCK(ctx);
  cudaStream_t st = (cudaStream_t)stream;
  MaskPrep mp;
  rc = prepare_mask(ctx, vm, false, st, &mp);
  if (rc) return rc;
  THCB_CUDA_TRY(cudaStreamSynchronize(st));
  memcpy(count_host, (char *)ctx->host_slot + kHostCountOffset, 8);
  ctx->prep_count_known = 1;   // the pinned slot now holds the count of exactly this mask
  return THCB200_OK;
}

static int masked_move(thcb200_ctx *ctx, bool select, const thcb200_tensor *strided, const thcb200_tensor *packed,
                       const thcb200_tensor *mask_u8, void *stream, int flags, const char *what) {
  if (!ctx) { set_error("%s: null context", what); return THCB200_ERR_ARG; }
  HostView vs, vp, vm;
  int rc = to_host_view(strided, &vs, what);
  if (!rc) rc = to_host_view(packed, &vp, what);
  if (!rc) rc = check_mask(mask_u8, &vm, what);
  if (rc) return rc;
  if (vs.dtype != vp.dtype) { set_error("%s: operands have different dtypes", what); return THCB200_ERR_ARG; }
  if (vs.numel != vm.numel) { set_error("%s: tensor and mask have different element counts", what); return THCB200_ERR_SIZE; }
  if (vm.numel == 0) return THCB200_OK;
  THCB_CTX_LOCK(ctx);
  const bool reuse = (flags & THCB200_FLAG_MASK_COUNTED) != 0;
  cudaStream_t st = (cudaStream_t)stream;
#define THCB_MOVE(W) (select ? masked_move_sized<W, true>(ctx, vs, vp, vm, reuse, st) : masked_move_sized<W, false>(ctx, vs, vp, vm, reuse, st))
  switch (dtype_size(vs.dtype)) {
    case 1: return THCB_MOVE(uint8_t);
    case 2: return THCB_MOVE(uint16_t);
    case 4: return THCB_MOVE(uint32_t);
    default: return THCB_MOVE(uint64_t);
  }
#undef THCB_MOVE
}

int thcb200_mask_coords(thcb200_ctx *ctx, const thcb200_tensor *out_i64, const thcb200_tensor *mask_u8, const int64_t *sizes,
                        int nd, void *stream, int flags) {
  if (!ctx || !sizes) { set_error("mask_coords: null argument"); return THCB200_ERR_ARG; }
  if (nd < 1 || nd > THCB200_MAX_DIMS) { set_error("mask_coords: %d dims", nd); return THCB200_ERR_DIMS; }
  HostView vo, vm;
  int rc = to_host_view(out_i64, &vo, "mask_coords output");
  if (!rc) rc = check_mask(mask_u8, &vm, "mask_coords");
  if (rc) return rc;
  if (vo.dtype != THCB200_I64) { set_error("mask_coords: the output must be an I64 view"); return THCB200_ERR_ARG; }
  int64_t total = 1;
  CoordShape shape;
  shape.nd = nd;
  for (int d = 0; d < nd; ++d) { shape.size[d] = (uint64_t)sizes[d]; total *= sizes[d]; }
  if (total != vm.numel) { set_error("mask_coords: the sizes do not multiply to the mask's element count"); return THCB200_ERR_SIZE; }
  if (vm.numel == 0 || vo.numel == 0) return THCB200_OK;
  THCB_CTX_LOCK(ctx);
  cudaStream_t st = (cudaStream_t)stream;
  MaskPrep mp;
  rc = prepare_mask(ctx, vm, (flags & THCB200_FLAG_MASK_COUNTED) != 0, st, &mp);
  if (rc) return rc;
  Collapsed co;
  if (!mp.cm.unit || !collapse_view(vo, &co) || !co.unit) { set_error("mask_coords: the mask and the output must be dense"); return THCB200_ERR_ARG; }
  // with the count already on the host (the caller counted this mask and said so) a short output is refused
  if (mp.hit && counted_on_host(ctx, &rc, vo.numel, (int64_t)nd, "mask_coords")) return rc;
  const bool mvec = aligned16(vm.data);
  set_plan_name(mvec ? "mask_coords" : "mask_coords_bytes");
  launch_pdl(mask_coords_kernel, (unsigned)mp.ntiles, kThreads, 0, st, reinterpret_cast<const uint8_t *>(vm.data), (uint64_t)vm.numel, mvec, mp.offsets,
                                                              shape, reinterpret_cast<int64_t *>(vo.data));
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return THCB200_OK;
}

int thcb200_masked_copy(thcb200_ctx *ctx, const thcb200_tensor *t, const thcb200_tensor *mask_u8,
                        const thcb200_tensor *src, void *stream, int flags) {
  return masked_move(ctx, false, t, src, mask_u8, stream, flags, "masked_copy");
}

int thcb200_masked_select(thcb200_ctx *ctx, const thcb200_tensor *out, const thcb200_tensor *src,
                          const thcb200_tensor *mask_u8, void *stream, int flags) {
  return masked_move(ctx, true, src, out, mask_u8, stream, flags, "masked_select");
}

}  // extern "C"
