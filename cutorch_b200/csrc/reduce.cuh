// Reduction kernels for sm_100a: full reduction (one launch, fixed order, last-block
// finalize) and dimension reductions over inner-contiguous rows, outer-strided columns and
// arbitrary layouts, each with a plain-value and a (value, first position) form.
//
// Replaces kernelReduceAll/Pass1/Pass2 (lib/THC/THCReduceAll.cuh:21-123),
// kernelReduceContigDim / kernelReduceNoncontigDim(_shared) (lib/THC/THCReduce.cuh:25-214) and
// kernelTransformReduceInnermostDimIndex / OuterDimIndex
// (lib/THC/THCTensorMathReduce.cuh:453-585).
#pragma once

#include <math.h>

#include <type_traits>

#include "core.cuh"
#include "ops.cuh"

namespace thcb {

// Fold modes: the (reduce op, pre-transform) pairs that exist in the C API.
enum ReduceMode {
  kSum = 0, kSumAbs, kSumSquare, kSumPowAbs, kSumNonZero, kSumSqDev,
  kProd, kMin, kMax, kAll, kAny, kSumMoments, kNumReduceModes
};

inline int reduce_mode(int rop, int pre) {
  if (rop == THCB200_RED_SUM) {
    switch (pre) {
      case THCB200_PRE_IDENTITY: return kSum;
      case THCB200_PRE_ABS: return kSumAbs;
      case THCB200_PRE_SQUARE: return kSumSquare;
      case THCB200_PRE_POWABS: return kSumPowAbs;
      case THCB200_PRE_NONZERO: return kSumNonZero;
      case THCB200_PRE_SQDEV: return kSumSqDev;
      case THCB200_PRE_MOMENTS: return kSumMoments;
    }
    return -1;
  }
  if (pre != THCB200_PRE_IDENTITY) return -1;
  switch (rop) {
    case THCB200_RED_PROD: return kProd;
    case THCB200_RED_MIN: return kMin;
    case THCB200_RED_MAX: return kMax;
    case THCB200_RED_ALL: return kAll;
    case THCB200_RED_ANY: return kAny;
  }
  return -1;
}

template <typename M> __device__ __forceinline__ bool is_nan(M v) { return v != v; }

// ---------------------------------------------------------------------------------
// Folder<T, MODE>: accumulator type, element transform and combine of one fold mode.
//   Sum-like modes accumulate in TypeTraits<T>::Acc (double for float/double, float for
//   half, int64 for integers) -- the accumulate types of TH's CPU reductions, with the
//   transform applied in that type as TH does.
//   Min/Max compare in the element's math type; a NaN wins, as in TH's scans.
// ---------------------------------------------------------------------------------
// running sums of x and x*x (var / std along a dim)
template <typename A> struct Moments { A s, s2; };

template <typename T, int MODE>
struct Folder {
  static constexpr bool kMinMax = (MODE == kMin || MODE == kMax);
  static constexpr bool kLogical = (MODE == kAll || MODE == kAny);
  static constexpr bool kMoments = (MODE == kSumMoments);
  using SumAcc = typename TypeTraits<T>::Acc;
  using M = typename TypeTraits<T>::Math;
  using Scalar = typename std::conditional<kMinMax, M, typename std::conditional<kLogical, int, SumAcc>::type>::type;
  using Acc = typename std::conditional<kMoments, Moments<SumAcc>, Scalar>::type;
  struct Params { Scalar s; };

  __host__ __device__ static Acc init() {
    if constexpr (kMoments) { Acc a; a.s = 0; a.s2 = 0; return a; }
    else if constexpr (MODE == kProd) return (Acc)1;
    else if constexpr (MODE == kAll) return 1;
    else if constexpr (kMinMax) return Acc();  // unused: min/max folds start from an element
    else return (Acc)0;
  }
  __device__ __forceinline__ static Acc pre(T x, const Params &p) {
    if constexpr (kMinMax) return to_math<T>(x);
    else if constexpr (kLogical) return to_math<T>(x) != (M)0 ? 1 : 0;
    else if constexpr (kMoments) {
      const SumAcc v = (SumAcc)to_math<T>(x);
      Acc a; a.s = v; a.s2 = v * v;
      return a;
    } else {
      const Acc v = (Acc)to_math<T>(x);
      if constexpr (MODE == kSumAbs) return v < 0 ? -v : v;
      else if constexpr (MODE == kSumSquare) return v * v;
      else if constexpr (MODE == kSumPowAbs) {
        if constexpr (std::is_same<Acc, float>::value) return powf(fabsf(v), p.s);
        else return (Acc)pow(fabs((double)v), (double)p.s);
      }
      else if constexpr (MODE == kSumNonZero) return v != 0 ? (Acc)1 : (Acc)0;
      else if constexpr (MODE == kSumSqDev) return (v - p.s) * (v - p.s);
      else return v;
    }
  }
  __device__ __forceinline__ static Acc combine(Acc a, Acc b) {
    if constexpr (kMoments) { Acc r; r.s = a.s + b.s; r.s2 = a.s2 + b.s2; return r; }
    else if constexpr (MODE == kProd) {
      if constexpr (TypeTraits<T>::is_fp) return a * b;
      else return (Acc)((uint64_t)a * (uint64_t)b);
    }
    else if constexpr (MODE == kAll) return a && b;
    else if constexpr (MODE == kAny) return a || b;
    else if constexpr (MODE == kMax) {
      if constexpr (TypeTraits<T>::is_fp) { if (is_nan(a)) return a; if (is_nan(b)) return b; }
      return a > b ? a : b;
    }
    else if constexpr (MODE == kMin) {
      if constexpr (TypeTraits<T>::is_fp) { if (is_nan(a)) return a; if (is_nan(b)) return b; }
      return a < b ? a : b;
    }
    else {
      if constexpr (TypeTraits<T>::is_fp) return a + b;
      else return (Acc)((uint64_t)a + (uint64_t)b);
    }
  }
};

// (value, position) accumulator of max/min along a dim.  `better(a, b)`: a is kept over b.
// Total order: NaN beats numbers, then the larger (smaller) value, then the lower position,
// which makes the combine associative and commutative: any tree gives the first occurrence.
template <typename M>
struct ValIdx {
  M v;
  int64_t i;  // 0-based position along the reduced dim; -1 = empty
};

template <typename T, bool IS_MAX>
struct IndexFolder {
  using M = typename TypeTraits<T>::Math;
  using Acc = ValIdx<M>;
  __device__ __forceinline__ static Acc empty() { Acc a; a.v = M(); a.i = -1; return a; }
  __device__ __forceinline__ static bool better(const Acc &a, const Acc &b) {
    if (b.i < 0) return true;
    if (a.i < 0) return false;
    if constexpr (TypeTraits<T>::is_fp) {
      const bool an = is_nan(a.v), bn = is_nan(b.v);
      if (an || bn) return an && (!bn || a.i < b.i);
    }
    if (a.v == b.v) return a.i < b.i;
    return IS_MAX ? (a.v > b.v) : (a.v < b.v);
  }
  __device__ __forceinline__ static Acc combine(const Acc &a, const Acc &b) { return better(a, b) ? a : b; }
  __device__ __forceinline__ static void feed(Acc &acc, T x, int64_t pos) {
    Acc e; e.v = to_math<T>(x); e.i = pos;
    if (!better(acc, e)) acc = e;
  }
};

// Per-thread running extreme for the value+position reductions.  A thread meets its elements
// in increasing position, so a strict comparison keeps the first occurrence and the only
// other rule needed is "the first NaN wins and ends the contest".  It starts from a sentinel
// (lowest / highest value) instead of a validity flag: a thread that only ever saw the
// sentinel reports "empty", which the final write resolves to (sentinel, first position) --
// correct, because in that case every element of the slice equals the sentinel.
// Positions are 32-bit offsets from `origin` (a unit never spans more than 2^32 - 2 elements).
template <typename M, bool FP> struct Sentinel;
template <typename M> struct Sentinel<M, true> {
  __device__ __forceinline__ static M lowest() { return (M)-INFINITY; }
  __device__ __forceinline__ static M highest() { return (M)INFINITY; }
};
template <typename M> struct Sentinel<M, false> {
  __device__ __forceinline__ static M lowest() { return ((M)-1 > (M)0) ? (M)0 : (M)((uint64_t)1 << (sizeof(M) * 8 - 1)); }
  __device__ __forceinline__ static M highest() { return (M)~lowest(); }
};

template <typename T, bool IS_MAX>
struct FastIdx {
  using M = typename TypeTraits<T>::Math;
  static constexpr bool FP = TypeTraits<T>::is_fp;
  static constexpr uint32_t kEmpty = 0xFFFFFFFFu;
  M bv;
  uint32_t bi;
  bool bnan;
  __device__ __forceinline__ static M sentinel() { return IS_MAX ? Sentinel<M, FP>::lowest() : Sentinel<M, FP>::highest(); }
  __device__ __forceinline__ void reset() { bv = sentinel(); bi = kEmpty; bnan = false; }
  __device__ __forceinline__ void feed(T xe, uint32_t rel) {
    const M x = to_math<T>(xe);
    bool take = IS_MAX ? (x > bv) : (x < bv);
    if constexpr (FP) {
      const bool xn = (x != x);
      take = take || (xn && !bnan);
      bnan = bnan || xn;
    }
    if (take) { bv = x; bi = rel; }
  }
  __device__ __forceinline__ ValIdx<M> result(uint64_t origin) const {
    ValIdx<M> r;
    r.v = bv;
    r.i = (bi == kEmpty) ? (int64_t)-1 : (int64_t)(origin + bi);
    return r;
  }
  // final value of an output whose merged result is still "empty": all elements equal the sentinel
  __device__ __forceinline__ static ValIdx<M> resolve(ValIdx<M> r) {
    if (r.i < 0) { r.v = sentinel(); r.i = 0; }
    return r;
  }
};

// ---- warp / block combine in a fixed order -------------------------------------------
template <typename A> __device__ __forceinline__ A shfl_xor(A v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
template <> __device__ __forceinline__ int64_t shfl_xor<int64_t>(int64_t v, int m) { return (int64_t)__shfl_xor_sync(0xffffffffu, (long long)v, m); }
template <> __device__ __forceinline__ int16_t shfl_xor<int16_t>(int16_t v, int m) { return (int16_t)__shfl_xor_sync(0xffffffffu, (int)v, m); }
template <> __device__ __forceinline__ int8_t shfl_xor<int8_t>(int8_t v, int m) { return (int8_t)__shfl_xor_sync(0xffffffffu, (int)v, m); }
template <> __device__ __forceinline__ uint8_t shfl_xor<uint8_t>(uint8_t v, int m) { return (uint8_t)__shfl_xor_sync(0xffffffffu, (int)v, m); }
template <> __device__ __forceinline__ Moments<double> shfl_xor<Moments<double>>(Moments<double> v, int m) {
  Moments<double> r;
  r.s = __shfl_xor_sync(0xffffffffu, v.s, m);
  r.s2 = __shfl_xor_sync(0xffffffffu, v.s2, m);
  return r;
}
template <> __device__ __forceinline__ Moments<float> shfl_xor<Moments<float>>(Moments<float> v, int m) {
  Moments<float> r;
  r.s = __shfl_xor_sync(0xffffffffu, v.s, m);
  r.s2 = __shfl_xor_sync(0xffffffffu, v.s2, m);
  return r;
}
template <typename M> __device__ __forceinline__ ValIdx<M> shfl_xor_vi(ValIdx<M> a, int m) {
  ValIdx<M> r;
  r.v = shfl_xor<M>(a.v, m);
  r.i = shfl_xor<int64_t>(a.i, m);
  return r;
}

// Butterfly over the 32 lanes; every lane ends with the same value.  For the min/max value
// folds an "empty" flag travels with the value (lanes that saw no element).
template <typename F> __device__ __forceinline__ typename F::Acc warp_fold(typename F::Acc v) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) v = F::combine(v, shfl_xor<typename F::Acc>(v, m));
  return v;
}
template <typename F> __device__ __forceinline__ typename F::Acc warp_fold_vi(typename F::Acc v) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) v = F::combine(v, shfl_xor_vi(v, m));
  return v;
}

// Value accumulator with validity, so that min/max need no sentinel start value.
template <typename F>
struct Opt {
  typename F::Acc v;
  int has;
  __device__ __forceinline__ void feed(typename F::Acc x) {
    if constexpr (F::kMinMax) { v = has ? F::combine(v, x) : x; has = 1; }
    else v = F::combine(v, x);
  }
  __device__ __forceinline__ void merge(const Opt &o) {
    if constexpr (F::kMinMax) { if (o.has) { v = has ? F::combine(v, o.v) : o.v; has = 1; } }
    else v = F::combine(v, o.v);
  }
  __device__ __forceinline__ static Opt start() { Opt o; o.v = F::init(); o.has = 0; return o; }
};
template <typename F> __device__ __forceinline__ Opt<F> warp_fold_opt(Opt<F> a) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) {
    Opt<F> o;
    o.v = shfl_xor<typename F::Acc>(a.v, m);
    o.has = __shfl_xor_sync(0xffffffffu, a.has, m);
    // keep the operand order independent of the lane so both partners compute the same
    const bool low = (threadIdx.x & m) == 0;
    Opt<F> x = low ? a : o, y = low ? o : a;
    x.merge(y);
    a = x;
  }
  return a;
}

// One step of a mixed-radix decode: lin = q * size + r.  The outermost dim needs no division, and
// operands below 2^32 take the 32-bit divide: a 64-bit division is over a hundred instructions,
// which a warp reducing a row of a thousand elements notices (two of them per row were 40 % of
// the instructions of `sum` over the last dim of a 3-D window).
__device__ __forceinline__ void radix_step(uint64_t lin, uint64_t size, bool outermost, uint64_t &q, uint64_t &r) {
  if (outermost) { q = 0; r = lin; }
  else if (((lin | size) >> 32) == 0) {
    const uint32_t l = (uint32_t)lin, s = (uint32_t)size, qq = l / s;
    q = qq;
    r = l - qq * s;
  } else {
    q = lin / size;
    r = lin - q * size;
  }
}

// Decodes a slice number into element offsets of the input and output(s); the dims are the
// non-reduced ones.  Evaluated once per slice.
struct SliceMap {
  int n;
  uint64_t size[kMaxDims];
  int64_t in_stride[kMaxDims];
  int64_t out_stride[kMaxDims];
  int64_t idx_stride[kMaxDims];
  __device__ __forceinline__ void decode(uint64_t lin, int64_t &in_off, int64_t &out_off, int64_t &idx_off) const {
    in_off = 0; out_off = 0; idx_off = 0;
    for (int d = n - 1; d >= 0; --d) {
      uint64_t q, r;
      radix_step(lin, size[d], d == 0, q, r);
      in_off += (int64_t)r * in_stride[d];
      out_off += (int64_t)r * out_stride[d];
      idx_off += (int64_t)r * idx_stride[d];
      lin = q;
    }
  }
};

constexpr int kRedThreads = 256;
constexpr int kRedWarps = kRedThreads / 32;
constexpr int kRedUnroll = 4;

// Ticket draw that publishes this CTA's earlier stores and, in the CTA that draws the last ticket,
// makes the other CTAs' stores visible: one acquire-release atomic at GPU scope in place of a fence,
// an atomic and a second fence.  Call from one thread after a __syncthreads() that follows the
// CTA's stores; the stores of the CTA's other threads are covered through that barrier.
__device__ __forceinline__ unsigned int draw_ticket(unsigned int *ticket) {
  unsigned int old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(ticket) : "memory");
  return old;
}

// Loads a partial that another CTA stored, from the L2 (never from a line an earlier kernel may
// have left in this SM's L1).
template <typename P> __device__ __forceinline__ P load_partial(const P *p) {
  static_assert(sizeof(P) % 4 == 0, "partials are made of 32-bit words");
  P r;
  const unsigned int *src = reinterpret_cast<const unsigned int *>(p);
  unsigned int *dst = reinterpret_cast<unsigned int *>(&r);
#pragma unroll
  for (int i = 0; i < (int)(sizeof(P) / 4); ++i) dst[i] = __ldcg(src + i);
  return r;
}

// ====================================================================================
// Cross-GPU part of a full reduction (see ExchangeBlock in core.cuh).  Called by the 32 lanes of
// warp 0 of the finishing CTA with the rank's accumulator bits; lane 0 stores the folded result.
// ====================================================================================
__device__ __forceinline__ unsigned long long slot_fold(int fold, int is_fp, unsigned long long a, unsigned long long b) {
  if (is_fp) {
    const double x = __longlong_as_double((long long)a), y = __longlong_as_double((long long)b);
    double r;
    switch (fold) {
      case THCB200_RED_PROD: r = x * y; break;
      case THCB200_RED_MIN: r = (x != x) ? x : (y != y) ? y : (x < y ? x : y); break;   // a NaN wins, the first one
      case THCB200_RED_MAX: r = (x != x) ? x : (y != y) ? y : (x > y ? x : y); break;
      default: r = x + y; break;
    }
    return (unsigned long long)__double_as_longlong(r);
  }
  const long long x = (long long)a, y = (long long)b;
  switch (fold) {
    case THCB200_RED_PROD: return a * b;
    case THCB200_RED_MIN: return (unsigned long long)(x < y ? x : y);
    case THCB200_RED_MAX: return (unsigned long long)(x > y ? x : y);
    default: return a + b;
  }
}

__device__ __forceinline__ void peer_exchange(const PeerExchange &px, unsigned long long mine, void *result) {
  const int lane = threadIdx.x & 31;
  const int par = (int)(px.epoch & 1u);
  if (lane < px.nranks) {
    // my accumulator, then the epoch, into my column of rank `lane`'s block
    ExchangeBlock *peer = px.block[lane];
    *reinterpret_cast<volatile unsigned long long *>(&peer->slot[par][px.rank]) = mine;
    __threadfence_system();
    *reinterpret_cast<volatile unsigned int *>(&peer->flag[par][px.rank]) = px.epoch;
  }
  // every rank's column of my own block must show this epoch; a bounded number of polls each
  ExchangeBlock *own = px.block[px.rank];
  bool arrived = true;
  if (lane < px.nranks) {
    const volatile unsigned int *f = &own->flag[par][lane];
    unsigned int polls = 0;
    while ((int)(*f - px.epoch) < 0) {
      if (++polls > px.max_polls) { arrived = false; break; }
      __nanosleep(200);
    }
  }
  arrived = __all_sync(0xffffffffu, arrived);
  __threadfence_system();
  if (lane == 0) {
    unsigned long long r = mine;
    if (arrived) {
      r = *reinterpret_cast<volatile unsigned long long *>(&own->slot[par][0]);
      for (int k = 1; k < px.nranks; ++k)
        r = slot_fold(px.fold, px.is_fp, r, *reinterpret_cast<volatile unsigned long long *>(&own->slot[par][k]));
    } else {
      *px.status = 1;   // the host reads this; the slot keeps this rank's own accumulator
    }
    *reinterpret_cast<unsigned long long *>(result) = r;
  }
}

// ====================================================================================
// Tail shared by the full-reduction kernels: fold the CTA's accumulators, store the CTA's
// partial, and let the CTA that draws the last ticket fold all partials in index order.
// ====================================================================================
template <typename T, int MODE>
__device__ __forceinline__ void reduce_all_finish(Opt<Folder<T, MODE>> acc, void *partials_raw, unsigned int *ticket, void *result,
                                                  const PeerExchange &px) {
  using F = Folder<T, MODE>;
  using Acc = typename F::Acc;
  struct Partial { Acc v; int has; };
  Partial *partials = reinterpret_cast<Partial *>(partials_raw);
  __shared__ Partial sm[kRedWarps];
  __shared__ bool is_last;
  acc = warp_fold_opt<F>(acc);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sm[warp].v = acc.v; sm[warp].has = acc.has; }
  __syncthreads();
  if (warp == 0) {
    // the 8 warp results fold as a butterfly over the first lanes (fixed order)
    Opt<F> b = Opt<F>::start();
    if (lane < kRedWarps) { b.v = sm[lane].v; b.has = sm[lane].has; }
    b = warp_fold_opt<F>(b);
    if (lane == 0) {
      partials[blockIdx.x].v = b.v;
      partials[blockIdx.x].has = b.has;
      is_last = (draw_ticket(ticket) == gridDim.x - 1);
    }
  }
  __syncthreads();
  if (!is_last) return;
  Opt<F> f = Opt<F>::start();
  for (unsigned int i = threadIdx.x; i < gridDim.x; i += kRedThreads) {
    const Partial p = load_partial(partials + i);
    Opt<F> o;
    o.v = p.v; o.has = p.has;
    f.merge(o);
  }
  f = warp_fold_opt<F>(f);
  if (lane == 0) { sm[warp].v = f.v; sm[warp].has = f.has; }
  __syncthreads();
  if (warp == 0) {
    Opt<F> b = Opt<F>::start();
    if (lane < kRedWarps) { b.v = sm[lane].v; b.has = sm[lane].has; }
    b = warp_fold_opt<F>(b);
    if (lane == 0) *ticket = 0;  // ready for the next launch on this stream
    // result slot: double for floating element types, int64 for integer ones
    if (px.nranks > 1) {
      // the other GPUs' accumulators are folded in here, by this warp, before the kernel ends
      unsigned long long bits;
      if constexpr (TypeTraits<T>::is_fp) bits = (unsigned long long)__double_as_longlong((double)b.v);
      else bits = (unsigned long long)(int64_t)b.v;
      peer_exchange(px, bits, result);
    } else if (lane == 0) {
      if constexpr (TypeTraits<T>::is_fp) *reinterpret_cast<double *>(result) = (double)b.v;
      else *reinterpret_cast<int64_t *>(result) = (int64_t)b.v;
    }
  }
}

// ====================================================================================
// reduce_all over a view that is not one dense run but whose innermost dim (after sorting the
// dims by stride: a full reduction is order-free) has stride 1: padded rows, windows of larger
// tensors.  Tiles are [ty rows x (tx * kRedRowsSlots) vectors]; a row's offset is decoded from its
// number once per thread and tile.
// ====================================================================================
constexpr int kRedRowsOuterDims = 7;
struct RedRowsView {
  int nouter;
  FastDiv32 outer_size[kRedRowsOuterDims];
  int64_t outer_stride[kRedRowsOuterDims];
  uint32_t R, Cunits;       // rows; elements per row
  uint32_t tiles_c;
  FastDiv32 tiles_c_div;
  int log2_tx;
  __device__ __forceinline__ int64_t row_offset(uint32_t r) const {
    int64_t off = 0;
    uint32_t rem = r;
#pragma unroll 1
    for (int i = nouter - 1; i >= 1; --i) {
      uint32_t q, m;
      outer_size[i].divmod(rem, q, m);
      off += (int64_t)m * outer_stride[i];
      rem = q;
    }
    return off + (int64_t)rem * outer_stride[0];
  }
};

// Rows need not start on a 16-byte boundary: per row the elements before the first boundary and
// after the last whole vector (at most 2 * (V - 1) of them) are read one by one by the first
// threads of the row's first column tile; everything between moves as 16-byte vectors.  A thread
// takes kRedRowsSlots vectors of one row per tile, tx apart, so the row's offset and alignment are
// worked out once per kRedRowsSlots loads (with one vector per decode the kernel was bound by
// instruction issue: 104 M warp instructions for 134 M floats).
constexpr int kRedRowsSlots = 8;
template <typename T, int MODE>
__global__ void __launch_bounds__(kRedThreads)
reduce_all_rows_kernel(const T *in, RedRowsView rv, uint32_t ntiles, typename Folder<T, MODE>::Params prm,
                       void *partials_raw, unsigned int *ticket, void *result, PeerExchange px) {
  pdl_prologue();
  using F = Folder<T, MODE>;
  constexpr int V = 16 / (int)sizeof(T);
  constexpr int W = kRedRowsSlots;
  const unsigned tx = 1u << rv.log2_tx, ty = kRedThreads >> rv.log2_tx;
  const unsigned x = threadIdx.x & (tx - 1), y = threadIdx.x >> rv.log2_tx;
  const uint32_t C = rv.Cunits;   // elements per row
  Opt<F> acc = Opt<F>::start();
  for (uint32_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    uint32_t rtile, ctile;
    rv.tiles_c_div.divmod(t, rtile, ctile);
    const uint32_t r = rtile * ty + y;
    if (r >= rv.R) continue;
    const T *row = in + rv.row_offset(r);
    const uint32_t mis = (uint32_t)((reinterpret_cast<uintptr_t>(row) / sizeof(T)) % V);
    uint32_t head = mis ? V - mis : 0;
    if (head > C) head = C;
    const uint32_t nvec = (C - head) / V;
    const uint32_t tail0 = head + nvec * V;          // first element after the vectors
    const T *vrow = row + head;
    const uint32_t cu0 = ctile * (tx * W) + x;        // this thread's first vector of the row's aligned part
    Bytes16 v[W];
#pragma unroll
    for (int w = 0; w < W; ++w)
      if (cu0 + (uint32_t)w * tx < nvec) v[w] = ld16_stream(vrow + (uint64_t)(cu0 + (uint32_t)w * tx) * V);
    // edge elements: x < head takes row[x], head <= x < head + (C - tail0) takes the tail
    T edge = T();
    const bool eok = ctile == 0 && x < head + (C - tail0);
    if (eok) edge = row[x < head ? x : tail0 + (x - head)];
#pragma unroll
    for (int w = 0; w < W; ++w) {
      if (cu0 + (uint32_t)w * tx < nvec) {
        const T *e = reinterpret_cast<const T *>(&v[w]);
#pragma unroll
        for (int j = 0; j < V; ++j) acc.feed(F::pre(e[j], prm));
      }
    }
    if (eok) acc.feed(F::pre(edge, prm));
  }
  reduce_all_finish<T, MODE>(acc, partials_raw, ticket, result, px);
}

// ====================================================================================
// reduce_all: persistent CTAs walk 16 KiB tiles block-cyclically; partial per CTA; the CTA
// that draws the last ticket folds the partials in index order and writes the result.
// ====================================================================================
template <typename T, int MODE, int VB /* vector bytes: 32, 16, or 0 = strided walk */>
__global__ void __launch_bounds__(kRedThreads)
reduce_all_kernel(const T *in, StridedView<uint64_t> view, uint64_t n, typename Folder<T, MODE>::Params prm,
                  void *partials_raw, unsigned int *ticket, void *result, const T *edge, uint32_t nedge, PeerExchange px) {
  pdl_prologue();
  using F = Folder<T, MODE>;
  constexpr bool VEC = VB != 0;
  constexpr int V = VEC ? VB / (int)sizeof(T) : 1;
  constexpr uint64_t kTile = (uint64_t)kRedThreads * kRedUnroll * V;
  Opt<F> acc = Opt<F>::start();
  // elements in front of the first vector boundary of a dense run (fewer than one vector)
  if (blockIdx.x == 0 && threadIdx.x < nedge) acc.feed(F::pre(edge[threadIdx.x], prm));
  const uint64_t ntiles = (n + kTile - 1) / kTile;
  for (uint64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t base = t * kTile;
    if constexpr (VEC) {
      if (base + kTile <= n) {
        typename VecBytes<VEC ? VB : 16>::type v[kRedUnroll];
#pragma unroll
        for (int u = 0; u < kRedUnroll; ++u) v[u] = ldv_stream<VEC ? VB : 16>(in + base + ((uint64_t)u * kRedThreads + threadIdx.x) * V);
#pragma unroll
        for (int u = 0; u < kRedUnroll; ++u) {
          const T *e = reinterpret_cast<const T *>(&v[u]);
#pragma unroll
          for (int k = 0; k < V; ++k) acc.feed(F::pre(e[k], prm));
        }
      } else {
        for (uint64_t i = base + threadIdx.x; i < n; i += kRedThreads) acc.feed(F::pre(in[i], prm));
      }
    } else {
      T x[kRedUnroll];
      bool ok[kRedUnroll];
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * kRedThreads + threadIdx.x;
        ok[u] = i < n;
        if (ok[u]) x[u] = in[view.offset(i)];
      }
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u) if (ok[u]) acc.feed(F::pre(x[u], prm));
    }
  }
  reduce_all_finish<T, MODE>(acc, partials_raw, ticket, result, px);
}

// ====================================================================================
// Output conversion of the dimension reductions: accumulator -> element type.
// ====================================================================================
template <typename T, typename Acc> __device__ __forceinline__ T acc_to_elem(Acc a) {
  if constexpr (std::is_same<T, __half>::value) return __float2half_rn((float)a);
  else return (T)a;
}

// Optional step applied to each output after the fold, for the entry points cutorch composes
// from two calls: mean = sum then div by the length (lib/THC/generic/THCTensorMathReduce.cu:37-43),
// norm = fold then pow (:160-187).  The fold result is first rounded to the element type, then
// the step runs in the element's math type and rounds again -- the values of the two-call form.
enum PostKind { kPostNone = 0, kPostDiv = 1, kPostPow = 2, kPostVarBiased = 3, kPostVarUnbiased = 4, kPostStdBiased = 5, kPostStdUnbiased = 6 };
struct PostOp {
  int kind;
  double f;     // operand for floating element types
  int64_t i;    // operand for integer element types
};

// var / std from the running sums, in the accumulate type (TH: sum and sum of squares over the
// slice, E[x^2] - E[x]^2 with the n/(n-1) correction when unbiased, clamped at zero); post.f = n.
template <typename T, typename A> __device__ __forceinline__ T finalize_moments(Moments<A> a, const PostOp &post) {
  const A n = (A)post.f;
  const A mean = a.s / n;
  const bool unbiased = (post.kind == kPostVarUnbiased || post.kind == kPostStdUnbiased);
  A v = unbiased ? a.s2 / (n - (A)1) - (n / (n - (A)1)) * mean * mean : a.s2 / n - mean * mean;
  v = v < (A)0 ? (A)0 : v;
  if (post.kind == kPostStdBiased || post.kind == kPostStdUnbiased) v = (A)sqrt((double)v);
  return acc_to_elem<T, A>(v);
}

template <typename A> struct IsMoments : std::false_type {};
template <typename A> struct IsMoments<Moments<A>> : std::true_type {};

template <typename T, typename Acc> __device__ __forceinline__ T finalize_out(Acc a, const PostOp &post) {
  if constexpr (IsMoments<Acc>::value) {
    return finalize_moments<T>(a, post);
  } else {
    T r = acc_to_elem<T, Acc>(a);
    if (post.kind == kPostNone) return r;
    using M = typename TypeTraits<T>::Math;
    if constexpr (TypeTraits<T>::is_fp) {
      const M x = to_math<T>(r);
      if (post.kind == kPostDiv) return from_math<T>(x / (M)post.f);
      return from_math<T>(fp_apply<THCB200_OP_POW, M>((M)post.f, (M)0, x, (M)0, (M)0));
    } else {
      using P = typename Promoted<T>::type;
      if (post.kind == kPostDiv) return (T)((P)r / (P)post.i);
      return r;
    }
  }
}

// Partial accumulators of split reductions, kept in the workspace between the two stages.
template <typename Acc> struct PartialVal { Acc v; int has; };

constexpr int kFinishBatch = 16;

// Folds the nsplit partials of output `o` in split order and writes the result: the second
// stage of a split reduction, run either by reduce_finish_kernel or by the last CTA of a tile.
template <typename T, int MODE, bool INDEX, bool IS_MAX>
__device__ __forceinline__ void finish_output(T *out_elem, int64_t *idx_elem, uint64_t o, uint32_t nsplit,
                                              const void *partials_raw, const PostOp &post) {
  using F = Folder<T, MODE>;
  using IF = IndexFolder<T, IS_MAX>;
  if constexpr (INDEX) {
    // the partials are loaded kFinishBatch at a time (independent loads in flight) and folded in split order
    const typename IF::Acc *pp = reinterpret_cast<const typename IF::Acc *>(partials_raw) + o * nsplit;
    typename IF::Acc r = IF::empty();
    for (uint32_t s0 = 0; s0 < nsplit; s0 += kFinishBatch) {
      typename IF::Acc b[kFinishBatch];
#pragma unroll
      for (int u = 0; u < kFinishBatch; ++u) if (s0 + u < nsplit) b[u] = load_partial(pp + s0 + u);
#pragma unroll
      for (int u = 0; u < kFinishBatch; ++u) if (s0 + u < nsplit) r = IF::combine(r, b[u]);
    }
    r = FastIdx<T, IS_MAX>::resolve(r);
    *out_elem = from_math<T>(r.v);
    *idx_elem = r.i + 1;  // TH_INDEX_BASE
  } else {
    const PartialVal<typename F::Acc> *pp = reinterpret_cast<const PartialVal<typename F::Acc> *>(partials_raw) + o * nsplit;
    Opt<F> r = Opt<F>::start();
    for (uint32_t s0 = 0; s0 < nsplit; s0 += kFinishBatch) {
      PartialVal<typename F::Acc> b[kFinishBatch];
#pragma unroll
      for (int u = 0; u < kFinishBatch; ++u) if (s0 + u < nsplit) b[u] = load_partial(pp + s0 + u);
#pragma unroll
      for (int u = 0; u < kFinishBatch; ++u) if (s0 + u < nsplit) { Opt<F> x; x.v = b[u].v; x.has = b[u].has; r.merge(x); }
    }
    *out_elem = finalize_out<T, typename F::Acc>(r.v, post);
  }
}

// Draws a ticket for `tile`; true in the CTA that drew the last of `count` (all partials of
// the tile are then visible to it).  Call with every thread of the CTA, after the partial stores.
__device__ __forceinline__ bool last_cta_of_tile(unsigned int *tickets, uint64_t tile, uint32_t count) {
  __shared__ bool s_last;
  __syncthreads();
  if (threadIdx.x == 0) s_last = (draw_ticket(&tickets[tile]) == count - 1);
  __syncthreads();
  return s_last;
}

// ====================================================================================
// ROW: the reduced dim has stride 1.  A unit of work is (slice, split); WARP_PER_UNIT picks
// one warp per unit (8 units per CTA) or the whole CTA per unit.  With nsplit > 1 the unit's
// partial goes to the workspace [slice][split] and finish_kernel completes the fold.
// ====================================================================================
template <typename T, int MODE, bool INDEX, bool IS_MAX, bool VEC, bool WARP_PER_UNIT>
__global__ void __launch_bounds__(kRedThreads, 4)
reduce_row_kernel(const T *in, T *out, int64_t *idx_out, SliceMap map, uint64_t nslices, uint64_t K,
                  uint32_t nsplit, uint64_t split_len, typename Folder<T, MODE>::Params prm, void *partials_raw,
                  unsigned int *tickets, PostOp post) {
  pdl_prologue();
  using F = Folder<T, MODE>;
  using IF = IndexFolder<T, IS_MAX>;
  constexpr int V = 16 / sizeof(T);
  constexpr int GROUP = WARP_PER_UNIT ? 32 : kRedThreads;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gt = WARP_PER_UNIT ? lane : threadIdx.x;  // thread index inside the group
  const uint64_t unit = WARP_PER_UNIT ? (uint64_t)blockIdx.x * kRedWarps + warp : blockIdx.x;
  const uint64_t nunits = nslices * nsplit;
  const bool active = unit < nunits;
  const uint64_t slice = active ? div_by_u32(unit, nsplit) : 0;
  const uint32_t split = active ? (uint32_t)(unit - slice * nsplit) : 0;
  int64_t in_off = 0, out_off = 0, idx_off = 0;
  if (active) map.decode(slice, in_off, out_off, idx_off);
  const T *row = in + in_off;
  const uint64_t k0 = (uint64_t)split * split_len;
  const uint64_t k1 = active ? (k0 + split_len < K ? k0 + split_len : K) : k0;

  Opt<F> acc = Opt<F>::start();
  FastIdx<T, IS_MAX> fast;
  fast.reset();
  uint64_t k = k0;
  if constexpr (VEC) {
    // A unit need not start on a 16-byte boundary (odd row lengths, windows): the up to V - 1
    // elements before the first boundary and after the last whole vector go one to a lane.  They
    // are loaded first and fed in position order (head, vectors, tail: the position scans keep the
    // first occurrence by replacing on strictly better values only), the head after the first
    // batch of vector loads is under way, so a short row costs one memory latency, not three.
    const uint64_t mis = (reinterpret_cast<uintptr_t>(row + k0) / sizeof(T)) % V;
    uint64_t head = mis ? V - mis : 0;
    if (head > k1 - k0) head = k1 - k0;
    const uint64_t tail0 = k0 + head + (k1 - k0 - head) / V * V;   // first element after the whole vectors
    const bool has_head = (uint64_t)gt < head, has_tail = (uint64_t)gt < k1 - tail0;
    T eh = T(), et = T();
    if (has_head) eh = row[k0 + gt];
    if (has_tail) et = row[tail0 + gt];
    bool head_fed = false;
    // whole 16-byte vectors, kRedUnroll of them in flight per thread
    constexpr uint64_t kStep = (uint64_t)GROUP * V * kRedUnroll;
    for (k = k0 + head; k < tail0; k += kStep) {
      const uint64_t nrem = (tail0 - k) / V;
      Bytes16 v[kRedUnroll];
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u)
        if ((uint64_t)u * GROUP + gt < nrem) v[u] = ld16_stream(row + k + ((uint64_t)u * GROUP + gt) * V);
      if (!head_fed) {
        head_fed = true;
        if (has_head) {
          if constexpr (INDEX) fast.feed(eh, (uint32_t)gt);
          else acc.feed(F::pre(eh, prm));
        }
      }
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u) {
        if ((uint64_t)u * GROUP + gt < nrem) {
          const T *e = reinterpret_cast<const T *>(&v[u]);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            if constexpr (INDEX) fast.feed(e[j], (uint32_t)(k - k0) + (uint32_t)((u * GROUP + gt) * V + j));
            else acc.feed(F::pre(e[j], prm));
          }
        }
      }
    }
    if (!head_fed && has_head) {
      if constexpr (INDEX) fast.feed(eh, (uint32_t)gt);
      else acc.feed(F::pre(eh, prm));
    }
    if (has_tail) {
      if constexpr (INDEX) fast.feed(et, (uint32_t)(tail0 - k0) + (uint32_t)gt);
      else acc.feed(F::pre(et, prm));
    }
    k = k1;
  }
  for (uint64_t i = k + gt; i < k1; i += GROUP) {
    if constexpr (INDEX) fast.feed(row[i], (uint32_t)(i - k0));
    else acc.feed(F::pre(row[i], prm));
  }

  // fold inside the group
  typename IF::Acc best = fast.result(k0);
  if constexpr (INDEX) best = warp_fold_vi<IF>(best);
  else acc = warp_fold_opt<F>(acc);
  if constexpr (!WARP_PER_UNIT) {
    __shared__ PartialVal<typename F::Acc> smv[kRedWarps];
    __shared__ typename IF::Acc smi[kRedWarps];
    if (lane == 0) {
      if constexpr (INDEX) smi[warp] = best;
      else { smv[warp].v = acc.v; smv[warp].has = acc.has; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if constexpr (INDEX) {
        best = smi[0];
        for (int w = 1; w < kRedWarps; ++w) best = IF::combine(best, smi[w]);
      } else {
        acc = Opt<F>::start();
        for (int w = 0; w < kRedWarps; ++w) { Opt<F> o; o.v = smv[w].v; o.has = smv[w].has; acc.merge(o); }
      }
    }
  }
  if (nsplit > 1) {
    // only the CTA-per-unit form splits
    if (active && gt == 0) {
      if constexpr (INDEX) reinterpret_cast<typename IF::Acc *>(partials_raw)[unit] = best;
      else {
        PartialVal<typename F::Acc> *pp = reinterpret_cast<PartialVal<typename F::Acc> *>(partials_raw);
        pp[unit].v = acc.v; pp[unit].has = acc.has;
      }
    }
    if constexpr (!WARP_PER_UNIT) {
      if (tickets && last_cta_of_tile(tickets, slice, nsplit)) {
        if (threadIdx.x == 0) {
          finish_output<T, MODE, INDEX, IS_MAX>(out + out_off, idx_out + idx_off, slice, nsplit, partials_raw, post);
          tickets[slice] = 0;
        }
      }
    }
    return;
  }
  if (!active || gt != 0) return;
  if constexpr (INDEX) {
    best = FastIdx<T, IS_MAX>::resolve(best);
    out[out_off] = from_math<T>(best.v);
    idx_out[idx_off] = best.i + 1;  // TH_INDEX_BASE
  } else {
    out[out_off] = finalize_out<T, typename F::Acc>(acc.v, post);
  }
}

// Column loads: 16-byte vectors where the layout allows, 4-byte words for the 1-byte types
// (their accumulators would not fit shared memory at 16 columns per lane), else one element.
template <int BYTES, typename T> struct ColVec {
  using type = T;
  __device__ __forceinline__ static T load(const T *p) { return *p; }
};
template <typename T> struct ColVec<16, T> {
  using type = Bytes16;
  __device__ __forceinline__ static Bytes16 load(const T *p) { return ld16_stream(p); }
};
template <> struct ColVec<4, uint8_t> {
  using type = uint32_t;
  __device__ __forceinline__ static uint32_t load(const uint8_t *p) { return *reinterpret_cast<const uint32_t *>(p); }
};
template <> struct ColVec<4, int8_t> {
  using type = uint32_t;
  __device__ __forceinline__ static uint32_t load(const int8_t *p) { return *reinterpret_cast<const uint32_t *>(p); }
};
// elements per lane of the vector form of reduce_col_kernel
template <typename T> constexpr int col_vec_elems() { return sizeof(T) == 1 ? 4 : 16 / (int)sizeof(T); }

// ====================================================================================
// COL: some non-reduced dim ("inner", size I) has stride 1 in the input and the reduced dim
// is strided.  A CTA owns 32 lanes x V adjacent inner positions and one K split; its 8 warps
// take the rows of the split round-robin, kRedUnroll row loads in flight per thread, and are
// merged through shared memory in warp order.
// ====================================================================================
template <typename T, int MODE, bool INDEX, bool IS_MAX, int V, int U /* row loads in flight per thread */>
__global__ void __launch_bounds__(kRedThreads, 4)
reduce_col_kernel(const T *in, T *out, int64_t *idx_out, SliceMap map /* dims other than K and inner */,
                  uint64_t nouter, uint64_t K, int64_t strideK, uint64_t I, int64_t out_inner_stride,
                  int64_t idx_inner_stride, uint32_t nsplit, uint64_t split_len, uint32_t tiles_i,
                  typename Folder<T, MODE>::Params prm, void *partials_raw, unsigned int *tickets, PostOp post) {
  pdl_prologue();
  using F = Folder<T, MODE>;
  using IF = IndexFolder<T, IS_MAX>;
  using VecT = typename ColVec<V * sizeof(T), T>::type;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // blockIdx.x -> (outer, split, inner tile)
  uint32_t b = blockIdx.x;
  const uint32_t ti = b % tiles_i; b /= tiles_i;
  const uint32_t split = b % nsplit; b /= nsplit;
  const uint64_t outer = b;
  int64_t in_off, out_off, idx_off;
  map.decode(outer, in_off, out_off, idx_off);
  const uint64_t i0 = ((uint64_t)ti * 32 + lane) * V;
  const bool col_ok = i0 < I;  // I is a multiple of V on the vector path
  const uint64_t k0 = (uint64_t)split * split_len;
  const uint64_t k1 = k0 + split_len < K ? k0 + split_len : K;
  const T *col = in + in_off + (int64_t)i0;

  Opt<F> acc[V];
  FastIdx<T, IS_MAX> fast[V];
#pragma unroll
  for (int j = 0; j < V; ++j) { acc[j] = Opt<F>::start(); fast[j].reset(); }
  if (col_ok) {
    uint64_t k = k0 + warp;
    for (; k + (uint64_t)(U - 1) * kRedWarps < k1; k += (uint64_t)U * kRedWarps) {
      VecT v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const T *p = col + (int64_t)(k + (uint64_t)u * kRedWarps) * strideK;
        v[u] = ColVec<V * sizeof(T), T>::load(p);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const T *e = reinterpret_cast<const T *>(&v[u]);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          if constexpr (INDEX) fast[j].feed(e[j], (uint32_t)(k - k0) + (uint32_t)(u * kRedWarps));
          else acc[j].feed(F::pre(e[j], prm));
        }
      }
    }
    // the last rows of the split: one more batch, each load guarded (a single round trip)
    if (k < k1) {
      VecT v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t kk = k + (uint64_t)u * kRedWarps;
        if (kk < k1) v[u] = ColVec<V * sizeof(T), T>::load(col + (int64_t)kk * strideK);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t kk = k + (uint64_t)u * kRedWarps;
        if (kk < k1) {
          const T *e = reinterpret_cast<const T *>(&v[u]);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            if constexpr (INDEX) fast[j].feed(e[j], (uint32_t)(kk - k0));
            else acc[j].feed(F::pre(e[j], prm));
          }
        }
      }
    }
  }
  // merge the 8 warps in warp order through shared memory
  __shared__ PartialVal<typename F::Acc> smv[INDEX ? 1 : kRedWarps][32 * V + 1];
  __shared__ typename IF::Acc smi[INDEX ? kRedWarps : 1][32 * V + 1];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    if constexpr (INDEX) smi[warp][lane * V + j] = fast[j].result(k0);
    else { smv[warp][lane * V + j].v = acc[j].v; smv[warp][lane * V + j].has = acc[j].has; }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 32 * V; c += kRedThreads) {
    const uint64_t i = (uint64_t)ti * 32 * V + c;
    if (i >= I) continue;
    const uint64_t slot = (outer * I + i) * nsplit + split;  // [outer][inner][split]
    if constexpr (INDEX) {
      typename IF::Acc r = smi[0][c];
      for (int w = 1; w < kRedWarps; ++w) r = IF::combine(r, smi[w][c]);
      if (nsplit > 1) reinterpret_cast<typename IF::Acc *>(partials_raw)[slot] = r;
      else {
        r = FastIdx<T, IS_MAX>::resolve(r);
        out[out_off + (int64_t)i * out_inner_stride] = from_math<T>(r.v);
        idx_out[idx_off + (int64_t)i * idx_inner_stride] = r.i + 1;
      }
    } else {
      Opt<F> r = Opt<F>::start();
      for (int w = 0; w < kRedWarps; ++w) { Opt<F> o; o.v = smv[w][c].v; o.has = smv[w][c].has; r.merge(o); }
      if (nsplit > 1) {
        PartialVal<typename F::Acc> *pp = reinterpret_cast<PartialVal<typename F::Acc> *>(partials_raw);
        pp[slot].v = r.v; pp[slot].has = r.has;
      } else {
        out[out_off + (int64_t)i * out_inner_stride] = finalize_out<T, typename F::Acc>(r.v, post);
      }
    }
  }
  // the CTA that completes a column tile folds its partials right away (no second launch)
  if (nsplit > 1 && tickets) {
    const uint64_t tile = outer * tiles_i + ti;
    if (last_cta_of_tile(tickets, tile, nsplit)) {
      for (int c = threadIdx.x; c < 32 * V; c += kRedThreads) {
        const uint64_t i = (uint64_t)ti * 32 * V + c;
        if (i >= I) continue;
        finish_output<T, MODE, INDEX, IS_MAX>(out + out_off + (int64_t)i * out_inner_stride,
                                              idx_out + idx_off + (int64_t)i * idx_inner_stride, outer * I + i, nsplit,
                                              partials_raw, post);
      }
      if (threadIdx.x == 0) tickets[tile] = 0;
    }
  }
}

// ====================================================================================
// finish: folds the nsplit partials of every output in split order (one thread per output).
// Output o = outer * I + inner for COL (I = 1 for ROW, where outer is the slice).
// ====================================================================================
template <typename T, int MODE, bool INDEX, bool IS_MAX>
__global__ void __launch_bounds__(kRedThreads)
reduce_finish_kernel(T *out, int64_t *idx_out, SliceMap map, uint64_t nouter, uint64_t I,
                     int64_t out_inner_stride, int64_t idx_inner_stride, uint32_t nsplit,
                     const void *partials_raw, PostOp post) {
  pdl_prologue();
  const uint64_t o = (uint64_t)blockIdx.x * kRedThreads + threadIdx.x;
  if (o >= nouter * I) return;
  const uint64_t outer = o / I, i = o - outer * I;
  int64_t in_off, out_off, idx_off;
  map.decode(outer, in_off, out_off, idx_off);
  finish_output<T, MODE, INDEX, IS_MAX>(out + out_off + (int64_t)i * out_inner_stride,
                                        idx_out + idx_off + (int64_t)i * idx_inner_stride, o, nsplit, partials_raw, post);
}

// ====================================================================================
// STRIDED (fallback): one thread per output slice walks the reduced dim with its stride.
// ====================================================================================
template <typename T, int MODE, bool INDEX, bool IS_MAX>
__global__ void __launch_bounds__(kRedThreads)
reduce_strided_kernel(const T *in, T *out, int64_t *idx_out, SliceMap map, uint64_t nslices, uint64_t K,
                      int64_t strideK, typename Folder<T, MODE>::Params prm, PostOp post) {
  pdl_prologue();
  using F = Folder<T, MODE>;
  using IF = IndexFolder<T, IS_MAX>;
  const uint64_t s = (uint64_t)blockIdx.x * kRedThreads + threadIdx.x;
  if (s >= nslices) return;
  int64_t in_off, out_off, idx_off;
  map.decode(s, in_off, out_off, idx_off);
  const T *p = in + in_off;
  Opt<F> acc = Opt<F>::start();
  typename IF::Acc best = IF::empty();
  uint64_t k = 0;
  for (; k + kRedUnroll <= K; k += kRedUnroll) {
    T x[kRedUnroll];
#pragma unroll
    for (int u = 0; u < kRedUnroll; ++u) x[u] = p[(int64_t)(k + u) * strideK];
#pragma unroll
    for (int u = 0; u < kRedUnroll; ++u) {
      if constexpr (INDEX) IF::feed(best, x[u], (int64_t)(k + u));
      else acc.feed(F::pre(x[u], prm));
    }
  }
  for (; k < K; ++k) {
    if constexpr (INDEX) IF::feed(best, p[(int64_t)k * strideK], (int64_t)k);
    else acc.feed(F::pre(p[(int64_t)k * strideK], prm));
  }
  if constexpr (INDEX) {
    out[out_off] = from_math<T>(best.v);
    idx_out[idx_off] = best.i + 1;
  } else {
    out[out_off] = finalize_out<T, typename F::Acc>(acc.v, post);
  }
}

}  // namespace thcb
