// Inclusive scans along one dim (cumsum / cumprod): lib/THC/THCTensorMathScan.cu:24-129 and
// generic/THCTensorMathScan.cu:5-118 in cutorch, which copies both tensors to contiguous form and
// runs one of two kernels (16x32-thread shared-memory scan of the innermost dim, or one thread per
// column for outer dims) or thrust for 1-D.
//
// Here the operands keep their strides.  Three walks:
//   row      the scanned dim has stride 1 in both tensors: a warp scans a row (or a chunk of one)
//            in steps of 32 vectors, thread-local scan + warp shuffle scan + running carry;
//   col      some dims after the scanned one form a stride-1 run in both tensors: a thread owns V
//            adjacent columns and walks down the scanned dim, lanes side by side;
//   strided  anything else: a thread per slice.
// When there are too few rows / columns to fill the GPU the scanned dim is cut into chunks:
// pass 1 folds every chunk, pass 2 turns the chunk totals into carries, pass 3 scans each chunk
// starting from its carry.  Accumulation is in the accumulate type of the reductions (double for
// float and double, float for half, int64 for integers), each output rounded from the running
// accumulator, as TH's cumsum / cumprod do.  Fixed partition and order: results repeat bit for bit.
#include <string.h>

#include "context.h"
#include "core.cuh"
#include "plan.h"

namespace thcb {
namespace {

constexpr int kScanThreads = 256;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kScanUnroll = 4;

struct ScanMap {
  int n;
  uint64_t size[kMaxDims];
  int64_t in_stride[kMaxDims];
  int64_t out_stride[kMaxDims];
  __device__ __forceinline__ void decode(uint64_t lin, int64_t &in_off, int64_t &out_off) const {
    in_off = 0; out_off = 0;
    for (int d = n - 1; d >= 0; --d) {
      uint64_t q, r;
      if (d == 0) { q = 0; r = lin; }                    // the outermost dim needs no division
      else if (((lin | size[d]) >> 32) == 0) {           // 32-bit operands: the short divide
        const uint32_t l = (uint32_t)lin, s = (uint32_t)size[d], qq = l / s;
        q = qq;
        r = l - qq * s;
      } else {
        q = lin / size[d];
        r = lin - q * size[d];
      }
      in_off += (int64_t)r * in_stride[d];
      out_off += (int64_t)r * out_stride[d];
      lin = q;
    }
  }
};

template <typename T, int V> struct alignas(V * sizeof(T)) Pack { T v[V]; };

template <typename A, bool PROD> __device__ __forceinline__ A scan_identity() { return PROD ? (A)1 : (A)0; }
template <typename A, bool PROD> __device__ __forceinline__ A scan_op(A earlier, A later) {
  return PROD ? earlier * later : earlier + later;
}
template <typename T, typename A> __device__ __forceinline__ A to_acc(T x) { return (A)to_math<T>(x); }
template <typename T, typename A> __device__ __forceinline__ T from_acc(A a) {
  return from_math<T>((typename TypeTraits<T>::Math)a);
}

// ---------------------------------------------------------------------------------
// row walk.  unit = row * S + chunk; a warp per unit.
// ---------------------------------------------------------------------------------
template <typename T, bool PROD, bool VEC, bool TOTAL_ONLY>
__global__ void __launch_bounds__(kScanThreads)
scan_row_kernel(const T *in, T *out, ScanMap map, uint64_t nrows, uint64_t K, uint32_t S, uint64_t chunk_len,
                typename TypeTraits<T>::Acc *carries) {
  pdl_prologue();
  using A = typename TypeTraits<T>::Acc;
  constexpr int V = VEC ? 16 / (int)sizeof(T) : 1;
  constexpr int U = kScanUnroll;
  const unsigned lane = threadIdx.x & 31;
  const uint64_t unit = (uint64_t)blockIdx.x * kScanWarps + (threadIdx.x >> 5);
  if (unit >= nrows * S) return;
  const uint64_t row = div_by_u32(unit, S);
  const uint64_t k0 = (unit - row * S) * chunk_len;
  const uint64_t k1 = k0 + chunk_len < K ? k0 + chunk_len : K;
  int64_t ioff, ooff;
  map.decode(row, ioff, ooff);
  const T *ip = in + ioff;
  T *op = out + ooff;
  A carry = scan_identity<A, PROD>();
  // Vector layout: a unit need not start on a 16-byte boundary (input and output rows share their
  // misalignment); [k0, kb) before the first boundary and [ke, k1) after the last whole vector
  // (fewer than V elements each) are taken one element per lane.
  uint64_t kb = k0, ke = k1;
  if constexpr (VEC) {
    const uint64_t mis = (reinterpret_cast<uintptr_t>(ip + k0) / sizeof(T)) % V;
    uint64_t head = mis ? V - mis : 0;
    if (head > k1 - k0) head = k1 - k0;
    kb = k0 + head;
    ke = kb + (k1 - kb) / V * V;
  }
  if constexpr (TOTAL_ONLY) {
    // only the fold of the chunk is wanted: every lane folds what it loads, one butterfly at the end
    A acc = scan_identity<A, PROD>();
    if constexpr (VEC) {
      if (lane < kb - k0) acc = to_acc<T, A>(ip[k0 + lane]);
      if (lane < k1 - ke) acc = scan_op<A, PROD>(acc, to_acc<T, A>(ip[ke + lane]));
    }
    for (uint64_t base = kb; base < ke; base += (uint64_t)32 * V * U) {
      Pack<T, V> x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t pos = base + ((uint64_t)u * 32 + lane) * V;
        if (pos < ke) x[u] = *reinterpret_cast<const Pack<T, V> *>(ip + pos);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t pos = base + ((uint64_t)u * 32 + lane) * V;
        if (pos < ke) {
#pragma unroll
          for (int j = 0; j < V; ++j) acc = scan_op<A, PROD>(acc, to_acc<T, A>(x[u].v[j]));
        }
      }
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) acc = scan_op<A, PROD>(acc, __shfl_xor_sync(0xffffffffu, acc, d));
    if (lane == 0) carries[unit] = acc;
    return;
  }
  if (carries) carry = carries[unit];
  // one element per lane: the pieces in front of and behind the whole vectors
  auto lane_step = [&](uint64_t start, uint64_t count) {
    if (count == 0) return;   // uniform over the warp
    const bool live = lane < count;
    const A e = live ? to_acc<T, A>(ip[start + lane]) : scan_identity<A, PROD>();
    const A incl = [&] {
      A v = e;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const A y = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= (unsigned)d) v = scan_op<A, PROD>(y, v);
      }
      return v;
    }();
    A excl = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) excl = scan_identity<A, PROD>();
    if (live) op[start + lane] = from_acc<T, A>(scan_op<A, PROD>(scan_op<A, PROD>(carry, excl), e));
    carry = scan_op<A, PROD>(carry, __shfl_sync(0xffffffffu, incl, 31));
  };
  if constexpr (VEC) lane_step(k0, kb - k0);
  for (uint64_t base = kb; base < ke; base += (uint64_t)32 * V * U) {
    Pack<T, V> x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t pos = base + ((uint64_t)u * 32 + lane) * V;
      if (pos < ke) x[u] = *reinterpret_cast<const Pack<T, V> *>(ip + pos);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t pos = base + ((uint64_t)u * 32 + lane) * V;
      const bool live = pos < ke;
      A a[V];
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const A e = live ? to_acc<T, A>(x[u].v[j]) : scan_identity<A, PROD>();
        a[j] = j == 0 ? e : scan_op<A, PROD>(a[j - 1], e);
      }
      A incl = a[V - 1];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const A y = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= (unsigned)d) incl = scan_op<A, PROD>(y, incl);
      }
      A excl = __shfl_up_sync(0xffffffffu, incl, 1);
      if (lane == 0) excl = scan_identity<A, PROD>();
      const A pre = scan_op<A, PROD>(carry, excl);
      if (live) {
        Pack<T, V> y;
#pragma unroll
        for (int j = 0; j < V; ++j) y.v[j] = from_acc<T, A>(scan_op<A, PROD>(pre, a[j]));
        *reinterpret_cast<Pack<T, V> *>(op + pos) = y;
      }
      carry = scan_op<A, PROD>(carry, __shfl_sync(0xffffffffu, incl, 31));
    }
  }
  if constexpr (VEC) lane_step(ke, k1 - ke);
}

// chunk totals -> exclusive carries, in place; a CTA per row, threads own consecutive segments
template <typename A, bool PROD>
__global__ void __launch_bounds__(kScanThreads) scan_row_carry_kernel(A *carries, uint64_t nrows, uint32_t S) {
  pdl_prologue();
  __shared__ A wtot[kScanWarps];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  A *c = carries + (uint64_t)blockIdx.x * S;
  const uint32_t per = (S + kScanThreads - 1) / kScanThreads;
  const uint32_t lo = threadIdx.x * per < S ? threadIdx.x * per : S;
  const uint32_t hi = lo + per < S ? lo + per : S;
  A tot = scan_identity<A, PROD>();
  for (uint32_t i = lo; i < hi; ++i) tot = scan_op<A, PROD>(tot, c[i]);
  A incl = tot;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const A y = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl = scan_op<A, PROD>(y, incl);
  }
  if (lane == 31) wtot[warp] = incl;
  __syncthreads();
  A run = scan_identity<A, PROD>();
  for (unsigned w = 0; w < warp; ++w) run = scan_op<A, PROD>(run, wtot[w]);
  A excl = __shfl_up_sync(0xffffffffu, incl, 1);
  if (lane != 0) run = scan_op<A, PROD>(run, excl);
  for (uint32_t i = lo; i < hi; ++i) {
    const A v = c[i];
    c[i] = run;
    run = scan_op<A, PROD>(run, v);
  }
}

// ---------------------------------------------------------------------------------
// column walk.  unit = (outer * S + chunk) * tiles_i + tile; a warp per unit, 32 * V columns.
// carries: [outer][chunk][I]
// ---------------------------------------------------------------------------------
template <typename T, bool PROD, int V, bool TOTAL_ONLY>
__global__ void __launch_bounds__(kScanThreads)
scan_col_kernel(const T *in, T *out, ScanMap map, uint64_t nouter, uint64_t K, int64_t sKi, int64_t sKo, uint64_t I,
                uint32_t tiles_i, uint32_t S, uint64_t chunk_len, typename TypeTraits<T>::Acc *carries) {
  pdl_prologue();
  using A = typename TypeTraits<T>::Acc;
  constexpr int U = kScanUnroll;
  const unsigned lane = threadIdx.x & 31;
  const uint64_t unit = (uint64_t)blockIdx.x * kScanWarps + (threadIdx.x >> 5);
  if (unit >= nouter * S * tiles_i) return;
  const uint64_t oc = div_by_u32(unit, tiles_i);
  const uint32_t ti = (uint32_t)(unit - oc * tiles_i);
  const uint64_t o = div_by_u32(oc, S);
  const uint64_t col = ((uint64_t)ti * 32 + lane) * V;
  if (col >= I) return;
  const uint64_t k0 = (oc - o * S) * chunk_len;
  const uint64_t k1 = k0 + chunk_len < K ? k0 + chunk_len : K;
  int64_t ioff, ooff;
  map.decode(o, ioff, ooff);
  const T *ip = in + ioff + (int64_t)col + (int64_t)k0 * sKi;
  T *op = out + ooff + (int64_t)col + (int64_t)k0 * sKo;
  A acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = scan_identity<A, PROD>();
  A *cslot = carries ? carries + oc * I + col : nullptr;
  if (!TOTAL_ONLY && cslot) {
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = cslot[j];
  }
  for (uint64_t k = k0; k < k1; k += U) {
    Pack<T, V> x[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (k + u < k1) x[u] = *reinterpret_cast<const Pack<T, V> *>(ip + (int64_t)u * sKi);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (k + u < k1) {
        Pack<T, V> y;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          acc[j] = scan_op<A, PROD>(acc[j], to_acc<T, A>(x[u].v[j]));
          y.v[j] = from_acc<T, A>(acc[j]);
        }
        if (!TOTAL_ONLY) *reinterpret_cast<Pack<T, V> *>(op + (int64_t)u * sKo) = y;
      }
    }
    ip += (int64_t)U * sKi;
    op += (int64_t)U * sKo;
  }
  if (TOTAL_ONLY) {
#pragma unroll
    for (int j = 0; j < V; ++j) cslot[j] = acc[j];
  }
}

// chunk totals -> exclusive carries along the chunk index; a thread per (outer, column)
template <typename A, bool PROD>
__global__ void __launch_bounds__(kScanThreads) scan_col_carry_kernel(A *carries, uint64_t nouter, uint64_t I, uint32_t S) {
  pdl_prologue();
  const uint64_t t = (uint64_t)blockIdx.x * kScanThreads + threadIdx.x;
  if (t >= nouter * I) return;
  const uint64_t o = t / I, col = t - o * I;
  A *c = carries + o * S * I + col;
  A run = scan_identity<A, PROD>();
  // eight totals are loaded before the first carry is stored (loads and stores alias otherwise)
  for (uint32_t i0 = 0; i0 < S; i0 += 8) {
    A v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i0 + u < S) v[u] = c[(uint64_t)(i0 + u) * I];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (i0 + u < S) {
        c[(uint64_t)(i0 + u) * I] = run;
        run = scan_op<A, PROD>(run, v[u]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// strided walk: a thread per slice
// ---------------------------------------------------------------------------------
template <typename T, bool PROD>
__global__ void __launch_bounds__(kScanThreads)
scan_strided_kernel(const T *in, T *out, ScanMap map, uint64_t nslices, uint64_t K, int64_t sKi, int64_t sKo) {
  pdl_prologue();
  using A = typename TypeTraits<T>::Acc;
  const uint64_t s = (uint64_t)blockIdx.x * kScanThreads + threadIdx.x;
  if (s >= nslices) return;
  int64_t ioff, ooff;
  map.decode(s, ioff, ooff);
  const T *ip = in + ioff;
  T *op = out + ooff;
  A acc = scan_identity<A, PROD>();
  for (uint64_t k = 0; k < K; ++k) {
    acc = scan_op<A, PROD>(acc, to_acc<T, A>(ip[(int64_t)k * sKi]));
    op[(int64_t)k * sKo] = from_acc<T, A>(acc);
  }
}
// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
enum ScanKind { kScanRow, kScanCol, kScanStrided };

struct ScanPlan {
  ScanKind kind;
  bool vec;
  ScanMap map;
  uint64_t nslices;   // rows (row), outer slices (col), slices (strided)
  uint64_t K, I;
  int64_t sKi, sKo;
  uint32_t tiles_i, S;
  uint64_t chunk_len;
};

// appends dim (size, is, os) to the map, merging it into the previous entry when it continues
// that entry's run in both tensors
void map_push(ScanMap *m, bool adjacent, int64_t size, int64_t is, int64_t os) {
  if (adjacent && m->n > 0 && m->in_stride[m->n - 1] == size * is && m->out_stride[m->n - 1] == size * os) {
    m->size[m->n - 1] *= (uint64_t)size;
    m->in_stride[m->n - 1] = is;
    m->out_stride[m->n - 1] = os;
    return;
  }
  m->size[m->n] = (uint64_t)size;
  m->in_stride[m->n] = is;
  m->out_stride[m->n] = os;
  ++m->n;
}

void plan_scan(const thcb200_ctx *ctx, const HostView &in, const HostView &out, int dim, size_t esz, ScanPlan *pl) {
  const int vfull = (int)(16 / esz);
  const int vcol = esz == 1 ? 4 : vfull;
  pl->K = (uint64_t)in.sizes[dim];
  pl->sKi = in.strides[dim];
  pl->sKo = out.strides[dim];
  pl->I = 1;
  pl->tiles_i = 1;
  pl->S = 1;
  pl->chunk_len = pl->K;
  pl->vec = false;
  pl->map.n = 0;
  const bool aligned = ((uintptr_t)in.data % 16 == 0) && ((uintptr_t)out.data % 16 == 0);
  const uint64_t target_warps = (uint64_t)ctx->num_sms * 4 * kScanWarps;
  uint64_t nother = 1;
  for (int i = 0; i < in.ndim; ++i) if (i != dim) nother *= (uint64_t)in.sizes[i];

  if (pl->sKi == 1 && pl->sKo == 1 && pl->K >= 64) {
    pl->kind = kScanRow;
    int prev = -2;
    for (int i = 0; i < in.ndim; ++i) {
      if (i == dim || in.sizes[i] == 1) continue;
      map_push(&pl->map, prev >= 0, in.sizes[i], in.strides[i], out.strides[i]);
      prev = i;
    }
    pl->nslices = nother;
    // vectors from each unit's first 16-byte boundary: input and output rows only have to share
    // their misalignment
    bool vec = ((uintptr_t)in.data % 16) == ((uintptr_t)out.data % 16);
    for (int i = 0; i < pl->map.n; ++i)
      if ((pl->map.in_stride[i] - pl->map.out_stride[i]) % vfull != 0) vec = false;
    pl->vec = vec;
    const uint64_t step = 32ull * (vec ? vfull : 1) * kScanUnroll;
    if (nother < target_warps / 2 && pl->K >= 4 * step) {
      uint64_t want = target_warps / nother;
      const uint64_t maxs = pl->K / (2 * step);
      if (want > maxs) want = maxs;
      if (want > 1) {
        uint64_t len = (pl->K + want - 1) / want;
        len = (len + step - 1) / step * step;
        pl->chunk_len = len;
        pl->S = (uint32_t)((pl->K + len - 1) / len);
      }
    }
    return;
  }
  // column walk: the dims after `dim`, from the last one outward, while they form one stride-1 run
  int inner_from = in.ndim;   // dims [inner_from, ndim) are the inner run
  {
    int64_t run = 1;
    for (int i = in.ndim - 1; i > dim; --i) {
      if (in.sizes[i] == 1) { if (inner_from == i + 1) inner_from = i; continue; }
      if (in.strides[i] == run && out.strides[i] == run) { run *= in.sizes[i]; inner_from = i; } else break;
    }
    if (run >= 32 && pl->K > 1) {
      pl->kind = kScanCol;
      pl->I = (uint64_t)run;
      int prev = -2;
      for (int i = 0; i < inner_from; ++i) {
        if (i == dim) { prev = -2; continue; }
        if (in.sizes[i] == 1) continue;
        map_push(&pl->map, prev >= 0, in.sizes[i], in.strides[i], out.strides[i]);
        prev = i;
      }
      uint64_t nouter = 1;
      for (int i = 0; i < pl->map.n; ++i) nouter *= pl->map.size[i];
      pl->nslices = nouter;
      bool vec = aligned && pl->I % vcol == 0 && pl->sKi % vcol == 0 && pl->sKo % vcol == 0;
      for (int i = 0; i < pl->map.n; ++i)
        if (pl->map.in_stride[i] % vcol != 0 || pl->map.out_stride[i] % vcol != 0) vec = false;
      pl->vec = vec;
      const int v = vec ? vcol : 1;
      pl->tiles_i = (uint32_t)((pl->I + 32ull * v - 1) / (32ull * v));
      const uint64_t units = nouter * pl->tiles_i;
      const uint64_t min_chunk = 16ull * kScanUnroll;
      if (units < target_warps / 2 && pl->K >= 4 * min_chunk) {
        uint64_t want = target_warps / units;
        const uint64_t maxs = pl->K / (2 * min_chunk);
        if (want > maxs) want = maxs;
        if (want > 1) {
          uint64_t len = (pl->K + want - 1) / want;
          len = (len + kScanUnroll - 1) / kScanUnroll * kScanUnroll;
          pl->chunk_len = len;
          pl->S = (uint32_t)((pl->K + len - 1) / len);
        }
      }
      return;
    }
  }
  pl->kind = kScanStrided;
  pl->map.n = 0;
  int prev = -2;
  for (int i = 0; i < in.ndim; ++i) {
    if (i == dim) { prev = -2; continue; }
    if (in.sizes[i] == 1) continue;
    map_push(&pl->map, prev >= 0, in.sizes[i], in.strides[i], out.strides[i]);
    prev = i;
  }
  pl->nslices = nother;
}

int blocks_for(uint64_t units, uint64_t per_cta, unsigned *grid) {
  const uint64_t blocks = (units + per_cta - 1) / per_cta;
  if (blocks >= (1ull << 31)) { set_error("scan_dim: tensor too large"); return THCB200_ERR_DIMS; }
  *grid = (unsigned)(blocks ? blocks : 1);
  return 0;
}

template <typename T, bool PROD>
int launch_scan(thcb200_ctx *ctx, const HostView &in, const HostView &out, int dim, cudaStream_t st) {
  using A = typename TypeTraits<T>::Acc;
  constexpr int VC = sizeof(T) == 1 ? 4 : 16 / (int)sizeof(T);
  ScanPlan pl;
  plan_scan(ctx, in, out, dim, sizeof(T), &pl);
  const T *ip = reinterpret_cast<const T *>(in.data);
  T *op = reinterpret_cast<T *>(out.data);
  A *carries = nullptr;
  if (pl.S > 1) {
    const uint64_t slots = pl.kind == kScanCol ? pl.nslices * pl.S * pl.I : pl.nslices * pl.S;
    carries = reinterpret_cast<A *>(ctx_workspace(ctx, slots * sizeof(A)));
    if (!carries) return THCB200_ERR_NOMEM;
  }
  unsigned grid;
  int rc;
  int launches = 1;
  switch (pl.kind) {
    case kScanRow: {
      if ((rc = blocks_for(pl.nslices * pl.S, kScanWarps, &grid))) return rc;
      set_plan_name(pl.S > 1 ? (pl.vec ? "scan_row_vec_chunked" : "scan_row_chunked") : (pl.vec ? "scan_row_vec" : "scan_row"));
      if (pl.S > 1) {
        if (pl.vec) launch_pdl(scan_row_kernel<T, PROD, true, true>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.S, pl.chunk_len, carries);
        else launch_pdl(scan_row_kernel<T, PROD, false, true>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.S, pl.chunk_len, carries);
        unsigned g2;
        if ((rc = blocks_for(pl.nslices, 1, &g2))) return rc;
        launch_pdl(scan_row_carry_kernel<A, PROD>, g2, kScanThreads, 0, st, carries, pl.nslices, pl.S);
        launches += 2;
      }
      if (pl.vec) launch_pdl(scan_row_kernel<T, PROD, true, false>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.S, pl.chunk_len, carries);
      else launch_pdl(scan_row_kernel<T, PROD, false, false>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.S, pl.chunk_len, carries);
      break;
    }
    case kScanCol: {
      if ((rc = blocks_for(pl.nslices * pl.S * pl.tiles_i, kScanWarps, &grid))) return rc;
      set_plan_name(pl.S > 1 ? (pl.vec ? "scan_col_vec_chunked" : "scan_col_chunked") : (pl.vec ? "scan_col_vec" : "scan_col"));
      if (pl.S > 1) {
        if (pl.vec) launch_pdl(scan_col_kernel<T, PROD, VC, true>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.sKi, pl.sKo, pl.I, pl.tiles_i, pl.S, pl.chunk_len, carries);
        else launch_pdl(scan_col_kernel<T, PROD, 1, true>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.sKi, pl.sKo, pl.I, pl.tiles_i, pl.S, pl.chunk_len, carries);
        unsigned g2;
        if ((rc = blocks_for(pl.nslices * pl.I, kScanThreads, &g2))) return rc;
        launch_pdl(scan_col_carry_kernel<A, PROD>, g2, kScanThreads, 0, st, carries, pl.nslices, pl.I, pl.S);
        launches += 2;
      }
      if (pl.vec) launch_pdl(scan_col_kernel<T, PROD, VC, false>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.sKi, pl.sKo, pl.I, pl.tiles_i, pl.S, pl.chunk_len, carries);
      else launch_pdl(scan_col_kernel<T, PROD, 1, false>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.sKi, pl.sKo, pl.I, pl.tiles_i, pl.S, pl.chunk_len, carries);
      break;
    }
    default: {
      if ((rc = blocks_for(pl.nslices, kScanThreads, &grid))) return rc;
      set_plan_name("scan_strided");
      launch_pdl(scan_strided_kernel<T, PROD>, grid, kScanThreads, 0, st, ip, op, pl.map, pl.nslices, pl.K, pl.sKi, pl.sKo);
      break;
    }
  }
  count_launch(launches);
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

template <typename T>
int scan_typed(thcb200_ctx *ctx, bool prod, const HostView &in, const HostView &out, int dim, cudaStream_t st) {
  return prod ? launch_scan<T, true>(ctx, in, out, dim, st) : launch_scan<T, false>(ctx, in, out, dim, st);
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" int thcb200_scan_dim(thcb200_ctx *ctx, int rop, const thcb200_tensor *out, const thcb200_tensor *in, int dim,
                                void *stream) {
  if (!ctx) { set_error("scan_dim: null context"); return THCB200_ERR_ARG; }
  if (rop != THCB200_RED_SUM && rop != THCB200_RED_PROD) { set_error("scan_dim: only sum and prod scans exist"); return THCB200_ERR_ARG; }
  HostView vin, vout;
  int rc = to_host_view(in, &vin, "scan_dim input");
  if (!rc) rc = to_host_view(out, &vout, "scan_dim output");
  if (rc) return rc;
  if (vin.dtype != vout.dtype) { set_error("scan_dim: operands have different dtypes"); return THCB200_ERR_ARG; }
  if (dim < 0 || dim >= vin.ndim) { set_error("scan_dim: dimension %d out of range", dim); return THCB200_ERR_ARG; }
  if (vin.ndim != vout.ndim) { set_error("scan_dim: output and input have different shapes"); return THCB200_ERR_SIZE; }
  for (int i = 0; i < vin.ndim; ++i)
    if (vin.sizes[i] != vout.sizes[i]) { set_error("scan_dim: output and input have different shapes"); return THCB200_ERR_SIZE; }
  if (vin.numel == 0) return THCB200_OK;
  THCB_CTX_LOCK(ctx);
  cudaStream_t st = (cudaStream_t)stream;
  const bool prod = rop == THCB200_RED_PROD;
  switch (vin.dtype) {
    case THCB200_U8: return scan_typed<uint8_t>(ctx, prod, vin, vout, dim, st);
    case THCB200_I8: return scan_typed<int8_t>(ctx, prod, vin, vout, dim, st);
    case THCB200_I16: return scan_typed<int16_t>(ctx, prod, vin, vout, dim, st);
    case THCB200_I32: return scan_typed<int32_t>(ctx, prod, vin, vout, dim, st);
    case THCB200_I64: return scan_typed<int64_t>(ctx, prod, vin, vout, dim, st);
    case THCB200_F16: return scan_typed<__half>(ctx, prod, vin, vout, dim, st);
    case THCB200_F32: return scan_typed<float>(ctx, prod, vin, vout, dim, st);
    default: return scan_typed<double>(ctx, prod, vin, vout, dim, st);
  }
}
