/*
 * THCReduce.cuh -- C++ template forms of the dimension reduction and the full reduction for
 * user-defined functors, with the contracts of cutorch's installed templates:
 *
 *   template <typename TensorType, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
 *   bool THC_reduceDim(THCState*, TensorType* out, TensorType* in, const ModifyOp&, const ReduceOp&,
 *                      const ReduceAccOp&, AccT init, int dim, int keepdim);        (lib/THC/THCReduce.cuh:258-271)
 *   bool THC_reduceAll(THCState*, TensorType* in, const ModifyOp&, const ReduceOp&, const ReduceAccOp&,
 *                      AccT init, AccT* out, int outOnDevice);                      (lib/THC/THCReduceAll.cuh:234-246)
 *
 * out[..., 0, ...] = (T) fold_i reduceOp(acc, modifyOp(in[..., i, ...])), acc starting at `init`;
 * partial accumulators are merged with reduceAccOp.  `init` must be an identity of the fold: as in
 * the reference every thread starts from it.  THC_reduceDim resizes `out` to in's sizes with
 * size[dim] = 1 and squeezes that dim unless keepdim (lib/THC/THCReduce.cuh:328-332, 449-451).
 * THC_reduceAll writes *out on the host, returning once the stream has finished as the reference's
 * synchronous copy does, or on the device when outOnDevice (lib/THC/THCReduceAll.cuh:259-270,
 * 333-335); a tensor without dimensions yields init.  It is one launch: the CTA that finishes last
 * folds the CTAs' partials in index order and writes the result (for a host result into a pinned
 * slot of the calling thread, so no copy follows the kernel).
 * Both return false for more than 25 dims.
 *
 * The built-in reductions (sum, prod, min, max, norm ...) do not come through here: they use the
 * kernels behind the C API.  These templates serve arbitrary functors and arbitrary trivially
 * copyable accumulator types.  The functors take values, so elements are loaded 16 bytes at a time
 * where the layout allows and eight loads ahead of the first fold; a reduced dim that is dense gets a
 * warp per slice (many slices) or a CTA per slice, a strided one with a dense neighbour gets lanes
 * along that neighbour.  Partials are merged by shuffles and through shared memory in a fixed
 * order, so results repeat bit for bit.
 *
 * Include from a .cu file compiled for sm_100a and link libthcb200.
 */
#ifndef THCB200_THC_REDUCE_CUH
#define THCB200_THC_REDUCE_CUH

#include <string.h>

#include "THCApply.cuh"

namespace thcb_user {

constexpr int kReduceThreads = 256;

// slice number -> element offsets of the input and the output (dims other than the reduced one)
struct SliceView {
  int n;
  uint64_t size[THCB200_MAX_DIMS];
  int64_t in_stride[THCB200_MAX_DIMS];
  int64_t out_stride[THCB200_MAX_DIMS];
  __device__ __forceinline__ void decode(uint64_t lin, int64_t &in_off, int64_t &out_off) const {
    in_off = 0;
    out_off = 0;
    for (int d = n - 1; d >= 0; --d) {
      const uint64_t q = lin / size[d], r = lin - q * size[d];
      in_off += (int64_t)r * in_stride[d];
      out_off += (int64_t)r * out_stride[d];
      lin = q;
    }
  }
};

// V elements loaded as one aligned unit (V * sizeof(T) = 16 bytes in the vector kernels)
template <typename T, int V> struct alignas(V * sizeof(T)) ValuePack { T v[V]; };

// shuffle of any trivially copyable accumulator, 32 bits at a time
template <typename AccT>
__device__ __forceinline__ AccT shfl_down_any(const AccT &v, unsigned delta) {
  constexpr int W = (int)((sizeof(AccT) + 3) / 4);
  uint32_t w[W];
  for (int i = 0; i < W; ++i) w[i] = 0;
  memcpy(w, &v, sizeof(AccT));
#pragma unroll
  for (int i = 0; i < W; ++i) w[i] = __shfl_down_sync(0xffffffffu, w[i], delta);
  AccT r;
  memcpy(&r, w, sizeof(AccT));
  return r;
}

// Folds the accumulators of a CTA in thread order (0 with 1, 2 with 3, then 0-1 with 2-3 ...: a
// binary tree over thread numbers), result in thread 0 only.  Inside a warp the tree runs on
// shuffles, across warps thread 0 finishes it from `buf` (one accumulator per warp).  blockDim.x is
// a power of two of at least 32 and every thread of the CTA calls this.
template <typename AccT, typename ReduceAccOp>
__device__ __forceinline__ AccT block_fold(AccT acc, AccT *buf, const ReduceAccOp &accOp) {
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (unsigned s = 1; s < 32; s <<= 1) {
    const AccT other = shfl_down_any(acc, s);
    if ((lane & (2 * s - 1)) == 0) acc = accOp(acc, other);
  }
  if (nwarps == 1) return acc;
  if (lane == 0) buf[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (unsigned s = 1; s < nwarps; s <<= 1)
      for (unsigned i = 0; i + s < nwarps; i += 2 * s) buf[i] = accOp(buf[i], buf[i + s]);
    acc = buf[0];
  }
  return acc;
}

constexpr int kLoadsInFlight = 8;   // elements a thread loads before it folds the first of them

// one CTA per slice; threads stride over the reduced dim.  V > 1 (the reduced dim is dense and every
// slice starts on a 16-byte boundary): whole 16-byte packs first, then the K % V elements left.
template <typename T, int V, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
__global__ void __launch_bounds__(kReduceThreads)
reduce_dim_cta_kernel(T *out, const T *in, SliceView sv, uint64_t K, int64_t strideK, AccT init, ModifyOp modifyOp,
                      ReduceOp reduceOp, ReduceAccOp accOp) {
  extern __shared__ __align__(16) unsigned char thcb_user_smem[];
  AccT *buf = reinterpret_cast<AccT *>(thcb_user_smem);
  int64_t in_off, out_off;
  sv.decode(blockIdx.x, in_off, out_off);
  const T *p = in + in_off;
  AccT acc = init;
  // kLoadsInFlight loads are issued before the first value is folded (the functors take values, so
  // the loads do not depend on one another); a thread folds its values in the order it loaded them
  if (V > 1) {
    const uint64_t packs = K / V;
    const ValuePack<T, V> *pp = reinterpret_cast<const ValuePack<T, V> *>(p);
    for (uint64_t k0 = threadIdx.x; k0 < packs; k0 += (uint64_t)blockDim.x * kLoadsInFlight) {
      ValuePack<T, V> x[kLoadsInFlight];
#pragma unroll
      for (int u = 0; u < kLoadsInFlight; ++u) {
        const uint64_t k = k0 + (uint64_t)u * blockDim.x;
        if (k < packs) x[u] = pp[k];
      }
#pragma unroll
      for (int u = 0; u < kLoadsInFlight; ++u)
        if (k0 + (uint64_t)u * blockDim.x < packs) {
#pragma unroll
          for (int j = 0; j < V; ++j) acc = reduceOp(acc, modifyOp(x[u].v[j]));
        }
    }
    for (uint64_t k = packs * V + threadIdx.x; k < K; k += blockDim.x) acc = reduceOp(acc, modifyOp(p[k]));
  } else {
    for (uint64_t k0 = threadIdx.x; k0 < K; k0 += (uint64_t)blockDim.x * kLoadsInFlight) {
      T x[kLoadsInFlight];
#pragma unroll
      for (int u = 0; u < kLoadsInFlight; ++u) {
        const uint64_t k = k0 + (uint64_t)u * blockDim.x;
        if (k < K) x[u] = p[(int64_t)k * strideK];
      }
#pragma unroll
      for (int u = 0; u < kLoadsInFlight; ++u)
        if (k0 + (uint64_t)u * blockDim.x < K) acc = reduceOp(acc, modifyOp(x[u]));
    }
  }
  acc = block_fold(acc, buf, accOp);
  if (threadIdx.x == 0) out[out_off] = (T)acc;
}

// A warp per slice (many slices): no shared memory and no barrier, the lanes' accumulators are folded
// by shuffles in lane order.  CTAs stride over groups of blockDim.x / 32 slices.
template <typename T, int V, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
__global__ void __launch_bounds__(kReduceThreads)
reduce_dim_warp_kernel(T *out, const T *in, SliceView sv, uint64_t nslices, uint64_t K, int64_t strideK, AccT init,
                       ModifyOp modifyOp, ReduceOp reduceOp, ReduceAccOp accOp) {
  const unsigned lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (uint64_t slice = (uint64_t)blockIdx.x * warps + (threadIdx.x >> 5); slice < nslices; slice += (uint64_t)gridDim.x * warps) {
    int64_t in_off, out_off;
    sv.decode(slice, in_off, out_off);
    const T *p = in + in_off;
    AccT acc = init;
    if (V > 1) {
      const uint64_t packs = K / V;
      const ValuePack<T, V> *pp = reinterpret_cast<const ValuePack<T, V> *>(p);
      for (uint64_t k0 = lane; k0 < packs; k0 += 32 * kLoadsInFlight) {
        ValuePack<T, V> x[kLoadsInFlight];
#pragma unroll
        for (int u = 0; u < kLoadsInFlight; ++u)
          if (k0 + 32 * u < packs) x[u] = pp[k0 + 32 * u];
#pragma unroll
        for (int u = 0; u < kLoadsInFlight; ++u)
          if (k0 + 32 * u < packs) {
#pragma unroll
            for (int j = 0; j < V; ++j) acc = reduceOp(acc, modifyOp(x[u].v[j]));
          }
      }
      for (uint64_t k = packs * V + lane; k < K; k += 32) acc = reduceOp(acc, modifyOp(p[k]));
    } else {
      for (uint64_t k0 = lane; k0 < K; k0 += 32 * kLoadsInFlight) {
        T x[kLoadsInFlight];
#pragma unroll
        for (int u = 0; u < kLoadsInFlight; ++u)
          if (k0 + 32 * u < K) x[u] = p[(int64_t)(k0 + 32 * u) * strideK];
#pragma unroll
        for (int u = 0; u < kLoadsInFlight; ++u)
          if (k0 + 32 * u < K) acc = reduceOp(acc, modifyOp(x[u]));
      }
    }
#pragma unroll
    for (unsigned s = 1; s < 32; s <<= 1) {
      const AccT other = shfl_down_any(acc, s);
      if ((lane & (2 * s - 1)) == 0) acc = accOp(acc, other);
    }
    if (lane == 0) out[out_off] = (T)acc;
  }
}

// The reduced dim is strided and some other dim (`inner` elements, stride 1 in the input) is dense:
// a lane sits on V neighbouring slices (V * sizeof(T) = 16 bytes when alignment allows, else V = 1),
// so every load of a warp is whole lines; the CTA's warps take the reduced positions round-robin
// with kLoadsInFlight of them in flight per thread, and the warps' accumulators are merged in warp
// order through shared memory.
template <typename T, int V, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
__global__ void __launch_bounds__(kReduceThreads)
reduce_dim_col_kernel(T *out, const T *in, SliceView sv /* the dims other than the reduced and the inner one */, uint64_t inner,
                      int64_t out_inner_stride, uint32_t tiles_i, uint64_t K, int64_t strideK, AccT init, ModifyOp modifyOp,
                      ReduceOp reduceOp, ReduceAccOp accOp, uint32_t nsplit, uint64_t split_len, AccT *partials) {
  extern __shared__ __align__(16) unsigned char thcb_user_smem[];
  AccT *buf = reinterpret_cast<AccT *>(thcb_user_smem);     // [warp][lane][V]
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  // blockIdx.x -> (outer slice, split of the reduced dim, tile of 32 * V inner positions)
  uint32_t b = blockIdx.x;
  const uint32_t ti = b % tiles_i; b /= tiles_i;
  const uint32_t split = b % nsplit;
  const uint64_t outer = b / nsplit;
  const uint64_t i = ((uint64_t)ti * 32 + lane) * V;
  int64_t in_off, out_off;
  sv.decode(outer, in_off, out_off);
  const T *p = in + in_off + (int64_t)i;
  const uint64_t kbeg = (uint64_t)split * split_len, kend = kbeg + split_len < K ? kbeg + split_len : K;
  AccT acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = init;
  if (i < inner) {
    for (uint64_t k0 = kbeg + warp; k0 < kend; k0 += (uint64_t)nwarps * kLoadsInFlight) {
      ValuePack<T, V> x[kLoadsInFlight];
#pragma unroll
      for (int u = 0; u < kLoadsInFlight; ++u) {
        const uint64_t k = k0 + (uint64_t)u * nwarps;
        if (k < kend) x[u] = *reinterpret_cast<const ValuePack<T, V> *>(p + (int64_t)k * strideK);
      }
#pragma unroll
      for (int u = 0; u < kLoadsInFlight; ++u)
        if (k0 + (uint64_t)u * nwarps < kend) {
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] = reduceOp(acc[j], modifyOp(x[u].v[j]));
        }
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) buf[(warp * 32 + lane) * V + j] = acc[j];
  __syncthreads();
  if (warp == 0 && i < inner) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      AccT r = buf[lane * V + j];
      for (unsigned w = 1; w < nwarps; ++w) r = accOp(r, buf[(w * 32 + lane) * V + j]);
      if (nsplit > 1) partials[(outer * nsplit + split) * inner + i + j] = r;   // [outer][split][inner]
      else out[out_off + (int64_t)(i + j) * out_inner_stride] = (T)r;
    }
  }
}

// second stage of a split column reduction: partials [outer][split][inner] folded in split order
template <typename T, typename ReduceAccOp, typename AccT>
__global__ void __launch_bounds__(kReduceThreads)
reduce_dim_col_finish_kernel(T *out, SliceView sv, uint64_t nouter, uint64_t inner, int64_t out_inner_stride, uint32_t nsplit,
                             const AccT *partials, ReduceAccOp accOp) {
  const uint64_t o = (uint64_t)blockIdx.x * kReduceThreads + threadIdx.x;
  if (o >= nouter * inner) return;
  const uint64_t outer = o / inner, i = o - outer * inner;
  int64_t in_off, out_off;
  sv.decode(outer, in_off, out_off);
  const AccT *pp = partials + outer * nsplit * inner + i;
  AccT r = pp[0];
  for (uint32_t s2 = 1; s2 < nsplit; ++s2) r = accOp(r, pp[(uint64_t)s2 * inner]);
  out[out_off + (int64_t)i * out_inner_stride] = (T)r;
}

// one thread per slice; neighbouring threads take neighbouring slices
template <typename T, typename ModifyOp, typename ReduceOp, typename AccT>
__global__ void __launch_bounds__(kReduceThreads)
reduce_dim_thread_kernel(T *out, const T *in, SliceView sv, uint64_t nslices, uint64_t K, int64_t strideK, AccT init,
                         ModifyOp modifyOp, ReduceOp reduceOp) {
  const uint64_t s = (uint64_t)blockIdx.x * kReduceThreads + threadIdx.x;
  if (s >= nslices) return;
  int64_t in_off, out_off;
  sv.decode(s, in_off, out_off);
  const T *p = in + in_off;
  AccT acc = init;
  for (uint64_t k0 = 0; k0 < K; k0 += kLoadsInFlight) {
    T x[kLoadsInFlight];
#pragma unroll
    for (int u = 0; u < kLoadsInFlight; ++u)
      if (k0 + u < K) x[u] = p[(int64_t)(k0 + u) * strideK];
#pragma unroll
    for (int u = 0; u < kLoadsInFlight; ++u)
      if (k0 + u < K) acc = reduceOp(acc, modifyOp(x[u]));
  }
  out[out_off] = (T)acc;
}

// Tail of the full reduction, run by every CTA after its own fold: the CTA's partial goes to
// `partials`, and the CTA that draws the last ticket folds all partials in index order (thread t takes
// t, t + 256, ..., then the fixed tree of block_fold) and writes the result -- to device memory or to a
// pinned host slot the device can see.  One launch; the result does not depend on which CTA was last.
template <typename ReduceAccOp, typename AccT>
__device__ __forceinline__ void reduce_all_finish(AccT acc, AccT *buf, AccT *partials, unsigned int *ticket, AccT init,
                                                  const ReduceAccOp &accOp, AccT *result) {
  __shared__ bool thcb_user_last;
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = acc;
    __threadfence();
    thcb_user_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!thcb_user_last) return;
  __threadfence();
  AccT f = init;
  const volatile AccT *vp = partials;
  for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) {
    AccT p;
    // other CTAs wrote these: read them past the L1
    const volatile unsigned char *src = reinterpret_cast<const volatile unsigned char *>(vp + i);
    unsigned char *dst = reinterpret_cast<unsigned char *>(&p);
    if (sizeof(AccT) % 4 == 0) {
      for (unsigned w = 0; w < sizeof(AccT) / 4; ++w)
        reinterpret_cast<uint32_t *>(dst)[w] = reinterpret_cast<const volatile uint32_t *>(src)[w];
    } else {
      for (unsigned w = 0; w < sizeof(AccT); ++w) dst[w] = src[w];
    }
    f = accOp(f, p);
  }
  f = block_fold(f, buf, accOp);
  if (threadIdx.x == 0) {
    *result = f;
    __threadfence_system();
  }
}

// full reduction: every CTA strides over the logical index space, then reduce_all_finish
template <typename T, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
__global__ void __launch_bounds__(kReduceThreads)
reduce_all_kernel(const T *in, View<uint64_t> v, uint64_t n, AccT init, ModifyOp modifyOp, ReduceOp reduceOp,
                  ReduceAccOp accOp, AccT *partials, unsigned int *ticket, AccT *result) {
  extern __shared__ __align__(16) unsigned char thcb_user_smem[];
  AccT *buf = reinterpret_cast<AccT *>(thcb_user_smem);
  AccT acc = init;
  const uint64_t step = (uint64_t)gridDim.x * kReduceThreads;
  for (uint64_t i0 = (uint64_t)blockIdx.x * kReduceThreads + threadIdx.x; i0 < n; i0 += step * kLoadsInFlight) {
    T x[kLoadsInFlight];
#pragma unroll
    for (int u = 0; u < kLoadsInFlight; ++u) {
      const uint64_t i = i0 + (uint64_t)u * step;
      if (i < n) x[u] = in[v.offset(i)];
    }
#pragma unroll
    for (int u = 0; u < kLoadsInFlight; ++u)
      if (i0 + (uint64_t)u * step < n) acc = reduceOp(acc, modifyOp(x[u]));
  }
  acc = block_fold(acc, buf, accOp);
  __syncthreads();     // buf is used again by the finishing CTA
  reduce_all_finish(acc, buf, partials, ticket, init, accOp, result);
}

// the same for one dense run starting on a 16-byte boundary: 16-byte packs, the n % V elements left go to CTA 0
template <typename T, int V, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
__global__ void __launch_bounds__(kReduceThreads)
reduce_all_dense_kernel(const T *in, uint64_t n, AccT init, ModifyOp modifyOp, ReduceOp reduceOp, ReduceAccOp accOp,
                        AccT *partials, unsigned int *ticket, AccT *result) {
  extern __shared__ __align__(16) unsigned char thcb_user_smem[];
  AccT *buf = reinterpret_cast<AccT *>(thcb_user_smem);
  AccT acc = init;
  const uint64_t packs = n / V, step = (uint64_t)gridDim.x * kReduceThreads;
  const ValuePack<T, V> *pp = reinterpret_cast<const ValuePack<T, V> *>(in);
  for (uint64_t i0 = (uint64_t)blockIdx.x * kReduceThreads + threadIdx.x; i0 < packs; i0 += step * kLoadsInFlight) {
    ValuePack<T, V> x[kLoadsInFlight];
#pragma unroll
    for (int u = 0; u < kLoadsInFlight; ++u) {
      const uint64_t i = i0 + (uint64_t)u * step;
      if (i < packs) x[u] = pp[i];
    }
#pragma unroll
    for (int u = 0; u < kLoadsInFlight; ++u)
      if (i0 + (uint64_t)u * step < packs) {
#pragma unroll
        for (int j = 0; j < V; ++j) acc = reduceOp(acc, modifyOp(x[u].v[j]));
      }
  }
  if (blockIdx.x == 0)
    for (uint64_t i = packs * V + threadIdx.x; i < n; i += kReduceThreads) acc = reduceOp(acc, modifyOp(in[i]));
  acc = block_fold(acc, buf, accOp);
  __syncthreads();
  reduce_all_finish(acc, buf, partials, ticket, init, accOp, result);
}

// One pinned slot per host thread that the device can write (for results that go to the host): 256
// bytes, allocated on first use and kept.  Null when pinned memory cannot be had.
inline void *host_result_slot() {
  static thread_local void *slot = 0;
  if (!slot && cudaHostAlloc(&slot, 256, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
    cudaGetLastError();
    slot = 0;
  }
  return slot;
}

template <typename TensorType> struct TensorShape;
#define THCB_USER_SHAPE(TENSOR)                                                                       \
  template <> struct TensorShape<TENSOR> {                                                            \
    static void resize(THCState *s, TENSOR *t, THLongStorage *size) { TENSOR##_resize(s, t, size, 0); } \
    static void squeeze1d(THCState *s, TENSOR *t, int dim) { TENSOR##_squeeze1d(s, t, t, dim); }      \
  };
THCB_USER_SHAPE(THCudaByteTensor)
THCB_USER_SHAPE(THCudaCharTensor)
THCB_USER_SHAPE(THCudaShortTensor)
THCB_USER_SHAPE(THCudaIntTensor)
THCB_USER_SHAPE(THCudaLongTensor)
THCB_USER_SHAPE(THCudaHalfTensor)
THCB_USER_SHAPE(THCudaTensor)
THCB_USER_SHAPE(THCudaDoubleTensor)
#undef THCB_USER_SHAPE

}  // namespace thcb_user

template <typename TensorType, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
bool THC_reduceDim(THCState *state, TensorType *out, TensorType *in, const ModifyOp &modifyOp, const ReduceOp &reduceOp,
                   const ReduceAccOp &reduceAccOp, AccT init, int dim, int keepdim) {
  using namespace thcb_user;
  typedef typename TensorAccess<TensorType>::DataType T;
  if (in->nDimension > THCB200_MAX_DIMS || out->nDimension > THCB200_MAX_DIMS) return false;
  if (in->nDimension == 0) return true;
  if (dim < 0 || dim >= in->nDimension) return false;
  // out takes in's sizes with the reduced dim set to 1
  THLongStorage *sizes = THLongStorage_newWithSize(in->nDimension);
  for (int d = 0; d < in->nDimension; ++d) THLongStorage_set(sizes, d, d == dim ? 1 : in->size[d]);
  TensorShape<TensorType>::resize(state, out, sizes);
  THLongStorage_free(sizes);

  SliceView sv;
  sv.n = 0;
  uint64_t nslices = 1;
  for (int d = 0; d < in->nDimension; ++d) {
    if (d == dim || in->size[d] == 1) continue;
    sv.size[sv.n] = (uint64_t)in->size[d];
    sv.in_stride[sv.n] = in->stride[d];
    sv.out_stride[sv.n] = out->stride[d];
    nslices *= (uint64_t)in->size[d];
    ++sv.n;
  }
  const uint64_t K = (uint64_t)in->size[dim];
  const int64_t strideK = in->stride[dim];
  thcb200_tensor din = describe(in), dout = describe(out);
  cudaStream_t st = THCState_getCurrentStream(state);
  bool ok = true;
  // a dense dim other than the reduced one (the innermost such): lanes go along it
  int inner_dim = -1;
  if (strideK != 1)
    for (int d = in->nDimension - 1; d >= 0; --d)
      if (d != dim && in->stride[d] == 1 && in->size[d] >= 32) { inner_dim = d; break; }
  if (nslices > 0 && K > 0 && inner_dim >= 0 && sizeof(AccT) * kReduceThreads <= 48 * 1024) {
    SliceView so;
    so.n = 0;
    uint64_t nouter = 1;
    for (int d = 0; d < in->nDimension; ++d) {
      if (d == dim || d == inner_dim || in->size[d] == 1) continue;
      so.size[so.n] = (uint64_t)in->size[d];
      so.in_stride[so.n] = in->stride[d];
      so.out_stride[so.n] = out->stride[d];
      nouter *= (uint64_t)in->size[d];
      ++so.n;
    }
    const uint64_t inner = (uint64_t)in->size[inner_dim];
    // 16 bytes of neighbouring slices per lane when every row of the walk starts on a 16-byte boundary
    constexpr int VEC = sizeof(T) < 16 ? 16 / (int)sizeof(T) : 1;
    bool vec = VEC > 1 && ((uintptr_t)din.data & 15) == 0 && inner % VEC == 0 && strideK % VEC == 0 &&
               sizeof(AccT) * kReduceThreads * VEC <= 48 * 1024;
    for (int d = 0; d < so.n; ++d)
      if (so.in_stride[d] % VEC != 0) vec = false;
    const uint64_t tiles_i = (inner + 32 * (vec ? VEC : 1) - 1) / (32 * (vec ? VEC : 1));
    // few tiles: the reduced dim is cut into splits (one CTA each) whose partials a second small kernel
    // folds in split order; about eight CTAs per SM in all
    uint64_t nsplit = 1, split_len = K;
    const uint64_t ctas = nouter * tiles_i, want_ctas = 148ull * 8;
    if (ctas < want_ctas && K >= 512) {
      nsplit = want_ctas / ctas;
      if (nsplit > K / 256) nsplit = K / 256;
      if (nsplit < 1) nsplit = 1;
      split_len = (K + nsplit - 1) / nsplit;
      nsplit = (K + split_len - 1) / split_len;
    }
    AccT *partials = 0;
    if (ctas * nsplit >= (1ull << 31)) ok = false;
    if (ok && nsplit > 1 && cudaMallocAsync((void **)&partials, sizeof(AccT) * nouter * nsplit * inner, st) != cudaSuccess) {
      cudaGetLastError();
      ok = false;
    }
    if (ok) {
      if (vec)
        reduce_dim_col_kernel<T, VEC, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<(unsigned)(ctas * nsplit), kReduceThreads,
                                                                             sizeof(AccT) * kReduceThreads * VEC, st>>>(
            (T *)dout.data, (const T *)din.data, so, inner, out->stride[inner_dim], (uint32_t)tiles_i, K, strideK, init, modifyOp,
            reduceOp, reduceAccOp, (uint32_t)nsplit, split_len, partials);
      else
        reduce_dim_col_kernel<T, 1, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<(unsigned)(ctas * nsplit), kReduceThreads,
                                                                           sizeof(AccT) * kReduceThreads, st>>>(
            (T *)dout.data, (const T *)din.data, so, inner, out->stride[inner_dim], (uint32_t)tiles_i, K, strideK, init, modifyOp,
            reduceOp, reduceAccOp, (uint32_t)nsplit, split_len, partials);
      if (nsplit > 1) {
        const uint64_t outs = nouter * inner;
        reduce_dim_col_finish_kernel<T, ReduceAccOp, AccT><<<(unsigned)((outs + kReduceThreads - 1) / kReduceThreads), kReduceThreads, 0, st>>>(
            (T *)dout.data, so, nouter, inner, out->stride[inner_dim], (uint32_t)nsplit, partials, reduceAccOp);
        cudaFreeAsync(partials, st);
      }
    }
  } else if (nslices > 0 && K > 0) {
    // lanes along the reduced dim when it is the dense one or when there are too few slices to
    // fill the GPU with a thread each; otherwise a thread per slice
    const bool cta_per_slice = strideK == 1 || nslices < 148ull * 8 * kReduceThreads / 32;
    if (cta_per_slice && nslices < (1ull << 31)) {
      constexpr int VEC = sizeof(T) < 16 ? 16 / (int)sizeof(T) : 1;
      bool vec = VEC > 1 && strideK == 1 && ((uintptr_t)din.data & 15) == 0 && K >= (uint64_t)VEC * 32;
      for (int d = 0; d < sv.n; ++d)
        if (sv.in_stride[d] % VEC != 0) vec = false;
      int threads = 32;
      while (threads < kReduceThreads && (uint64_t)threads * 4 * (vec ? VEC : 1) < K) threads <<= 1;
      const size_t smem = (size_t)threads * sizeof(AccT);
      // many slices: a warp each, CTAs striding over them; few: a CTA each
      const uint64_t warps_per_cta = kReduceThreads / 32, groups = (nslices + warps_per_cta - 1) / warps_per_cta;
      if (strideK == 1 && nslices >= 148ull * 4 * warps_per_cta) {
        const unsigned grid = (unsigned)(groups < 148ull * 8 ? groups : 148ull * 8);
        if (vec)
          reduce_dim_warp_kernel<T, VEC, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<grid, kReduceThreads, 0, st>>>(
              (T *)dout.data, (const T *)din.data, sv, nslices, K, strideK, init, modifyOp, reduceOp, reduceAccOp);
        else
          reduce_dim_warp_kernel<T, 1, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<grid, kReduceThreads, 0, st>>>(
              (T *)dout.data, (const T *)din.data, sv, nslices, K, strideK, init, modifyOp, reduceOp, reduceAccOp);
      } else if (smem > 48 * 1024) ok = false;
      else if (vec)
        reduce_dim_cta_kernel<T, VEC, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<(unsigned)nslices, threads, smem, st>>>(
            (T *)dout.data, (const T *)din.data, sv, K, strideK, init, modifyOp, reduceOp, reduceAccOp);
      else
        reduce_dim_cta_kernel<T, 1, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<(unsigned)nslices, threads, smem, st>>>(
            (T *)dout.data, (const T *)din.data, sv, K, strideK, init, modifyOp, reduceOp, reduceAccOp);
    } else {
      const uint64_t blocks = (nslices + kReduceThreads - 1) / kReduceThreads;
      if (blocks >= (1ull << 31)) ok = false;
      else
        reduce_dim_thread_kernel<T, ModifyOp, ReduceOp, AccT><<<(unsigned)blocks, kReduceThreads, 0, st>>>(
            (T *)dout.data, (const T *)din.data, sv, nslices, K, strideK, init, modifyOp, reduceOp);
    }
  }
  if (ok && !keepdim) TensorShape<TensorType>::squeeze1d(state, out, dim);
  return ok;
}

template <typename TensorType, typename ModifyOp, typename ReduceOp, typename ReduceAccOp, typename AccT>
bool THC_reduceAll(THCState *state, TensorType *in, const ModifyOp &modifyOp, const ReduceOp &reduceOp,
                   const ReduceAccOp &reduceAccOp, AccT init, AccT *out, int outOnDevice) {
  using namespace thcb_user;
  typedef typename TensorAccess<TensorType>::DataType T;
  if (in->nDimension > THCB200_MAX_DIMS) return false;
  cudaStream_t st = THCState_getCurrentStream(state);
  thcb200_tensor din = describe(in);
  const int64_t n = numel(din);
  if (in->nDimension == 0 || n == 0) {
    if (!outOnDevice) { *out = init; return true; }
    return cudaMemcpyAsync(out, &init, sizeof(AccT), cudaMemcpyHostToDevice, st) == cudaSuccess &&
           cudaStreamSynchronize(st) == cudaSuccess;   // `init` lives on this frame: finish before returning
  }
  if (sizeof(AccT) * kReduceThreads > 48 * 1024) return false;
  uint64_t blocks = ((uint64_t)n + (uint64_t)kReduceThreads * 8 - 1) / ((uint64_t)kReduceThreads * 8);
  const uint64_t cap = 148 * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  // scratch: a ticket, `blocks` partials and one slot for a host result that cannot use the pinned slot
  unsigned char *scratch = 0;
  if (cudaMallocAsync((void **)&scratch, 16 + sizeof(AccT) * (blocks + 1), st) != cudaSuccess) { cudaGetLastError(); return false; }
  unsigned int *ticket = reinterpret_cast<unsigned int *>(scratch);
  AccT *partials = reinterpret_cast<AccT *>(scratch + 16);
  // a host result is written by the finishing CTA straight into pinned host memory when the
  // accumulator fits the thread's slot; otherwise it is copied back from the scratch
  void *slot = (!outOnDevice && sizeof(AccT) <= 256) ? host_result_slot() : 0;
  void *slot_dev = 0;
  if (slot && cudaHostGetDevicePointer(&slot_dev, slot, 0) != cudaSuccess) { cudaGetLastError(); slot = 0; }
  AccT *result = outOnDevice ? out : (slot ? reinterpret_cast<AccT *>(slot_dev) : partials + blocks);
  bool ok = cudaMemsetAsync(ticket, 0, sizeof(unsigned int), st) == cudaSuccess;
  const size_t smem = sizeof(AccT) * kReduceThreads;
  const View<uint64_t> vin = collapse<uint64_t>(din);
  constexpr int VEC = sizeof(T) < 16 ? 16 / (int)sizeof(T) : 1;
  if (VEC > 1 && dense_aligned(vin, din.data))
    reduce_all_dense_kernel<T, VEC, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<(unsigned)blocks, kReduceThreads, smem, st>>>(
        (const T *)din.data, (uint64_t)n, init, modifyOp, reduceOp, reduceAccOp, partials, ticket, result);
  else
    reduce_all_kernel<T, ModifyOp, ReduceOp, ReduceAccOp, AccT><<<(unsigned)blocks, kReduceThreads, smem, st>>>(
        (const T *)din.data, vin, (uint64_t)n, init, modifyOp, reduceOp, reduceAccOp, partials, ticket, result);
  ok = (cudaGetLastError() == cudaSuccess) && ok;
  if (ok && !outOnDevice && !slot) ok = cudaMemcpyAsync(out, result, sizeof(AccT), cudaMemcpyDeviceToHost, st) == cudaSuccess;
  // the scratch is released in stream order; only a host result waits for the stream
  cudaFreeAsync(scratch, st);
  if (!outOnDevice) {
    ok = (cudaStreamSynchronize(st) == cudaSuccess) && ok;
    if (ok && slot) memcpy(out, slot, sizeof(AccT));
  }
  return ok;
}

#endif /* THCB200_THC_REDUCE_CUH */
