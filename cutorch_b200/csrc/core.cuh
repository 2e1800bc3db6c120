// Shared device/host definitions of the B200 apply/reduce core: element-type traits,
// strided-view descriptors passed to kernels by value, fast integer division.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/thcb200.h"

namespace thcb {

constexpr int kMaxDims = THCB200_MAX_DIMS;
constexpr int kNumSM_B200 = 148;

// ---------------------------------------------------------------------------------
// Element-type traits.  Acc is the accumulator of sum/prod reductions: TH's CPU
// tensors (the parity target) accumulate float in double and every integer type in
// 64-bit; half accumulates in float.  Math is the type pointwise arithmetic runs in
// (half -> float, result rounded back once per op: cutorch never defines
// CUDA_HALF_INSTRUCTIONS, lib/THC/THCNumerics.cuh:126-533).
// ---------------------------------------------------------------------------------
template <typename T> struct TypeTraits;
template <> struct TypeTraits<uint8_t> { using Acc = int64_t; using Math = uint8_t; static constexpr int dtype = THCB200_U8; static constexpr bool is_fp = false; };
template <> struct TypeTraits<int8_t>  { using Acc = int64_t; using Math = int8_t;  static constexpr int dtype = THCB200_I8; static constexpr bool is_fp = false; };
template <> struct TypeTraits<int16_t> { using Acc = int64_t; using Math = int16_t; static constexpr int dtype = THCB200_I16; static constexpr bool is_fp = false; };
template <> struct TypeTraits<int32_t> { using Acc = int64_t; using Math = int32_t; static constexpr int dtype = THCB200_I32; static constexpr bool is_fp = false; };
template <> struct TypeTraits<int64_t> { using Acc = int64_t; using Math = int64_t; static constexpr int dtype = THCB200_I64; static constexpr bool is_fp = false; };
template <> struct TypeTraits<__half>  { using Acc = float;   using Math = float;   static constexpr int dtype = THCB200_F16; static constexpr bool is_fp = true; };
template <> struct TypeTraits<float>   { using Acc = double;  using Math = float;   static constexpr int dtype = THCB200_F32; static constexpr bool is_fp = true; };
template <> struct TypeTraits<double>  { using Acc = double;  using Math = double;  static constexpr int dtype = THCB200_F64; static constexpr bool is_fp = true; };

inline size_t dtype_size(int dt) {
  switch (dt) {
    case THCB200_U8: case THCB200_I8: return 1;
    case THCB200_I16: case THCB200_F16: return 2;
    case THCB200_I32: case THCB200_F32: return 4;
    case THCB200_I64: case THCB200_F64: return 8;
  }
  return 0;
}

template <typename T> __host__ __device__ __forceinline__ typename TypeTraits<T>::Math to_math(T v) { return v; }
template <> __host__ __device__ __forceinline__ float to_math<__half>(__half v) { return __half2float(v); }
template <typename T> __host__ __device__ __forceinline__ T from_math(typename TypeTraits<T>::Math v) { return v; }
template <> __host__ __device__ __forceinline__ __half from_math<__half>(float v) { return __float2half_rn(v); }

// ---------------------------------------------------------------------------------
// Division by a run-time constant without a hardware divide: n / d for 32-bit n via a
// 64-bit multiply-high (d in [1, 2^31]).  Used by the index-to-offset walks.
// ---------------------------------------------------------------------------------
struct FastDiv32 {
  uint32_t d, mul, shift;
  FastDiv32() : d(1), mul(0), shift(0) {}
  explicit FastDiv32(uint32_t div) : d(div) {
    // Round-up method (Granlund-Montgomery): shift = ceil(log2 d), mul = floor(2^32 (2^shift - d) / d) + 1
    for (shift = 0; shift < 32; ++shift)
      if ((1ULL << shift) >= div) break;
    uint64_t one = 1;
    mul = (uint32_t)(((one << 32) * ((one << shift) - div)) / div + 1);
  }
  __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
    uint32_t t = __umulhi(n, mul);
#else
    uint32_t t = (uint32_t)(((uint64_t)n * mul) >> 32);
#endif
    return (uint32_t)(((uint64_t)t + n) >> shift);
  }
  // q and r may alias n
  __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t &q, uint32_t &r) const {
    const uint32_t qq = div(n);
    r = n - qq * d;
    q = qq;
  }
};

// ---------------------------------------------------------------------------------
// Strided view handed to the generic kernels (one per operand, individually collapsed
// the way TensorInfo::collapseDims does, lib/THC/THCTensorInfo.cuh:74-224).
// IndexT is uint32_t when both the element count and the largest offset fit, else
// uint64_t (lib/THC/THCTensorTypeUtils.cu:220-245).
// ---------------------------------------------------------------------------------
template <typename IndexT> struct DivHelper;
template <> struct DivHelper<uint32_t> {
  FastDiv32 f;
  DivHelper() {}
  explicit DivHelper(uint64_t d) : f((uint32_t)d) {}
  __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t &q, uint32_t &r) const { f.divmod(n, q, r); }
};
template <> struct DivHelper<uint64_t> {
  uint64_t d;
  DivHelper() : d(1) {}
  explicit DivHelper(uint64_t dd) : d(dd) {}
  __host__ __device__ __forceinline__ void divmod(uint64_t n, uint64_t &q, uint64_t &r) const {
    const uint64_t qq = n / d;
    r = n - qq * d;
    q = qq;
  }
};

constexpr int kGenericDims = 8;  // collapsed dims held inline; deeper views use the spill table

template <typename IndexT>
struct StridedView {
  int dims;                       // 1 and strides[0]==1 -> contiguous
  DivHelper<IndexT> sizes[kGenericDims];
  IndexT strides[kGenericDims];   // element strides (may be "negative" modulo 2^n)

  // logical row-major index -> element offset (lib/THC/THCTensorInfo.cuh:228-278)
  __host__ __device__ __forceinline__ IndexT offset(IndexT linear) const {
    if (dims == 1) return linear * strides[0];
    IndexT off = 0;
#pragma unroll
    for (int i = kGenericDims - 1; i >= 1; --i) {
      if (i < dims) {
        IndexT q, r;
        sizes[i].divmod(linear, q, r);
        off += r * strides[i];
        linear = q;
      }
    }
    return off + linear * strides[0];
  }
};

// a / b for a 32-bit divisor: nothing for b == 1, the 32-bit divide when a fits (a 64-bit
// division is over a hundred instructions on the GPU).
__device__ __forceinline__ uint64_t div_by_u32(uint64_t a, uint32_t b) {
  if (b == 1) return a;
  if ((a >> 32) == 0) return (uint32_t)a / b;
  return a / b;
}

// Host-side plain description of one operand after validation.
struct HostView {
  char *data;
  int dtype;
  int ndim;
  int64_t sizes[kMaxDims];
  int64_t strides[kMaxDims];
  int64_t numel;
};

// ---------------------------------------------------------------------------------
// 16-byte and 32-byte global accesses.  sm_100 has 256-bit ld/st.global; a contiguous
// stream moves one 32-byte sector per thread per instruction with them.
// ---------------------------------------------------------------------------------
struct alignas(16) Bytes16 { uint32_t w[4]; };
struct alignas(32) Bytes32 { uint32_t w[8]; };

__device__ __forceinline__ Bytes16 ld16(const void *p) {
  Bytes16 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
  return v;
}
__device__ __forceinline__ void st16(void *p, const Bytes16 &v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
}
// Streaming variants: data is touched once, keep it from displacing reusable lines.
__device__ __forceinline__ Bytes16 ld16_stream(const void *p) {
  Bytes16 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
  return v;
}
__device__ __forceinline__ Bytes32 ld32_stream(const void *p) {
  Bytes32 v;
  asm volatile("ld.global.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]),
                 "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
  return v;
}
__device__ __forceinline__ void st32(void *p, const Bytes32 &v) {
  asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]),
                  "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7]) : "memory");
}

// Width-generic forms: VecBytes<16> / VecBytes<32> and the matching streaming load / store.
template <int VB> struct VecBytes;
template <> struct VecBytes<16> { using type = Bytes16; };
template <> struct VecBytes<32> { using type = Bytes32; };
template <int VB> __device__ __forceinline__ typename VecBytes<VB>::type ldv_stream(const void *p) {
  if constexpr (VB == 16) return ld16_stream(p); else return ld32_stream(p);
}
template <int VB> __device__ __forceinline__ void stv(void *p, const typename VecBytes<VB>::type &v) {
  if constexpr (VB == 16) st16(p, v); else st32(p, v);
}

// ---------------------------------------------------------------------------------
// Exchange of full-reduction accumulators between the GPUs of a box through peer memory.
// Every rank owns one ExchangeBlock in its device memory, mapped into every other rank
// (cudaIpc between processes, plain peer access inside one).  The CTA that finishes a rank's
// full reduction STORES the rank's 8-byte accumulator and then the call's epoch into its
// column of every rank's block (peer stores over NVLink, no peer loads), waits -- for a
// bounded number of polls -- until its own block holds this epoch from every rank, and folds
// the accumulators in rank order: the reduction and its all-reduce are one kernel, and every
// rank computes the same bits.  Two parities alternate, so a rank that runs ahead by one call
// does not overwrite what a slower rank is still reading.
// ---------------------------------------------------------------------------------
constexpr int kMaxPeers = 16;
struct ExchangeBlock {
  unsigned long long slot[2][kMaxPeers];   // [parity][writer rank]: accumulator bits (double or int64)
  unsigned int flag[2][kMaxPeers];         // [parity][writer rank]: epoch of the call that wrote the slot
};
struct PeerExchange {
  int nranks;                 // 0 or 1: no exchange
  int rank;
  unsigned int epoch;         // grows by one per call, never 0
  unsigned int max_polls;     // per awaited rank; the wait gives up after that and sets *status
  int fold;                   // THCB200_RED_SUM / PROD / MIN / MAX
  int is_fp;                  // slots hold doubles (else int64)
  int *status;                // device word, set to 1 when a wait ran out
  ExchangeBlock *block[kMaxPeers];   // block[r]: rank r's block as this process addresses it
};

// ---------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the library starts with pdl_prologue() and is
// launched through launch_pdl(): the launch carries the programmatic-stream-serialization
// attribute, so the GPU may make the kernel's CTAs resident while the previous kernel of the stream
// is still running its tail, and the launch latency and ramp of one call overlap the end of the
// one before.  griddepcontrol.launch_dependents lets the NEXT kernel's CTAs come in as soon as all of
// this kernel's CTAs have started; griddepcontrol.wait returns once every earlier kernel of the
// stream has completed and its writes are visible, so it stands before the first access to global
// memory (arguments arrive with the launch and need no wait).  Under a plain launch both are no-ops.
// THCB200_PDL=0 in the environment turns the attribute off (plain stream order).
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

bool pdl_enabled();   // plan.cu: reads THCB200_PDL once

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace thcb
