// Type-converting element-wise copy between any two element types (C cast semantics, half
// through float): the CopyOp path of THC_copyTensor (lib/THC/THCTensorCopy.cu:12-21,114-121).
#include "apply.cuh"
#include "context.h"
#include "plan.h"

namespace thcb {
namespace {

template <typename TO, typename TI> __device__ __forceinline__ TO convert_elem(TI v) {
  if constexpr (std::is_same<TI, __half>::value) {
    if constexpr (std::is_same<TO, __half>::value) return v;
    else return (TO)__half2float(v);
  } else if constexpr (std::is_same<TO, __half>::value) {
    return __float2half_rn((float)v);
  } else {
    return (TO)v;
  }
}

template <typename TO, typename TI, typename IndexT>
__global__ void __launch_bounds__(kApplyThreads)
convert_kernel(TO *out, StridedView<IndexT> vo, const TI *in, StridedView<IndexT> vi, IndexT n) {
  pdl_prologue();
  constexpr int U = kApplyUnroll;
  const IndexT base = (IndexT)blockIdx.x * (IndexT)(kApplyThreads * U) + threadIdx.x;
  TI x[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const IndexT i = base + (IndexT)u * kApplyThreads;
    if (i < n) x[u] = in[vi.offset(i)];
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const IndexT i = base + (IndexT)u * kApplyThreads;
    if (i < n) out[vo.offset(i)] = convert_elem<TO, TI>(x[u]);
  }
}

template <typename TO, typename TI>
int launch_convert(const ApplyPlan &plan, void *out, const void *in, cudaStream_t st) {
  const uint64_t n = plan.numel;
  const uint64_t tile = (uint64_t)kApplyThreads * kApplyUnroll;
  const uint64_t blocks = (n + tile - 1) / tile;
  if (blocks >= (1ULL << 31)) { set_error("copy: tensor too large"); return THCB200_ERR_DIMS; }
  if (!plan.index64) {
    launch_pdl(convert_kernel<TO, TI, uint32_t>, (unsigned)blocks, kApplyThreads, 0, st, 
        (TO *)out, to_strided_view<uint32_t>(plan, 0), (const TI *)in, to_strided_view<uint32_t>(plan, 1), (uint32_t)n);
  } else {
    launch_pdl(convert_kernel<TO, TI, uint64_t>, (unsigned)blocks, kApplyThreads, 0, st, 
        (TO *)out, to_strided_view<uint64_t>(plan, 0), (const TI *)in, to_strided_view<uint64_t>(plan, 1), (uint64_t)n);
  }
  count_launch();
  set_plan_name("convert");
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

template <typename TO>
int convert_from(int in_dtype, const ApplyPlan &plan, void *out, const void *in, cudaStream_t st) {
  switch (in_dtype) {
    case THCB200_U8: return launch_convert<TO, uint8_t>(plan, out, in, st);
    case THCB200_I8: return launch_convert<TO, int8_t>(plan, out, in, st);
    case THCB200_I16: return launch_convert<TO, int16_t>(plan, out, in, st);
    case THCB200_I32: return launch_convert<TO, int32_t>(plan, out, in, st);
    case THCB200_I64: return launch_convert<TO, int64_t>(plan, out, in, st);
    case THCB200_F16: return launch_convert<TO, __half>(plan, out, in, st);
    case THCB200_F32: return launch_convert<TO, float>(plan, out, in, st);
    default: return launch_convert<TO, double>(plan, out, in, st);
  }
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" THCB200_API int thcb200_copy_convert(thcb200_ctx *ctx, const thcb200_tensor *out, const thcb200_tensor *in,
                                                void *stream) {
  if (!ctx) { set_error("copy_convert: null context"); return THCB200_ERR_ARG; }
  HostView v[2];
  int rc = to_host_view(out, &v[0], "copy_convert output");
  if (rc) return rc;
  rc = to_host_view(in, &v[1], "copy_convert input");
  if (rc) return rc;
  if (v[0].numel != v[1].numel) { set_error("copy_convert: operands have different element counts"); return THCB200_ERR_SIZE; }
  if (v[0].numel == 0) return THCB200_OK;
  ApplyPlan plan;
  // element size 0: never pick the vector or tiled forms, the two element sizes differ
  make_apply_plan(v, 2, 0, &plan);
  if (plan.kind == kApplyDeep) { set_error("copy_convert: more than %d non-collapsible dimensions", kGenericDims); return THCB200_ERR_DIMS; }
  cudaStream_t st = (cudaStream_t)stream;
  switch (v[0].dtype) {
    case THCB200_U8: return convert_from<uint8_t>(v[1].dtype, plan, v[0].data, v[1].data, st);
    case THCB200_I8: return convert_from<int8_t>(v[1].dtype, plan, v[0].data, v[1].data, st);
    case THCB200_I16: return convert_from<int16_t>(v[1].dtype, plan, v[0].data, v[1].data, st);
    case THCB200_I32: return convert_from<int32_t>(v[1].dtype, plan, v[0].data, v[1].data, st);
    case THCB200_I64: return convert_from<int64_t>(v[1].dtype, plan, v[0].data, v[1].data, st);
    case THCB200_F16: return convert_from<__half>(v[1].dtype, plan, v[0].data, v[1].data, st);
    case THCB200_F32: return convert_from<float>(v[1].dtype, plan, v[0].data, v[1].data, st);
    default: return convert_from<double>(v[1].dtype, plan, v[0].data, v[1].data, st);
  }
}
