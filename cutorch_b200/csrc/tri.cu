// tril / triu of a matrix view: out[r][c] = keep(r, c) ? in[r][c] : 0 with
// keep = (c - r <= k) for the lower and (c - r >= k) for the upper triangle
// (TensorTriOp, lib/THC/THCTensorMathPairwise.cu:373-406; entry points
// lib/THC/generic/THCTensorMathPairwise.cu:169-233).  The reference recovers (r, c) from pointer
// differences inside a generic apply; here the kernel walks the matrix by coordinates with lanes
// along whichever dim has the smaller output stride, and elements outside the triangle are not
// read at all (they cost the 0 store only).
#include <string.h>

#include "context.h"
#include "core.cuh"
#include "plan.h"

namespace thcb {
namespace {

constexpr int kTriThreads = 256;
constexpr int kTriUnroll = 4;

// fast dim f (lanes), slow dim s.  row_is_fast tells which of them is the matrix row.
template <typename W>
__global__ void __launch_bounds__(kTriThreads)
tri_kernel(W *out, const W *in, uint64_t nfast, uint64_t nslow, int64_t of, int64_t os, int64_t inf, int64_t ins,
           int64_t k, int upper, int row_is_fast, uint32_t tiles_f) {
  const uint64_t slow = blockIdx.x / tiles_f;
  const uint64_t f0 = (uint64_t)(blockIdx.x - slow * tiles_f) * (kTriThreads * kTriUnroll) + threadIdx.x;
  W x[kTriUnroll];
  bool keep[kTriUnroll];
#pragma unroll
  for (int u = 0; u < kTriUnroll; ++u) {
    const uint64_t f = f0 + (uint64_t)u * kTriThreads;
    const int64_t r = row_is_fast ? (int64_t)f : (int64_t)slow;
    const int64_t c = row_is_fast ? (int64_t)slow : (int64_t)f;
    keep[u] = f < nfast && (upper ? (c - r >= k) : (c - r <= k));
    x[u] = W(0);
    if (keep[u]) x[u] = in[(int64_t)f * inf + (int64_t)slow * ins];
  }
#pragma unroll
  for (int u = 0; u < kTriUnroll; ++u) {
    const uint64_t f = f0 + (uint64_t)u * kTriThreads;
    if (f < nfast) out[(int64_t)f * of + (int64_t)slow * os] = x[u];
  }
}

template <typename W>
int launch_tri(const HostView &vo, const HostView &vi, int64_t k, int upper, cudaStream_t st) {
  // lanes along the dim where the output's stride is smaller in magnitude
  auto mag = [](int64_t s) { return s < 0 ? -s : s; };
  const int fast = mag(vo.strides[1]) <= mag(vo.strides[0]) ? 1 : 0;
  const int slow = 1 - fast;
  const uint64_t nfast = (uint64_t)vo.sizes[fast], nslow = (uint64_t)vo.sizes[slow];
  const uint64_t tiles_f = (nfast + kTriThreads * kTriUnroll - 1) / (kTriThreads * kTriUnroll);
  const uint64_t blocks = tiles_f * nslow;
  if (blocks >= (1ull << 31) || tiles_f >= (1ull << 31)) { set_error("tri: matrix too large"); return THCB200_ERR_DIMS; }
  set_plan_name(fast == 1 ? "tri_rows" : "tri_cols");
  tri_kernel<W><<<(unsigned)blocks, kTriThreads, 0, st>>>(reinterpret_cast<W *>(vo.data), reinterpret_cast<const W *>(vi.data),
                                                          nfast, nslow, vo.strides[fast], vo.strides[slow], vi.strides[fast],
                                                          vi.strides[slow], k, upper, fast == 0 ? 1 : 0, (uint32_t)tiles_f);
  count_launch();
  THCB_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" int thcb200_tri(thcb200_ctx *ctx, int upper, int64_t k, const thcb200_tensor *out, const thcb200_tensor *in,
                           void *stream) {
  if (!ctx) { set_error("tri: null context"); return THCB200_ERR_ARG; }
  HostView vo, vi;
  int rc = to_host_view(out, &vo, "tri output");
  if (!rc) rc = to_host_view(in, &vi, "tri input");
  if (rc) return rc;
  if (vi.ndim != 2 || vo.ndim != 2) { set_error("tri: expected a matrix"); return THCB200_ERR_ARG; }
  if (vi.dtype != vo.dtype) { set_error("tri: operands have different dtypes"); return THCB200_ERR_ARG; }
  if (vi.sizes[0] != vo.sizes[0] || vi.sizes[1] != vo.sizes[1]) { set_error("tri: output and input have different shapes"); return THCB200_ERR_SIZE; }
  if (vi.numel == 0) return THCB200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype_size(vi.dtype)) {
    case 1: return launch_tri<uint8_t>(vo, vi, k, upper, st);
    case 2: return launch_tri<uint16_t>(vo, vi, k, upper, st);
    case 4: return launch_tri<uint32_t>(vo, vi, k, upper, st);
    default: return launch_tri<uint64_t>(vo, vi, k, upper, st);
  }
}
