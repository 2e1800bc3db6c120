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
constexpr int kTriUnroll = 4;   // fast-dim elements per thread
constexpr int kTriRows = 8;     // slow-dim lines per CTA

// fast dim f (lanes), slow dim s.  row_is_fast tells which of them is the matrix row.
// A CTA covers kTriThreads * kTriUnroll positions of the fast dim on kTriRows lines of the slow one.
template <typename W>
__global__ void __launch_bounds__(kTriThreads)
tri_kernel(W *out, const W *in, uint64_t nfast, uint64_t nslow, int64_t of, int64_t os, int64_t inf, int64_t ins,
           int64_t k, int upper, int row_is_fast, uint32_t tiles_f) {
  pdl_prologue();
  const uint64_t stile = blockIdx.x / tiles_f;
  const uint64_t f0 = (uint64_t)(blockIdx.x - stile * tiles_f) * (kTriThreads * kTriUnroll) + threadIdx.x;
  // two lines at a time: all of their loads are issued before the first store (out may be in)
  for (int line = 0; line < kTriRows; line += 2) {
    W x[2][kTriUnroll];
#pragma unroll
    for (int l = 0; l < 2; ++l) {
      const uint64_t slow = stile * kTriRows + line + l;
#pragma unroll
      for (int u = 0; u < kTriUnroll; ++u) {
        const uint64_t f = f0 + (uint64_t)u * kTriThreads;
        const int64_t r = row_is_fast ? (int64_t)f : (int64_t)slow;
        const int64_t c = row_is_fast ? (int64_t)slow : (int64_t)f;
        const bool keep = slow < nslow && f < nfast && (upper ? (c - r >= k) : (c - r <= k));
        x[l][u] = W(0);
        if (keep) x[l][u] = in[(int64_t)f * inf + (int64_t)slow * ins];
      }
    }
#pragma unroll
    for (int l = 0; l < 2; ++l) {
      const uint64_t slow = stile * kTriRows + line + l;
#pragma unroll
      for (int u = 0; u < kTriUnroll; ++u) {
        const uint64_t f = f0 + (uint64_t)u * kTriThreads;
        if (slow < nslow && f < nfast) out[(int64_t)f * of + (int64_t)slow * os] = x[l][u];
      }
    }
  }
}

// Rows with unit stride in both tensors, 16-byte aligned: a thread moves whole 16-byte vectors
// (V elements); a vector entirely outside the triangle is stored as zeros without being read.
template <typename W>
__global__ void __launch_bounds__(kTriThreads)
tri_vec_kernel(W *out, const W *in, uint64_t ncols, uint64_t nrows, int64_t orow, int64_t irow, int64_t k, int upper,
               uint32_t tiles_f) {
  pdl_prologue();
  constexpr int V = 16 / (int)sizeof(W);
  const uint64_t nvec = ncols / V;   // ncols is a multiple of V
  const uint64_t stile = blockIdx.x / tiles_f;
  const uint64_t v0 = (uint64_t)(blockIdx.x - stile * tiles_f) * (kTriThreads * kTriUnroll) + threadIdx.x;
  for (int line = 0; line < kTriRows; line += 2) {
    Bytes16 x[2][kTriUnroll];
#pragma unroll
    for (int l = 0; l < 2; ++l) {
      const uint64_t r = stile * kTriRows + line + l;
#pragma unroll
      for (int u = 0; u < kTriUnroll; ++u) {
        const uint64_t v = v0 + (uint64_t)u * kTriThreads;
        const int64_t c0 = (int64_t)(v * V);
        // d = column - row - k of the vector's first element; element j is kept when d + j >= 0
        // (upper) or d + j <= 0 (lower)
        const int64_t d = c0 - (int64_t)r - k;
        const bool inside = r < nrows && v < nvec;
        const bool any = inside && (upper ? d + (V - 1) >= 0 : d <= 0);
        const bool all = upper ? d >= 0 : d + (V - 1) <= 0;
        x[l][u] = Bytes16();
        if (any) {
          x[l][u] = ld16_stream(in + (int64_t)r * irow + c0);
          if (!all) {
            W *e = reinterpret_cast<W *>(&x[l][u]);
            const int dd = (int)d;   // |d| < V here
#pragma unroll
            for (int j = 0; j < V; ++j)
              if (!(upper ? dd + j >= 0 : dd + j <= 0)) e[j] = W(0);
          }
        }
      }
    }
#pragma unroll
    for (int l = 0; l < 2; ++l) {
      const uint64_t r = stile * kTriRows + line + l;
#pragma unroll
      for (int u = 0; u < kTriUnroll; ++u) {
        const uint64_t v = v0 + (uint64_t)u * kTriThreads;
        if (r < nrows && v < nvec) st16(out + (int64_t)r * orow + (int64_t)(v * V), x[l][u]);
      }
    }
  }
}

template <typename W>
int launch_tri(const HostView &vo, const HostView &vi, int64_t k, int upper, cudaStream_t st) {
  constexpr int V = 16 / (int)sizeof(W);
  W *op = reinterpret_cast<W *>(vo.data);
  const W *ip = reinterpret_cast<const W *>(vi.data);
  if (V > 1 && vo.strides[1] == 1 && vi.strides[1] == 1 && vo.sizes[1] % V == 0 && vo.strides[0] % V == 0 &&
      vi.strides[0] % V == 0 && (uintptr_t)op % 16 == 0 && (uintptr_t)ip % 16 == 0) {
    const uint64_t nvec = (uint64_t)vo.sizes[1] / V;
    const uint64_t tiles_f = (nvec + kTriThreads * kTriUnroll - 1) / (kTriThreads * kTriUnroll);
    const uint64_t blocks = tiles_f * (((uint64_t)vo.sizes[0] + kTriRows - 1) / kTriRows);
    if (blocks >= (1ull << 31)) { set_error("tri: matrix too large"); return THCB200_ERR_DIMS; }
    set_plan_name("tri_rows_vec");
    launch_pdl(tri_vec_kernel<W>, (unsigned)blocks, kTriThreads, 0, st, op, ip, (uint64_t)vo.sizes[1], (uint64_t)vo.sizes[0],
                                                                vo.strides[0], vi.strides[0], k, upper, (uint32_t)tiles_f);
    count_launch();
    THCB_CUDA_TRY(cudaGetLastError());
    return 0;
  }
  // lanes along the dim where the output's stride is smaller in magnitude
  auto mag = [](int64_t s) { return s < 0 ? -s : s; };
  const int fast = mag(vo.strides[1]) <= mag(vo.strides[0]) ? 1 : 0;
  const int slow = 1 - fast;
  const uint64_t nfast = (uint64_t)vo.sizes[fast], nslow = (uint64_t)vo.sizes[slow];
  const uint64_t tiles_f = (nfast + kTriThreads * kTriUnroll - 1) / (kTriThreads * kTriUnroll);
  const uint64_t blocks = tiles_f * ((nslow + kTriRows - 1) / kTriRows);
  if (blocks >= (1ull << 31) || tiles_f >= (1ull << 31)) { set_error("tri: matrix too large"); return THCB200_ERR_DIMS; }
  set_plan_name(fast == 1 ? "tri_rows" : "tri_cols");
  launch_pdl(tri_kernel<W>, (unsigned)blocks, kTriThreads, 0, st, op, ip, nfast, nslow, vo.strides[fast], vo.strides[slow],
                                                          vi.strides[fast], vi.strides[slow], k, upper, fast == 0 ? 1 : 0,
                                                          (uint32_t)tiles_f);
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
