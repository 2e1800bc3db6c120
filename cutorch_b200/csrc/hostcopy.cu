// Copies between a tensor in host memory and a tensor in device memory, with type conversion and
// any strides on both sides: what cutorch's :cuda(), :float() and copy between CPU and GPU tensors
// come down to (lib/THC/generic/THCTensorCopy.c:7-164).
//
// The reference makes both sides contiguous and of one type on the CPU (TH's strided, converting
// copy loops) and then issues one cudaMemcpy.  Here the host does only what it must: when the host
// view is one dense run its bytes cross the bus as they are, otherwise its runs are packed into a
// dense buffer first.  Striding on the device side and the type conversion are done by the device
// kernels (thcb200_copy_convert / thcb200_pointwise) from or into a dense device temporary of the
// host side's element type, which is skipped when the device side is dense and of the same type.
// Both calls return when the copy is complete, as the reference's do.
#include <stdlib.h>
#include <string.h>

#include "context.h"
#include "core.cuh"
#include "plan.h"

namespace thcb {
namespace {

// The view with size-1 dims dropped and neighbouring dims merged; `dense` when it is one run of
// numel elements in logical order.
struct PackedHostView {
  int nd;
  int64_t sizes[kMaxDims], strides[kMaxDims];
  bool dense;
};

PackedHostView pack_view(const HostView &v) {
  PackedHostView p;
  p.nd = v.ndim;
  for (int d = 0; d < v.ndim; ++d) { p.sizes[d] = v.sizes[d]; p.strides[d] = v.strides[d]; }
  if (p.nd == 0) { p.nd = 1; p.sizes[0] = 1; p.strides[0] = 1; }
  collapse_dims(p.sizes, p.strides, &p.nd, -1);
  p.dense = p.nd == 1 && (p.sizes[0] == 1 || p.strides[0] == 1);
  return p;
}

// Walks the runs of the innermost dim in logical order.  GATHER: strided -> dense, else dense -> strided.
template <bool GATHER>
void host_move(const PackedHostView &p, char *strided, char *dense, size_t esz) {
  const int L = p.nd - 1;
  const int64_t run = p.sizes[L], rs = p.strides[L];
  int64_t idx[kMaxDims] = {0};
  int64_t off = 0;
  for (;;) {
    char *s = strided + off * (int64_t)esz;
    if (rs == 1) {
      if (GATHER) memcpy(dense, s, (size_t)run * esz); else memcpy(s, dense, (size_t)run * esz);
    } else {
      for (int64_t i = 0; i < run; ++i) {
        if (GATHER) memcpy(dense + (size_t)i * esz, s + i * rs * (int64_t)esz, esz);
        else memcpy(s + i * rs * (int64_t)esz, dense + (size_t)i * esz, esz);
      }
    }
    dense += (size_t)run * esz;
    int d = L - 1;
    for (; d >= 0; --d) {
      off += p.strides[d];
      if (++idx[d] < p.sizes[d]) break;
      off -= p.strides[d] * p.sizes[d];
      idx[d] = 0;
    }
    if (d < 0) break;
  }
}

thcb200_tensor dense_desc(void *data, int dtype, int64_t numel) {
  thcb200_tensor t;
  memset(&t, 0, sizeof(t));
  t.data = data;
  t.dtype = dtype;
  t.ndim = 1;
  t.sizes[0] = numel;
  t.strides[0] = 1;
  return t;
}

bool host_view_ok(const HostView &v, const char *what) {
  for (int d = 0; d < v.ndim; ++d)
    if (v.strides[d] < 0) { set_error("%s: negative strides are not supported on the host side", what); return false; }
  return true;
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" THCB200_API int thcb200_copy_from_host(thcb200_ctx *ctx, const thcb200_tensor *dst, const thcb200_tensor *src_host,
                                                  void *stream) {
  if (!ctx) { set_error("copy_from_host: null context"); return THCB200_ERR_ARG; }
  HostView vd, vs;
  int rc = to_host_view(dst, &vd, "copy_from_host destination");
  if (!rc) rc = to_host_view(src_host, &vs, "copy_from_host source");
  if (rc) return rc;
  if (vd.numel != vs.numel) { set_error("copy_from_host: operands have different element counts"); return THCB200_ERR_SIZE; }
  if (vd.numel == 0) return THCB200_OK;
  if (!host_view_ok(vs, "copy_from_host")) return THCB200_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = dtype_size(vs.dtype);
  const size_t bytes = (size_t)vs.numel * esz;
  const PackedHostView ps = pack_view(vs), pd = pack_view(vd);
  // the bytes that cross the bus, in logical order
  char *packed = nullptr;
  const char *wire = vs.data;
  if (!ps.dense) {
    packed = (char *)malloc(bytes);
    if (!packed) { set_error("copy_from_host: out of host memory"); return THCB200_ERR_NOMEM; }
    host_move<true>(ps, vs.data, packed, esz);
    wire = packed;
  }
  cudaError_t e;
  if (pd.dense && vd.dtype == vs.dtype) {
    e = cudaMemcpyAsync(vd.data, wire, bytes, cudaMemcpyHostToDevice, st);
  } else {
    void *tmp = nullptr;
    e = cudaMallocAsync(&tmp, bytes, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, wire, bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
      thcb200_tensor dense = dense_desc(tmp, vs.dtype, vs.numel);
      rc = vd.dtype == vs.dtype ? thcb200_pointwise(ctx, THCB200_OP_COPY, dst, &dense, nullptr, nullptr, 1, thcb200_scalar{0.0, 0}, thcb200_scalar{0.0, 0}, stream)
                                : thcb200_copy_convert(ctx, dst, &dense, stream);
    }
    if (tmp) cudaFreeAsync(tmp, st);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  free(packed);
  if (e != cudaSuccess) { set_error("copy_from_host: %s", cudaGetErrorString(e)); return THCB200_ERR_CUDA; }
  return rc;
}

extern "C" THCB200_API int thcb200_copy_to_host(thcb200_ctx *ctx, const thcb200_tensor *dst_host, const thcb200_tensor *src,
                                                void *stream) {
  if (!ctx) { set_error("copy_to_host: null context"); return THCB200_ERR_ARG; }
  HostView vd, vs;
  int rc = to_host_view(dst_host, &vd, "copy_to_host destination");
  if (!rc) rc = to_host_view(src, &vs, "copy_to_host source");
  if (rc) return rc;
  if (vd.numel != vs.numel) { set_error("copy_to_host: operands have different element counts"); return THCB200_ERR_SIZE; }
  if (vd.numel == 0) return THCB200_OK;
  if (!host_view_ok(vd, "copy_to_host")) return THCB200_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = dtype_size(vd.dtype);
  const size_t bytes = (size_t)vd.numel * esz;
  const PackedHostView pd = pack_view(vd), ps = pack_view(vs);
  char *packed = nullptr;
  char *wire = vd.data;
  if (!pd.dense) {
    packed = (char *)malloc(bytes);
    if (!packed) { set_error("copy_to_host: out of host memory"); return THCB200_ERR_NOMEM; }
    wire = packed;
  }
  cudaError_t e = cudaSuccess;
  void *tmp = nullptr;
  if (ps.dense && vd.dtype == vs.dtype) {
    e = cudaMemcpyAsync(wire, vs.data, bytes, cudaMemcpyDeviceToHost, st);
  } else {
    // the device packs (and converts) into a dense temporary of the host side's type
    e = cudaMallocAsync(&tmp, bytes, st);
    if (e == cudaSuccess) {
      thcb200_tensor dense = dense_desc(tmp, vd.dtype, vd.numel);
      rc = vd.dtype == vs.dtype ? thcb200_pointwise(ctx, THCB200_OP_COPY, &dense, src, nullptr, nullptr, 1, thcb200_scalar{0.0, 0}, thcb200_scalar{0.0, 0}, stream)
                                : thcb200_copy_convert(ctx, &dense, src, stream);
      if (rc == 0) e = cudaMemcpyAsync(wire, tmp, bytes, cudaMemcpyDeviceToHost, st);
    }
    if (tmp) cudaFreeAsync(tmp, st);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e == cudaSuccess && rc == 0 && packed) host_move<false>(pd, vd.data, packed, esz);
  free(packed);
  if (e != cudaSuccess) { set_error("copy_to_host: %s", cudaGetErrorString(e)); return THCB200_ERR_CUDA; }
  return rc;
}
