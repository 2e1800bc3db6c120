// Copies between a tensor in host memory and a tensor in device memory, with type conversion and
// any strides on both sides: what cutorch's :cuda(), :float() and copy between CPU and GPU tensors
// come down to (lib/THC/generic/THCTensorCopy.c:7-164).
//
// The reference makes both sides contiguous and of one type on the CPU (TH's strided, converting
// copy loops) and then issues one cudaMemcpy.  Here the host only hands over bytes:
//  * a host view that is one dense run crosses the bus as it is;
//  * a strided host view (transposed, permuted, rows with padding) crosses as the span of memory it
//    covers, and the device kernels walk that span with the host view's own strides, as long as
//    the span is at most about twice the view's bytes (a transposed 16384 x 16384 float matrix
//    packed by one host thread takes 4.3 s; its span crosses in 20 ms);
//  * only views that are sparse in their span (a column of a wide matrix) are packed on the host.
// Striding on the device side and the type conversion are always done by the device kernels
// (thcb200_copy_convert / thcb200_pointwise).  Both calls return when the copy is complete, as the
// reference's do.
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

// The span of host memory a view with non-negative strides covers, in elements from its first one,
// and whether shipping that span instead of packed elements is worth it.
int64_t span_elems(const HostView &v) {
  int64_t hi = 0;
  for (int d = 0; d < v.ndim; ++d) hi += (v.sizes[d] - 1) * v.strides[d];
  return hi + 1;
}
bool ship_span(const HostView &v) { return span_elems(v) <= 2 * v.numel + (1 << 18); }

thcb200_tensor span_desc(void *data, const HostView &v) {
  thcb200_tensor t;
  memset(&t, 0, sizeof(t));
  t.data = data;
  t.dtype = v.dtype;
  t.ndim = v.ndim;
  for (int d = 0; d < v.ndim; ++d) { t.sizes[d] = v.sizes[d]; t.strides[d] = v.strides[d]; }
  return t;
}

int device_copy(thcb200_ctx *ctx, const thcb200_tensor *out, const thcb200_tensor *in, void *stream) {
  return out->dtype == in->dtype ? thcb200_pointwise(ctx, THCB200_OP_COPY, out, in, nullptr, nullptr, 1, thcb200_scalar{0.0, 0},
                                                     thcb200_scalar{0.0, 0}, stream)
                                 : thcb200_copy_convert(ctx, out, in, stream);
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
  if (!ps.dense && ship_span(vs)) {
    // the span the view covers goes up as it is; the device walks it with the view's strides
    const size_t span_bytes = (size_t)span_elems(vs) * esz;
    void *tmp = nullptr;
    cudaError_t e = device_alloc_async(&tmp, span_bytes, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, vs.data, span_bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
      thcb200_tensor up = span_desc(tmp, vs);
      rc = device_copy(ctx, dst, &up, stream);
    }
    if (tmp) cudaFreeAsync(tmp, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { set_error("copy_from_host: %s", cudaGetErrorString(e)); return THCB200_ERR_CUDA; }
    return rc;
  }
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
    e = device_alloc_async(&tmp, bytes, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, wire, bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
      thcb200_tensor dense = dense_desc(tmp, vs.dtype, vs.numel);
      rc = device_copy(ctx, dst, &dense, stream);
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
  if (!pd.dense && ship_span(vd) && !overlapping_indices(vd)) {
    // The device lays the elements out with the host view's strides inside a copy of the span the
    // view covers, and the span goes down in one piece.  Where the view leaves gaps in its span,
    // the span is fetched first so that the gaps go back unchanged.
    const int64_t span = span_elems(vd);
    const size_t span_bytes = (size_t)span * esz;
    void *tmp = nullptr;
    cudaError_t e = device_alloc_async(&tmp, span_bytes, st);
    if (e == cudaSuccess && span != vd.numel) e = cudaMemcpyAsync(tmp, vd.data, span_bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
      thcb200_tensor down = span_desc(tmp, vd);
      rc = device_copy(ctx, &down, src, stream);
      if (rc == 0) e = cudaMemcpyAsync(vd.data, tmp, span_bytes, cudaMemcpyDeviceToHost, st);
    }
    if (tmp) cudaFreeAsync(tmp, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { set_error("copy_to_host: %s", cudaGetErrorString(e)); return THCB200_ERR_CUDA; }
    return rc;
  }
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
    e = device_alloc_async(&tmp, bytes, st);
    if (e == cudaSuccess) {
      thcb200_tensor dense = dense_desc(tmp, vd.dtype, vd.numel);
      rc = device_copy(ctx, &dense, src, stream);
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
