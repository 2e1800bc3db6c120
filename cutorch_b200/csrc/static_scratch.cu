// thcb200_reduce_dim_static: the dimension reduction for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a reduction:
// code that runs after an application has handed every byte of device memory to its own
// pool, a plug-in whose contract forbids allocations after start-up, or a tight loop that
// cannot afford the implicit device synchronisation an allocation may bring.  The regular
// entry point keeps its split-reduction partials in a per-context workspace that it grows
// with cudaMalloc on demand; this variant keeps them in a fixed array that is part of the
// library image instead, so a call never allocates (no cudaMalloc/cudaFree, no context, no
// allocating library routine).
//
// The price: every GPU on which this library is loaded holds THCB200_STATIC_SCRATCH_BYTES for
// the life of the process, a reduction whose partials do not fit is refused, and all calls on
// one device share the one array.
#include <mutex>

#include "context.h"
#include "plan.h"
#include "reduce_launch.cuh"

namespace {

// Partial accumulators of split reductions ([output][split], kPartialSlotBytes each).  Device code may
// name this array directly; host code may not use the name as an address (on the host it is
// only a handle for cudaGetSymbolAddress), so the launches below receive g_scratch_dev[device].
static __device__ __align__(256) unsigned char g_static_scratch[THCB200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void *g_scratch_dev[kMaxDevices];  // device address of g_static_scratch, per device
int g_num_sms[kMaxDevices];
int g_setup_rc[kMaxDevices];
// The first call on a device, from whichever host thread, runs the set-up; every other caller
// waits for it and then sees what it published (std::call_once allocates nothing).
std::once_flag g_once[kMaxDevices];

// Once per device, with that device current.
int setup_device_once(int device) {
  void *p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
  if (e != cudaSuccess || !p) {
    cudaGetLastError();
    thcb::set_error("reduce_dim_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    return THCB200_ERR_CUDA;
  }
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) {
    cudaGetLastError();
    thcb::set_error("reduce_dim_static: cannot query the device: %s", cudaGetErrorString(e));
    return THCB200_ERR_CUDA;
  }
  g_scratch_dev[device] = p;
  g_num_sms[device] = sms;
  return 0;
}

int setup_device(int device) {
  std::call_once(g_once[device], [device] { g_setup_rc[device] = setup_device_once(device); });
  if (g_setup_rc[device]) thcb::set_error("reduce_dim_static: the set-up of device %d failed on its first call", device);
  return g_setup_rc[device];
}

}  // namespace

using namespace thcb;

// Same contract and results as thcb200_reduce_dim (the same kernels run), but without a
// context and without any allocation.
//  * The first call on a device looks up the device address of the scratch array (and, with
//    CUDA's lazy module loading, is the moment the runtime places the library's device code and
//    this array on that GPU: the free memory cudaMemGetInfo reports drops by the array's size
//    then, once).  Make that first call at start-up, outside any stream capture; every later
//    call leaves the device's memory as it found it.
//  * A reduction that needs more than THCB200_STATIC_SCRATCH_BYTES of partials is refused with
//    THCB200_ERR_LIMIT (only reductions that are split along the reduced dim need partials at
//    all; the others always pass).
//  * All calls on a device share the array and it keeps the previous call's contents.  Nothing
//    in it has to start at zero -- every slot a call reads was written earlier in that call --
//    but two calls that overlap on the GPU (different streams, or threads racing on one
//    device) would overwrite each other's partials: serialise them.
extern "C" THCB200_API int thcb200_reduce_dim_static(int rop, int pre, thcb200_scalar s, const thcb200_tensor *out,
                                                     const thcb200_tensor *in, int dim, void *stream) {
  HostView vin, vout;
  int rc = to_host_view(in, &vin, "reduce_dim_static input");
  if (rc) return rc;
  rc = to_host_view(out, &vout, "reduce_dim_static output");
  if (rc) return rc;
  if (vin.dtype != vout.dtype) { set_error("reduce_dim_static: input and output dtypes differ"); return THCB200_ERR_ARG; }
  const int mode = reduce_mode(rop, pre);
  if (mode < 0) { set_error("reduce_dim_static: unknown reduce op %d / pre op %d", rop, pre); return THCB200_ERR_ARG; }
  // the running sums of var / std need the post step that only thcb200_reduce_dim_post takes
  if (pre == THCB200_PRE_MOMENTS) { set_error("reduce_dim_static: THCB200_PRE_MOMENTS needs a var/std post step; use thcb200_reduce_dim_post"); return THCB200_ERR_ARG; }
  if (dim < 0 || dim >= vin.ndim) { set_error("reduce_dim_static: dimension %d out of range", dim); return THCB200_ERR_ARG; }
  if (vout.ndim != vin.ndim) { set_error("reduce_dim_static: output must have the input's dimension count"); return THCB200_ERR_ARG; }
  for (int i = 0; i < vin.ndim; ++i) {
    if (vout.sizes[i] != (i == dim ? 1 : vin.sizes[i])) { set_error("reduce_dim_static: output size mismatch in dim %d", i); return THCB200_ERR_SIZE; }
  }
  if (vin.sizes[dim] == 0) { set_error("reduce_dim_static: reduced dimension is empty"); return THCB200_ERR_ARG; }
  if (vout.numel == 0) return THCB200_OK;

  int device = 0;
  THCB_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) { set_error("reduce_dim_static: device index %d not supported", device); return THCB200_ERR_LIMIT; }
  rc = setup_device(device);
  if (rc) return rc;

  // A stand-in context whose workspace is the static array: the shared launch code then finds
  // its partials buffer large enough and never grows it.
  thcb200_ctx view_ctx{};
  view_ctx.device = device;
  view_ctx.num_sms = g_num_sms[device];
  view_ctx.ws = g_scratch_dev[device];
  view_ctx.ws_bytes = THCB200_STATIC_SCRATCH_BYTES;

  // How much scratch the plan for this call wants (same planner as the launch).
  const size_t esz = dtype_size(vin.dtype);
  const int vec_elems = (int)(16 / esz);
  const int col_vec = esz == 1 ? 4 : vec_elems;
  RedDimPlan pl;
  rc = plan_reduce_dim(&view_ctx, vin, vout, nullptr, dim, esz, vec_elems, col_vec, &pl);
  if (rc) return rc;
  if (pl.nsplit > 1) {
    const uint64_t noutputs = (pl.kind == kRedCol) ? pl.nslices * pl.I : pl.nslices;
    const uint64_t need = noutputs * pl.nsplit * kPartialSlotBytes;
    if (need > THCB200_STATIC_SCRATCH_BYTES) {
      set_error("reduce_dim_static: this reduction needs %llu bytes of partials, the static scratch holds %llu; "
                "use thcb200_reduce_dim", (unsigned long long)need, (unsigned long long)THCB200_STATIC_SCRATCH_BYTES);
      return THCB200_ERR_LIMIT;
    }
  }
  cudaStream_t st = (cudaStream_t)stream;
  switch (vin.dtype) {
    case THCB200_U8: return reduce_dim_u8(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
    case THCB200_I8: return reduce_dim_i8(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
    case THCB200_I16: return reduce_dim_i16(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
    case THCB200_I32: return reduce_dim_i32(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
    case THCB200_I64: return reduce_dim_i64(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
    case THCB200_F16: return reduce_dim_f16(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
    case THCB200_F32: return reduce_dim_f32(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
    default: return reduce_dim_f64(&view_ctx, mode, vin, vout, dim, s, PostOp{kPostNone, 0.0, 0}, st);
  }
}
