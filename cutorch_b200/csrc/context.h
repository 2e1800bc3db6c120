// Per-device context: reduction workspace, ticket counters, pinned result slot.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <mutex>

#include "../../include/thcb200.h"

namespace thcb {
constexpr int kNumTickets = 4096;
struct PeerExchange;
}

// The scratch of a context (workspace, ticket counters, result slots, mask offsets) is reused
// from call to call, which is safe in the order of ONE stream: calls on streams that may run
// concurrently need a context each.  Several host threads may share a context; `lock` serialises
// their calls (including the wait for a result that comes back through the pinned slot).
struct thcb200_ctx {
  std::recursive_mutex lock;
  int device;
  int num_sms;
  int max_smem_optin;
  void *ws;               // device workspace for partial results, grown on demand
  size_t ws_bytes;
  unsigned int *tickets;  // kNumTickets counters, zero between launches (kernels reset them)
  int *status;            // device word: kernels record bounded-wait failures here
  void *host_slot;        // pinned, mapped, 64 bytes
  void *host_slot_dev;    // the device-side address of host_slot: kernels store results straight to the host
  void *dev_slot;         // device, 64 bytes: result of reduce_all_host
  // masked copy / select: tile counts and offsets of the mask counted last, and which mask
  // view and stream they belong to (reused only when the caller says the mask is unchanged)
  void *mask_ws;
  size_t mask_ws_bytes;
  const void *prep_mask;
  uint64_t prep_layout;   // hash of the mask view's sizes and strides
  int64_t prep_numel;
  void *prep_stream;
  int prep_valid;
  int prep_count_known;   // the host has read the count of that mask from the pinned slot
  // set by a sharded full reduction for the duration of its launch: fold the other GPUs' accumulators
  // in the finishing CTA (see ExchangeBlock in core.cuh); null otherwise
  const thcb::PeerExchange *px;
};

#define THCB_CTX_LOCK(ctx) std::lock_guard<std::recursive_mutex> thcb_ctx_guard((ctx)->lock)

namespace thcb {

// Returns a device buffer of at least `bytes` (256-byte aligned), valid until the next call
// that asks for more.  Growing synchronises the device; nullptr on allocation failure.
void *ctx_workspace(thcb200_ctx *ctx, size_t bytes);

// Every device allocation the library makes for itself (workspaces, dense temporaries) goes through
// these two, so that a test can make the n-th one fail the way an exhausted GPU would, without
// exhausting a GPU: see thcb200_debug_fail_allocation in thcb200.h.
cudaError_t device_alloc(void **p, size_t bytes);
cudaError_t device_alloc_async(void **p, size_t bytes, cudaStream_t st);

#define THCB_CUDA_TRY(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      ::thcb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return THCB200_ERR_CUDA;                                                           \
    }                                                                                    \
  } while (0)

}  // namespace thcb
