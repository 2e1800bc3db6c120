// Sharded reductions over the GPUs of one box: one process (or thread) per GPU, each holding a
// block of rows, NCCL over NVLink / NVSwitch for the exchange.
//
// cutorch drives several devices from one process and has no collective layer of its own
// (lib/THC/THCGeneral.h.in:57-123, lib/THC/THCGeneral.c:100-115); what a sharded tensor needs on
// top of the per-device calls is small:
//   * a full reduction: every rank's kernel leaves its accumulator (double / int64) in device
//     memory and the ranks' accumulators are combined -- ncclAllReduce straight on that slot, on the
//     stream the kernel ran on, for sums and products and for integer min / max; an all-gather
//     followed by this library's own fold in rank order where NCCL's arithmetic would not keep the
//     rule of the unsharded call (a NaN wins a floating min / max);
//   * a reduction along the sharded dim: the same choice per (element type, fold), on the vector
//     of per-rank outputs;
//   * max / min with positions along the sharded dim: NCCL has no arg-reduce, so (value, global
//     position) pairs are all-gathered and combined with the first-occurrence rule by the same
//     kernels that serve the unsharded call (ranks are blocks of rows in order, so the lowest rank
//     among equals is the lowest global position).
// NCCL is bound at run time (dlopen of libnccl.so.2, or the path in THCB200_NCCL_LIB): a process that
// already loaded NCCL -- torch does -- shares that copy, and a program that never shards needs no
// NCCL at all.  No kernel here reads another GPU's memory.
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "context.h"
#include "plan.h"
#include "reduce.cuh"

struct thcb200_comm {
  ncclComm_t comm;
  int nranks, rank, device;
  // receive buffer of the all-gathers, grown on demand; separate from the context's workspace, which
  // the folds that follow a gather may use for their own partials
  void *buf;
  size_t buf_bytes;
  // overlapped mode: the all-reduce of a full reduction's accumulators runs on `side`, in the order
  // local fold (caller's stream) -> ev_local -> all-reduce (side) -> ev_done
  int overlap;
  int pending;            // an all-reduce has been issued on `side` and nobody has waited for it yet
  cudaStream_t side;
  cudaEvent_t ev_local, ev_done;
  // exchange through peer memory (ExchangeBlock in core.cuh): this rank's block, every rank's block as
  // mapped here, which of them were opened from an IPC handle, the call counter, the poll limit
  thcb::ExchangeBlock *own_block;
  thcb::ExchangeBlock *blocks[thcb::kMaxPeers];
  unsigned char ipc_opened[thcb::kMaxPeers];
  int peer_ready, peer_on;
  unsigned int epoch, max_polls;
  int *peer_status;       // device word the finishing CTA sets when its wait runs out
};

namespace thcb {
namespace {

struct NcclApi {
  void *handle;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *);
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommAbort)(ncclComm_t);
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*GetVersion)(int *);
  const char *(*GetErrorString)(ncclResult_t);
  char why[256];
};
NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
  NcclApi &n = g_nccl;
  const char *names[3] = {getenv("THCB200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  for (const char *name : names) {
    if (!name || !name[0]) continue;
    n.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (n.handle) break;
  }
  if (!n.handle) { snprintf(n.why, sizeof(n.why), "NCCL is not available: %s", dlerror()); return; }
#define THCB_SYM(field, sym)                                                          \
  *(void **)(&n.field) = dlsym(n.handle, sym);                                        \
  if (!n.field) { snprintf(n.why, sizeof(n.why), "NCCL lacks %s", sym); n.handle = nullptr; return; }
  THCB_SYM(GetUniqueId, "ncclGetUniqueId")
  THCB_SYM(CommInitRank, "ncclCommInitRank")
  THCB_SYM(CommDestroy, "ncclCommDestroy")
  THCB_SYM(CommAbort, "ncclCommAbort")
  THCB_SYM(AllReduce, "ncclAllReduce")
  THCB_SYM(AllGather, "ncclAllGather")
  THCB_SYM(GetVersion, "ncclGetVersion")
  THCB_SYM(GetErrorString, "ncclGetErrorString")
#undef THCB_SYM
}

const NcclApi *nccl() {
  std::call_once(g_nccl_once, load_nccl);
  if (!g_nccl.handle) { set_error("%s", g_nccl.why); return nullptr; }
  return &g_nccl;
}

#define THCB_NCCL_TRY(api, expr)                                                             \
  do {                                                                                       \
    ncclResult_t _r = (expr);                                                                \
    if (_r != ncclSuccess) {                                                                 \
      set_error("%s failed: %s", #expr, (api)->GetErrorString(_r));                          \
      return THCB200_ERR_CUDA;                                                               \
    }                                                                                        \
  } while (0)

ncclDataType_t nccl_type(int dtype) {
  switch (dtype) {
    case THCB200_U8: return ncclUint8;
    case THCB200_I8: return ncclInt8;
    case THCB200_I32: return ncclInt32;
    case THCB200_I64: return ncclInt64;
    case THCB200_F16: return ncclFloat16;
    case THCB200_F32: return ncclFloat32;
    case THCB200_F64: return ncclFloat64;
  }
  return ncclNumTypes;   // I16: NCCL has no 16-bit integer
}

// Whether ncclAllReduce computes this fold the way the unsharded call does.  Sums and products of
// float / double / 32- and 64-bit integers and integer min / max do.  Floating min / max would lose
// the "a NaN wins" rule, 8- and 16-bit integers have no (or a saturating-free but absent) NCCL
// type worth trusting for wrap-around, and half sums would be accumulated in half: those go
// through the all-gather and this library's fold.
bool all_reduce_keeps_the_rule(int dtype, int rop) {
  const bool fp = dtype >= THCB200_F16;
  if (dtype == THCB200_F16 || dtype == THCB200_U8 || dtype == THCB200_I8 || dtype == THCB200_I16) return false;
  if (rop == THCB200_RED_SUM || rop == THCB200_RED_PROD) return true;
  if (rop == THCB200_RED_MIN || rop == THCB200_RED_MAX) return !fp;
  return false;
}

ncclRedOp_t nccl_op(int rop) {
  switch (rop) {
    case THCB200_RED_PROD: return ncclProd;
    case THCB200_RED_MIN: return ncclMin;
    case THCB200_RED_MAX: return ncclMax;
    default: return ncclSum;
  }
}

thcb200_tensor dense2d(void *data, int dtype, int64_t rows, int64_t cols) {
  thcb200_tensor t;
  memset(&t, 0, sizeof(t));
  t.data = data;
  t.dtype = dtype;
  t.ndim = 2;
  t.sizes[0] = rows; t.sizes[1] = cols;
  t.strides[0] = cols; t.strides[1] = 1;
  return t;
}

bool is_dense(const HostView &v) {
  int64_t sizes[kMaxDims], strides[kMaxDims];
  int nd = v.ndim;
  for (int i = 0; i < nd; ++i) { sizes[i] = v.sizes[i]; strides[i] = v.strides[i]; }
  if (nd == 0) return true;
  collapse_dims(sizes, strides, &nd, -1);
  return nd == 1 && (strides[0] == 1 || sizes[0] == 1);
}

void *comm_buffer(thcb200_comm *comm, size_t bytes) {
  if (bytes <= comm->buf_bytes) return comm->buf;
  // earlier calls may still read the old buffer
  if (cudaDeviceSynchronize() != cudaSuccess) { set_error("comm buffer: device synchronize failed"); return nullptr; }
  if (comm->buf) cudaFree(comm->buf);
  comm->buf = nullptr;
  comm->buf_bytes = 0;
  size_t want = 1 << 16;
  while (want < bytes) want <<= 1;
  if (device_alloc(&comm->buf, want) != cudaSuccess) {
    cudaGetLastError();
    comm->buf = nullptr;
    set_error("comm buffer: cannot allocate %zu bytes", want);
    return nullptr;
  }
  comm->buf_bytes = want;
  return comm->buf;
}

// the exchange alone, for a rank whose block of the tensor is empty: one warp
__global__ void __launch_bounds__(32) peer_exchange_only_kernel(PeerExchange px, unsigned long long bits, void *result) {
  pdl_prologue();
  peer_exchange(px, bits, result);
}

int check_comm(thcb200_ctx *ctx, thcb200_comm *comm, const char *what) {
  if (!ctx || !comm) { set_error("%s: null context or communicator", what); return THCB200_ERR_ARG; }
  if (ctx->device != comm->device) { set_error("%s: the context and the communicator belong to different devices", what); return THCB200_ERR_ARG; }
  return 0;
}

}  // namespace
}  // namespace thcb

using namespace thcb;

extern "C" {

int thcb200_comm_unique_id(void *id, size_t bytes) {
  const NcclApi *n = nccl();
  if (!n) return THCB200_ERR_UNSUPPORTED;
  if (!id || bytes < sizeof(ncclUniqueId)) { set_error("comm_unique_id: the buffer must hold %zu bytes", sizeof(ncclUniqueId)); return THCB200_ERR_ARG; }
  ncclUniqueId u;
  THCB_NCCL_TRY(n, n->GetUniqueId(&u));
  memcpy(id, &u, sizeof(u));
  return THCB200_OK;
}

int thcb200_comm_create(thcb200_comm **out, int nranks, int rank, const void *id, size_t bytes) {
  const NcclApi *n = nccl();
  if (!n) return THCB200_ERR_UNSUPPORTED;
  if (!out || !id || bytes < sizeof(ncclUniqueId)) { set_error("comm_create: null argument or short id"); return THCB200_ERR_ARG; }
  if (nranks < 1 || rank < 0 || rank >= nranks) { set_error("comm_create: rank %d outside %d ranks", rank, nranks); return THCB200_ERR_ARG; }
  ncclUniqueId u;
  memcpy(&u, id, sizeof(u));
  if (nranks > 64) { set_error("comm_create: at most 64 ranks (the GPUs of one box)"); return THCB200_ERR_LIMIT; }
  thcb200_comm *c = new thcb200_comm();
  c->nranks = nranks;
  c->rank = rank;
  cudaError_t e = cudaGetDevice(&c->device);
  if (e != cudaSuccess) { delete c; set_error("comm_create: %s", cudaGetErrorString(e)); return THCB200_ERR_CUDA; }
  e = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_local, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    set_error("comm_create: %s", cudaGetErrorString(e));
    thcb200_comm_destroy(c);
    return THCB200_ERR_CUDA;
  }
  ncclResult_t r = n->CommInitRank(&c->comm, nranks, u, rank);
  if (r != ncclSuccess) {
    c->comm = nullptr;
    set_error("ncclCommInitRank failed: %s", n->GetErrorString(r));
    thcb200_comm_destroy(c);
    return THCB200_ERR_CUDA;
  }
  *out = c;
  return THCB200_OK;
}

int thcb200_comm_set_overlap(thcb200_comm *comm, int on) {
  if (!comm) { set_error("comm_set_overlap: null communicator"); return THCB200_ERR_ARG; }
  comm->overlap = on ? 1 : 0;
  return THCB200_OK;
}

int thcb200_comm_wait(thcb200_comm *comm, void *stream) {
  if (!comm) { set_error("comm_wait: null communicator"); return THCB200_ERR_ARG; }
  if (comm->pending) THCB_CUDA_TRY(cudaStreamWaitEvent((cudaStream_t)stream, comm->ev_done, 0));
  return THCB200_OK;
}

int thcb200_comm_create_local(thcb200_comm **out, int nranks, int rank) {
  if (!out) { set_error("comm_create_local: null output pointer"); return THCB200_ERR_ARG; }
  if (nranks < 1 || rank < 0 || rank >= nranks) { set_error("comm_create_local: rank %d outside %d ranks", rank, nranks); return THCB200_ERR_ARG; }
  if (nranks > kMaxPeers) { set_error("comm_create_local: at most %d ranks exchange through peer memory", kMaxPeers); return THCB200_ERR_LIMIT; }
  thcb200_comm *c = new thcb200_comm();
  c->nranks = nranks;
  c->rank = rank;
  cudaError_t e = cudaGetDevice(&c->device);
  if (e != cudaSuccess) { delete c; set_error("comm_create_local: %s", cudaGetErrorString(e)); return THCB200_ERR_CUDA; }
  *out = c;
  return THCB200_OK;
}

size_t thcb200_comm_peer_block_bytes(void) { return sizeof(ExchangeBlock); }

static int ensure_own_block(thcb200_comm *comm) {
  if (comm->own_block) return 0;
  if (comm->nranks > kMaxPeers) { set_error("peer exchange: at most %d ranks", kMaxPeers); return THCB200_ERR_LIMIT; }
  // cudaMalloc, not the stream-ordered pool: the block is exported to other processes
  void *p = nullptr;
  cudaError_t e = device_alloc(&p, sizeof(ExchangeBlock));
  if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(ExchangeBlock));
  void *st = nullptr;
  if (e == cudaSuccess) e = device_alloc(&st, 64);
  if (e == cudaSuccess) e = cudaMemset(st, 0, 64);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();   // zeroed before any peer learns the address
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (p) cudaFree(p);
    if (st) cudaFree(st);
    set_error("peer exchange: cannot set up this rank's block: %s", cudaGetErrorString(e));
    return THCB200_ERR_NOMEM;
  }
  comm->own_block = (ExchangeBlock *)p;
  comm->peer_status = (int *)st;
  comm->blocks[comm->rank] = comm->own_block;
  comm->max_polls = 1u << 22;   // about a second of polling before a wait gives up
  return 0;
}

int thcb200_comm_peer_export(thcb200_comm *comm, void *handle, size_t bytes) {
  if (!comm || !handle || bytes < sizeof(cudaIpcMemHandle_t)) { set_error("comm_peer_export: null argument or short buffer"); return THCB200_ERR_ARG; }
  int rc = ensure_own_block(comm);
  if (rc) return rc;
  cudaIpcMemHandle_t h;
  THCB_CUDA_TRY(cudaIpcGetMemHandle(&h, comm->own_block));
  memcpy(handle, &h, sizeof(h));
  return THCB200_OK;
}

int thcb200_comm_peer_attach(thcb200_comm *comm, const void *handles, size_t bytes_each) {
  if (!comm || !handles || bytes_each < sizeof(cudaIpcMemHandle_t)) { set_error("comm_peer_attach: null argument or short handles"); return THCB200_ERR_ARG; }
  int rc = ensure_own_block(comm);
  if (rc) return rc;
  for (int r = 0; r < comm->nranks; ++r) {
    if (r == comm->rank || comm->blocks[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char *)handles + (size_t)r * bytes_each, sizeof(h));
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_error("comm_peer_attach: cannot map rank %d's block: %s", r, cudaGetErrorString(e));
      return THCB200_ERR_CUDA;
    }
    comm->blocks[r] = (ExchangeBlock *)p;
    comm->ipc_opened[r] = 1;
  }
  comm->peer_ready = 1;
  return THCB200_OK;
}

int thcb200_comm_peer_attach_local(thcb200_comm *comm, void *const *blocks) {
  if (!comm || !blocks) { set_error("comm_peer_attach_local: null argument"); return THCB200_ERR_ARG; }
  if (comm->nranks > kMaxPeers) { set_error("peer exchange: at most %d ranks", kMaxPeers); return THCB200_ERR_LIMIT; }
  for (int r = 0; r < comm->nranks; ++r) {
    if (!blocks[r]) { set_error("comm_peer_attach_local: no block for rank %d", r); return THCB200_ERR_ARG; }
    comm->blocks[r] = (ExchangeBlock *)blocks[r];
  }
  if (!comm->peer_status) {
    void *st = nullptr;
    if (device_alloc(&st, 64) != cudaSuccess || cudaMemset(st, 0, 64) != cudaSuccess) {
      cudaGetLastError();
      if (st) cudaFree(st);
      set_error("comm_peer_attach_local: cannot allocate the status word");
      return THCB200_ERR_NOMEM;
    }
    comm->peer_status = (int *)st;
  }
  if (!comm->max_polls) comm->max_polls = 1u << 22;
  comm->peer_ready = 1;
  return THCB200_OK;
}

int thcb200_comm_set_peer_exchange(thcb200_comm *comm, int on, unsigned int max_polls) {
  if (!comm) { set_error("comm_set_peer_exchange: null communicator"); return THCB200_ERR_ARG; }
  if (on && !comm->peer_ready) { set_error("comm_set_peer_exchange: attach the ranks' blocks first"); return THCB200_ERR_ARG; }
  comm->peer_on = on ? 1 : 0;
  if (max_polls) comm->max_polls = max_polls;
  return THCB200_OK;
}

int thcb200_comm_peer_status(thcb200_comm *comm, int *timed_out, void *stream) {
  if (!comm || !timed_out) { set_error("comm_peer_status: null argument"); return THCB200_ERR_ARG; }
  *timed_out = 0;
  if (!comm->peer_status) return THCB200_OK;
  THCB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  int v = 0;
  THCB_CUDA_TRY(cudaMemcpy(&v, comm->peer_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (v) THCB_CUDA_TRY(cudaMemset(comm->peer_status, 0, sizeof(int)));
  *timed_out = v;
  return THCB200_OK;
}

void thcb200_comm_destroy(thcb200_comm *comm) {
  if (!comm) return;
  const NcclApi *n = comm->comm ? nccl() : nullptr;
  if (comm->side) cudaStreamSynchronize(comm->side);
  for (int r = 0; r < kMaxPeers; ++r)
    if (comm->ipc_opened[r] && comm->blocks[r]) cudaIpcCloseMemHandle(comm->blocks[r]);
  if (comm->own_block) cudaFree(comm->own_block);
  if (comm->peer_status) cudaFree(comm->peer_status);
  if (n && comm->comm) n->CommDestroy(comm->comm);
  if (comm->buf) cudaFree(comm->buf);
  if (comm->ev_local) cudaEventDestroy(comm->ev_local);
  if (comm->ev_done) cudaEventDestroy(comm->ev_done);
  if (comm->side) cudaStreamDestroy(comm->side);
  delete comm;
}

int thcb200_comm_info(const thcb200_comm *comm, int *nranks, int *rank, int *nccl_version) {
  if (!comm) { set_error("comm_info: null communicator"); return THCB200_ERR_ARG; }
  if (nranks) *nranks = comm->nranks;
  if (rank) *rank = comm->rank;
  if (nccl_version) {
    const NcclApi *n = nccl();
    if (!n) return THCB200_ERR_UNSUPPORTED;
    THCB_NCCL_TRY(n, n->GetVersion(nccl_version));
  }
  return THCB200_OK;
}

int thcb200_comm_all_reduce(thcb200_comm *comm, void *buf_dev, int64_t count, int dtype, int rop, void *stream) {
  const NcclApi *n = nccl();
  if (!n) return THCB200_ERR_UNSUPPORTED;
  if (!comm || !buf_dev || count < 0) { set_error("comm_all_reduce: bad argument"); return THCB200_ERR_ARG; }
  if (!comm->comm) { set_error("comm_all_reduce: this communicator was created without NCCL"); return THCB200_ERR_UNSUPPORTED; }
  if (nccl_type(dtype) == ncclNumTypes || rop < THCB200_RED_SUM || rop > THCB200_RED_MAX) {
    set_error("comm_all_reduce: dtype %d / fold %d has no NCCL form", dtype, rop);
    return THCB200_ERR_UNSUPPORTED;
  }
  if (count == 0) return THCB200_OK;
  THCB_NCCL_TRY(n, n->AllReduce(buf_dev, buf_dev, (size_t)count, nccl_type(dtype), nccl_op(rop), comm->comm, (cudaStream_t)stream));
  return THCB200_OK;
}

int thcb200_comm_all_gather(thcb200_comm *comm, const void *send_dev, void *recv_dev, int64_t bytes_per_rank, void *stream) {
  const NcclApi *n = nccl();
  if (!n) return THCB200_ERR_UNSUPPORTED;
  if (!comm || !send_dev || !recv_dev || bytes_per_rank < 0) { set_error("comm_all_gather: bad argument"); return THCB200_ERR_ARG; }
  if (!comm->comm) { set_error("comm_all_gather: this communicator was created without NCCL"); return THCB200_ERR_UNSUPPORTED; }
  if (bytes_per_rank == 0) return THCB200_OK;
  THCB_NCCL_TRY(n, n->AllGather(send_dev, recv_dev, (size_t)bytes_per_rank, ncclUint8, comm->comm, (cudaStream_t)stream));
  return THCB200_OK;
}

int thcb200_sharded_reduce_all(thcb200_ctx *ctx, thcb200_comm *comm, int rop, int pre, thcb200_scalar s,
                               const thcb200_tensor *in, void *result_dev, void *stream) {
  int rc = check_comm(ctx, comm, "sharded_reduce_all");
  if (rc) return rc;
  if (!in) { set_error("sharded_reduce_all: null tensor"); return THCB200_ERR_ARG; }
  THCB_CTX_LOCK(ctx);
  cudaStream_t st = (cudaStream_t)stream;
  if (comm->peer_on && comm->nranks > 1) {
    // one kernel: the finishing CTA stores this rank's accumulator into every rank's block, waits (bounded)
    // for the others' and folds them in rank order
    const int fold = rop == THCB200_RED_ALL ? THCB200_RED_MIN : rop == THCB200_RED_ANY ? THCB200_RED_MAX : rop;
    if (fold < THCB200_RED_SUM || fold > THCB200_RED_MAX) { set_error("sharded_reduce_all: unknown reduce op %d", rop); return THCB200_ERR_ARG; }
    PeerExchange px;
    memset(&px, 0, sizeof(px));
    px.nranks = comm->nranks;
    px.rank = comm->rank;
    if (++comm->epoch == 0) comm->epoch = 2;   // never 0, and the parity keeps alternating across the wrap
    px.epoch = comm->epoch;
    px.max_polls = comm->max_polls;
    px.fold = fold;
    px.is_fp = in->dtype >= THCB200_F16 ? 1 : 0;
    px.status = comm->peer_status;
    for (int r = 0; r < comm->nranks; ++r) px.block[r] = comm->blocks[r];
    if (view_numel(in) == 0) {
      // nothing to fold here, but the other ranks wait for this rank's column: send the identity
      if (fold == THCB200_RED_MIN || fold == THCB200_RED_MAX) { set_error("sharded_reduce_all: min/max over an empty block"); return THCB200_ERR_ARG; }
      const bool one = (rop == THCB200_RED_PROD || rop == THCB200_RED_ALL);
      unsigned long long bits;
      if (px.is_fp) { const double d = one ? 1.0 : 0.0; memcpy(&bits, &d, 8); } else bits = one ? 1ull : 0ull;
      launch_pdl(peer_exchange_only_kernel, 1, 32, 0, st, px, bits, result_dev);
      THCB_CUDA_TRY(cudaGetLastError());
      return THCB200_OK;
    }
    ctx->px = &px;
    rc = thcb200_reduce_all(ctx, rop, pre, s, in, result_dev, stream);
    ctx->px = nullptr;
    return rc;
  }
  if (comm->nranks > 1 && !comm->comm) { set_error("sharded_reduce_all: this communicator has no NCCL and its peer exchange is off"); return THCB200_ERR_UNSUPPORTED; }
  // an earlier overlapped all-reduce may still be using a slot: it finishes before this fold writes one
  if (comm->pending) THCB_CUDA_TRY(cudaStreamWaitEvent(st, comm->ev_done, 0));
  // this rank's accumulator, left in the result slot on the device by the finishing CTA
  rc = thcb200_reduce_all(ctx, rop, pre, s, in, result_dev, stream);
  if (rc || comm->nranks == 1) return rc;
  const bool fp = in->dtype >= THCB200_F16;
  const int slot_dtype = fp ? THCB200_F64 : THCB200_I64;
  // logical and / or of 0/1 accumulators are their min / max
  const int fold = rop == THCB200_RED_ALL ? THCB200_RED_MIN : rop == THCB200_RED_ANY ? THCB200_RED_MAX : rop;
  if (all_reduce_keeps_the_rule(slot_dtype, fold)) {
    if (!comm->overlap) {
      comm->pending = 0;
      return thcb200_comm_all_reduce(comm, result_dev, 1, slot_dtype, fold, stream);
    }
    // overlapped: the collective leaves the caller's stream free for the kernels that follow
    THCB_CUDA_TRY(cudaEventRecord(comm->ev_local, st));
    THCB_CUDA_TRY(cudaStreamWaitEvent(comm->side, comm->ev_local, 0));
    rc = thcb200_comm_all_reduce(comm, result_dev, 1, slot_dtype, fold, (void *)comm->side);
    if (rc) return rc;
    THCB_CUDA_TRY(cudaEventRecord(comm->ev_done, comm->side));
    comm->pending = 1;
    return THCB200_OK;
  }
  comm->pending = 0;
  // floating min / max: gather the ranks' slots and fold them here in rank order (a NaN wins)
  void *slots_dev = comm_buffer(comm, (size_t)comm->nranks * 8);
  if (!slots_dev) return THCB200_ERR_NOMEM;
  rc = thcb200_comm_all_gather(comm, result_dev, slots_dev, 8, stream);
  if (rc) return rc;
  thcb200_tensor slots = dense2d(slots_dev, slot_dtype, 1, comm->nranks);
  return thcb200_reduce_all(ctx, fold, THCB200_PRE_IDENTITY, thcb200_scalar{0.0, 0}, &slots, result_dev, stream);
}

int thcb200_sharded_reduce_dim(thcb200_ctx *ctx, thcb200_comm *comm, int rop, int pre, thcb200_scalar s,
                               const thcb200_tensor *out, const thcb200_tensor *in, int dim, void *stream) {
  int rc = check_comm(ctx, comm, "sharded_reduce_dim");
  if (rc) return rc;
  HostView vout;
  rc = to_host_view(out, &vout, "sharded_reduce_dim output");
  if (rc) return rc;
  if (!is_dense(vout)) { set_error("sharded_reduce_dim: the output must be one dense run (it is exchanged as it lies)"); return THCB200_ERR_ARG; }
  THCB_CTX_LOCK(ctx);
  rc = thcb200_reduce_dim(ctx, rop, pre, s, out, in, dim, stream);   // this rank's rows
  if (rc || comm->nranks == 1 || vout.numel == 0) return rc;
  // the per-rank outputs already carry the element transform: what is left is the plain fold
  const int fold = rop == THCB200_RED_ALL ? THCB200_RED_MIN : rop == THCB200_RED_ANY ? THCB200_RED_MAX : rop;
  if (all_reduce_keeps_the_rule(vout.dtype, fold))
    return thcb200_comm_all_reduce(comm, vout.data, vout.numel, vout.dtype, fold, stream);
  // gather the ranks' vectors [nranks][numel] and fold dim 0 with the library's own kernel
  const size_t esz = dtype_size(vout.dtype);
  const size_t row = (size_t)vout.numel * esz;
  const size_t need = (size_t)comm->nranks * row;
  char *rows = (char *)comm_buffer(comm, need);
  if (!rows) return THCB200_ERR_NOMEM;
  rc = thcb200_comm_all_gather(comm, vout.data, rows, (int64_t)row, stream);
  if (rc) return rc;
  thcb200_tensor gathered = dense2d(rows, vout.dtype, comm->nranks, vout.numel);
  thcb200_tensor folded = dense2d(vout.data, vout.dtype, 1, vout.numel);
  return thcb200_reduce_dim(ctx, fold, THCB200_PRE_IDENTITY, thcb200_scalar{0.0, 0}, &folded, &gathered, 0, stream);
}

int thcb200_sharded_reduce_dim_index(thcb200_ctx *ctx, thcb200_comm *comm, int rop, const thcb200_tensor *values,
                                     const thcb200_tensor *indices, const thcb200_tensor *in, int dim,
                                     int64_t shard_start, void *stream) {
  int rc = check_comm(ctx, comm, "sharded_reduce_dim_index");
  if (rc) return rc;
  HostView vval, vidx;
  rc = to_host_view(values, &vval, "sharded_reduce_dim_index values");
  if (!rc) rc = to_host_view(indices, &vidx, "sharded_reduce_dim_index indices");
  if (rc) return rc;
  if (!is_dense(vval) || !is_dense(vidx)) { set_error("sharded_reduce_dim_index: values and indices must be dense runs"); return THCB200_ERR_ARG; }
  if (shard_start < 0) { set_error("sharded_reduce_dim_index: negative shard start"); return THCB200_ERR_ARG; }
  THCB_CTX_LOCK(ctx);
  rc = thcb200_reduce_dim_index(ctx, rop, values, indices, in, dim, stream);   // positions 1-based inside this rank's block
  if (rc || vval.numel == 0) return rc;
  const thcb200_scalar start = {(double)shard_start, shard_start};
  if (shard_start) {
    rc = thcb200_pointwise(ctx, THCB200_OP_ADD_S, indices, indices, nullptr, nullptr, 1, start, thcb200_scalar{0.0, 0}, stream);
    if (rc) return rc;
  }
  if (comm->nranks == 1) return THCB200_OK;
  const int64_t n = vval.numel;
  const size_t esz = dtype_size(vval.dtype);
  const size_t vrow = (size_t)n * esz, prow = (size_t)n * 8;
  const size_t R = (size_t)comm->nranks;
  // buffer: [values R x n][positions R x n][which n]
  const size_t off_p = (R * vrow + 255) & ~(size_t)255, off_w = (off_p + R * prow + 255) & ~(size_t)255;
  char *buf = (char *)comm_buffer(comm, off_w + prow);
  if (!buf) return THCB200_ERR_NOMEM;
  char *gv = buf, *gp = buf + off_p, *which = buf + off_w;
  rc = thcb200_comm_all_gather(comm, vval.data, gv, (int64_t)vrow, stream);
  if (!rc) rc = thcb200_comm_all_gather(comm, vidx.data, gp, (int64_t)prow, stream);
  if (rc) return rc;
  // the winning rank per output: the same value+position kernel, over the rank dim (ranks are row
  // blocks in order, so the first occurrence among ranks is the lowest global position)
  thcb200_tensor tv = dense2d(gv, vval.dtype, (int64_t)R, n), tp = dense2d(gp, THCB200_I64, (int64_t)R, n);
  thcb200_tensor out_v = dense2d(vval.data, vval.dtype, 1, n), out_w = dense2d(which, THCB200_I64, 1, n);
  thcb200_tensor out_p = dense2d(vidx.data, THCB200_I64, 1, n);
  rc = thcb200_reduce_dim_index(ctx, rop, &out_v, &out_w, &tv, 0, stream);
  if (rc) return rc;
  // ... and its global position
  return thcb200_indexed(ctx, THCB200_INDEX_GATHER, &out_p, &tp, &out_w, 0, 0, thcb200_scalar{0.0, 0}, stream);
}

}  // extern "C"
