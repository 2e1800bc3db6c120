// The THC C API of the apply / reduce path (include/THC/THC.h) on top of the descriptor-level
// core (include/thcb200.h): tensor/storage metadata, output resizing, argument checks and the
// composition rules of the THCTensor_(op) entry points
// (lib/THC/generic/THCTensorMathPointwise.cu, THCTensorMathPairwise.cu, THCTensorMathReduce.cu,
// THCTensorCopy.cu, THCTensor.c, THCStorage.c).  Host code only; every kernel launch goes
// through thcb200_*.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <new>
#include <set>
#include <type_traits>
#include <utility>
#include <vector>
#include <string>

#include "../../include/THC/THC.h"
#include "../../include/thcb200.h"

// ======================================================================================
// Errors
// ======================================================================================
namespace {

struct THFailure {
  std::string msg;
  int arg;
};

THErrorHandlerFunction g_error_handler = nullptr;
void *g_error_handler_data = nullptr;
THArgErrorHandlerFunction g_arg_error_handler = nullptr;
void *g_arg_error_handler_data = nullptr;
thread_local bool g_failed = false;
thread_local char g_failure_msg[1024] = "";

[[noreturn]] void th_error(const char *fmt, ...) {
  char buf[900];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (g_error_handler) {
    g_error_handler(buf, g_error_handler_data);  // does not return by contract
    abort();
  }
  throw THFailure{buf, 0};
}

[[noreturn]] void th_arg_error(int arg, const char *fmt, ...) {
  char buf[900];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (g_arg_error_handler) {
    g_arg_error_handler(arg, buf, g_arg_error_handler_data);
    abort();
  }
  char full[1000];
  snprintf(full, sizeof(full), "invalid argument %d: %s", arg, buf);
  throw THFailure{full, arg};
}

void record_failure(const THFailure &f) {
  g_failed = true;
  snprintf(g_failure_msg, sizeof(g_failure_msg), "%s", f.msg.c_str());
}

#define THArgCheck(cond, arg, ...) do { if (!(cond)) th_arg_error(arg, __VA_ARGS__); } while (0)
#define THCudaCheck(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) th_error("cuda runtime error (%d) : %s at %s:%d", (int)_e, cudaGetErrorString(_e), __FILE__, __LINE__); } while (0)
#define CUTORCH_DIM_WARNING "tensor too large or too many (>25) dimensions"

#define API_BEGIN try {
#define API_END } catch (const THFailure &f) { record_failure(f); }
#define API_END_RET(v) } catch (const THFailure &f) { record_failure(f); return v; }

}  // namespace

// ======================================================================================
// State
// ======================================================================================
// Contexts of one device, one per stream that has been current on it: the scratch of a context
// is only safe in the order of a single stream (cutorch keeps its scratch space per stream for the
// same reason, lib/THC/THCGeneral.c:563-590).
struct CtxTable {
  std::mutex m;
  std::vector<std::pair<cudaStream_t, thcb200_ctx *>> v;
};

struct THCState {
  int numDevices;
  CtxTable *tables;           // per device; contexts are created on first use
  unsigned long long epoch;   // distinguishes this initialisation from earlier ones at the same address
  THCDeviceAllocator *allocator;
  THCDeviceAllocator defaultAllocator;
  int initialised;
  unsigned char *p2pOff;      // numDevices x numDevices: 1 = direct access switched off by the caller
  cudaDeviceProp *props;      // per device, filled on first request
  unsigned char *propsValid;
  void (*gcFunction)(void *); // called once when a device allocation fails, before one retry
  void *gcData;
};

namespace {

cudaStream_t state_stream(THCState *state);

// Default device allocator: stream-ordered (cudaMallocAsync / cudaFreeAsync from the device's
// default memory pool, which keeps freed blocks for reuse).  It plays the part of cutorch's
// caching allocator (lib/THC/THCCachingAllocator.cpp): temporaries and resized outputs on the hot
// path cost no device synchronisation.  A block is returned in the order of the stream that is
// current when it is freed, so a storage has to be freed while the stream that last used it is
// current (or after that stream was synchronised).
cudaError_t default_malloc(void *, void **p, size_t n, cudaStream_t st) { return cudaMallocAsync(p, n, st); }

// Device allocation as cutorch's THCudaMalloc does it (lib/THC/THCGeneral.c:842-854): when the
// allocator fails and the host language registered a garbage-collection callback, run it (it frees
// tensors nobody refers to any more) and try once more.  The failed attempt's error is cleared.
cudaError_t malloc_with_gc_retry(THCState *state, THCDeviceAllocator *a, void *actx, void **p, size_t n, cudaStream_t st) {
  cudaError_t e = a->malloc(actx, p, n, st);
  if (e != cudaSuccess && state && state->gcFunction) {
    cudaGetLastError();
    state->gcFunction(state->gcData);
    e = a->malloc(actx, p, n, st);
  }
  return e;
}

// States that are initialised right now: a storage may outlive its THCState, and must not follow a
// dangling pointer when it is finally freed (it is then released in the order of the null stream).
std::mutex g_live_states_mutex;
std::set<const void *> g_live_states;
void mark_state(const void *state, bool live) {
  std::lock_guard<std::mutex> lock(g_live_states_mutex);
  if (live) g_live_states.insert(state); else g_live_states.erase(state);
}
cudaError_t default_free(void *ctx, void *p) {
  bool live;
  {
    std::lock_guard<std::mutex> lock(g_live_states_mutex);
    live = g_live_states.count(ctx) != 0;
  }
  return cudaFreeAsync(p, live ? state_stream((THCState *)ctx) : (cudaStream_t)0);
}

int current_device() {
  int d = 0;
  THCudaCheck(cudaGetDevice(&d));
  return d;
}

// The current stream of each device is a property of the calling thread, as in cutorch
// (THCThreadLocal in lib/THC/THCGeneral.c:516-561): a thread that never called
// THCState_setStream works on the default stream whatever other threads have set.
std::atomic<unsigned long long> g_state_epoch{0};

struct ThreadStreams {
  struct Entry {
    const THCState *state;
    unsigned long long epoch;
    std::vector<THCStream *> current;   // per device; null = default stream
  };
  std::vector<Entry> entries;
  static void release(Entry &e) {
    for (THCStream *s : e.current) if (s) THCStream_free(s);
    e.current.clear();
  }
  // the calling thread's streams for this initialisation of `state` (created empty on demand)
  Entry *find(const THCState *state, bool create) {
    for (size_t i = 0; i < entries.size(); ++i) {
      if (entries[i].state != state) continue;
      if (entries[i].epoch == state->epoch) return &entries[i];
      release(entries[i]);               // left over from a state that was shut down
      entries.erase(entries.begin() + (long)i);
      break;
    }
    if (!create) return nullptr;
    entries.push_back(Entry{state, state->epoch, std::vector<THCStream *>((size_t)(state->numDevices > 0 ? state->numDevices : 1), nullptr)});
    return &entries.back();
  }
  void drop(const THCState *state) {
    for (size_t i = 0; i < entries.size(); ++i)
      if (entries[i].state == state) { release(entries[i]); entries.erase(entries.begin() + (long)i); return; }
  }
  ~ThreadStreams() { for (Entry &e : entries) release(e); }
};
thread_local ThreadStreams t_streams;

THCStream *thread_stream(THCState *state, int device) {
  if (!state || !state->initialised || device < 0 || device >= state->numDevices) return nullptr;
  ThreadStreams::Entry *e = t_streams.find(state, false);
  return e ? e->current[(size_t)device] : nullptr;
}

cudaStream_t state_stream(THCState *state) {
  THCStream *s = thread_stream(state, current_device());
  return s ? s->stream : (cudaStream_t)0;
}

// The context of the current device and the calling thread's current stream on it.
thcb200_ctx *state_ctx(THCState *state) {
  if (!state || !state->initialised) th_error("THCState is not initialised (call THCudaInit)");
  const int d = current_device();
  if (d >= state->numDevices) th_error("current device %d out of range", d);
  const cudaStream_t st = state_stream(state);
  struct Last { const THCState *state; unsigned long long epoch; int device; cudaStream_t stream; thcb200_ctx *ctx; };
  thread_local Last last = {nullptr, 0, -1, nullptr, nullptr};
  if (last.ctx && last.state == state && last.epoch == state->epoch && last.device == d && last.stream == st) return last.ctx;
  CtxTable &t = state->tables[d];
  thcb200_ctx *ctx = nullptr;
  {
    std::lock_guard<std::mutex> lock(t.m);
    for (auto &e : t.v) if (e.first == st) { ctx = e.second; break; }
    if (!ctx) {
      if (thcb200_ctx_create(&ctx, d) != 0) th_error("%s", thcb200_last_error());
      t.v.emplace_back(st, ctx);
    }
  }
  last = Last{state, state->epoch, d, st, ctx};
  return ctx;
}

}  // namespace

extern "C" {

void THSetErrorHandler(THErrorHandlerFunction f, void *data) { g_error_handler = f; g_error_handler_data = data; }
void THSetArgErrorHandler(THArgErrorHandlerFunction f, void *data) { g_arg_error_handler = f; g_arg_error_handler_data = data; }
int THCB200_errorOccurred(void) { return g_failed ? 1 : 0; }
const char *THCB200_errorMessage(void) { return g_failure_msg; }
void THCB200_clearError(void) { g_failed = false; g_failure_msg[0] = 0; }

THLongStorage *THLongStorage_newWithSize(ptrdiff_t size) {
  THLongStorage *s = (THLongStorage *)calloc(1, sizeof(THLongStorage));
  s->data = size > 0 ? (long *)calloc((size_t)size, sizeof(long)) : nullptr;
  s->size = size;
  s->refcount = 1;
  s->flag = TH_STORAGE_REFCOUNTED | TH_STORAGE_RESIZABLE | TH_STORAGE_FREEMEM;
  return s;
}
THLongStorage *THLongStorage_newWithSize1(long a) {
  THLongStorage *s = THLongStorage_newWithSize(1);
  s->data[0] = a;
  return s;
}
void THLongStorage_set(THLongStorage *s, ptrdiff_t i, long v) {
  API_BEGIN
  THArgCheck(i >= 0 && i < s->size, 2, "out of bounds");
  s->data[i] = v;
  API_END
}
long THLongStorage_get(const THLongStorage *s, ptrdiff_t i) {
  API_BEGIN
  THArgCheck(i >= 0 && i < s->size, 2, "out of bounds");
  return s->data[i];
  API_END_RET(0)
}
void THLongStorage_free(THLongStorage *s) {
  if (!s) return;
  if (--s->refcount > 0) return;
  free(s->data);
  free(s);
}

THCState *THCState_alloc(void) { return (THCState *)calloc(1, sizeof(THCState)); }
void THCState_free(THCState *state) { free(state); }

void THCudaInit(THCState *state) {
  API_BEGIN
  if (!state) th_error("THCudaInit: null state");
  int n = 0;
  THCudaCheck(cudaGetDeviceCount(&n));
  state->numDevices = n;
  state->tables = new CtxTable[(size_t)(n > 0 ? n : 1)];
  state->epoch = ++g_state_epoch;
  state->p2pOff = (unsigned char *)calloc((size_t)(n > 0 ? n * n : 1), 1);
  state->props = (cudaDeviceProp *)calloc((size_t)(n > 0 ? n : 1), sizeof(cudaDeviceProp));
  state->propsValid = (unsigned char *)calloc((size_t)(n > 0 ? n : 1), 1);
  state->defaultAllocator.malloc = default_malloc;
  state->defaultAllocator.realloc = nullptr;
  state->defaultAllocator.free = default_free;
  state->defaultAllocator.emptyCache = nullptr;
  state->defaultAllocator.cacheInfo = nullptr;
  state->defaultAllocator.state = state;
  state->allocator = &state->defaultAllocator;
  state->initialised = 1;
  mark_state(state, true);
  // keep freed blocks in the pools instead of returning them to the driver at every synchronise
  for (int d = 0; d < n; ++d) {
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, d) == cudaSuccess) {
      unsigned long long keep = ~0ull;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    } else {
      cudaGetLastError();
    }
  }
  API_END
}

void THCudaShutdown(THCState *state) {
  if (!state || !state->initialised) return;
  mark_state(state, false);
  for (int d = 0; d < state->numDevices; ++d)
    for (auto &e : state->tables[d].v) thcb200_ctx_destroy(e.second);
  delete[] state->tables;
  t_streams.drop(state);   // other threads' entries are recognised as stale by the epoch
  free(state->p2pOff);
  free(state->props);
  free(state->propsValid);
  state->tables = nullptr;
  state->p2pOff = nullptr;
  state->props = nullptr;
  state->propsValid = nullptr;
  state->initialised = 0;
}

int THCState_getNumDevices(THCState *state) { return state->numDevices; }
cudaStream_t THCState_getCurrentStream(THCState *state) {
  API_BEGIN
  return state_stream(state);
  API_END_RET(0)
}
cudaStream_t THCState_getCurrentStreamOnDevice(THCState *state, int device) {
  THCStream *s = thread_stream(state, device);
  return s ? s->stream : (cudaStream_t)0;
}
THCStream *THCState_getStream(THCState *state) {
  API_BEGIN
  return thread_stream(state, current_device());
  API_END_RET(nullptr)
}
void THCState_setStream(THCState *state, THCStream *stream) {
  API_BEGIN
  const int d = current_device();
  if (stream) {
    THArgCheck(stream->device == d, 2, "stream belongs to another device");
    THCStream_retain(stream);
  }
  if (!state->initialised || d >= state->numDevices) th_error("THCState_setStream: state not initialised for device %d", d);
  ThreadStreams::Entry *e = t_streams.find(state, true);
  if (e->current[(size_t)d]) THCStream_free(e->current[(size_t)d]);
  e->current[(size_t)d] = stream;
  API_END
}
THCDeviceAllocator *THCState_getDeviceAllocator(THCState *state) { return state->allocator; }
void THCState_setDeviceAllocator(THCState *state, THCDeviceAllocator *allocator) { state->allocator = allocator; }
int THCState_getPeerToPeerAccess(THCState *state, int dev, int devToAccess) {
  API_BEGIN
  THArgCheck(dev >= 0 && dev < state->numDevices, 2, "%d is not a device", dev);
  THArgCheck(devToAccess >= 0 && devToAccess < state->numDevices, 3, "%d is not a device", devToAccess);
  if (dev == devToAccess) return 1;
  if (state->p2pOff[dev * state->numDevices + devToAccess]) return 0;
  int can = 0;
  THCudaCheck(cudaDeviceCanAccessPeer(&can, dev, devToAccess));
  return can;
  API_END_RET(0)
}
void THCState_setPeerToPeerAccess(THCState *state, int dev, int devToAccess, int enable) {
  API_BEGIN
  THArgCheck(dev >= 0 && dev < state->numDevices, 2, "%d is not a device", dev);
  THArgCheck(devToAccess >= 0 && devToAccess < state->numDevices, 3, "%d is not a device", devToAccess);
  if (enable && dev != devToAccess) {
    int can = 0;
    THCudaCheck(cudaDeviceCanAccessPeer(&can, dev, devToAccess));
    if (!can) th_error("p2p access from device %d to device %d is not possible", dev, devToAccess);
  }
  state->p2pOff[dev * state->numDevices + devToAccess] = enable ? 0 : 1;
  API_END
}
struct cudaDeviceProp *THCState_getCurrentDeviceProperties(THCState *state) {
  API_BEGIN
  const int d = current_device();
  if (!state->propsValid[d]) {
    THCudaCheck(cudaGetDeviceProperties(&state->props[d], d));
    state->propsValid[d] = 1;
  }
  return &state->props[d];
  API_END_RET(nullptr)
}
void *THCState_getCurrentDeviceScratchSpace(THCState *state) {
  API_BEGIN
  size_t bytes = 0;
  return thcb200_ctx_workspace(state_ctx(state), 128 * 1024, &bytes);
  API_END_RET(nullptr)
}
size_t THCState_getCurrentDeviceScratchSpaceSize(THCState *state) {
  API_BEGIN
  size_t bytes = 0;
  thcb200_ctx_workspace(state_ctx(state), 128 * 1024, &bytes);
  return bytes;
  API_END_RET(0)
}
void __THCudaCheck(cudaError_t err, const char *file, const int line) {
  API_BEGIN
  if (err != cudaSuccess) {
    cudaGetLastError();
    th_error("cuda runtime error (%d) : %s at %s:%d", (int)err, cudaGetErrorString(err), file, line);
  }
  API_END
}
cudaError_t THCudaMalloc(THCState *state, void **ptr, size_t size) {
  return malloc_with_gc_retry(state, state->allocator, state->allocator->state, ptr, size, state_stream(state));
}
void THCSetGCHandler(THCState *state, void (*gc_function)(void *data), void *data) {
  state->gcFunction = gc_function;
  state->gcData = data;
}
cudaError_t THCudaFree(THCState *state, void *ptr) { return state->allocator->free(state->allocator->state, ptr); }

struct THCB200StreamOwned {
  THCStream s;
  int owns;
};
THCStream *THCStream_new(int flags) {
  API_BEGIN
  THCB200StreamOwned *o = (THCB200StreamOwned *)calloc(1, sizeof(THCB200StreamOwned));
  o->s.device = current_device();
  THCudaCheck(cudaStreamCreateWithFlags(&o->s.stream, (unsigned)flags));
  o->s.refcount = 1;
  o->owns = 1;
  return &o->s;
  API_END_RET(nullptr)
}
THCStream *THCStream_defaultStream(int device) {
  THCB200StreamOwned *o = (THCB200StreamOwned *)calloc(1, sizeof(THCB200StreamOwned));
  o->s.device = device;
  o->s.stream = 0;
  o->s.refcount = 1;
  o->owns = 0;
  return &o->s;
}
THCStream *THCB200_streamFromRaw(cudaStream_t stream, int device) {
  THCB200StreamOwned *o = (THCB200StreamOwned *)calloc(1, sizeof(THCB200StreamOwned));
  o->s.device = device;
  o->s.stream = stream;
  o->s.refcount = 1;
  o->owns = 0;
  return &o->s;
}
void THCStream_retain(THCStream *self) { if (self) __sync_fetch_and_add(&self->refcount, 1); }
void THCStream_free(THCStream *self) {
  if (!self) return;
  if (__sync_sub_and_fetch(&self->refcount, 1) > 0) return;
  THCB200StreamOwned *o = (THCB200StreamOwned *)self;
  if (o->owns && self->stream) cudaStreamDestroy(self->stream);
  free(o);
}
struct thcb200_ctx *THCB200_currentContext(THCState *state) {
  API_BEGIN
  return state_ctx(state);
  API_END_RET(nullptr)
}

half THC_float2half(float a) {
  __half h = __float2half_rn(a);
  half r;
  memcpy(&r, &h, sizeof(r));
  return r;
}
float THC_half2float(half a) {
  __half h;
  memcpy(&h, &a, sizeof(h));
  return __half2float(h);
}

}  // extern "C"

// ======================================================================================
// Typed storage / tensor templates.  StorageT<R> and TensorT<R> have the layout of the C
// structs declared per type in THC.h.
// ======================================================================================
namespace {

template <typename R> struct StorageT {
  R *data;
  ptrdiff_t size;
  int refcount;
  char flag;
  THCDeviceAllocator *allocator;
  void *allocatorContext;
  StorageT *view;
  int device;
};

template <typename R> struct TensorT {
  long *size;
  long *stride;
  int nDimension;
  StorageT<R> *storage;
  ptrdiff_t storageOffset;
  int refcount;
  char flag;
};

template <typename R> struct RealTraits;
template <> struct RealTraits<unsigned char> { static constexpr int dtype = THCB200_U8; static constexpr bool fp = false; using acc = long; };
template <> struct RealTraits<char> { static constexpr int dtype = THCB200_I8; static constexpr bool fp = false; using acc = long; };
template <> struct RealTraits<short> { static constexpr int dtype = THCB200_I16; static constexpr bool fp = false; using acc = long; };
template <> struct RealTraits<int> { static constexpr int dtype = THCB200_I32; static constexpr bool fp = false; using acc = long; };
template <> struct RealTraits<long> { static constexpr int dtype = THCB200_I64; static constexpr bool fp = false; using acc = long; };
template <> struct RealTraits<half> { static constexpr int dtype = THCB200_F16; static constexpr bool fp = true; using acc = float; };
template <> struct RealTraits<float> { static constexpr int dtype = THCB200_F32; static constexpr bool fp = true; using acc = float; };
template <> struct RealTraits<double> { static constexpr int dtype = THCB200_F64; static constexpr bool fp = true; using acc = double; };

template <typename R> thcb200_scalar to_scalar(R v) { thcb200_scalar s; s.f = (double)v; s.i = (int64_t)v; return s; }
template <> thcb200_scalar to_scalar<half>(half v) { thcb200_scalar s; s.f = (double)THC_half2float(v); s.i = (int64_t)s.f; return s; }
thcb200_scalar scalar_f(double v) { thcb200_scalar s; s.f = v; s.i = (int64_t)v; return s; }
thcb200_scalar scalar_i(int64_t v) { thcb200_scalar s; s.f = (double)v; s.i = v; return s; }
template <typename R> R from_double(double v) { return (R)v; }
template <> half from_double<half>(double v) { return THC_float2half((float)v); }
template <typename R> double real_to_double(R v) { return (double)v; }
template <> double real_to_double<half>(half v) { return (double)THC_half2float(v); }

// Makes device `d` current for a scope.
struct DeviceGuard {
  int prev;
  bool changed;
  explicit DeviceGuard(int d) : prev(0), changed(false) {
    THCudaCheck(cudaGetDevice(&prev));
    if (d >= 0 && d != prev) { THCudaCheck(cudaSetDevice(d)); changed = true; }
  }
  ~DeviceGuard() { if (changed) cudaSetDevice(prev); }
};

// ---- storage -------------------------------------------------------------------------
template <typename R> StorageT<R> *storage_new(THCState *state, ptrdiff_t size) {
  THArgCheck(size >= 0, 2, "invalid size");
  StorageT<R> *s = (StorageT<R> *)calloc(1, sizeof(StorageT<R>));
  s->allocator = state->allocator;
  s->allocatorContext = state->allocator->state;
  s->refcount = 1;
  s->flag = TH_STORAGE_REFCOUNTED | TH_STORAGE_RESIZABLE | TH_STORAGE_FREEMEM;
  s->device = current_device();
  s->size = size;
  if (size > 0) {
    cudaError_t e = malloc_with_gc_retry(state, s->allocator, s->allocatorContext, (void **)&s->data, (size_t)size * sizeof(R), state_stream(state));
    if (e != cudaSuccess) {
      cudaGetLastError();
      free(s);
      th_error("cuda runtime error (%d) : %s (allocating %zu bytes)", (int)e, cudaGetErrorString(e), (size_t)size * sizeof(R));
    }
  }
  return s;
}

template <typename R> void storage_free(THCState *, StorageT<R> *s) {
  if (!s) return;
  if (!(s->flag & TH_STORAGE_REFCOUNTED)) return;
  if (__sync_sub_and_fetch(&s->refcount, 1) > 0) return;
  if ((s->flag & TH_STORAGE_FREEMEM) && s->data) {
    // with the storage's own device current, the block goes back in the order of THAT device's
    // current stream, whatever device the caller is working on
    DeviceGuard g(s->device);
    s->allocator->free(s->allocatorContext, s->data);
  }
  if ((s->flag & TH_STORAGE_FREEMEM) == 0 && s->view) storage_free<R>(nullptr, s->view);
  free(s);
}

template <typename R> void storage_resize(THCState *state, StorageT<R> *s, ptrdiff_t size) {
  THArgCheck(size >= 0, 2, "invalid size");
  if (!(s->flag & TH_STORAGE_RESIZABLE)) th_error("Trying to resize storage that is not resizable");
  if (size == s->size) return;
  // a storage lives on one device: it is reallocated and its old block freed with that device current
  DeviceGuard g(s->data ? s->device : -1);
  if (!s->data) s->device = current_device();
  R *nd = nullptr;
  if (size > 0) {
    cudaError_t e = malloc_with_gc_retry(state, s->allocator, s->allocatorContext, (void **)&nd, (size_t)size * sizeof(R), state_stream(state));
    if (e != cudaSuccess) { cudaGetLastError(); th_error("cuda runtime error (%d) : %s", (int)e, cudaGetErrorString(e)); }
    if (s->data && s->size > 0) {
      const ptrdiff_t keep = size < s->size ? size : s->size;
      THCudaCheck(cudaMemcpyAsync(nd, s->data, (size_t)keep * sizeof(R), cudaMemcpyDeviceToDevice, state_stream(state)));
    }
  }
  if (s->data && (s->flag & TH_STORAGE_FREEMEM)) {
    // the old block may still be read by work queued on the stream: the default allocator frees in
    // stream order; any other allocator gets a quiet stream first
    if (s->allocator->free != default_free) THCudaCheck(cudaStreamSynchronize(state_stream(state)));
    s->allocator->free(s->allocatorContext, s->data);
  }
  s->data = nd;
  s->size = size;
  s->flag |= TH_STORAGE_FREEMEM;
}

// ---- tensor --------------------------------------------------------------------------
template <typename R> TensorT<R> *tensor_alloc() {
  TensorT<R> *t = (TensorT<R> *)calloc(1, sizeof(TensorT<R>));
  t->refcount = 1;
  t->flag = TH_TENSOR_REFCOUNTED;
  return t;
}

template <typename R> ptrdiff_t tensor_nelement(const TensorT<R> *t) {
  if (t->nDimension == 0) return 0;
  ptrdiff_t n = 1;
  for (int d = 0; d < t->nDimension; ++d) n *= t->size[d];
  return n;
}

template <typename R> bool tensor_is_contiguous(const TensorT<R> *t) {
  long z = 1;
  for (int d = t->nDimension - 1; d >= 0; --d) {
    if (t->size[d] != 1) {
      if (t->stride[d] != z) return false;
      z *= t->size[d];
    }
  }
  return true;
}

template <typename R> bool tensor_same_size(const TensorT<R> *a, const TensorT<R> *b) {
  if (a->nDimension != b->nDimension) return false;
  for (int d = 0; d < a->nDimension; ++d)
    if (a->size[d] != b->size[d]) return false;
  return true;
}

// Gives the tensor nd dims of the given sizes; strides default to row-major when `stride`
// is null or an entry is negative.  The storage only ever grows.
template <typename R> void tensor_raw_resize(THCState *state, TensorT<R> *t, int nd, const long *size, const long *stride) {
  bool same = (nd == t->nDimension);
  for (int d = 0; same && d < nd; ++d) {
    if (size[d] != t->size[d]) same = false;
    if (stride && stride[d] >= 0 && stride[d] != t->stride[d]) same = false;
  }
  if (same) return;
  if (nd <= 0) { t->nDimension = 0; return; }
  // the new strides and the extent they need are worked out first and the storage is grown before
  // the tensor's own fields change: if the allocation fails the tensor is left as it was
  long new_stride[THCB200_MAX_DIMS > 32 ? THCB200_MAX_DIMS : 32];
  if (nd > (int)(sizeof(new_stride) / sizeof(new_stride[0]))) th_arg_error(1, CUTORCH_DIM_WARNING);
  ptrdiff_t extent = 1;
  for (int d = nd - 1; d >= 0; --d) {
    if (stride && stride[d] >= 0) new_stride[d] = stride[d];
    else new_stride[d] = (d == nd - 1) ? 1 : size[d + 1] * new_stride[d + 1];
    extent += (ptrdiff_t)(size[d] - 1) * new_stride[d];
  }
  if (extent + t->storageOffset > 0) {
    if (!t->storage) t->storage = storage_new<R>(state, 0);
    if (extent + t->storageOffset > t->storage->size) storage_resize<R>(state, t->storage, extent + t->storageOffset);
  }
  if (nd != t->nDimension) {
    t->size = (long *)realloc(t->size, sizeof(long) * nd);
    t->stride = (long *)realloc(t->stride, sizeof(long) * nd);
    t->nDimension = nd;
  }
  for (int d = 0; d < nd; ++d) { t->size[d] = size[d]; t->stride[d] = new_stride[d]; }
}

template <typename R> void tensor_raw_set(THCState *state, TensorT<R> *t, StorageT<R> *storage, ptrdiff_t offset, int nd,
                                          const long *size, const long *stride) {
  THArgCheck(offset >= 0, 3, "Tensor: invalid storage offset");
  if (t->storage != storage) {
    if (t->storage) storage_free<R>(state, t->storage);
    t->storage = storage;
    if (storage) __sync_fetch_and_add(&storage->refcount, 1);
  }
  t->storageOffset = offset;
  tensor_raw_resize<R>(state, t, nd, size, stride);
}

template <typename R> void tensor_free(THCState *state, TensorT<R> *t) {
  if (!t) return;
  if (!(t->flag & TH_TENSOR_REFCOUNTED)) return;
  if (__sync_sub_and_fetch(&t->refcount, 1) > 0) return;
  free(t->size);
  free(t->stride);
  if (t->storage) storage_free<R>(state, t->storage);
  free(t);
}

template <typename R> TensorT<R> *tensor_new_with_tensor(THCState *state, TensorT<R> *src) {
  TensorT<R> *t = tensor_alloc<R>();
  tensor_raw_set<R>(state, t, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  return t;
}

template <typename R> void tensor_narrow(THCState *state, TensorT<R> *self, TensorT<R> *src, int dim, long first, long size) {
  if (!src) src = self;
  THArgCheck(dim >= 0 && dim < src->nDimension, 3, "out of range");
  THArgCheck(first >= 0 && first < src->size[dim], 4, "out of range");
  THArgCheck(size > 0 && first + size <= src->size[dim], 5, "out of range");
  if (self != src) tensor_raw_set<R>(state, self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  if (first > 0) self->storageOffset += first * self->stride[dim];
  self->size[dim] = size;
}

template <typename R> void tensor_select(THCState *state, TensorT<R> *self, TensorT<R> *src, int dim, long index) {
  if (!src) src = self;
  THArgCheck(src->nDimension > 1, 1, "cannot select on a vector");
  THArgCheck(dim >= 0 && dim < src->nDimension, 3, "out of range");
  THArgCheck(index >= 0 && index < src->size[dim], 4, "out of range");
  if (self != src) tensor_raw_set<R>(state, self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  tensor_narrow<R>(state, self, nullptr, dim, index, 1);
  for (int d = dim; d < self->nDimension - 1; ++d) {
    self->size[d] = self->size[d + 1];
    self->stride[d] = self->stride[d + 1];
  }
  self->nDimension--;
}

template <typename R> void tensor_transpose(THCState *state, TensorT<R> *self, TensorT<R> *src, int d1, int d2) {
  if (!src) src = self;
  THArgCheck(d1 >= 0 && d1 < src->nDimension, 1, "out of range");
  THArgCheck(d2 >= 0 && d2 < src->nDimension, 2, "out of range");
  if (self != src) tensor_raw_set<R>(state, self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  if (d1 == d2) return;
  long z = self->stride[d1]; self->stride[d1] = self->stride[d2]; self->stride[d2] = z;
  z = self->size[d1]; self->size[d1] = self->size[d2]; self->size[d2] = z;
}

template <typename R> void tensor_squeeze1d(THCState *state, TensorT<R> *self, TensorT<R> *src, int dim) {
  if (!src) src = self;
  THArgCheck(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  if (self != src) tensor_raw_set<R>(state, self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  if (src->size[dim] == 1 && src->nDimension > 1) {
    for (int d = dim; d < self->nDimension - 1; ++d) {
      self->size[d] = self->size[d + 1];
      self->stride[d] = self->stride[d + 1];
    }
    self->nDimension--;
  }
}

template <typename R> void tensor_resize_as(THCState *state, TensorT<R> *self, TensorT<R> *src) {
  if (!tensor_same_size<R>(self, src)) tensor_raw_resize<R>(state, self, src->nDimension, src->size, nullptr);
}

// expand (lib/THC/generic/THCTensor.c:297-330; the geometry rule is TH's inferExpandGeometry): the
// tensor's dims are matched to the last dims of `sizes`; a dim of size 1 (or a new leading dim) is
// repeated with stride 0, any other dim must already have the requested size (-1 keeps it).
template <typename R> void tensor_expand(THCState *state, TensorT<R> *r, TensorT<R> *t, const long *sizes, int nsizes) {
  THArgCheck(t->nDimension > 0, 0, "can't expand an empty tensor");
  THArgCheck(nsizes >= t->nDimension, 1, "the number of sizes provided must be greater or equal to the number of dimensions in the tensor");
  if (nsizes > THCB200_MAX_DIMS) th_arg_error(1, CUTORCH_DIM_WARNING);
  long esize[THCB200_MAX_DIMS], estride[THCB200_MAX_DIMS];
  for (int i = nsizes - 1; i >= 0; --i) {
    const int d = i - (nsizes - t->nDimension);     // the tensor's dim under position i, or negative
    long size = d >= 0 ? t->size[d] : 1;
    long stride = d >= 0 ? t->stride[d] : 0;
    long want = sizes[i];
    if (want == -1) {
      if (d < 0) th_error("The expanded size of the tensor (-1) isn't allowed in a leading, non-existing dimension %d", i);
      want = size;
    }
    if (size != want) {
      if (size != 1) th_error("The expanded size of the tensor (%ld) must match the existing size (%ld) at non-singleton dimension %d.", want, size, i);
      size = want;
      stride = 0;
    }
    esize[i] = size;
    estride[i] = stride;
  }
  tensor_raw_set<R>(state, r, t->storage, t->storageOffset, nsizes, esize, estride);
}

// ---- descriptors and the math layer ----------------------------------------------------
template <typename R> thcb200_tensor describe(const TensorT<R> *t) {
  thcb200_tensor d;
  memset(&d, 0, sizeof(d));
  d.dtype = RealTraits<R>::dtype;
  d.ndim = t->nDimension;
  if (t->nDimension > THCB200_MAX_DIMS) th_arg_error(2, CUTORCH_DIM_WARNING);
  for (int i = 0; i < t->nDimension; ++i) { d.sizes[i] = t->size[i]; d.strides[i] = t->stride[i]; }
  d.data = (t->storage && t->storage->data) ? (void *)(t->storage->data + t->storageOffset) : nullptr;
  // Every kernel trusts the view: the smallest and the largest element offset it can reach (as
  // canUse32BitIndexMath works out the largest, lib/THC/THCTensorTypeUtils.cu:220-245) have to lie
  // inside the storage.  cutorch's kernels assert on their offsets in debug builds
  // (lib/THC/THCTensorInfo.cuh:228-278); here the view is refused on the host, before any launch.
  if (t->storage && t->nDimension > 0) {
    int64_t lo = 0, hi = 0;
    if (thcb200_view_extent(&d, &lo, &hi) == 1) {
      const int64_t first = (int64_t)t->storageOffset + lo, last = (int64_t)t->storageOffset + hi;
      if (first < 0 || last >= (int64_t)t->storage->size)
        th_error("tensor view reaches elements %lld..%lld of a storage of %lld elements", (long long)first, (long long)last,
                 (long long)t->storage->size);
    }
  }
  return d;
}

void check_core(int rc, int arg = 2) {
  if (rc == 0) return;
  if (rc == THCB200_ERR_DIMS) th_arg_error(arg, CUTORCH_DIM_WARNING);
  if (rc == THCB200_ERR_SIZE) th_arg_error(arg, "sizes do not match");
  th_error("%s", thcb200_last_error());
}

template <typename R> void check_gpu1(THCState *, const TensorT<R> *t, int cur) {
  if (t && t->storage && t->storage->data && t->storage->device != cur) th_error("arguments are located on different GPUs");
}
template <typename R> void check_gpu(THCState *state, std::initializer_list<const TensorT<R> *> ts) {
  const int cur = current_device();
  for (const TensorT<R> *t : ts) check_gpu1<R>(state, t, cur);
}

template <typename R>
void pointwise(THCState *state, int op, TensorT<R> *out, TensorT<R> *a, TensorT<R> *b, TensorT<R> *c, thcb200_scalar s0,
               thcb200_scalar s1, int flags = 0) {
  thcb200_tensor dout = describe<R>(out), da, db, dc;
  int nin = 0;
  if (a) { da = describe<R>(a); nin = 1; }
  if (b) { db = describe<R>(b); nin = 2; }
  if (c) { dc = describe<R>(c); nin = 3; }
  check_core(thcb200_pointwise_ex(state_ctx(state), op, &dout, a ? &da : nullptr, b ? &db : nullptr, c ? &dc : nullptr, nin,
                                  s0, s1, (void *)state_stream(state), flags));
}

const thcb200_scalar kZero = {0.0, 0};

// self = op(src) (in place when self == src)
template <typename R> void unary(THCState *state, int op, TensorT<R> *self, TensorT<R> *src, thcb200_scalar s0 = kZero,
                                 thcb200_scalar s1 = kZero) {
  check_gpu<R>(state, {self, src});
  if (self != src) tensor_resize_as<R>(state, self, src);
  pointwise<R>(state, op, self, src, nullptr, nullptr, s0, s1);
}

// self = op(src1, src2) (in place when self == src1)
template <typename R> void binary(THCState *state, int op, TensorT<R> *self, TensorT<R> *src1, TensorT<R> *src2,
                                  thcb200_scalar s0 = kZero) {
  check_gpu<R>(state, {self, src1, src2});
  THArgCheck(tensor_nelement<R>(src1) == tensor_nelement<R>(src2), 3, "sizes do not match");
  if (self != src1) tensor_resize_as<R>(state, self, src1);
  pointwise<R>(state, op, self, src1, src2, nullptr, s0, kZero);
}

// byte ranges [lo, hi) of the elements a view can touch
template <typename R> bool may_alias(const TensorT<R> *a, const TensorT<R> *b) {
  if (!a->storage || !b->storage || !a->storage->data || !b->storage->data) return false;
  auto range = [](const TensorT<R> *t, const R *&lo, const R *&hi) {
    ptrdiff_t mn = 0, mx = 0;
    for (int d = 0; d < t->nDimension; ++d) {
      if (t->size[d] == 0) { lo = hi = nullptr; return; }
      const ptrdiff_t span = (ptrdiff_t)(t->size[d] - 1) * t->stride[d];
      if (span > 0) mx += span; else mn += span;
    }
    lo = t->storage->data + t->storageOffset + mn;
    hi = t->storage->data + t->storageOffset + mx + 1;
  };
  const R *alo, *ahi, *blo, *bhi;
  range(a, alo, ahi);
  range(b, blo, bhi);
  if (!alo || !blo) return false;
  return alo < bhi && blo < ahi;
}

// ---- copies, same device or across devices (THC_copyTensor, lib/THC/THCTensorCopy.cu:24-205) ----

template <typename R> int tensor_device(const TensorT<R> *t, int fallback) {
  return (t->storage && t->storage->data) ? t->storage->device : fallback;
}

// lets kernels on `from` address memory of `to`
bool enable_peer_access(int from, int to) {
  if (from == to) return true;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, from, to) != cudaSuccess || !can) { cudaGetLastError(); return false; }
  DeviceGuard g(from);
  const cudaError_t e = cudaDeviceEnablePeerAccess(to, 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (e != cudaErrorPeerAccessAlreadyEnabled) return false;
  }
  // blocks of the stream-ordered allocator live in `to`'s default pool, which grants access per device
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, to) == cudaSuccess) {
    cudaMemAccessDesc desc;
    memset(&desc, 0, sizeof(desc));
    desc.location.type = cudaMemLocationTypeDevice;
    desc.location.id = from;
    desc.flags = cudaMemAccessFlagsProtReadWrite;
    if (cudaMemPoolSetAccess(pool, &desc, 1) != cudaSuccess) { cudaGetLastError(); return false; }
  } else {
    cudaGetLastError();
  }
  return true;
}

// `waiter` (a stream of device wdev) waits for everything queued so far on `signal` (device sdev)
void stream_wait_stream(int wdev, cudaStream_t waiter, int sdev, cudaStream_t signal) {
  cudaEvent_t ev;
  {
    DeviceGuard g(sdev);
    THCudaCheck(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    THCudaCheck(cudaEventRecord(ev, signal));
  }
  {
    DeviceGuard g(wdev);
    THCudaCheck(cudaStreamWaitEvent(waiter, ev, 0));
  }
  THCudaCheck(cudaEventDestroy(ev));
}

template <typename R> TensorT<R> *tensor_new_contiguous(THCState *state, TensorT<R> *t);

// dst = convert(src) with both tensors on the current device
template <typename RD, typename RS> void copy_on_device(THCState *state, TensorT<RD> *dst, TensorT<RS> *src, int flags) {
  const ptrdiff_t n = tensor_nelement<RD>(dst);
  if constexpr (std::is_same<RD, RS>::value) {
    if ((tensor_is_contiguous<RD>(dst) && tensor_is_contiguous<RS>(src)) || n == 1) {
      THCudaCheck(cudaMemcpyAsync(dst->storage->data + dst->storageOffset, src->storage->data + src->storageOffset,
                                  (size_t)n * sizeof(RD), cudaMemcpyDeviceToDevice, state_stream(state)));
      return;
    }
    pointwise<RD>(state, THCB200_OP_COPY, dst, src, nullptr, nullptr, kZero, kZero, flags);
  } else {
    thcb200_tensor dd = describe<RD>(dst), ds = describe<RS>(src);
    check_core(thcb200_copy_convert(state_ctx(state), &dd, &ds, (void *)state_stream(state)));
  }
}

// The copy runs on the source device, on that device's current stream, bracketed by a two-way
// wait with the destination device's current stream.  Contiguous same-type tensors go through
// cudaMemcpyAsync; anything else through the copy / convert kernel writing the peer's memory
// directly over NVLink when peer access can be enabled, else through contiguous temporaries.
template <typename RD, typename RS>
void copy_across_devices(THCState *state, TensorT<RD> *dst, TensorT<RS> *src, int src_dev, int dst_dev, int flags) {
  const ptrdiff_t n = tensor_nelement<RD>(dst);
  cudaStream_t sstream = THCState_getCurrentStreamOnDevice(state, src_dev);
  cudaStream_t dstream = THCState_getCurrentStreamOnDevice(state, dst_dev);
  stream_wait_stream(src_dev, sstream, dst_dev, dstream);
  {
    DeviceGuard g(src_dev);
    const bool memcpy_ok = std::is_same<RD, RS>::value &&
                           ((tensor_is_contiguous<RD>(dst) && tensor_is_contiguous<RS>(src)) || n == 1);
    const bool peer = !state->p2pOff[src_dev * state->numDevices + dst_dev] && enable_peer_access(src_dev, dst_dev);
    if (memcpy_ok) {
      THCudaCheck(cudaMemcpyPeerAsync(dst->storage->data + dst->storageOffset, dst_dev, src->storage->data + src->storageOffset,
                                      src_dev, (size_t)n * sizeof(RD), sstream));
    } else if (peer) {
      copy_on_device<RD, RS>(state, dst, src, flags);   // kernel on the source device, stores to the peer
    } else {
      // no peer access: dense temporaries of dst's type on both sides and one memcpy between them
      TensorT<RD> *sc = tensor_alloc<RD>();
      tensor_raw_resize<RD>(state, sc, dst->nDimension, dst->size, nullptr);
      copy_on_device<RD, RS>(state, sc, src, 0);
      TensorT<RD> *dc;
      {
        DeviceGuard gd(dst_dev);
        dc = tensor_alloc<RD>();
        tensor_raw_resize<RD>(state, dc, dst->nDimension, dst->size, nullptr);
      }
      THCudaCheck(cudaMemcpyPeerAsync(dc->storage->data, dst_dev, sc->storage->data, src_dev, (size_t)n * sizeof(RD), sstream));
      stream_wait_stream(dst_dev, dstream, src_dev, sstream);
      {
        DeviceGuard gd(dst_dev);
        copy_on_device<RD, RD>(state, dst, dc, flags);
        tensor_free<RD>(state, dc);
      }
      tensor_free<RD>(state, sc);
    }
  }
  stream_wait_stream(dst_dev, dstream, src_dev, sstream);
}

template <typename RD, typename RS> void copy_any(THCState *state, TensorT<RD> *dst, TensorT<RS> *src, int flags) {
  THArgCheck(tensor_nelement<RD>(dst) == tensor_nelement<RS>(src), 2, "sizes do not match");
  if (tensor_nelement<RD>(dst) == 0) return;
  const int cur = current_device();
  const int sd = tensor_device<RS>(src, cur), dd = tensor_device<RD>(dst, cur);
  if (sd == dd) {
    DeviceGuard g(sd);
    copy_on_device<RD, RS>(state, dst, src, flags);
  } else {
    copy_across_devices<RD, RS>(state, dst, src, sd, dd, flags);
  }
}

template <typename R> void tensor_copy(THCState *state, TensorT<R> *self, TensorT<R> *src, int flags = 0) {
  if (self == src) return;
  copy_any<R, R>(state, self, src, flags);
}

template <typename RD, typename RS> void tensor_copy_convert(THCState *state, TensorT<RD> *dst, TensorT<RS> *src) {
  copy_any<RD, RS>(state, dst, src, 0);
}

template <typename R> TensorT<R> *tensor_new_contiguous(THCState *state, TensorT<R> *t) {
  if (tensor_is_contiguous<R>(t)) { __sync_fetch_and_add(&t->refcount, 1); return t; }
  TensorT<R> *c = tensor_alloc<R>();
  tensor_raw_resize<R>(state, c, t->nDimension, t->size, nullptr);
  tensor_copy<R>(state, c, t);
  return c;
}

template <typename R> TensorT<R> *tensor_new_clone(THCState *state, TensorT<R> *t) {
  TensorT<R> *c = tensor_alloc<R>();
  tensor_raw_resize<R>(state, c, t->nDimension, t->size, nullptr);
  tensor_copy<R>(state, c, t);
  return c;
}

// out = t + value * (src1 (*|/) src2).  cutorch copies t into self and then updates self in
// place (lib/THC/generic/THCTensorMathPointwise.cu:582-629); when self shares no memory with
// src1/src2 the copy is folded into one four-operand kernel, which computes the same values.
template <typename R> void addc(THCState *state, int op, TensorT<R> *self, TensorT<R> *t, R value, TensorT<R> *src1,
                                TensorT<R> *src2) {
  check_gpu<R>(state, {self, t, src1, src2});
  THArgCheck(tensor_nelement<R>(src1) == tensor_nelement<R>(src2), 3, "sizes do not match");
  if (self != t) {
    tensor_resize_as<R>(state, self, t);
    if (!may_alias<R>(self, src1) && !may_alias<R>(self, src2) && !may_alias<R>(self, t)) {
      pointwise<R>(state, op, self, t, src1, src2, to_scalar<R>(value), kZero);
      return;
    }
    tensor_copy<R>(state, self, t);
  }
  pointwise<R>(state, op, self, self, src1, src2, to_scalar<R>(value), kZero);
}

template <typename R> R negate(R v) { return (R)(-v); }
template <> half negate<half>(half v) { return THC_float2half(-THC_half2float(v)); }
template <typename R> bool is_one(R v) { return v == (R)1; }
template <> bool is_one<half>(half v) { return THC_half2float(v) == 1.0f; }

// cross product along `dimension` of two tensors holding 3-vectors there
// (lib/THC/generic/THCTensorMathPointwise.cu:111-144): out_i = x_j * y_k - x_k * y_j.
template <typename R> void cross(THCState *state, TensorT<R> *self, TensorT<R> *x, TensorT<R> *y, int dimension) {
  check_gpu<R>(state, {self, x, y});
  THArgCheck(x->nDimension == y->nDimension, 2, "inconsistent tensor dimension");
  for (int i = 0; i < x->nDimension; ++i) THArgCheck(x->size[i] == y->size[i], 2, "inconsistent tensor sizes");
  THArgCheck(dimension >= 0 && dimension < x->nDimension, 3, "dimension out of range");
  THArgCheck(x->size[dimension] == 3, 3, "dimension must have size 3");
  TensorT<R> *xs = x, *ys = y;
  bool ox = false, oy = false;
  if (self == x || may_alias<R>(self, x)) { xs = tensor_new_clone<R>(state, x); ox = true; }
  if (self == y || may_alias<R>(self, y)) { ys = tensor_new_clone<R>(state, y); oy = true; }
  tensor_resize_as<R>(state, self, xs);
  for (int i = 0; i < 3; ++i) {
    const int j = (i + 1) % 3, k = (i + 2) % 3;
    TensorT<R> *o = tensor_new_with_tensor<R>(state, self), *xj = tensor_new_with_tensor<R>(state, xs),
               *xk = tensor_new_with_tensor<R>(state, xs), *yj = tensor_new_with_tensor<R>(state, ys),
               *yk = tensor_new_with_tensor<R>(state, ys);
    tensor_narrow<R>(state, o, nullptr, dimension, i, 1);
    tensor_narrow<R>(state, xj, nullptr, dimension, j, 1);
    tensor_narrow<R>(state, xk, nullptr, dimension, k, 1);
    tensor_narrow<R>(state, yj, nullptr, dimension, j, 1);
    tensor_narrow<R>(state, yk, nullptr, dimension, k, 1);
    pointwise<R>(state, THCB200_OP_MUL, o, xj, yk, nullptr, kZero, kZero);
    pointwise<R>(state, THCB200_OP_ADDCMUL, o, o, xk, yj, scalar_i(-1), kZero);
    tensor_free<R>(state, o); tensor_free<R>(state, xj); tensor_free<R>(state, xk);
    tensor_free<R>(state, yj); tensor_free<R>(state, yk);
  }
  if (ox) tensor_free<R>(state, xs);
  if (oy) tensor_free<R>(state, ys);
}

// ---- reductions ----------------------------------------------------------------------
template <typename R> void resize_reduced(THCState *state, TensorT<R> *out, const long *src_size, int nd, long dim) {
  long sz[THCB200_MAX_DIMS];
  for (int i = 0; i < nd; ++i) sz[i] = src_size[i];
  sz[dim] = 1;
  tensor_raw_resize<R>(state, out, nd, sz, nullptr);
}

template <typename R>
void reduce_dim(THCState *state, int rop, int pre, thcb200_scalar s, TensorT<R> *self, TensorT<R> *src, long dim, int keepdim,
                int post_kind = THCB200_POST_NONE, thcb200_scalar post_value = kZero) {
  check_gpu<R>(state, {self, src});
  THArgCheck(src->nDimension <= THCB200_MAX_DIMS, 2, CUTORCH_DIM_WARNING);
  THArgCheck(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  THArgCheck(self != src, 1, "output must differ from the input");
  resize_reduced<R>(state, self, src->size, src->nDimension, dim);
  thcb200_tensor dout = describe<R>(self), din = describe<R>(src);
  check_core(thcb200_reduce_dim_post(state_ctx(state), rop, pre, s, post_kind, post_value, &dout, &din, (int)dim,
                                     (void *)state_stream(state)));
  if (!keepdim) tensor_squeeze1d<R>(state, self, nullptr, (int)dim);
}

template <typename R>
void reduce_dim_index(THCState *state, int rop, TensorT<R> *values, TensorT<long> *indices, TensorT<R> *src, long dim, int keepdim) {
  check_gpu<R>(state, {values, src});
  check_gpu<long>(state, {indices});
  THArgCheck(src->nDimension <= THCB200_MAX_DIMS, 4, CUTORCH_DIM_WARNING);
  THArgCheck(dim >= 0 && dim < src->nDimension, 5, "dimension out of range");
  THArgCheck(values != src, 1, "output must differ from the input");
  resize_reduced<R>(state, values, src->size, src->nDimension, dim);
  resize_reduced<long>(state, indices, src->size, src->nDimension, dim);
  thcb200_tensor dv = describe<R>(values), di = describe<long>(indices), din = describe<R>(src);
  check_core(thcb200_reduce_dim_index(state_ctx(state), rop, &dv, &di, &din, (int)dim, (void *)state_stream(state)), 4);
  if (!keepdim) {
    tensor_squeeze1d<R>(state, values, nullptr, (int)dim);
    tensor_squeeze1d<long>(state, indices, nullptr, (int)dim);
  }
}

// Full reduction to the host.  The core returns a double (floating types) or int64.
template <typename R> double reduce_all_f(THCState *state, int rop, int pre, thcb200_scalar s, TensorT<R> *self) {
  check_gpu<R>(state, {self});
  thcb200_tensor d = describe<R>(self);
  union { double f; int64_t i; } r;
  r.i = 0;
  check_core(thcb200_reduce_all_host(state_ctx(state), rop, pre, s, &d, &r, (void *)state_stream(state)), 1);
  return RealTraits<R>::fp ? r.f : (double)r.i;
}
template <typename R> int64_t reduce_all_i(THCState *state, int rop, int pre, thcb200_scalar s, TensorT<R> *self) {
  check_gpu<R>(state, {self});
  thcb200_tensor d = describe<R>(self);
  union { double f; int64_t i; } r;
  r.i = 0;
  check_core(thcb200_reduce_all_host(state_ctx(state), rop, pre, s, &d, &r, (void *)state_stream(state)), 1);
  return RealTraits<R>::fp ? (int64_t)r.f : r.i;
}
template <typename R> typename RealTraits<R>::acc reduce_all_acc(THCState *state, int rop, int pre, thcb200_scalar s, TensorT<R> *self) {
  using A = typename RealTraits<R>::acc;
  if (RealTraits<R>::fp) return (A)reduce_all_f<R>(state, rop, pre, s, self);
  return (A)reduce_all_i<R>(state, rop, pre, s, self);
}

// self = inclusive scan of src along `dimension` (THCTensor_(scanDim),
// lib/THC/generic/THCTensorMathScan.cu:76-104)
template <typename R> void scan_dim(THCState *state, int rop, TensorT<R> *self, TensorT<R> *src, long dimension) {
  check_gpu<R>(state, {self, src});
  THArgCheck(dimension >= 0 && dimension < src->nDimension, 3, "dimension %d out of range", (int)dimension + TH_INDEX_BASE);
  if (self != src) tensor_resize_as<R>(state, self, src);
  thcb200_tensor dout = describe<R>(self), din = describe<R>(src);
  check_core(thcb200_scan_dim(state_ctx(state), rop, &dout, &din, (int)dimension, (void *)state_stream(state)));
}

// self = lower / upper triangle of the matrix src (lib/THC/generic/THCTensorMathPairwise.cu:169-233)
template <typename R> void tri(THCState *state, int upper, TensorT<R> *self, TensorT<R> *src, long k) {
  check_gpu<R>(state, {self, src});
  THArgCheck(src->nDimension == 2, 1, "expected a matrix");
  if (self != src) tensor_resize_as<R>(state, self, src);
  thcb200_tensor dout = describe<R>(self), din = describe<R>(src);
  check_core(thcb200_tri(state_ctx(state), upper, (int64_t)k, &dout, &din, (void *)state_stream(state)));
}

// renorm: every slice src.select(dimension, j) whose p-norm exceeds maxnorm is scaled to norm
// maxnorm (lib/THC/generic/THCTensorMathReduce.cu:47-74).  Composed from the dimension
// reductions (sums of |x|^p over every other dim), the factor step and a broadcast multiply;
// no transposed clone of the tensor is made.
template <typename R>
void renorm(THCState *state, TensorT<R> *self, TensorT<R> *src, R value, long dimension, R maxnorm) {
  check_gpu<R>(state, {self, src});
  THArgCheck(dimension >= 0 && dimension < src->nDimension, 3, "invalid dimension");
  THArgCheck(real_to_double<R>(value) > 0, 2, "non-positive-norm not supported");
  THArgCheck(src->nDimension > 1, 1, "need at least 2 dimensions");
  const double p = real_to_double<R>(value);
  thcb200_ctx *ctx = state_ctx(state);
  void *st = (void *)state_stream(state);
  if (self != src) tensor_resize_as<R>(state, self, src);
  {  // slices that are short dense runs: one pass
    thcb200_tensor dout = describe<R>(self), din = describe<R>(src);
    const int rc = thcb200_renorm_rows(ctx, &dout, &din, (int)dimension, p, real_to_double<R>(maxnorm), st);
    if (rc == THCB200_OK) return;
    if (rc != THCB200_ERR_UNSUPPORTED) check_core(rc);
  }
  // sums of |x|^p over every dim but `dimension`, one dim at a time from the innermost outward
  TensorT<R> *cur = src;
  bool first = true;
  for (int d = src->nDimension - 1; d >= 0; --d) {
    if (d == dimension) continue;
    TensorT<R> *next = tensor_alloc<R>();
    resize_reduced<R>(state, next, cur->size, cur->nDimension, d);
    const int pre = !first ? THCB200_PRE_IDENTITY : (p == 1.0 ? THCB200_PRE_ABS : (p == 2.0 ? THCB200_PRE_SQUARE : THCB200_PRE_POWABS));
    thcb200_tensor dout = describe<R>(next), din = describe<R>(cur);
    thcb200_scalar s = {p, 0};
    const int rc = thcb200_reduce_dim(ctx, THCB200_RED_SUM, pre, s, &dout, &din, d, st);
    if (cur != src) tensor_free<R>(state, cur);
    cur = next;
    first = false;
    if (rc) { tensor_free<R>(state, cur); check_core(rc); }
  }
  // cur: all sizes 1 except `dimension`
  thcb200_tensor dsum = describe<R>(cur);
  int rc = thcb200_renorm_factor(ctx, &dsum, &dsum, p, real_to_double<R>(maxnorm), st);
  if (rc == 0) {
    // the factors seen through src's shape: stride 0 along every other dim
    long strides[THCB200_MAX_DIMS];
    for (int d = 0; d < src->nDimension; ++d) strides[d] = d == dimension ? cur->stride[d] : 0;
    TensorT<R> *wide = tensor_alloc<R>();
    tensor_raw_set<R>(state, wide, cur->storage, cur->storageOffset, src->nDimension, src->size, strides);
    thcb200_tensor dout = describe<R>(self), din = describe<R>(src), dw = describe<R>(wide);
    rc = thcb200_pointwise(ctx, THCB200_OP_MUL, &dout, &din, &dw, nullptr, 2, kZero, kZero, st);
    tensor_free<R>(state, wide);
  }
  tensor_free<R>(state, cur);
  check_core(rc);
}

// Half tensors renorm as float tensors and round once at the end (the half parity target is
// FloatTensor math on the half values); sums of |x|^p would overflow half anyway.
template <>
void renorm<half>(THCState *state, TensorT<half> *self, TensorT<half> *src, half value, long dimension, half maxnorm) {
  check_gpu<half>(state, {self, src});
  THArgCheck(dimension >= 0 && dimension < src->nDimension, 3, "invalid dimension");
  THArgCheck(src->nDimension > 1, 1, "need at least 2 dimensions");
  THArgCheck(THC_half2float(value) > 0, 2, "non-positive-norm not supported");
  if (self != src) tensor_resize_as<half>(state, self, src);
  {
    thcb200_tensor dout = describe<half>(self), din = describe<half>(src);
    const int rc = thcb200_renorm_rows(state_ctx(state), &dout, &din, (int)dimension, (double)THC_half2float(value),
                                       (double)THC_half2float(maxnorm), (void *)state_stream(state));
    if (rc == THCB200_OK) return;
    if (rc != THCB200_ERR_UNSUPPORTED) check_core(rc);
  }
  TensorT<float> *wide = tensor_alloc<float>();
  tensor_raw_resize<float>(state, wide, src->nDimension, src->size, nullptr);
  try {
    tensor_copy_convert<float, half>(state, wide, src);
    renorm<float>(state, wide, wide, THC_half2float(value), dimension, THC_half2float(maxnorm));
    tensor_copy_convert<half, float>(state, self, wide);
  } catch (...) {
    tensor_free<float>(state, wide);
    throw;
  }
  tensor_free<float>(state, wide);
}

// ---- construction calls that are thin callers of fill / copy / sumall ------------------------
// (lib/THC/generic/THCTensorMath.cu:36-82,358-422).  A diagonal is a 1-D view with stride
// stride0 + stride1, so diag / eye / trace need no kernels of their own.
thcb200_scalar one_scalar() { thcb200_scalar s; s.f = 1.0; s.i = 1; return s; }

template <typename R> void fill_with(THCState *state, TensorT<R> *t, thcb200_scalar v) {
  pointwise<R>(state, THCB200_OP_FILL, t, nullptr, nullptr, nullptr, v, kZero);
}
// the k-th diagonal of a matrix as a 1-D view of `len` elements (k > 0 above the main diagonal)
template <typename R> TensorT<R> *diagonal_view(THCState *state, TensorT<R> *m, long k, long len) {
  TensorT<R> *d = tensor_alloc<R>();
  const long start = k >= 0 ? k * m->stride[1] : -k * m->stride[0];
  const long stride = m->stride[0] + m->stride[1];
  tensor_raw_set<R>(state, d, m->storage, m->storageOffset + start, 1, &len, &stride);
  return d;
}
template <typename R> void diag(THCState *state, TensorT<R> *self, TensorT<R> *src, long k) {
  check_gpu<R>(state, {self, src});
  THArgCheck(src->nDimension == 2 || src->nDimension == 1, 1, "expected a matrix or a vector");
  if (src->nDimension == 2) {
    const long size0 = src->size[0], size1 = src->size[1];
    long len = k > 0 ? std::min(size0, size1 - k) : std::min(size0 + k, size1);
    if (len < 0) len = 0;
    tensor_raw_resize<R>(state, self, 1, &len, nullptr);
    if (len == 0) return;
    TensorT<R> *d = diagonal_view<R>(state, src, k, len);
    try { tensor_copy<R>(state, self, d); } catch (...) { tensor_free<R>(state, d); throw; }
    tensor_free<R>(state, d);
  } else {
    const long n = (long)tensor_nelement<R>(src);
    const long side = k > 0 ? n + k : n - k;
    const long sizes[2] = {side, side};
    TensorT<R> *keep = src;
    __sync_fetch_and_add(&keep->refcount, 1);            // src may be self
    TensorT<R> *from = src;
    if (self == src) { from = tensor_alloc<R>(); tensor_raw_resize<R>(state, from, 1, &n, nullptr); tensor_copy<R>(state, from, src); }
    tensor_raw_resize<R>(state, self, 2, sizes, nullptr);
    fill_with<R>(state, self, kZero);
    if (n > 0) {
      TensorT<R> *d = diagonal_view<R>(state, self, k, n);
      try { tensor_copy<R>(state, d, from); } catch (...) { tensor_free<R>(state, d); throw; }
      tensor_free<R>(state, d);
    }
    if (from != src) tensor_free<R>(state, from);
    tensor_free<R>(state, keep);
  }
}
template <typename R> void eye(THCState *state, TensorT<R> *self, long n, long m) {
  check_gpu<R>(state, {self});
  THArgCheck(n > 0, 1, "invalid argument");
  if (m <= 0) m = n;
  const long sizes[2] = {n, m};
  tensor_raw_resize<R>(state, self, 2, sizes, nullptr);
  fill_with<R>(state, self, kZero);
  TensorT<R> *d = diagonal_view<R>(state, self, 0, std::min(n, m));
  try { fill_with<R>(state, d, one_scalar()); } catch (...) { tensor_free<R>(state, d); throw; }
  tensor_free<R>(state, d);
}

// cat (lib/THC/generic/THCTensorMath.cu:84-260): the result is sized from the inputs (missing
// trailing dims count as 1, empty inputs are skipped, a dimension of -1 in cutorch's 1-based
// convention means the last one) and every input is copied into its narrowed slice of the result.
// The reference batches many small contiguous inputs into one launch; here each input is one copy.
template <typename R> void cat_array(THCState *state, TensorT<R> *result, TensorT<R> **inputs, int num, int dimension) {
  auto dim_size = [](const TensorT<R> *t, int i) -> long { return i < t->nDimension ? t->size[i] : std::min(t->nDimension, 1); };
  int max_dim = dimension + 1;
  for (int i = 0; i < num; ++i) max_dim = std::max(max_dim, inputs[i]->nDimension);
  int cat_dim = dimension;
  if (dimension + TH_INDEX_BASE == -1) cat_dim = max_dim ? max_dim - 1 : 0;
  if (num <= 0) th_arg_error(3, "invalid number of inputs");
  if (cat_dim < 0) th_arg_error(4, "invalid dimension");
  if (max_dim > THCB200_MAX_DIMS) th_arg_error(2, CUTORCH_DIM_WARNING);
  for (int i = 0; i < num; ++i) check_gpu<R>(state, {result, inputs[i]});
  long size[THCB200_MAX_DIMS];
  for (int i = 0; i < max_dim; ++i) {
    long d = dim_size(inputs[0], i);
    for (int j = 1; j < num; ++j) {
      const long sz = dim_size(inputs[j], i);
      if (i == cat_dim) d += sz;
      else if (d != sz && d && sz) th_error("inconsistent tensor sizes");
      else if (!d) d = sz;
    }
    size[i] = d;
  }
  // an input may be the result itself: keep the inputs alive and unchanged while the result is resized
  bool aliased = false;
  for (int i = 0; i < num; ++i) aliased = aliased || inputs[i] == result || (inputs[i]->storage && inputs[i]->storage == result->storage);
  TensorT<R> *out = result;
  if (aliased) out = tensor_alloc<R>();
  tensor_raw_resize<R>(state, out, max_dim, size, nullptr);
  long offset = 0;
  TensorT<R> *slice = tensor_alloc<R>();
  try {
    for (int j = 0; j < num; ++j) {
      const long len = dim_size(inputs[j], cat_dim);
      if (inputs[j]->nDimension == 0 || len == 0) continue;
      tensor_narrow<R>(state, slice, out, cat_dim, offset, len);
      tensor_copy<R>(state, slice, inputs[j]);
      offset += len;
    }
    if (aliased) {
      tensor_raw_resize<R>(state, result, max_dim, size, nullptr);
      tensor_copy<R>(state, result, out);
    }
  } catch (...) {
    tensor_free<R>(state, slice);
    if (aliased) tensor_free<R>(state, out);
    throw;
  }
  tensor_free<R>(state, slice);
  if (aliased) tensor_free<R>(state, out);
}

// ---- single elements (lib/THC/generic/THCStorage.c:20-34, generic/THCTensor.c:840-900) ------
// One element crosses in the order of the current stream of the storage's device, and the call
// waits for it (the reference uses a plain cudaMemcpy, which is not ordered with non-blocking streams).
template <typename R> void storage_set(THCState *state, StorageT<R> *s, ptrdiff_t index, R value) {
  THArgCheck(s && index >= 0 && index < s->size, 2, "index out of bounds");
  DeviceGuard guard(s->device);
  const cudaStream_t st = THCState_getCurrentStreamOnDevice(state, s->device);
  THCudaCheck(cudaMemcpyAsync(s->data + index, &value, sizeof(R), cudaMemcpyHostToDevice, st));
  THCudaCheck(cudaStreamSynchronize(st));
}
template <typename R> R storage_get(THCState *state, const StorageT<R> *s, ptrdiff_t index) {
  THArgCheck(s && index >= 0 && index < s->size, 2, "index out of bounds");
  DeviceGuard guard(s->device);
  const cudaStream_t st = THCState_getCurrentStreamOnDevice(state, s->device);
  R value;
  THCudaCheck(cudaMemcpyAsync(&value, s->data + index, sizeof(R), cudaMemcpyDeviceToHost, st));
  THCudaCheck(cudaStreamSynchronize(st));
  return value;
}
template <typename R> ptrdiff_t element_index(const TensorT<R> *t, int nd, const long *x) {
  static const char *const kCount[5] = {"", "tensor must have one dimension", "tensor must have two dimensions",
                                        "tensor must have three dimensions", "tensor must have four dimensions"};
  THArgCheck(t->nDimension == nd, 1, kCount[nd]);
  ptrdiff_t off = t->storageOffset;
  for (int d = 0; d < nd; ++d) {
    THArgCheck(x[d] >= 0 && x[d] < t->size[d], 2, "out of range");
    off += x[d] * t->stride[d];
  }
  return off;
}

// ---- CPU <-> GPU tensors (lib/THC/generic/THCTensorCopy.c:7-164) --------------------------
// Every TH CPU tensor has the same layout apart from the element type of its storage.
struct CpuStorageAny { char *data; ptrdiff_t size; int refcount; char flag; void *allocator; void *allocatorContext; void *view; };
struct CpuTensorAny { long *size; long *stride; int nDimension; CpuStorageAny *storage; ptrdiff_t storageOffset; int refcount; char flag; };

thcb200_tensor describe_cpu(const void *tensor, int dtype) {
  const CpuTensorAny *t = (const CpuTensorAny *)tensor;
  if (!t) th_error("null CPU tensor");
  thcb200_tensor d;
  memset(&d, 0, sizeof(d));
  d.dtype = dtype;
  d.ndim = t->nDimension;
  if (t->nDimension > THCB200_MAX_DIMS) th_arg_error(2, CUTORCH_DIM_WARNING);
  for (int i = 0; i < t->nDimension; ++i) { d.sizes[i] = t->size[i]; d.strides[i] = t->stride[i]; }
  static const size_t esz[8] = {1, 1, 2, 4, 8, 2, 4, 8};
  d.data = (t->storage && t->storage->data) ? (void *)(t->storage->data + t->storageOffset * (ptrdiff_t)esz[dtype]) : nullptr;
  return d;
}
ptrdiff_t cpu_nelement(const void *tensor) {
  const CpuTensorAny *t = (const CpuTensorAny *)tensor;
  if (!t || t->nDimension == 0) return 0;
  ptrdiff_t n = 1;
  for (int i = 0; i < t->nDimension; ++i) n *= t->size[i];
  return n;
}
bool cpu_contiguous(const void *tensor) {
  const CpuTensorAny *t = (const CpuTensorAny *)tensor;
  long run = 1;
  for (int d = t->nDimension - 1; d >= 0; --d) {
    if (t->size[d] != 1 && t->stride[d] != run) return false;
    run *= t->size[d];
  }
  return true;
}

template <typename R>
void copy_from_cpu(THCState *state, TensorT<R> *self, const void *src, int src_dtype) {
  THArgCheck(tensor_nelement<R>(self) == cpu_nelement(src), 2, "sizes do not match");
  if (cpu_nelement(src) == 0) return;
  DeviceGuard guard(tensor_device<R>(self, current_device()));   // the GPU tensor may live on another device than the current one
  thcb200_tensor dd = describe<R>(self), ds = describe_cpu(src, src_dtype);
  check_core(thcb200_copy_from_host(state_ctx(state), &dd, &ds, (void *)state_stream(state)));
}
template <typename R>
void copy_to_cpu(THCState *state, void *self, int self_dtype, TensorT<R> *src) {
  THArgCheck(cpu_nelement(self) == tensor_nelement<R>(src), 2, "sizes do not match");
  if (cpu_nelement(self) == 0) return;
  DeviceGuard guard(tensor_device<R>(src, current_device()));
  thcb200_tensor dd = describe_cpu(self, self_dtype), ds = describe<R>(src);
  check_core(thcb200_copy_to_host(state_ctx(state), &dd, &ds, (void *)state_stream(state)));
}
// The asynchronous forms (lib/THC/generic/THCTensorCopy.c:112-164): same sizes, both contiguous,
// one cudaMemcpyAsync on the current stream of the GPU tensor's device.
template <typename R>
void copy_async(THCState *state, TensorT<R> *gpu, void *cpu, bool to_gpu) {
  THArgCheck(tensor_nelement<R>(gpu) == cpu_nelement(cpu), 2, "sizes do not match");
  THArgCheck(tensor_is_contiguous<R>(gpu), to_gpu ? 2 : 3, "Target tensor must be contiguous");
  THArgCheck(cpu_contiguous(cpu), to_gpu ? 3 : 2, "Source tensor must be contiguous");
  const ptrdiff_t n = tensor_nelement<R>(gpu);
  if (n == 0) return;
  thcb200_tensor dg = describe<R>(gpu), dc = describe_cpu(cpu, RealTraits<R>::dtype);
  DeviceGuard guard(gpu->storage->device);
  const cudaStream_t st = THCState_getCurrentStreamOnDevice(state, gpu->storage->device);
  if (to_gpu) THCudaCheck(cudaMemcpyAsync(dg.data, dc.data, (size_t)n * sizeof(R), cudaMemcpyHostToDevice, st));
  else THCudaCheck(cudaMemcpyAsync(dc.data, dg.data, (size_t)n * sizeof(R), cudaMemcpyDeviceToHost, st));
}

// ---- storage copies (lib/THC/generic/THCStorageCopy.h): a storage is copied as the 1-D tensor
// over all of it, through the tensor copies above ------------------------------------------
template <typename R> TensorT<R> *storage_as_tensor(THCState *state, StorageT<R> *s) {
  TensorT<R> *t = tensor_alloc<R>();
  const long n = (long)s->size, one = 1;
  tensor_raw_set<R>(state, t, s, 0, 1, &n, &one);
  return t;
}
// a CPU storage (same fields for every element type) as a 1-D CPU tensor on the caller's stack
struct CpuStorageView {
  long size, stride;
  CpuTensorAny t;
  explicit CpuStorageView(const void *storage) {
    CpuStorageAny *s = (CpuStorageAny *)storage;
    if (!s) th_error("null CPU storage");
    size = (long)s->size;
    stride = 1;
    t.size = &size; t.stride = &stride; t.nDimension = 1; t.storage = s; t.storageOffset = 0; t.refcount = 1; t.flag = 0;
  }
};
template <typename RD, typename RS> void storage_copy_convert(THCState *state, StorageT<RD> *self, StorageT<RS> *src) {
  THArgCheck(self->size == src->size, 2, "size does not match");
  if (self->size == 0) return;
  TensorT<RD> *d = storage_as_tensor<RD>(state, self);
  TensorT<RS> *f = storage_as_tensor<RS>(state, src);
  try {
    if constexpr (std::is_same<RD, RS>::value) tensor_copy<RD>(state, d, f); else tensor_copy_convert<RD, RS>(state, d, f);
  } catch (...) { tensor_free<RD>(state, d); tensor_free<RS>(state, f); throw; }
  tensor_free<RD>(state, d);
  tensor_free<RS>(state, f);
}
template <typename R> void storage_from_cpu(THCState *state, StorageT<R> *self, const void *cpu_storage, int cpu_dtype) {
  CpuStorageView v(cpu_storage);
  THArgCheck(self->size == v.size, 2, "size does not match");
  if (self->size == 0) return;
  TensorT<R> *d = storage_as_tensor<R>(state, self);
  try { copy_from_cpu<R>(state, d, &v.t, cpu_dtype); } catch (...) { tensor_free<R>(state, d); throw; }
  tensor_free<R>(state, d);
}
template <typename R> void storage_to_cpu(THCState *state, void *cpu_storage, int cpu_dtype, StorageT<R> *src) {
  CpuStorageView v(cpu_storage);
  THArgCheck(v.size == src->size, 2, "size does not match");
  if (src->size == 0) return;
  TensorT<R> *f = storage_as_tensor<R>(state, src);
  try { copy_to_cpu<R>(state, &v.t, cpu_dtype, f); } catch (...) { tensor_free<R>(state, f); throw; }
  tensor_free<R>(state, f);
}

// ---- indexed moves (lib/THC/generic/THCTensorIndex.cu, THCTensorScatterGather.cu) --------
using LongT = TensorT<long>;
template <typename R> R zero_real() { return R(); }

template <typename R>
void indexed(THCState *state, int mode, TensorT<R> *dst, TensorT<R> *src, LongT *index, int dim, bool vector, thcb200_scalar v) {
  thcb200_tensor dd = describe<R>(dst), di = describe<long>(index), ds;
  if (src) ds = describe<R>(src);
  check_core(thcb200_indexed(state_ctx(state), mode, &dd, src ? &ds : nullptr, &di, dim, vector ? 1 : 0, v,
                             (void *)state_stream(state)));
}

template <typename R> void index_vector_checks(THCState *state, TensorT<R> *a, TensorT<R> *b, LongT *indices, int dim, TensorT<R> *src) {
  check_gpu<R>(state, {a, b});
  check_gpu<long>(state, {indices});
  THArgCheck(indices->nDimension == 1, 3, "expecting vector of indices");
  THArgCheck(dim >= 0 && dim < src->nDimension, 4, "Indexing dim is out of bounds");
  THArgCheck(src->nDimension > 0, 2, "Source tensor is empty");
}

template <typename R> void index_select(THCState *state, TensorT<R> *dst, TensorT<R> *src, int dim, LongT *indices) {
  index_vector_checks<R>(state, dst, src, indices, dim, src);
  THArgCheck(dst != src, 1, "output must differ from the input");
  long sz[THCB200_MAX_DIMS];
  THArgCheck(src->nDimension <= THCB200_MAX_DIMS, 3, CUTORCH_DIM_WARNING);
  for (int d = 0; d < src->nDimension; ++d) sz[d] = src->size[d];
  sz[dim] = indices->size[0];
  tensor_raw_resize<R>(state, dst, src->nDimension, sz, nullptr);
  indexed<R>(state, THCB200_INDEX_GATHER, dst, src, indices, dim, true, kZero);
}

template <typename R> void index_copy_or_add(THCState *state, int mode, TensorT<R> *dst, int dim, LongT *indices, TensorT<R> *src) {
  index_vector_checks<R>(state, dst, src, indices, dim, src);
  THArgCheck(indices->size[0] == src->size[dim], 4, "length of src.size[dim] is not equal to length of indices");
  THArgCheck(dst->nDimension == src->nDimension, 2, "destination and source must have the same number of dimensions");
  indexed<R>(state, mode, dst, src, indices, dim, true, kZero);
}

template <typename R> void index_fill(THCState *state, TensorT<R> *dst, int dim, LongT *indices, R value) {
  index_vector_checks<R>(state, dst, nullptr, indices, dim, dst);
  indexed<R>(state, THCB200_INDEX_SCATTER_FILL, dst, nullptr, indices, dim, true, to_scalar<R>(value));
}

template <typename R> void gather(THCState *state, TensorT<R> *tensor, TensorT<R> *src, int dim, LongT *index) {
  check_gpu<R>(state, {tensor, src});
  check_gpu<long>(state, {index});
  THArgCheck(src->nDimension == tensor->nDimension, 2, "Input tensor must have same dimensions as output tensor");
  THArgCheck(dim >= 0 && dim < tensor->nDimension, 3, "Index dimension is out of bounds");
  THArgCheck(index->nDimension == src->nDimension, 4, "Index tensor must have same dimensions as input tensor");
  for (int d = 0; d < tensor->nDimension; ++d) {
    THArgCheck(index->size[d] == tensor->size[d], 4, "Index tensor must have the same size as output tensor.");
    if (d != dim)
      THArgCheck(tensor->size[d] == src->size[d], 2,
                 "Input tensor must have same size as output tensor apart from the specified dimension");
  }
  indexed<R>(state, THCB200_INDEX_GATHER, tensor, src, index, dim, false, kZero);
}

template <typename R> void scatter(THCState *state, int mode, TensorT<R> *tensor, int dim, LongT *index, TensorT<R> *src, R value) {
  check_gpu<R>(state, {tensor, src});
  check_gpu<long>(state, {index});
  THArgCheck(dim >= 0 && dim < tensor->nDimension, 2, "Index dimension is out of bounds");
  if (src) {
    THArgCheck(index->nDimension == src->nDimension, 3, "Index tensor must have same dimensions as input tensor");
    THArgCheck(src->nDimension == tensor->nDimension, 4, "Input tensor must have same dimensions as output tensor");
    for (int d = 0; d < tensor->nDimension; ++d) {
      THArgCheck(index->size[d] == src->size[d], 3, "Index tensor must have the same size as input tensor.");
      if (d != dim)
        THArgCheck(tensor->size[d] == src->size[d], 4,
                   "Input tensor must have same size as output tensor apart from the specified dimension");
    }
  } else {
    THArgCheck(index->nDimension == tensor->nDimension, 3, "Index tensor must have same dimensions as output tensor");
    for (int d = 0; d < tensor->nDimension; ++d)
      if (d != dim)
        THArgCheck(tensor->size[d] == index->size[d], 4,
                   "Index tensor must have same size as output tensor apart from the specified dimension");
  }
  indexed<R>(state, mode, tensor, src, index, dim, false, to_scalar<R>(value));
}

// ---- comparisons into a ByteTensor, Byte masks -----------------------------------------
using ByteT = TensorT<unsigned char>;

// self_ = (src1 CMP src2) or (src1 CMP value) as 0/1 bytes; self_ takes src1's size
// (THC_logicalValue / THC_logicalTensor, lib/THC/THCTensorMathCompare.cuh:69-85,
// THCTensorMathCompareT.cuh:52-72).
template <typename R>
void compare_to_byte(THCState *state, int op, ByteT *self_, TensorT<R> *src1, TensorT<R> *src2, thcb200_scalar s) {
  check_gpu<unsigned char>(state, {self_});
  check_gpu<R>(state, {src1, src2});
  if ((void *)self_ != (void *)src1) tensor_raw_resize<unsigned char>(state, self_, src1->nDimension, src1->size, nullptr);
  if (src2) THArgCheck(tensor_nelement<R>(src1) == tensor_nelement<R>(src2), 3, "sizes do not match");
  thcb200_tensor dout = describe<unsigned char>(self_), da = describe<R>(src1), db;
  if (src2) db = describe<R>(src2);
  check_core(thcb200_compare(state_ctx(state), op, &dout, &da, src2 ? &db : nullptr, s, (void *)state_stream(state)));
}

template <typename R> void masked_fill(THCState *state, TensorT<R> *tensor, ByteT *mask, R value) {
  check_gpu<R>(state, {tensor});
  check_gpu<unsigned char>(state, {mask});
  THArgCheck(tensor_nelement<R>(tensor) == tensor_nelement<unsigned char>(mask), 2, "sizes do not match");
  thcb200_tensor dt = describe<R>(tensor), dm = describe<unsigned char>(mask);
  check_core(thcb200_masked_fill(state_ctx(state), &dt, &dm, to_scalar<R>(value), (void *)state_stream(state)));
}

// lib/THC/generic/THCTensorMasked.cu:35-104.  `src` is read through its own strides, so no
// contiguous copy of it is made.
template <typename R> void masked_copy(THCState *state, TensorT<R> *tensor, ByteT *mask, TensorT<R> *src) {
  check_gpu<R>(state, {tensor, src});
  check_gpu<unsigned char>(state, {mask});
  THArgCheck(tensor_nelement<unsigned char>(mask) == tensor_nelement<R>(tensor), 2,
             "mask and tensor must have the same number of elements");
  thcb200_tensor dt = describe<R>(tensor), dm = describe<unsigned char>(mask), ds = describe<R>(src);
  int64_t total = 0;
  check_core(thcb200_masked_count(state_ctx(state), &dm, &total, (void *)state_stream(state)));
  THArgCheck(total <= (int64_t)tensor_nelement<R>(src), 2, "source nElements must be == mask `1` elements");
  if (total == 0) return;
  check_core(thcb200_masked_copy(state_ctx(state), &dt, &dm, &ds, (void *)state_stream(state), THCB200_FLAG_MASK_COUNTED));
}

// lib/THC/generic/THCTensorMasked.cu:119-177: `tensor` becomes 1-D with one element per set
// mask element, in src's logical order.
template <typename R> void masked_select(THCState *state, TensorT<R> *tensor, TensorT<R> *src, ByteT *mask) {
  check_gpu<R>(state, {tensor, src});
  check_gpu<unsigned char>(state, {mask});
  THArgCheck(tensor_nelement<unsigned char>(mask) == tensor_nelement<R>(src), 2, "sizes do not match");
  THArgCheck(tensor != src, 1, "output must differ from the input");
  thcb200_tensor dm = describe<unsigned char>(mask), ds = describe<R>(src);
  int64_t total = 0;
  check_core(thcb200_masked_count(state_ctx(state), &dm, &total, (void *)state_stream(state)));
  long sz[1] = {(long)total};
  tensor_raw_resize<R>(state, tensor, 1, sz, nullptr);
  if (total == 0) return;
  thcb200_tensor dt = describe<R>(tensor);
  check_core(thcb200_masked_select(state_ctx(state), &dt, &ds, &dm, (void *)state_stream(state), THCB200_FLAG_MASK_COUNTED));
}

// nonzero (lib/THC/generic/THCTensorMath.cu:262-356): a comparison with zero into a dense byte
// mask, the count of its set bytes, then one row of 1-based coordinates per set element.  The
// reference copies the tensor to a contiguous clone and runs thrust copy_if over linear indices.
template <typename R> void nonzero(THCState *state, LongT *out, TensorT<R> *self) {
  check_gpu<R>(state, {self});
  check_gpu<long>(state, {out});
  const int nd = self->nDimension;
  long shape[2] = {0, (long)nd};
  if (tensor_nelement<R>(self) == 0) { tensor_raw_resize<long>(state, out, 2, shape, nullptr); return; }
  ByteT *mask = tensor_alloc<unsigned char>();
  try {
    compare_to_byte<R>(state, THCB200_OP_NE_S, mask, self, nullptr, kZero);
    thcb200_tensor dm = describe<unsigned char>(mask);
    int64_t total = 0;
    check_core(thcb200_masked_count(state_ctx(state), &dm, &total, (void *)state_stream(state)));
    shape[0] = (long)total;
    tensor_raw_resize<long>(state, out, 2, shape, nullptr);
    if (total > 0) {
      int64_t sizes[THCB200_MAX_DIMS];
      for (int d = 0; d < nd; ++d) sizes[d] = self->size[d];
      thcb200_tensor dout = describe<long>(out);
      check_core(thcb200_mask_coords(state_ctx(state), &dout, &dm, sizes, nd, (void *)state_stream(state), THCB200_FLAG_MASK_COUNTED));
    }
  } catch (...) { tensor_free<unsigned char>(state, mask); throw; }
  tensor_free<unsigned char>(state, mask);
}

// The index* calls with a CPU LongTensor of positions (lib/THC/generic/THCTensorIndex.cu:5-15,
// 133-143,261-272,383-394): the positions go up into a temporary CudaLongTensor, then the call
// with device indices runs.
struct UploadedIndex {
  THCState *state;
  LongT *gpu;
  UploadedIndex(THCState *st, const void *cpu_long_tensor) : state(st), gpu(nullptr) {
    const CpuTensorAny *t = (const CpuTensorAny *)cpu_long_tensor;
    THArgCheck(t && t->nDimension == 1, 3, "expecting vector of indices");
    gpu = tensor_alloc<long>();
    long n = t->size[0];
    tensor_raw_resize<long>(state, gpu, 1, &n, nullptr);
    copy_from_cpu<long>(state, gpu, cpu_long_tensor, THCB200_I64);
  }
  ~UploadedIndex() { if (gpu) tensor_free<long>(state, gpu); }
};
// A CPU ByteTensor mask as a CudaByteTensor of the same sizes (lib/THC/generic/THCTensorMasked.cu:
// the ...Byte variants).
struct UploadedMask {
  THCState *state;
  ByteT *gpu;
  UploadedMask(THCState *st, const void *cpu_byte_tensor) : state(st), gpu(nullptr) {
    const CpuTensorAny *t = (const CpuTensorAny *)cpu_byte_tensor;
    if (!t) th_error("null mask");
    gpu = tensor_alloc<unsigned char>();
    tensor_raw_resize<unsigned char>(state, gpu, t->nDimension, t->size, nullptr);
    copy_from_cpu<unsigned char>(state, gpu, cpu_byte_tensor, THCB200_U8);
  }
  ~UploadedMask() { if (gpu) tensor_free<unsigned char>(state, gpu); }
};

}  // namespace

// ======================================================================================
// Per-type extern "C" wrappers
// ======================================================================================
#define real unsigned char
#define accreal long
#define CReal CudaByte
#define Real Byte
#define THC_T_FLOATING 0
#define THC_T_SIGNED 0
#define THC_T_HALF 0
#include "thc_compat_type.inc"
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_SIGNED

#define real char
#define accreal long
#define CReal CudaChar
#define Real Char
#define THC_T_SIGNED 0
#include "thc_compat_type.inc"
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_SIGNED
#define THC_T_SIGNED 1

#define real short
#define accreal long
#define CReal CudaShort
#define Real Short
#include "thc_compat_type.inc"
#undef real
#undef accreal
#undef CReal
#undef Real

#define real int
#define accreal long
#define CReal CudaInt
#define Real Int
#include "thc_compat_type.inc"
#undef real
#undef accreal
#undef CReal
#undef Real

#define real long
#define accreal long
#define CReal CudaLong
#define Real Long
#include "thc_compat_type.inc"
#undef real
#undef accreal
#undef CReal
#undef Real

#undef THC_T_FLOATING
#define THC_T_FLOATING 1

#define real half
#define accreal float
#define CReal CudaHalf
#define Real Half
#undef THC_T_HALF
#define THC_T_HALF 1
#include "thc_compat_type.inc"
#undef THC_T_HALF
#define THC_T_HALF 0
#undef real
#undef accreal
#undef CReal
#undef Real

#define real float
#define accreal float
#define CReal Cuda
#define Real Float
#include "thc_compat_type.inc"
#undef real
#undef accreal
#undef CReal
#undef Real

#define real double
#define accreal double
#define CReal CudaDouble
#define Real Double
#include "thc_compat_type.inc"
#undef real
#undef accreal
#undef CReal
#undef Real

extern "C" {
int THCudaByteTensor_logicalall(THCState *state, THCudaByteTensor *self) {
  API_BEGIN
  return (int)reduce_all_i<unsigned char>(state, THCB200_RED_ALL, THCB200_PRE_IDENTITY, kZero, (TensorT<unsigned char> *)self);
  API_END_RET(0)
}
int THCudaByteTensor_logicalany(THCState *state, THCudaByteTensor *self) {
  API_BEGIN
  return (int)reduce_all_i<unsigned char>(state, THCB200_RED_ANY, THCB200_PRE_IDENTITY, kZero, (TensorT<unsigned char> *)self);
  API_END_RET(0)
}
}
