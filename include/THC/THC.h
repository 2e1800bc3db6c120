/*
 * THC.h -- the THC C API of the apply / reduce path, served by the B200 core.
 *
 * Exports, for the eight cutorch tensor types, the entry points that cutorch's
 * cwrap-generated TensorMath.c binds for pointwise math, tensor-scalar math, dimension
 * reductions and full reductions, with the signatures of
 *   lib/THC/generic/THCTensorMathPointwise.h:1-69
 *   lib/THC/generic/THCTensorMathPairwise.h:4-17
 *   lib/THC/generic/THCTensorMathReduce.h:5-45
 *   lib/THC/generic/THCTensorMath.h:5-6           (fill, zero)
 *   lib/THC/generic/THCTensorCopy.h:5-6,35        (copy, copyIgnoringOverlaps, copyCuda<Type>)
 *   lib/THC/THCTensorMath.h:52-53                 (logicalall, logicalany)
 * plus the slice of the tensor/storage/state API those calls and their tests need
 * (lib/THC/generic/THCTensor.h, lib/THC/generic/THCStorage.h, lib/THC/THCGeneral.h.in,
 * lib/THC/THCStream.h).  Struct layouts of THCStorage and THCTensor follow
 * lib/THC/generic/THCStorage.h:9-19 and lib/THC/generic/THCTensor.h:7-19 field by field
 * because cutorch's FFI.lua mirrors them.
 *
 * This header stands in for torch7's TH + THC headers when the library is built and tested
 * on its own; inside a cutorch build the real headers declare the same symbols.
 */
#ifndef THCB200_THC_H
#define THCB200_THC_H

#include <cuda_runtime_api.h>
#include <cuda_fp16.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#define THC_EXTERNC extern "C"
#else
#define THC_EXTERNC extern
typedef __half_raw half;
#endif
#if defined(__GNUC__)
#define THC_API THC_EXTERNC __attribute__((visibility("default")))
#else
#define THC_API THC_EXTERNC
#endif

#define TH_INDEX_BASE 1
#define TH_CONCAT_2_EXPAND(a, b) a##b
#define TH_CONCAT_2(a, b) TH_CONCAT_2_EXPAND(a, b)
#define TH_CONCAT_3_EXPAND(a, b, c) a##b##c
#define TH_CONCAT_3(a, b, c) TH_CONCAT_3_EXPAND(a, b, c)
#define TH_CONCAT_4_EXPAND(a, b, c, d) a##b##c##d
#define TH_CONCAT_4(a, b, c, d) TH_CONCAT_4_EXPAND(a, b, c, d)

/* ---- the piece of TH the path touches ------------------------------------------------ */
typedef struct THLongStorage {
  long *data;
  ptrdiff_t size;
  int refcount;
  char flag;
  void *allocator;
  void *allocatorContext;
  struct THLongStorage *view;
} THLongStorage;

THC_API THLongStorage *THLongStorage_newWithSize(ptrdiff_t size);
THC_API THLongStorage *THLongStorage_newWithSize1(long a);
THC_API void THLongStorage_set(THLongStorage *s, ptrdiff_t i, long v);
THC_API long THLongStorage_get(const THLongStorage *s, ptrdiff_t i);
THC_API void THLongStorage_free(THLongStorage *s);

/* Errors: TH reports through handlers that do not return (luaT raises a Lua error).  With
 * no handler installed, the failing THC call records the message and returns; the caller
 * polls THCB200_errorOccurred(). */
typedef void (*THErrorHandlerFunction)(const char *msg, void *data);
typedef void (*THArgErrorHandlerFunction)(int argNumber, const char *msg, void *data);
THC_API void THSetErrorHandler(THErrorHandlerFunction f, void *data);
THC_API void THSetArgErrorHandler(THArgErrorHandlerFunction f, void *data);
THC_API int THCB200_errorOccurred(void);          /* 1 if a THC call failed since the last clear */
THC_API const char *THCB200_errorMessage(void);
THC_API void THCB200_clearError(void);

/* ---- state and streams --------------------------------------------------------------- */
typedef struct THCState THCState;
typedef struct THCStream {
  cudaStream_t stream;
  int device;
  int refcount;
} THCStream;

typedef struct _THCDeviceAllocator {
  cudaError_t (*malloc)(void *, void **, size_t, cudaStream_t);
  cudaError_t (*realloc)(void *, void **, size_t, size_t, cudaStream_t);
  cudaError_t (*free)(void *, void *);
  cudaError_t (*emptyCache)(void *);
  cudaError_t (*cacheInfo)(void *, int, size_t *, size_t *);
  void *state;
} THCDeviceAllocator;

THC_API THCState *THCState_alloc(void);
THC_API void THCState_free(THCState *state);
THC_API void THCudaInit(THCState *state);
THC_API void THCudaShutdown(THCState *state);
THC_API int THCState_getNumDevices(THCState *state);
THC_API cudaStream_t THCState_getCurrentStream(THCState *state);
THC_API cudaStream_t THCState_getCurrentStreamOnDevice(THCState *state, int device);
THC_API THCStream *THCState_getStream(THCState *state);
THC_API void THCState_setStream(THCState *state, THCStream *stream);
THC_API THCDeviceAllocator *THCState_getDeviceAllocator(THCState *state);
THC_API void THCState_setDeviceAllocator(THCState *state, THCDeviceAllocator *allocator);
/* 1 if copies may let device `dev` address memory of `devToAccess` directly (the hardware allows
 * it and it has not been switched off with ..._setPeerToPeerAccess); lib/THC/THCGeneral.h.in:131-138 */
THC_API int THCState_getPeerToPeerAccess(THCState *state, int dev, int devToAccess);
THC_API void THCState_setPeerToPeerAccess(THCState *state, int dev, int devToAccess, int enable);
THC_API struct cudaDeviceProp *THCState_getCurrentDeviceProperties(THCState *state);
/* scratch space of the current device (lib/THC/THCGeneral.h.in:188-192): at least 128 KiB */
THC_API void *THCState_getCurrentDeviceScratchSpace(THCState *state);
THC_API size_t THCState_getCurrentDeviceScratchSpaceSize(THCState *state);
THC_API void __THCudaCheck(cudaError_t err, const char *file, const int line);
/* Registers the callback THCudaMalloc and the storage allocations run once, before one retry, when
 * the device allocator fails (lib/THC/THCGeneral.c:836-854: cutorch hands Lua's collector here). */
THC_API void THCSetGCHandler(THCState *state, void (*cutorchGCFunction_)(void *data), void *data);
THC_API cudaError_t THCudaMalloc(THCState *state, void **ptr, size_t size);
THC_API cudaError_t THCudaFree(THCState *state, void *ptr);
THC_API THCStream *THCStream_new(int flags);
THC_API THCStream *THCStream_defaultStream(int device);
THC_API void THCStream_free(THCStream *self);
THC_API void THCStream_retain(THCStream *self);
/* Wraps a stream created elsewhere (not destroyed by THCStream_free). */
THC_API THCStream *THCB200_streamFromRaw(cudaStream_t stream, int device);
/* The descriptor-level context of the current device (see thcb200.h). */
THC_API struct thcb200_ctx *THCB200_currentContext(THCState *state);

THC_API half THC_float2half(float a);
THC_API float THC_half2float(half a);

#define TH_STORAGE_REFCOUNTED 1
#define TH_STORAGE_RESIZABLE 2
#define TH_STORAGE_FREEMEM 4
#define TH_TENSOR_REFCOUNTED 1

/* torch7's CPU storages and tensors as the copies between CPU and GPU tensors see them
 * (lib/TH/generic/THStorage.h, THTensor.h: the same field order for every element type; the
 * sources of TH are not part of cutorch, a build inside torch7 uses TH's own headers instead). */
#ifndef THCB200_HAVE_TH
#define THCB200_DECLARE_TH_STORAGE(Name, ctype)                                        \
  typedef struct TH##Name##Storage {                                                   \
    ctype *data;                                                                       \
    ptrdiff_t size;                                                                    \
    int refcount;                                                                      \
    char flag;                                                                         \
    void *allocator;                                                                   \
    void *allocatorContext;                                                            \
    struct TH##Name##Storage *view;                                                    \
  } TH##Name##Storage;
#define THCB200_DECLARE_TH_TENSOR(Name)                                                \
  typedef struct TH##Name##Tensor {                                                    \
    long *size;                                                                        \
    long *stride;                                                                      \
    int nDimension;                                                                    \
    TH##Name##Storage *storage;                                                        \
    ptrdiff_t storageOffset;                                                           \
    int refcount;                                                                      \
    char flag;                                                                         \
  } TH##Name##Tensor;
THCB200_DECLARE_TH_STORAGE(Byte, unsigned char)
THCB200_DECLARE_TH_STORAGE(Char, char)
THCB200_DECLARE_TH_STORAGE(Short, short)
THCB200_DECLARE_TH_STORAGE(Int, int)
THCB200_DECLARE_TH_STORAGE(Half, half)
THCB200_DECLARE_TH_STORAGE(Float, float)
THCB200_DECLARE_TH_STORAGE(Double, double)
THCB200_DECLARE_TH_TENSOR(Byte)
THCB200_DECLARE_TH_TENSOR(Char)
THCB200_DECLARE_TH_TENSOR(Short)
THCB200_DECLARE_TH_TENSOR(Int)
THCB200_DECLARE_TH_TENSOR(Long)   /* THLongStorage is declared above */
THCB200_DECLARE_TH_TENSOR(Half)
THCB200_DECLARE_TH_TENSOR(Float)
THCB200_DECLARE_TH_TENSOR(Double)
#undef THCB200_DECLARE_TH_STORAGE
#undef THCB200_DECLARE_TH_TENSOR
#endif

/* ---- per-type storage, tensor and math API ------------------------------------------- */
#define THC_B200_DECLARE_STRUCTS
#include "THCForEachType.h"
#undef THC_B200_DECLARE_STRUCTS
#define THC_B200_DECLARE_API
#include "THCForEachType.h"
#undef THC_B200_DECLARE_API

THC_API int THCudaByteTensor_logicalall(THCState *state, THCudaByteTensor *self);
THC_API int THCudaByteTensor_logicalany(THCState *state, THCudaByteTensor *self);

#endif /* THCB200_THC_H */
