/* Per-type declarations, expanded by THCForEachType.h with `real`, `accreal`, `CReal`,
 * THC_T_FLOATING, THC_T_SIGNED and THC_T_HALF defined.  Not include-guarded on purpose. */
#define THCTensor TH_CONCAT_3(TH, CReal, Tensor)
#define THCStorage TH_CONCAT_3(TH, CReal, Storage)
#define THCTensor_(NAME) TH_CONCAT_4(TH, CReal, Tensor_, NAME)
#define THCStorage_(NAME) TH_CONCAT_4(TH, CReal, Storage_, NAME)
/* torch7's names for the CPU tensor of the same element type (lib/TH/THTensor.h) */
#define THTensor TH_CONCAT_3(TH, Real, Tensor)
#define THTensor_(NAME) TH_CONCAT_4(TH, Real, Tensor_, NAME)

#ifdef THC_B200_DECLARE_STRUCTS

/* lib/THC/generic/THCStorage.h:9-19 */
typedef struct THCStorage {
  real *data;
  ptrdiff_t size;
  int refcount;
  char flag;
  THCDeviceAllocator *allocator;
  void *allocatorContext;
  struct THCStorage *view;
  int device;
} THCStorage;

/* lib/THC/generic/THCTensor.h:7-19 */
typedef struct THCTensor {
  long *size;
  long *stride;
  int nDimension;
  THCStorage *storage;
  ptrdiff_t storageOffset;
  int refcount;
  char flag;
} THCTensor;

#endif /* THC_B200_DECLARE_STRUCTS */

#ifdef THC_B200_DECLARE_API

/* ---- storage (lib/THC/generic/THCStorage.h) ---- */
THC_API real *THCStorage_(data)(THCState *state, const THCStorage *self);
THC_API ptrdiff_t THCStorage_(size)(THCState *state, const THCStorage *self);
THC_API int THCStorage_(elementSize)(THCState *state);
THC_API THCStorage *THCStorage_(new)(THCState *state);
THC_API THCStorage *THCStorage_(newWithSize)(THCState *state, ptrdiff_t size);
/* takes ownership of data (cudaMalloc'ed); clear TH_STORAGE_FREEMEM to only borrow it */
THC_API THCStorage *THCStorage_(newWithData)(THCState *state, real *data, ptrdiff_t size);
THC_API void THCStorage_(setFlag)(THCState *state, THCStorage *storage, const char flag);
THC_API void THCStorage_(clearFlag)(THCState *state, THCStorage *storage, const char flag);
THC_API void THCStorage_(retain)(THCState *state, THCStorage *storage);
THC_API void THCStorage_(free)(THCState *state, THCStorage *storage);
THC_API void THCStorage_(resize)(THCState *state, THCStorage *storage, ptrdiff_t size);
THC_API int THCStorage_(getDevice)(THCState *state, const THCStorage *storage);
/* whole storages: between storages of any two element types on the GPU, and between CPU and
 * GPU storages (lib/THC/generic/THCStorageCopy.h); sizes must match */
THC_API void THCStorage_(rawCopy)(THCState *state, THCStorage *storage, real *src);
THC_API void THCStorage_(copy)(THCState *state, THCStorage *storage, THCStorage *src);
THC_API void THCStorage_(copyCuda)(THCState *state, THCStorage *self, THCStorage *src);
THC_API void THCStorage_(copyCudaByte)(THCState *state, THCStorage *storage, struct THCudaByteStorage *src);
THC_API void THCStorage_(copyCudaChar)(THCState *state, THCStorage *storage, struct THCudaCharStorage *src);
THC_API void THCStorage_(copyCudaShort)(THCState *state, THCStorage *storage, struct THCudaShortStorage *src);
THC_API void THCStorage_(copyCudaInt)(THCState *state, THCStorage *storage, struct THCudaIntStorage *src);
THC_API void THCStorage_(copyCudaLong)(THCState *state, THCStorage *storage, struct THCudaLongStorage *src);
THC_API void THCStorage_(copyCudaHalf)(THCState *state, THCStorage *storage, struct THCudaHalfStorage *src);
THC_API void THCStorage_(copyCudaFloat)(THCState *state, THCStorage *storage, struct THCudaStorage *src);
THC_API void THCStorage_(copyCudaDouble)(THCState *state, THCStorage *storage, struct THCudaDoubleStorage *src);
THC_API void THCStorage_(copyByte)(THCState *state, THCStorage *storage, struct THByteStorage *src);
THC_API void THCStorage_(copyChar)(THCState *state, THCStorage *storage, struct THCharStorage *src);
THC_API void THCStorage_(copyShort)(THCState *state, THCStorage *storage, struct THShortStorage *src);
THC_API void THCStorage_(copyInt)(THCState *state, THCStorage *storage, struct THIntStorage *src);
THC_API void THCStorage_(copyLong)(THCState *state, THCStorage *storage, struct THLongStorage *src);
THC_API void THCStorage_(copyHalf)(THCState *state, THCStorage *storage, struct THHalfStorage *src);
THC_API void THCStorage_(copyFloat)(THCState *state, THCStorage *storage, struct THFloatStorage *src);
THC_API void THCStorage_(copyDouble)(THCState *state, THCStorage *storage, struct THDoubleStorage *src);
THC_API void TH_CONCAT_2(THByteStorage_copyCuda, Real)(THCState *state, struct THByteStorage *self, THCStorage *src);
THC_API void TH_CONCAT_2(THCharStorage_copyCuda, Real)(THCState *state, struct THCharStorage *self, THCStorage *src);
THC_API void TH_CONCAT_2(THShortStorage_copyCuda, Real)(THCState *state, struct THShortStorage *self, THCStorage *src);
THC_API void TH_CONCAT_2(THIntStorage_copyCuda, Real)(THCState *state, struct THIntStorage *self, THCStorage *src);
THC_API void TH_CONCAT_2(THLongStorage_copyCuda, Real)(THCState *state, struct THLongStorage *self, THCStorage *src);
THC_API void TH_CONCAT_2(THHalfStorage_copyCuda, Real)(THCState *state, struct THHalfStorage *self, THCStorage *src);
THC_API void TH_CONCAT_2(THFloatStorage_copyCuda, Real)(THCState *state, struct THFloatStorage *self, THCStorage *src);
THC_API void TH_CONCAT_2(THDoubleStorage_copyCuda, Real)(THCState *state, struct THDoubleStorage *self, THCStorage *src);
THC_API void THCStorage_(copyCPU)(THCState *state, THCStorage *self, struct TH_CONCAT_3(TH, Real, Storage) *src);
THC_API void TH_CONCAT_3(TH, Real, Storage_copyCuda)(THCState *state, struct TH_CONCAT_3(TH, Real, Storage) *self, THCStorage *src);
/* one element, blocking (lib/THC/generic/THCStorage.h:22-23) */
THC_API void THCStorage_(set)(THCState *state, THCStorage *self, ptrdiff_t index, real value);
THC_API real THCStorage_(get)(THCState *state, const THCStorage *self, ptrdiff_t index);

/* ---- tensor (lib/THC/generic/THCTensor.h) ---- */
THC_API THCStorage *THCTensor_(storage)(THCState *state, const THCTensor *self);
THC_API ptrdiff_t THCTensor_(storageOffset)(THCState *state, const THCTensor *self);
THC_API int THCTensor_(nDimension)(THCState *state, const THCTensor *self);
THC_API long THCTensor_(size)(THCState *state, const THCTensor *self, int dim);
THC_API long THCTensor_(stride)(THCState *state, const THCTensor *self, int dim);
THC_API THLongStorage *THCTensor_(newSizeOf)(THCState *state, THCTensor *self);
THC_API THLongStorage *THCTensor_(newStrideOf)(THCState *state, THCTensor *self);
THC_API real *THCTensor_(data)(THCState *state, const THCTensor *self);

THC_API THCTensor *THCTensor_(new)(THCState *state);
THC_API THCTensor *THCTensor_(newWithTensor)(THCState *state, THCTensor *tensor);
THC_API THCTensor *THCTensor_(newWithStorage)(THCState *state, THCStorage *storage_, ptrdiff_t storageOffset_,
                                              THLongStorage *size_, THLongStorage *stride_);
THC_API THCTensor *THCTensor_(newWithStorage1d)(THCState *state, THCStorage *storage_, ptrdiff_t storageOffset_,
                                                long size0_, long stride0_);
THC_API THCTensor *THCTensor_(newWithStorage2d)(THCState *state, THCStorage *storage_, ptrdiff_t storageOffset_,
                                                long size0_, long stride0_, long size1_, long stride1_);
THC_API THCTensor *THCTensor_(newWithStorage3d)(THCState *state, THCStorage *storage_, ptrdiff_t storageOffset_,
                                                long size0_, long stride0_, long size1_, long stride1_,
                                                long size2_, long stride2_);
THC_API THCTensor *THCTensor_(newWithStorage4d)(THCState *state, THCStorage *storage_, ptrdiff_t storageOffset_,
                                                long size0_, long stride0_, long size1_, long stride1_,
                                                long size2_, long stride2_, long size3_, long stride3_);
THC_API THCTensor *THCTensor_(newWithSize)(THCState *state, THLongStorage *size_, THLongStorage *stride_);
THC_API THCTensor *THCTensor_(newWithSize1d)(THCState *state, long size0_);
THC_API THCTensor *THCTensor_(newWithSize2d)(THCState *state, long size0_, long size1_);
THC_API THCTensor *THCTensor_(newWithSize3d)(THCState *state, long size0_, long size1_, long size2_);
THC_API THCTensor *THCTensor_(newWithSize4d)(THCState *state, long size0_, long size1_, long size2_, long size3_);
THC_API THCTensor *THCTensor_(newClone)(THCState *state, THCTensor *self);
THC_API THCTensor *THCTensor_(newContiguous)(THCState *state, THCTensor *tensor);
THC_API THCTensor *THCTensor_(newSelect)(THCState *state, THCTensor *tensor, int dimension_, long sliceIndex_);
THC_API THCTensor *THCTensor_(newNarrow)(THCState *state, THCTensor *tensor, int dimension_, long firstIndex_, long size_);
THC_API THCTensor *THCTensor_(newTranspose)(THCState *state, THCTensor *tensor, int dimension1_, int dimension2_);

THC_API void THCTensor_(resize)(THCState *state, THCTensor *tensor, THLongStorage *size, THLongStorage *stride);
THC_API void THCTensor_(resizeAs)(THCState *state, THCTensor *tensor, THCTensor *src);
THC_API void THCTensor_(resize1d)(THCState *state, THCTensor *tensor, long size0_);
THC_API void THCTensor_(resize2d)(THCState *state, THCTensor *tensor, long size0_, long size1_);
THC_API void THCTensor_(resize3d)(THCState *state, THCTensor *tensor, long size0_, long size1_, long size2_);
THC_API void THCTensor_(resize4d)(THCState *state, THCTensor *tensor, long size0_, long size1_, long size2_, long size3_);
THC_API void THCTensor_(set)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(setStorage)(THCState *state, THCTensor *self, THCStorage *storage_, ptrdiff_t storageOffset_,
                                    THLongStorage *size_, THLongStorage *stride_);
THC_API void THCTensor_(narrow)(THCState *state, THCTensor *self, THCTensor *src, int dimension_, long firstIndex_, long size_);
THC_API void THCTensor_(select)(THCState *state, THCTensor *self, THCTensor *src, int dimension_, long sliceIndex_);
THC_API void THCTensor_(transpose)(THCState *state, THCTensor *self, THCTensor *src, int dimension1_, int dimension2_);
THC_API void THCTensor_(squeeze1d)(THCState *state, THCTensor *self, THCTensor *src, int dimension_);
THC_API int THCTensor_(isContiguous)(THCState *state, const THCTensor *self);
THC_API int THCTensor_(isSameSizeAs)(THCState *state, const THCTensor *self, const THCTensor *src);
THC_API ptrdiff_t THCTensor_(nElement)(THCState *state, const THCTensor *self);
THC_API void THCTensor_(retain)(THCState *state, THCTensor *self);
THC_API void THCTensor_(free)(THCState *state, THCTensor *self);
THC_API void THCTensor_(freeCopyTo)(THCState *state, THCTensor *self, THCTensor *dst);
THC_API int THCTensor_(getDevice)(THCState *state, const THCTensor *self);
/* broadcast views: dims of size 1 and new leading dims repeat with stride 0 (lib/THC/generic/THCTensor.h:78-80) */
THC_API void THCTensor_(expand)(THCState *state, THCTensor *r, THCTensor *tensor, THLongStorage *sizes);
THC_API THCTensor *THCTensor_(newExpand)(THCState *state, THCTensor *tensor, THLongStorage *sizes);
/* one element by its coordinates, blocking (lib/THC/generic/THCTensor.h:115-124) */
THC_API void THCTensor_(set1d)(THCState *state, THCTensor *tensor, long x0, real value);
THC_API void THCTensor_(set2d)(THCState *state, THCTensor *tensor, long x0, long x1, real value);
THC_API void THCTensor_(set3d)(THCState *state, THCTensor *tensor, long x0, long x1, long x2, real value);
THC_API void THCTensor_(set4d)(THCState *state, THCTensor *tensor, long x0, long x1, long x2, long x3, real value);
THC_API real THCTensor_(get1d)(THCState *state, const THCTensor *tensor, long x0);
THC_API real THCTensor_(get2d)(THCState *state, const THCTensor *tensor, long x0, long x1);
THC_API real THCTensor_(get3d)(THCState *state, const THCTensor *tensor, long x0, long x1, long x2);
THC_API real THCTensor_(get4d)(THCState *state, const THCTensor *tensor, long x0, long x1, long x2, long x3);
THC_API int THCTensor_(checkGPU)(THCState *state, unsigned int nTensors, ...);

/* ---- fill / copy (lib/THC/generic/THCTensorMath.h:5-6, THCTensorCopy.h) ---- */
THC_API void THCTensor_(fill)(THCState *state, THCTensor *self, real value);
THC_API void THCTensor_(zero)(THCState *state, THCTensor *self);
/* thin callers of fill / copy / sumall (lib/THC/generic/THCTensorMath.h:7-12,20-22) */
THC_API void THCTensor_(zeros)(THCState *state, THCTensor *r_, THLongStorage *size);
THC_API void THCTensor_(zerosLike)(THCState *state, THCTensor *r_, THCTensor *input);
THC_API void THCTensor_(ones)(THCState *state, THCTensor *r_, THLongStorage *size);
THC_API void THCTensor_(onesLike)(THCState *state, THCTensor *r_, THCTensor *input);
THC_API void THCTensor_(reshape)(THCState *state, THCTensor *r_, THCTensor *t, THLongStorage *size);
THC_API ptrdiff_t THCTensor_(numel)(THCState *state, THCTensor *t);
/* concatenation along `dimension` (0-based; -2 = the last dim, cutorch's -1 in 1-based counting):
 * every input is copied into its slice of the result (lib/THC/generic/THCTensorMath.h:13-14) */
/* rows of 1-based coordinates of the non-zero elements, in order (lib/THC/generic/THCTensorMath.h:15) */
THC_API void THCTensor_(nonzero)(THCState *state, struct THCudaLongTensor *tensor, THCTensor *self);
THC_API void THCTensor_(cat)(THCState *state, THCTensor *result, THCTensor *ta, THCTensor *tb, int dimension);
THC_API void THCTensor_(catArray)(THCState *state, THCTensor *result, THCTensor **inputs, int numInputs, int dimension);
THC_API void THCTensor_(diag)(THCState *state, THCTensor *self, THCTensor *src, long k);
THC_API void THCTensor_(eye)(THCState *state, THCTensor *self, long n, long m);
THC_API accreal THCTensor_(trace)(THCState *state, THCTensor *self);
THC_API void THCTensor_(copy)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(copyIgnoringOverlaps)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(copyCudaByte)(THCState *state, THCTensor *dst, struct THCudaByteTensor *src);
THC_API void THCTensor_(copyCudaChar)(THCState *state, THCTensor *dst, struct THCudaCharTensor *src);
THC_API void THCTensor_(copyCudaShort)(THCState *state, THCTensor *dst, struct THCudaShortTensor *src);
THC_API void THCTensor_(copyCudaInt)(THCState *state, THCTensor *dst, struct THCudaIntTensor *src);
THC_API void THCTensor_(copyCudaLong)(THCState *state, THCTensor *dst, struct THCudaLongTensor *src);
THC_API void THCTensor_(copyCudaHalf)(THCState *state, THCTensor *dst, struct THCudaHalfTensor *src);
THC_API void THCTensor_(copyCudaFloat)(THCState *state, THCTensor *dst, struct THCudaTensor *src);
THC_API void THCTensor_(copyCudaDouble)(THCState *state, THCTensor *dst, struct THCudaDoubleTensor *src);
THC_API void THCTensor_(copyCuda)(THCState *state, THCTensor *self, THCTensor *src);
/* between CPU and GPU tensors, any strides and element types on both sides; blocking
 * (lib/THC/generic/THCTensorCopy.h:7-14,26-39, generic/THCTensorCopy.c:7-164) */
THC_API void THCTensor_(copyByte)(THCState *state, THCTensor *self, struct THByteTensor *src);
THC_API void THCTensor_(copyChar)(THCState *state, THCTensor *self, struct THCharTensor *src);
THC_API void THCTensor_(copyShort)(THCState *state, THCTensor *self, struct THShortTensor *src);
THC_API void THCTensor_(copyInt)(THCState *state, THCTensor *self, struct THIntTensor *src);
THC_API void THCTensor_(copyLong)(THCState *state, THCTensor *self, struct THLongTensor *src);
THC_API void THCTensor_(copyFloat)(THCState *state, THCTensor *self, struct THFloatTensor *src);
THC_API void THCTensor_(copyDouble)(THCState *state, THCTensor *self, struct THDoubleTensor *src);
THC_API void THCTensor_(copyHalf)(THCState *state, THCTensor *self, struct THHalfTensor *src);
THC_API void TH_CONCAT_2(THByteTensor_copyCuda, Real)(THCState *state, struct THByteTensor *self, THCTensor *src);
THC_API void TH_CONCAT_2(THCharTensor_copyCuda, Real)(THCState *state, struct THCharTensor *self, THCTensor *src);
THC_API void TH_CONCAT_2(THShortTensor_copyCuda, Real)(THCState *state, struct THShortTensor *self, THCTensor *src);
THC_API void TH_CONCAT_2(THIntTensor_copyCuda, Real)(THCState *state, struct THIntTensor *self, THCTensor *src);
THC_API void TH_CONCAT_2(THLongTensor_copyCuda, Real)(THCState *state, struct THLongTensor *self, THCTensor *src);
THC_API void TH_CONCAT_2(THFloatTensor_copyCuda, Real)(THCState *state, struct THFloatTensor *self, THCTensor *src);
THC_API void TH_CONCAT_2(THDoubleTensor_copyCuda, Real)(THCState *state, struct THDoubleTensor *self, THCTensor *src);
THC_API void TH_CONCAT_2(THHalfTensor_copyCuda, Real)(THCState *state, struct THHalfTensor *self, THCTensor *src);
/* same element type on both sides */
THC_API void THCTensor_(copyCPU)(THCState *state, THCTensor *self, struct THTensor *src);
THC_API void THTensor_(copyCuda)(THCState *state, struct THTensor *self, THCTensor *src);
/* asynchronous on the current stream: both sides contiguous, the CPU side in pinned memory */
THC_API void THCTensor_(copyAsyncCPU)(THCState *state, THCTensor *self, struct THTensor *src);
THC_API void THTensor_(copyAsyncCuda)(THCState *state, struct THTensor *self, THCTensor *src);

/* ---- pointwise math (lib/THC/generic/THCTensorMathPointwise.h) ---- */
#if THC_T_FLOATING
THC_API void THCTensor_(sigmoid)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(log)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(lgamma)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(log1p)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(exp)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(cos)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(acos)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(cosh)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(sin)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(asin)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(sinh)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(tan)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(atan)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(atan2)(THCState *state, THCTensor *r_, THCTensor *tx, THCTensor *ty);
THC_API void THCTensor_(tanh)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(pow)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(tpow)(THCState *state, THCTensor *self, real value, THCTensor *src);
THC_API void THCTensor_(sqrt)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(rsqrt)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(ceil)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(floor)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(round)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(trunc)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(frac)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(lerp)(THCState *state, THCTensor *result, THCTensor *a, THCTensor *b, real w);
THC_API void THCTensor_(cinv)(THCState *state, THCTensor *self, THCTensor *src);
#endif
#if THC_T_FLOATING || THC_T_SIGNED
THC_API void THCTensor_(neg)(THCState *state, THCTensor *self, THCTensor *src);
#endif
THC_API void THCTensor_(abs)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(sign)(THCState *state, THCTensor *self, THCTensor *src);
THC_API void THCTensor_(clamp)(THCState *state, THCTensor *self, THCTensor *src, real min_value, real max_value);
THC_API void THCTensor_(cross)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2, int dimension);
THC_API void THCTensor_(cadd)(THCState *state, THCTensor *self, THCTensor *src1, real value, THCTensor *src2);
THC_API void THCTensor_(csub)(THCState *state, THCTensor *self, THCTensor *src1, real value, THCTensor *src2);
THC_API void THCTensor_(cmul)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cpow)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cdiv)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(clshift)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(crshift)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cmax)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cmin)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cfmod)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cremainder)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cmaxValue)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(cminValue)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(cbitand)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cbitor)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(cbitxor)(THCState *state, THCTensor *self, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(addcmul)(THCState *state, THCTensor *self, THCTensor *t, real value, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(addcdiv)(THCState *state, THCTensor *self, THCTensor *t, real value, THCTensor *src1, THCTensor *src2);

/* ---- tensor (op) scalar (lib/THC/generic/THCTensorMathPairwise.h) ---- */
THC_API void THCTensor_(add)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(sub)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(mul)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(div)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(lshift)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(rshift)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(fmod)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(remainder)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(bitand)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(bitor)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(bitxor)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API int THCTensor_(equal)(THCState *state, THCTensor *self, THCTensor *src);

/* ---- comparisons (lib/THC/generic/THCTensorMathCompare.h:5-18, THCTensorMathCompareT.h:5-18):
 * <op>Value / <op>Tensor write 0/1 into a ByteTensor resized to src's shape, the ...T forms
 * into a tensor of the operands' own type ---- */
THC_API void THCTensor_(ltValue)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(ltValueT)(THCState *state, THCTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(ltTensor)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(ltTensorT)(THCState *state, THCTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(gtValue)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(gtValueT)(THCState *state, THCTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(gtTensor)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(gtTensorT)(THCState *state, THCTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(leValue)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(leValueT)(THCState *state, THCTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(leTensor)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(leTensorT)(THCState *state, THCTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(geValue)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(geValueT)(THCState *state, THCTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(geTensor)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(geTensorT)(THCState *state, THCTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(eqValue)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(eqValueT)(THCState *state, THCTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(eqTensor)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(eqTensorT)(THCState *state, THCTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(neValue)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(neValueT)(THCState *state, THCTensor *self_, THCTensor *src, real value);
THC_API void THCTensor_(neTensor)(THCState *state, struct THCudaByteTensor *self_, THCTensor *src1, THCTensor *src2);
THC_API void THCTensor_(neTensorT)(THCState *state, THCTensor *self_, THCTensor *src1, THCTensor *src2);

/* ---- scans (lib/THC/generic/THCTensorMathScan.h:5-6) ---- */
THC_API void THCTensor_(cumsum)(THCState *state, THCTensor *self, THCTensor *src, long dim);
THC_API void THCTensor_(cumprod)(THCState *state, THCTensor *self, THCTensor *src, long dim);

/* ---- indexed moves; positions are 1-based (lib/THC/generic/THCTensorIndex.h:5-8,
 * THCTensorScatterGather.h:5-8) ---- */
THC_API void THCTensor_(indexSelect)(THCState *state, THCTensor *tensor, THCTensor *src, int dim, struct THCudaLongTensor *index);
THC_API void THCTensor_(indexCopy)(THCState *state, THCTensor *res_, int dim, struct THCudaLongTensor *indices, THCTensor *src);
THC_API void THCTensor_(indexAdd)(THCState *state, THCTensor *res_, int dim, struct THCudaLongTensor *indices, THCTensor *src);
THC_API void THCTensor_(indexFill)(THCState *state, THCTensor *tensor, int dim, struct THCudaLongTensor *index, real val);
/* positions in a CPU LongTensor (lib/THC/generic/THCTensorIndex.h:10-13) */
THC_API void THCTensor_(indexSelect_long)(THCState *state, THCTensor *tensor, THCTensor *src, int dim, struct THLongTensor *index);
THC_API void THCTensor_(indexCopy_long)(THCState *state, THCTensor *res_, int dim, struct THLongTensor *indices, THCTensor *src);
THC_API void THCTensor_(indexAdd_long)(THCState *state, THCTensor *res_, int dim, struct THLongTensor *indices, THCTensor *src);
THC_API void THCTensor_(indexFill_long)(THCState *state, THCTensor *tensor, int dim, struct THLongTensor *index, real val);
THC_API void THCTensor_(gather)(THCState *state, THCTensor *tensor, THCTensor *src, int dim, struct THCudaLongTensor *index);
THC_API void THCTensor_(scatter)(THCState *state, THCTensor *tensor, int dim, struct THCudaLongTensor *index, THCTensor *src);
THC_API void THCTensor_(scatterAdd)(THCState *state, THCTensor *tensor, int dim, struct THCudaLongTensor *index, THCTensor *src);
THC_API void THCTensor_(scatterFill)(THCState *state, THCTensor *tensor, int dim, struct THCudaLongTensor *index, real value);

/* ---- triangles of a matrix (lib/THC/generic/THCTensorMath.h: tril, triu) ---- */
THC_API void THCTensor_(tril)(THCState *state, THCTensor *self, THCTensor *src, long k);
THC_API void THCTensor_(triu)(THCState *state, THCTensor *self, THCTensor *src, long k);

/* ---- Byte masks (lib/THC/generic/THCTensorMasked.h:5-36); the ...Byte variants take the mask as a
 * CPU ByteTensor, which is uploaded first ---- */
THC_API void THCTensor_(maskedFill)(THCState *state, THCTensor *tensor, struct THCudaByteTensor *mask, real value);
THC_API void THCTensor_(maskedCopy)(THCState *state, THCTensor *tensor, struct THCudaByteTensor *mask, THCTensor *src);
THC_API void THCTensor_(maskedSelect)(THCState *state, THCTensor *tensor, THCTensor *src, struct THCudaByteTensor *mask);
THC_API void THCTensor_(maskedFillByte)(THCState *state, THCTensor *tensor, struct THByteTensor *mask, real value);
THC_API void THCTensor_(maskedCopyByte)(THCState *state, THCTensor *tensor, struct THByteTensor *mask, THCTensor *src);
THC_API void THCTensor_(maskedSelectByte)(THCState *state, THCTensor *tensor, THCTensor *src, struct THByteTensor *mask);

/* ---- reductions (lib/THC/generic/THCTensorMathReduce.h) ---- */
#if THC_T_FLOATING
THC_API void THCTensor_(norm)(THCState *state, THCTensor *self, THCTensor *src, real value, long dimension, int keepdim);
THC_API void THCTensor_(std)(THCState *state, THCTensor *self, THCTensor *src, long dim, int biased, int keepdim);
THC_API void THCTensor_(var)(THCState *state, THCTensor *self, THCTensor *src, long dim, int biased, int keepdim);
THC_API accreal THCTensor_(dist)(THCState *state, THCTensor *self, THCTensor *src, real value);
THC_API void THCTensor_(renorm)(THCState *state, THCTensor *self, THCTensor *src, real value, long dimension, real max_norm);
THC_API accreal THCTensor_(normall)(THCState *state, THCTensor *self, real value);
THC_API accreal THCTensor_(varall)(THCState *state, THCTensor *self, int biased);
THC_API accreal THCTensor_(stdall)(THCState *state, THCTensor *self, int biased);
#endif
THC_API void THCTensor_(sum)(THCState *state, THCTensor *self, THCTensor *src, long dim, int keepdim);
THC_API void THCTensor_(prod)(THCState *state, THCTensor *self, THCTensor *src, long dim, int keepdim);
THC_API void THCTensor_(mean)(THCState *state, THCTensor *self, THCTensor *src, long dim, int keepdim);
THC_API accreal THCTensor_(sumall)(THCState *state, THCTensor *self);
THC_API accreal THCTensor_(prodall)(THCState *state, THCTensor *self);
THC_API accreal THCTensor_(meanall)(THCState *state, THCTensor *self);
THC_API void THCTensor_(min)(THCState *state, THCTensor *values, struct THCudaLongTensor *indices, THCTensor *src, long dim, int keepdim);
THC_API void THCTensor_(max)(THCState *state, THCTensor *values, struct THCudaLongTensor *indices, THCTensor *src, long dim, int keepdim);
THC_API real THCTensor_(minall)(THCState *state, THCTensor *self);
THC_API real THCTensor_(maxall)(THCState *state, THCTensor *self);

/* Extensions with no counterpart in cutorch: the full-reduction result stays on the device
 * as a double (floating types) or int64 (integer types) so that a collective can consume
 * it without a host round trip. */
THC_API void THCTensor_(sumallToDevice)(THCState *state, THCTensor *self, void *result_dev);

#endif /* THC_B200_DECLARE_API */

#undef THCTensor
#undef THCStorage
#undef THCTensor_
#undef THCStorage_
#undef THTensor
#undef THTensor_
