/* TEST INFRASTRUCTURE.  Pre-included (-include) when cutorch's own header files are compiled
 * as host C++ by g++ for oracle/ref_check.cpp.  It (1) turns the CUDA function qualifiers
 * into nothing so that the functor bodies become ordinary host functions, and (2) pre-defines
 * the include guards of the cutorch headers that need torch7's TH or launch kernels, so that
 * only the functor / TensorInfo / THCNumerics definitions are compiled. */
#ifndef REF_HOST_SHIM_H
#define REF_HOST_SHIM_H

#define __device__
#define __host__
#define __global__
#define __forceinline__ inline
#define __launch_bounds__(...)

/* headers whose content is not wanted */
#define THC_APPLY_INC              /* THCApply.cuh */
#define THC_REDUCE_INC             /* THCReduce.cuh */
#define THC_REDUCEALL_INC          /* THCReduceAll.cuh */
#define TH_CUDA_TENSOR_MATH_INC    /* THCTensorMath.h */
#define TH_CUDA_TENSOR_COPY_INC    /* THCTensorCopy.h */
#define THC_HALF_CONVERSION_INC    /* THCHalf.h: CUDA_HALF_TENSOR stays undefined, half specialisations drop out */
#define THC_THRUST_ALLOCATOR_INC   /* THCThrustAllocator.cuh */
#define THC_TENSOR_INC             /* THCTensor.h (needs TH) */

#include <math.h>
#include <stdlib.h>
#include <limits.h>
#include <float.h>
#include <stdint.h>
#include <stddef.h>

/* thrust is only named by THCTensorMasked.cuh's includes: its headers are parsed for the host system */
#define THRUST_DEVICE_SYSTEM 4 /* THRUST_DEVICE_SYSTEM_CPP: plain host code */

/* names that the (never instantiated) launch helpers of the compare headers mention */
struct THLongStorage;
void THLongStorage_free(THLongStorage *);
template <typename TensorType> struct TensorUtils;
#define THArgCheck(...) ((void)0)
#define THCudaCheck(x) ((void)0)
/* cudaGetLastError comes from the CUDA runtime header thrust pulls in (declared only; never called) */

/* CUDA math functions without a libm namesake */
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline double rsqrt(double x) { return 1.0 / sqrt(x); }

#endif
