/* Expands THCTypeAPI.h once per cutorch tensor type.  Not include-guarded on purpose. */
#define THC_T_FLOATING 0
#define THC_T_SIGNED 1
#define THC_T_HALF 0

#define real unsigned char
#define accreal long
#define CReal CudaByte
#define Real Byte
#define THC_T_DTYPE 0
#undef THC_T_SIGNED
#define THC_T_SIGNED 0
#include "THCTypeAPI.h"
#undef THC_T_SIGNED
#define THC_T_SIGNED 1
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#define real char
#define accreal long
#define CReal CudaChar
#define Real Char
#define THC_T_DTYPE 1
#undef THC_T_SIGNED
#define THC_T_SIGNED 0 /* neg is not defined for Char (lib/THC/generic/THCTensorMathPointwise.h:37-42) */
#include "THCTypeAPI.h"
#undef THC_T_SIGNED
#define THC_T_SIGNED 1
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#define real short
#define accreal long
#define CReal CudaShort
#define Real Short
#define THC_T_DTYPE 2
#include "THCTypeAPI.h"
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#define real int
#define accreal long
#define CReal CudaInt
#define Real Int
#define THC_T_DTYPE 3
#include "THCTypeAPI.h"
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#define real long
#define accreal long
#define CReal CudaLong
#define Real Long
#define THC_T_DTYPE 4
#include "THCTypeAPI.h"
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#undef THC_T_FLOATING
#define THC_T_FLOATING 1

#define real half
#define accreal float
#define CReal CudaHalf
#define Real Half
#define THC_T_DTYPE 5
#undef THC_T_HALF
#define THC_T_HALF 1
#include "THCTypeAPI.h"
#undef THC_T_HALF
#define THC_T_HALF 0
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#define real float
#define accreal float
#define CReal Cuda
#define Real Float
#define THC_T_DTYPE 6
#include "THCTypeAPI.h"
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#define real double
#define accreal double
#define CReal CudaDouble
#define Real Double
#define THC_T_DTYPE 7
#include "THCTypeAPI.h"
#undef real
#undef accreal
#undef CReal
#undef Real
#undef THC_T_DTYPE

#undef THC_T_FLOATING
#undef THC_T_SIGNED
#undef THC_T_HALF
