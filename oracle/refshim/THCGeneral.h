/* TEST INFRASTRUCTURE.  Stand-in for the generated THCGeneral.h (lib/THC/THCGeneral.h.in needs
 * torch7's TH and cuBLAS headers): just the macros the functor headers use. */
#ifndef REFSHIM_THC_GENERAL_H
#define REFSHIM_THC_GENERAL_H
#define THC_EXTERNC extern "C"
#define THC_API THC_EXTERNC
#define THC_CLASS
typedef struct THCState THCState;
#ifndef TH_INDEX_BASE
#define TH_INDEX_BASE 1
#endif
#endif
