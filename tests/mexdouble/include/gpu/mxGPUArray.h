/* gpu/mxGPUArray.h -- stand-in for MATLAB's GPU array interface (TEST INFRASTRUCTURE ONLY; see mex.h).
 * A gpuArray is an mxArray whose memory block lives on the device; an mxGPUArray is a second handle on the same block. */
#ifndef MEXDOUBLE_MXGPUARRAY_H
#define MEXDOUBLE_MXGPUARRAY_H
#include "mex.h"

typedef struct mxGPUArray_tag mxGPUArray;
typedef enum { MX_GPU_DO_NOT_INITIALIZE = 0, MX_GPU_INITIALIZE_VALUES = 1 } mxGPUInitialize;
enum { MX_GPU_SUCCESS = 0, MX_GPU_FAILURE = 1 };

#ifdef __cplusplus
extern "C" {
#endif
int mxInitGPU(void);
bool mxIsGPUArray(mxArray const* pa);
bool mxGPUIsValidGPUData(mxArray const* pa);
mxGPUArray const* mxGPUCreateFromMxArray(mxArray const* pa);
mxGPUArray* mxGPUCreateGPUArray(mwSize ndims, mwSize const* dims, mxClassID cid, mxComplexity ccx, mxGPUInitialize init);
mxArray* mxGPUCreateMxArrayOnGPU(mxGPUArray const* pa);
void mxGPUDestroyGPUArray(mxGPUArray const* pa);
mxClassID mxGPUGetClassID(mxGPUArray const* pa);
mwSize mxGPUGetNumberOfDimensions(mxGPUArray const* pa);
mwSize const* mxGPUGetDimensions(mxGPUArray const* pa);
size_t mxGPUGetNumberOfElements(mxGPUArray const* pa);
void const* mxGPUGetDataReadOnly(mxGPUArray const* pa);
void* mxGPUGetData(mxGPUArray* pa);
#ifdef __cplusplus
}
#endif
#endif
