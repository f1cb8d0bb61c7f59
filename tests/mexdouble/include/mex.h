/* mex.h -- a stand-in for MATLAB's MEX interface (TEST INFRASTRUCTURE ONLY).
 *
 * Just enough of the mx / mex API for the reference's unmodified gateways -- matlab/src/vl_nnconv.cu, vl_nnbnorm.cu,
 * vl_nnpool.cu, vl_nnroipool.cu, vl_nnbilinearsampler.cu with bits/datamex.cu and bits/mexutils.h -- to compile and run
 * without MATLAB: an mxArray is a small descriptor (class, dimensions, a reference-counted block of host or device
 * memory); mexErrMsgTxt and friends throw a C++ exception that the test driver turns into an error string, as MATLAB
 * turns it into an error.  The functions are defined in mxdouble.cpp.  Nothing in the library proper includes this.
 */
#ifndef MEXDOUBLE_MEX_H
#define MEXDOUBLE_MEX_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>

typedef size_t mwSize;
typedef size_t mwIndex;
typedef uint16_t mxChar;
typedef bool mxLogical;

typedef enum {
  mxUNKNOWN_CLASS = 0, mxCELL_CLASS, mxSTRUCT_CLASS, mxLOGICAL_CLASS, mxCHAR_CLASS, mxVOID_CLASS, mxDOUBLE_CLASS,
  mxSINGLE_CLASS, mxINT8_CLASS, mxUINT8_CLASS, mxINT16_CLASS, mxUINT16_CLASS, mxINT32_CLASS, mxUINT32_CLASS,
  mxINT64_CLASS, mxUINT64_CLASS, mxFUNCTION_CLASS
} mxClassID;

typedef enum { mxREAL = 0, mxCOMPLEX } mxComplexity;

typedef struct mxArray_tag mxArray;

#ifdef __cplusplus
extern "C" {
#endif

/* creation / destruction */
mxArray* mxCreateNumericArray(mwSize ndim, mwSize const* dims, mxClassID classid, mxComplexity flag);
mxArray* mxCreateNumericMatrix(mwSize m, mwSize n, mxClassID classid, mxComplexity flag);
mxArray* mxCreateDoubleMatrix(mwSize m, mwSize n, mxComplexity flag);
mxArray* mxCreateDoubleScalar(double value);
mxArray* mxCreateString(char const* str);
mxArray* mxDuplicateArray(mxArray const* in);
void mxDestroyArray(mxArray* pa);
void* mxMalloc(size_t n);
void* mxCalloc(size_t n, size_t size);
void mxFree(void* ptr);

/* queries */
mxClassID mxGetClassID(mxArray const* pa);
mwSize mxGetNumberOfDimensions(mxArray const* pa);
mwSize const* mxGetDimensions(mxArray const* pa);
size_t mxGetNumberOfElements(mxArray const* pa);
size_t mxGetM(mxArray const* pa);
size_t mxGetN(mxArray const* pa);
size_t mxGetElementSize(mxArray const* pa);
void* mxGetData(mxArray const* pa);
double* mxGetPr(mxArray const* pa);
double mxGetScalar(mxArray const* pa);
int mxGetString(mxArray const* pa, char* buf, mwSize buflen);
bool mxIsNumeric(mxArray const* pa);
bool mxIsComplex(mxArray const* pa);
bool mxIsSparse(mxArray const* pa);
bool mxIsChar(mxArray const* pa);
bool mxIsDouble(mxArray const* pa);
bool mxIsSingle(mxArray const* pa);
bool mxIsLogical(mxArray const* pa);
bool mxIsCell(mxArray const* pa);
bool mxIsStruct(mxArray const* pa);
bool mxIsEmpty(mxArray const* pa);
bool mxIsClass(mxArray const* pa, char const* name);
double mxGetInf(void);
double mxGetNaN(void);
double mxGetEps(void);

/* modification */
void mxSetData(mxArray* pa, void* newdata);
int mxSetDimensions(mxArray* pa, mwSize const* dims, mwSize ndim);

/* mex */
int mexPrintf(char const* fmt, ...);
void mexErrMsgTxt(char const* msg);
void mexErrMsgIdAndTxt(char const* id, char const* fmt, ...);
void mexWarnMsgTxt(char const* msg);
void mexWarnMsgIdAndTxt(char const* id, char const* fmt, ...);
int mexAtExit(void (*fn)(void));
void mexMakeArrayPersistent(mxArray* pa);
void mexMakeMemoryPersistent(void* ptr);
void mexLock(void);
void mexUnlock(void);

/* the entry point every gateway defines */
void mexFunction(int nlhs, mxArray* plhs[], int nrhs, mxArray const* prhs[]);

#ifdef __cplusplus
}
#endif

#endif /* MEXDOUBLE_MEX_H */
