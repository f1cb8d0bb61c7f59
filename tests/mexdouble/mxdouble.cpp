// The MEX stand-in's implementation (TEST INFRASTRUCTURE ONLY; see include/mex.h) and the few helpers the Python driver
// uses to build arguments and call a gateway's mexFunction.
#include "mex.h"
#include "gpu/mxGPUArray.h"

#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>

namespace {

// A reference-counted block of host or device memory; `owned` blocks are released with their last handle.
struct Block {
  void* ptr;
  size_t bytes;
  bool gpu, owned;
  int refs;
};

Block* new_block(size_t bytes, bool gpu, bool zero)
{
  Block* b = new Block{nullptr, bytes, gpu, true, 1};
  if (bytes) {
    if (gpu) {
      if (cudaMalloc(&b->ptr, bytes) != cudaSuccess) { cudaGetLastError(); b->ptr = nullptr; }
      else if (zero) cudaMemset(b->ptr, 0, bytes);
    } else {
      b->ptr = zero ? calloc(1, bytes) : malloc(bytes);
    }
  }
  return b;
}

void release(Block* b)
{
  if (!b || --b->refs > 0) return;
  if (b->owned && b->ptr) { if (b->gpu) cudaFree(b->ptr); else free(b->ptr); }
  delete b;
}

size_t element_size(mxClassID c)
{
  switch (c) {
    case mxDOUBLE_CLASS: case mxINT64_CLASS: case mxUINT64_CLASS: return 8;
    case mxSINGLE_CLASS: case mxINT32_CLASS: case mxUINT32_CLASS: return 4;
    case mxCHAR_CLASS: case mxINT16_CLASS: case mxUINT16_CLASS: return 2;
    case mxLOGICAL_CLASS: case mxINT8_CLASS: case mxUINT8_CLASS: return 1;
    default: return 0;
  }
}

struct MexError { std::string id, message; };
std::vector<void (*)(void)> g_atExit;
std::string g_warnings;

}  // namespace

struct mxArray_tag {
  mxClassID cls;
  mwSize ndim;
  mwSize dims[16];
  Block* blk;
};

struct mxGPUArray_tag {
  mxClassID cls;
  mwSize ndim;
  mwSize dims[16];
  Block* blk;
};

namespace {

size_t count(mwSize ndim, mwSize const* dims)
{
  size_t n = 1;
  for (mwSize i = 0; i < ndim; ++i) n *= dims[i];
  return n;
}

mxArray* make(mwSize ndim, mwSize const* dims, mxClassID cls, bool gpu, bool zero)
{
  mxArray* a = new mxArray_tag();
  a->cls = cls;
  // MATLAB arrays have at least two dimensions
  a->ndim = ndim < 2 ? 2 : ndim;
  for (mwSize i = 0; i < 16; ++i) a->dims[i] = 1;
  for (mwSize i = 0; i < ndim && i < 16; ++i) a->dims[i] = dims[i];
  if (ndim == 1) { a->dims[0] = dims[0]; a->dims[1] = 1; }
  if (ndim == 0) { a->dims[0] = 0; a->dims[1] = 0; }
  while (a->ndim > 2 && a->dims[a->ndim - 1] == 1) --a->ndim;      // MATLAB drops trailing singleton dimensions
  a->blk = new_block(count(a->ndim, a->dims) * element_size(cls), gpu, zero);
  return a;
}

}  // namespace

extern "C" {

mxArray* mxCreateNumericArray(mwSize ndim, mwSize const* dims, mxClassID classid, mxComplexity) { return make(ndim, dims, classid, false, true); }
mxArray* mxCreateNumericMatrix(mwSize m, mwSize n, mxClassID classid, mxComplexity) { mwSize d[2] = {m, n}; return make(2, d, classid, false, true); }
mxArray* mxCreateDoubleMatrix(mwSize m, mwSize n, mxComplexity) { mwSize d[2] = {m, n}; return make(2, d, mxDOUBLE_CLASS, false, true); }
mxArray* mxCreateDoubleScalar(double value) { mxArray* a = mxCreateDoubleMatrix(1, 1, mxREAL); *(double*)a->blk->ptr = value; return a; }

mxArray* mxCreateString(char const* str)
{
  mwSize d[2] = {1, strlen(str)};
  mxArray* a = make(2, d, mxCHAR_CLASS, false, true);
  for (size_t i = 0; i < d[1]; ++i) ((mxChar*)a->blk->ptr)[i] = (mxChar)(unsigned char)str[i];
  return a;
}

mxArray* mxDuplicateArray(mxArray const* in)
{
  mxArray* a = new mxArray_tag(*in);
  a->blk = new_block(in->blk->bytes, in->blk->gpu, false);
  if (in->blk->bytes) {
    if (in->blk->gpu) cudaMemcpy(a->blk->ptr, in->blk->ptr, in->blk->bytes, cudaMemcpyDeviceToDevice);
    else memcpy(a->blk->ptr, in->blk->ptr, in->blk->bytes);
  }
  return a;
}

void mxDestroyArray(mxArray* pa) { if (pa) { release(pa->blk); delete pa; } }
void* mxMalloc(size_t n) { return malloc(n ? n : 1); }
void* mxCalloc(size_t n, size_t size) { return calloc(n ? n : 1, size ? size : 1); }
void mxFree(void* ptr) { free(ptr); }

mxClassID mxGetClassID(mxArray const* pa) { return pa->cls; }
mwSize mxGetNumberOfDimensions(mxArray const* pa) { return pa->ndim; }
mwSize const* mxGetDimensions(mxArray const* pa) { return pa->dims; }
size_t mxGetNumberOfElements(mxArray const* pa) { return count(pa->ndim, pa->dims); }
size_t mxGetM(mxArray const* pa) { return pa->dims[0]; }
size_t mxGetN(mxArray const* pa) { size_t n = 1; for (mwSize i = 1; i < pa->ndim; ++i) n *= pa->dims[i]; return n; }
size_t mxGetElementSize(mxArray const* pa) { return element_size(pa->cls); }
void* mxGetData(mxArray const* pa) { return pa->blk->gpu ? nullptr : pa->blk->ptr; }
double* mxGetPr(mxArray const* pa) { return (pa->cls == mxDOUBLE_CLASS && !pa->blk->gpu) ? (double*)pa->blk->ptr : nullptr; }

double mxGetScalar(mxArray const* pa)
{
  if (pa->blk->gpu || !pa->blk->ptr) return 0.0;
  switch (pa->cls) {
    case mxDOUBLE_CLASS: return *(double*)pa->blk->ptr;
    case mxSINGLE_CLASS: return *(float*)pa->blk->ptr;
    case mxINT32_CLASS: return *(int32_t*)pa->blk->ptr;
    case mxLOGICAL_CLASS: return *(bool*)pa->blk->ptr;
    default: return 0.0;
  }
}

int mxGetString(mxArray const* pa, char* buf, mwSize buflen)
{
  if (pa->cls != mxCHAR_CLASS || buflen == 0) return 1;
  size_t n = mxGetNumberOfElements(pa);
  size_t m = n < buflen - 1 ? n : buflen - 1;
  for (size_t i = 0; i < m; ++i) buf[i] = (char)((mxChar*)pa->blk->ptr)[i];
  buf[m] = 0;
  return n > buflen - 1 ? 1 : 0;
}

bool mxIsNumeric(mxArray const* pa) { return !pa->blk->gpu && pa->cls >= mxDOUBLE_CLASS && pa->cls <= mxUINT64_CLASS; }
bool mxIsComplex(mxArray const*) { return false; }
bool mxIsSparse(mxArray const*) { return false; }
bool mxIsChar(mxArray const* pa) { return pa->cls == mxCHAR_CLASS; }
bool mxIsDouble(mxArray const* pa) { return pa->cls == mxDOUBLE_CLASS && !pa->blk->gpu; }
bool mxIsSingle(mxArray const* pa) { return pa->cls == mxSINGLE_CLASS && !pa->blk->gpu; }
bool mxIsLogical(mxArray const* pa) { return pa->cls == mxLOGICAL_CLASS; }
bool mxIsCell(mxArray const*) { return false; }
bool mxIsStruct(mxArray const*) { return false; }
bool mxIsEmpty(mxArray const* pa) { return mxGetNumberOfElements(pa) == 0; }
bool mxIsClass(mxArray const* pa, char const* name) { return pa->blk->gpu && strcmp(name, "gpuArray") == 0; }
double mxGetInf(void) { return INFINITY; }
double mxGetNaN(void) { return NAN; }
double mxGetEps(void) { return 2.220446049250313e-16; }

void mxSetData(mxArray* pa, void* newdata)
{
  release(pa->blk);
  pa->blk = new Block{newdata, 0, false, true, 1};      // memory from mxMalloc: released with free()
}

int mxSetDimensions(mxArray* pa, mwSize const* dims, mwSize ndim)
{
  pa->ndim = ndim < 2 ? 2 : ndim;
  for (mwSize i = 0; i < 16; ++i) pa->dims[i] = 1;
  for (mwSize i = 0; i < ndim && i < 16; ++i) pa->dims[i] = dims[i];
  while (pa->ndim > 2 && pa->dims[pa->ndim - 1] == 1) --pa->ndim;
  pa->blk->bytes = count(pa->ndim, pa->dims) * element_size(pa->cls);
  return 0;
}

int mexPrintf(char const* fmt, ...)
{
  va_list ap;
  va_start(ap, fmt);
  int n = vprintf(fmt, ap);
  va_end(ap);
  return n;
}

void mexErrMsgTxt(char const* msg) { throw MexError{"", msg ? msg : ""}; }

void mexErrMsgIdAndTxt(char const* id, char const* fmt, ...)
{
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  throw MexError{id ? id : "", buf};
}

void mexWarnMsgTxt(char const* msg) { g_warnings += msg; g_warnings += "\n"; }

void mexWarnMsgIdAndTxt(char const* id, char const* fmt, ...)
{
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_warnings += std::string(id ? id : "") + ": " + buf + "\n";
}

int mexAtExit(void (*fn)(void))
{
  for (auto f : g_atExit) if (f == fn) return 0;
  g_atExit.push_back(fn);
  return 0;
}

void mexMakeArrayPersistent(mxArray*) {}
void mexMakeMemoryPersistent(void*) {}
void mexLock(void) {}
void mexUnlock(void) {}

// ---- gpu/mxGPUArray.h
int mxInitGPU(void) { return cudaFree(0) == cudaSuccess ? MX_GPU_SUCCESS : MX_GPU_FAILURE; }
bool mxIsGPUArray(mxArray const* pa) { return pa && pa->blk->gpu; }
bool mxGPUIsValidGPUData(mxArray const* pa) { return pa != nullptr; }

mxGPUArray const* mxGPUCreateFromMxArray(mxArray const* pa)
{
  mxGPUArray* g = new mxGPUArray_tag();
  g->cls = pa->cls; g->ndim = pa->ndim;
  memcpy(g->dims, pa->dims, sizeof(g->dims));
  g->blk = pa->blk; ++g->blk->refs;
  return g;
}

mxGPUArray* mxGPUCreateGPUArray(mwSize ndims, mwSize const* dims, mxClassID cid, mxComplexity, mxGPUInitialize init)
{
  mxArray* tmp = make(ndims, dims, cid, true, init == MX_GPU_INITIALIZE_VALUES);
  mxGPUArray* g = new mxGPUArray_tag();
  g->cls = tmp->cls; g->ndim = tmp->ndim;
  memcpy(g->dims, tmp->dims, sizeof(g->dims));
  g->blk = tmp->blk;
  delete tmp;      // the block stays with the handle
  return g;
}

mxArray* mxGPUCreateMxArrayOnGPU(mxGPUArray const* pa)
{
  mxArray* a = new mxArray_tag();
  a->cls = pa->cls; a->ndim = pa->ndim;
  memcpy(a->dims, pa->dims, sizeof(a->dims));
  a->blk = pa->blk; ++a->blk->refs;
  return a;
}

void mxGPUDestroyGPUArray(mxGPUArray const* pa) { if (pa) { release(pa->blk); delete pa; } }
mxClassID mxGPUGetClassID(mxGPUArray const* pa) { return pa->cls; }
mwSize mxGPUGetNumberOfDimensions(mxGPUArray const* pa) { return pa->ndim; }
mwSize const* mxGPUGetDimensions(mxGPUArray const* pa) { return pa->dims; }
size_t mxGPUGetNumberOfElements(mxGPUArray const* pa) { return count(pa->ndim, pa->dims); }
void const* mxGPUGetDataReadOnly(mxGPUArray const* pa) { return pa->blk->ptr; }
void* mxGPUGetData(mxGPUArray* pa) { return pa->blk->ptr; }

// ---- helpers of the test driver
// A gpuArray over device memory the caller owns (a torch tensor's storage).
mxArray* mxd_wrap_gpu(void* devptr, int ndim, size_t const* dims, int classid)
{
  mxArray* a = new mxArray_tag();
  a->cls = (mxClassID)classid;
  a->ndim = ndim < 2 ? 2 : (mwSize)ndim;
  for (int i = 0; i < 16; ++i) a->dims[i] = 1;
  for (int i = 0; i < ndim && i < 16; ++i) a->dims[i] = dims[i];
  a->blk = new Block{devptr, count(a->ndim, a->dims) * element_size(a->cls), true, false, 1};
  return a;
}

// An array filled from host memory: a gpuArray (uploaded) or a plain array.
mxArray* mxd_from_host(void const* src, int ndim, size_t const* dims, int classid, int gpu)
{
  mwSize d[16];
  for (int i = 0; i < ndim && i < 16; ++i) d[i] = dims[i];
  mxArray* a = make((mwSize)ndim, d, (mxClassID)classid, gpu != 0, false);
  if (a->blk->bytes && !a->blk->ptr) { mxDestroyArray(a); return nullptr; }
  if (a->blk->bytes) {
    if (gpu) {
      if (cudaMemcpy(a->blk->ptr, src, a->blk->bytes, cudaMemcpyHostToDevice) != cudaSuccess) { cudaGetLastError(); mxDestroyArray(a); return nullptr; }
    } else memcpy(a->blk->ptr, src, a->blk->bytes);
  }
  return a;
}

// Copies an array's elements to host memory (after waiting for the device); 0 on success.
int mxd_to_host(mxArray const* pa, void* dst)
{
  size_t bytes = count(pa->ndim, pa->dims) * element_size(pa->cls);
  if (!bytes) return 0;
  if (pa->blk->gpu) {
    cudaError_t e = cudaMemcpy(dst, pa->blk->ptr, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
  } else memcpy(dst, pa->blk->ptr, bytes);
  return 0;
}

void* mxd_device_pointer(mxArray const* pa) { return pa && pa->blk->gpu ? pa->blk->ptr : nullptr; }

// Calls a gateway; 0 on success, 1 when it raised an error (message "id: text" in err), as MATLAB would.
int mxd_call(void (*fn)(int, mxArray**, int, mxArray const**), int nlhs, mxArray** plhs, int nrhs, mxArray const** prhs,
             char* err, size_t errlen)
{
  try {
    fn(nlhs, plhs, nrhs, prhs);
  } catch (MexError const& e) {
    if (err && errlen) snprintf(err, errlen, "%s%s%s", e.id.c_str(), e.id.empty() ? "" : ": ", e.message.c_str());
    return 1;
  }
  if (err && errlen) err[0] = 0;
  return 0;
}

void mxd_run_at_exit(void)
{
  for (auto f : g_atExit) f();
  g_atExit.clear();
}

char const* mxd_warnings(void) { return g_warnings.c_str(); }
void mxd_clear_warnings(void) { g_warnings.clear(); }

}  // extern "C"
