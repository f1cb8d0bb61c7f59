// vl::Tensor / vl::TensorShape / vl::Context / vl::ErrorCode with the reference's names and
// semantics (reference matlab/src/bits/data.hpp:38-253), as a thin header-only layer over the C ABI
// of vlb.h.  Written for code that is used to MatConvNet's C++ operator interface: a Tensor is a
// non-owning view (shape of up to 8 dimensions, data type, device type, pointer), a Context carries
// the stream, the scratch memory and the last error.  Only VLDT_GPU x VLDT_Float is computed; the
// operators answer VLE_Unsupported to anything else -- there is no CPU implementation behind them.
#ifndef VLB_DATA_HPP
#define VLB_DATA_HPP

#include <cstddef>
#include <string>
#include "../vlb.h"

namespace vl {

enum ErrorCode {           // numeric values shared with the C ABI (data.hpp:38-52)
  VLE_Success = 0, VLE_Unsupported, VLE_Cuda, VLE_Cudnn, VLE_Cublas, VLE_OutOfMemory, VLE_OutOfGPUMemeory,
  VLE_IllegalArgument, VLE_Unknown, VLE_Timeout, VLE_NoData, VLE_IllegalMessage, VLE_Interrupted
};
enum DeviceType { VLDT_CPU = 0, VLDT_GPU };
enum DataType { VLDT_Char, VLDT_Float, VLDT_Double };

inline char const* getErrorMessage(ErrorCode e) { return vlb_error_message((int)e); }
inline size_t getDataTypeSizeInBytes(DataType t) { return t == VLDT_Char ? 1 : (t == VLDT_Float ? 4 : (t == VLDT_Double ? 8 : 0)); }

#define VL_TENSOR_SHAPE_MAX_NUM_DIMENSIONS 8

class TensorShape {
public:
  TensorShape() : numDimensions(0) {}
  TensorShape(size_t height, size_t width, size_t depth, size_t size) : numDimensions(4)
  { dimensions[0] = height; dimensions[1] = width; dimensions[2] = depth; dimensions[3] = size; }
  TensorShape(size_t const* dims, size_t n) { setDimensions(dims, n); }
  void clear() { numDimensions = 0; }
  void setDimensions(size_t const* dims, size_t n)
  { numDimensions = n > VL_TENSOR_SHAPE_MAX_NUM_DIMENSIONS ? VL_TENSOR_SHAPE_MAX_NUM_DIMENSIONS : n;
    for (size_t k = 0; k < numDimensions; ++k) dimensions[k] = dims[k]; }
  void setDimension(size_t num, size_t d)
  { if (num >= VL_TENSOR_SHAPE_MAX_NUM_DIMENSIONS) return;
    while (numDimensions <= num) dimensions[numDimensions++] = 1;
    dimensions[num] = d; }
  void setHeight(size_t x) { setDimension(0, x); }
  void setWidth(size_t x) { setDimension(1, x); }
  void setDepth(size_t x) { setDimension(2, x); }
  void setSize(size_t x) { setDimension(3, x); }
  // squash the trailing dimensions into the last one, or pad with singleton dimensions (data.cu:585-601)
  void reshape(size_t n)
  { if (n >= VL_TENSOR_SHAPE_MAX_NUM_DIMENSIONS) n = VL_TENSOR_SHAPE_MAX_NUM_DIMENSIONS;
    if (n > 0 && numDimensions > n) { size_t m = 1; for (size_t k = n - 1; k < numDimensions; ++k) m *= dimensions[k]; dimensions[n - 1] = m; }
    else for (size_t k = numDimensions; k < n; ++k) dimensions[k] = 1;
    numDimensions = n; }
  void reshape(TensorShape const& s) { *this = s; }
  size_t getDimension(size_t num) const { return num < numDimensions ? dimensions[num] : 1; }
  size_t const* getDimensions() const { return dimensions; }
  size_t getNumDimensions() const { return numDimensions; }
  size_t getHeight() const { return getDimension(0); }
  size_t getWidth() const { return getDimension(1); }
  size_t getDepth() const { return getDimension(2); }
  size_t getSize() const { return getDimension(3); }
  size_t getNumElements() const
  { if (numDimensions == 0) return 0; size_t n = 1; for (size_t k = 0; k < numDimensions; ++k) n *= dimensions[k]; return n; }
  bool isEmpty() const { return getNumElements() == 0; }
protected:
  size_t dimensions[VL_TENSOR_SHAPE_MAX_NUM_DIMENSIONS];
  size_t numDimensions;
};

inline bool operator==(TensorShape const& a, TensorShape const& b)
{
  size_t n = a.getNumDimensions() > b.getNumDimensions() ? a.getNumDimensions() : b.getNumDimensions();
  for (size_t k = 0; k < n; ++k) if (a.getDimension(k) != b.getDimension(k)) return false;
  return true;
}
inline bool operator!=(TensorShape const& a, TensorShape const& b) { return !(a == b); }

class Tensor : public TensorShape {
public:
  Tensor() : TensorShape(), deviceType(VLDT_CPU), dataType(VLDT_Char), memory(NULL), memorySize(0) {}
  Tensor(TensorShape const& shape, DataType dataType, DeviceType deviceType, void* memory, size_t memorySize)
  : TensorShape(shape), deviceType(deviceType), dataType(dataType), memory(memory), memorySize(memorySize) {}
  void* getMemory() { return memory; }
  void const* getMemory() const { return memory; }
  DeviceType getDeviceType() const { return deviceType; }
  TensorShape getShape() const { return TensorShape(*this); }
  DataType getDataType() const { return dataType; }
  operator bool() const { return memory != NULL; }
  bool isNull() const { return memory == NULL; }
  void setMemory(void* x) { memory = x; }
protected:
  DeviceType deviceType;
  DataType dataType;
  void* memory;
  size_t memorySize;
};

inline bool areCompatible(Tensor const& a, Tensor const& b)
{
  return (a.isEmpty() || a.isNull()) || (b.isEmpty() || b.isNull()) ||
         ((a.getDeviceType() == b.getDeviceType()) & (a.getDataType() == b.getDataType()));
}

// The engine context (stream, scratch, errors) behind the reference's vl::Context interface
// (data.hpp:150-179).  Created lazily so that a Context can be a global object, as in the MEX files.
class Context {
public:
  Context() : handle(NULL), lastError(VLE_Success) {}
  ~Context() { clear(); }
  void clear() { if (handle) { vlb_ctx_destroy(handle); handle = NULL; } }
  void* getWorkspace(DeviceType device, size_t size)
  { if (device != VLDT_GPU || !get()) return NULL; return vlb_ctx_reserve_workspace(handle, size) == 0 ? (void*)1 : NULL; }
  void clearWorkspace(DeviceType) { if (handle) vlb_ctx_clear_workspace(handle); }
  void setStream(void* cudaStream) { if (get()) vlb_ctx_set_stream(handle, cudaStream); }
  ErrorCode setError(ErrorCode e, char const* msg = NULL)
  { if (e != VLE_Success) { lastError = e; lastErrorMessage = getErrorMessage(e); if (msg) { lastErrorMessage += " ["; lastErrorMessage += msg; lastErrorMessage += "]"; } } return e; }
  ErrorCode passError(ErrorCode e, char const* msg = NULL)
  { if (e != VLE_Success && msg) lastErrorMessage = std::string(msg) + ": " + lastErrorMessage; return e; }
  void resetLastError() { lastError = VLE_Success; lastErrorMessage.clear(); if (handle) vlb_ctx_reset_error(handle); }
  ErrorCode getLastError() const { return lastError; }
  std::string const& getLastErrorMessage() const { return lastErrorMessage; }
  // the C-ABI context; NULL (and VLE_Cuda recorded) when no B200 is the current device
  vlb_ctx* get()
  { if (!handle) { int rc = vlb_ctx_create(&handle); if (rc) { handle = NULL; setError((ErrorCode)rc, "cannot create the engine context"); } } return handle; }
  // turn a C-ABI return code into the context's error state
  ErrorCode check(int rc, char const* where)
  { if (rc == 0) return VLE_Success; setError((ErrorCode)rc, handle ? vlb_ctx_last_error(handle) : NULL); if (handle) vlb_ctx_reset_error(handle); return passError((ErrorCode)rc, where); }
private:
  Context(Context const&);
  Context& operator=(Context const&);
  vlb_ctx* handle;
  ErrorCode lastError;
  std::string lastErrorMessage;
};

namespace impl {
// The operators compute single precision on the GPU only (the reference dispatches on the last
// non-null tensor, impl/dispatcher.hpp:41-53).
inline bool gpuFloat(Tensor const& t) { return t.isNull() || (t.getDeviceType() == VLDT_GPU && t.getDataType() == VLDT_Float); }
inline float* f(Tensor& t) { return (float*)t.getMemory(); }
inline float const* f(Tensor const& t) { return (float const*)t.getMemory(); }
}

}  // namespace vl
#endif
