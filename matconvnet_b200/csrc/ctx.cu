// Context management and error reporting of the C ABI.
#include "common.cuh"

namespace vlb {

static char const* const kMessages[] = {
  "success", "unsupported feature", "CUDA error", "cuDNN error", "cuBLAS error", "out of memory",
  "out of GPU memory", "illegal argument", "unknown error", "timeout", "no data", "illegal message",
  "interrupted"};

int set_error(vlb_ctx* ctx, int code, char const* msg)
{
  if (!ctx) return code;
  if (code != VLB_Success) {
    ctx->lastError = code;
    ctx->lastErrorMessage = std::string(vlb_error_message(code));
    if (msg) { ctx->lastErrorMessage += " ["; ctx->lastErrorMessage += msg; ctx->lastErrorMessage += "]"; }
  }
  return code;
}

int pass_error(vlb_ctx* ctx, int code, char const* where)
{
  if (ctx && code != VLB_Success && where) {
    ctx->lastErrorMessage = std::string(where) + ": " + ctx->lastErrorMessage;
  }
  return code;
}

void* workspace(vlb_ctx* ctx, size_t bytes)
{
  if (bytes <= ctx->workspaceBytes && ctx->workspace) return ctx->workspace;
  if (bytes == 0) bytes = 256;
  if (ctx->workspace) {
    // Work enqueued earlier may still be using the old buffer.
    cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->workspace);
    ctx->workspace = nullptr;
    ctx->workspaceBytes = 0;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(ctx, VLB_OutOfGPUMemeory, cudaGetErrorString(e));
    return nullptr;
  }
  ctx->workspace = p;
  ctx->workspaceBytes = bytes;
  return p;
}

int check_launch(vlb_ctx* ctx, char const* where)
{
  cudaError_t e = cudaPeekAtLastError();
  if (e == cudaSuccess) return VLB_Success;
  cudaGetLastError();      // reported once: a launch error that stayed pending would be blamed on every later call
  set_error(ctx, VLB_Cuda, cudaGetErrorString(e));
  return pass_error(ctx, VLB_Cuda, where);
}

}  // namespace vlb

extern "C" {

int vlb_version(void) { return 100; }

char const* vlb_error_message(int code)
{
  if (code < 0 || code > VLB_Interrupted) code = VLB_Unknown;
  return vlb::kMessages[code];
}

int vlb_ctx_create(vlb_ctx** out)
{
  if (!out) return VLB_IllegalArgument;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { cudaGetLastError(); return VLB_Cuda; }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) { cudaGetLastError(); return VLB_Cuda; }
  if (prop.major != 10) {
    // The kernels are built for sm_100a only; refuse anything else up front.
    return VLB_Unsupported;
  }
  vlb_ctx* c = new vlb_ctx();
  c->device = dev;
  c->smCount = prop.multiProcessorCount;
  if (cudaMalloc((void**)&c->deviceStatus, 256 + 4 * 4096) != cudaSuccess || cudaMemset(c->deviceStatus, 0, 256 + 4 * 4096) != cudaSuccess) {
    cudaGetLastError();
    delete c;
    return VLB_OutOfGPUMemeory;
  }
  *out = c;
  return VLB_Success;
}

int vlb_ctx_destroy(vlb_ctx* ctx)
{
  if (!ctx) return VLB_Success;
  if (ctx->workspace) { cudaStreamSynchronize(ctx->stream); cudaFree(ctx->workspace); }
  if (ctx->deviceStatus) cudaFree(ctx->deviceStatus);
  delete ctx;
  return VLB_Success;
}

int vlb_ctx_set_stream(vlb_ctx* ctx, void* s) { if (!ctx) return VLB_IllegalArgument; ctx->stream = (cudaStream_t)s; return VLB_Success; }
void* vlb_ctx_get_stream(vlb_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int vlb_ctx_set_precision(vlb_ctx* ctx, int p)
{
  if (!ctx) return VLB_IllegalArgument;
  if (p < VLB_PRECISION_3XTF32 || p > VLB_PRECISION_FP32) return vlb::set_error(ctx, VLB_IllegalArgument, "precision");
  ctx->precision = p;
  return VLB_Success;
}
int vlb_ctx_get_precision(vlb_ctx* ctx) { return ctx ? ctx->precision : -1; }

char const* vlb_ctx_last_error(vlb_ctx* ctx) { return ctx ? ctx->lastErrorMessage.c_str() : "null context"; }
void vlb_ctx_reset_error(vlb_ctx* ctx) { if (ctx) { ctx->lastError = VLB_Success; ctx->lastErrorMessage.clear(); } }

int vlb_ctx_reserve_workspace(vlb_ctx* ctx, size_t bytes)
{
  if (!ctx) return VLB_IllegalArgument;
  return vlb::workspace(ctx, bytes) ? VLB_Success : ctx->lastError;
}
size_t vlb_ctx_workspace_bytes(vlb_ctx* ctx) { return ctx ? ctx->workspaceBytes : 0; }
int vlb_ctx_clear_workspace(vlb_ctx* ctx)
{
  if (!ctx) return VLB_IllegalArgument;
  if (ctx->workspace) { cudaStreamSynchronize(ctx->stream); cudaFree(ctx->workspace); }
  ctx->workspace = nullptr; ctx->workspaceBytes = 0;
  return VLB_Success;
}
long long vlb_ctx_launch_count(vlb_ctx* ctx) { return ctx ? ctx->launches : 0; }

int vlb_ctx_profile_begin(vlb_ctx* ctx)
{
  if (!ctx) return VLB_IllegalArgument;
  for (auto& r : ctx->prof) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
  ctx->prof.clear();
  ctx->profiling = true;
  return VLB_Success;
}

int vlb_ctx_profile_end(vlb_ctx* ctx, double* ms, double* flops, long long* launches)
{
  if (!ctx) return VLB_IllegalArgument;
  ctx->profiling = false;
  cudaError_t e = cudaStreamSynchronize(ctx->stream);
  double tms = 0, tf = 0;
  for (int k = 0; k < 4; ++k) { ctx->profKindMs[k] = 0; ctx->profKindFlops[k] = 0; ctx->profKindCount[k] = 0; }
  for (auto& r : ctx->prof) {
    float t = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, r.start, r.stop);
    tms += t; tf += r.flops;
    if (r.kind >= 0 && r.kind < 4) { ctx->profKindMs[r.kind] += t; ctx->profKindFlops[r.kind] += r.flops; ++ctx->profKindCount[r.kind]; }
    cudaEventDestroy(r.start); cudaEventDestroy(r.stop);
  }
  if (ms) *ms = tms;
  if (flops) *flops = tf;
  if (launches) *launches = (long long)ctx->prof.size();
  ctx->prof.clear();
  if (e != cudaSuccess) return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e));
  return VLB_Success;
}

int vlb_ctx_profile_kind(vlb_ctx* ctx, int kind, double* ms, double* flops, long long* count)
{
  if (!ctx || kind < 0 || kind > 3) return VLB_IllegalArgument;
  if (ms) *ms = ctx->profKindMs[kind];
  if (flops) *flops = ctx->profKindFlops[kind];
  if (count) *count = ctx->profKindCount[kind];
  return VLB_Success;
}

int vlb_ctx_device_status(vlb_ctx* ctx, int* status)
{
  if (!ctx || !status) return VLB_IllegalArgument;
  cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (e == cudaSuccess) e = cudaMemcpy(status, ctx->deviceStatus, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e));
  if (*status != 0) {
    cudaMemset(ctx->deviceStatus, 0, sizeof(int));
    if (*status == kStatusBadLabel)
      return vlb::set_error(ctx, VLB_IllegalArgument, "softmaxloss: a class label is larger than the number of classes");
    return vlb::set_error(ctx, VLB_Timeout, "a tensor-core kernel gave up waiting on a pipeline barrier");
  }
  return VLB_Success;
}

int vlb_ctx_set_test_switch(vlb_ctx* ctx, int switches)
{
  if (!ctx) return VLB_IllegalArgument;
  ctx->testSwitch = switches;
  return VLB_Success;
}

}  // extern "C"
