// Shared declarations for the engine's translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>
#include "../../include/vlb.h"

// The context: stream, grow-only scratch, sticky error message chain.
// Mirrors the parts of vl::Context / vl::CudaHelper the operators use
// (reference bits/data.hpp:150-179, bits/datacu.hpp:60-158).
struct vlb_ctx {
  int device = 0;
  cudaStream_t stream = 0;
  int precision = VLB_PRECISION_3XTF32;
  void* workspace = nullptr;
  size_t workspaceBytes = 0;
  int lastError = VLB_Success;
  std::string lastErrorMessage;
  long long launches = 0;
  int smCount = 148;
  int* deviceStatus = nullptr;   // one word the tensor-core kernels set when a bounded wait expires; behind it (byte 256)
                                 // 4096 zeroed ticket counters for last-block-finishes reductions, left at zero by their users
  // optional timing of the tensor-core launches with events on the launching stream
  struct ProfRec { cudaEvent_t start, stop; double flops; int kind; };
  int profDepth = 0;             // > 0: inside a bracket that spans several launches (vlb::ProfScope); the launches inside record nothing
  double profKindMs[4] = {0, 0, 0, 0}, profKindFlops[4] = {0, 0, 0, 0};     // per kind, filled by vlb_ctx_profile_end
  long long profKindCount[4] = {0, 0, 0, 0};
  // set by vlb_conv_relu_forward around its call of the forward convolution: the path that ran applies max(., 0) in its
  // epilogue and says so, otherwise the caller runs the ReLU kernel on the result
  bool fuseRelu = false, reluDone = false;
  // set by vlb_relu_conv_backward around its call of the backward convolution: the data-gradient path that ran zeroes dX
  // where reluMask (the convolution's input, a ReLU's output) is not positive and says so, otherwise the caller masks dX
  float const* reluMask = nullptr;
  bool maskDone = false;
  bool profiling = false;
  std::vector<ProfRec> prof;
  // vlb_ctx_set_test_switch: bit 0 makes the filter-tile loader of the tensor-memory convolution kernel stay idle, so that
  // the bounded waits behind it run out (a test of the time-out path: nothing faults or spins, the kernel gives up and returns)
  int testSwitch = 0;
};

// Values of the device status word (vlb_ctx::deviceStatus[0]).  1..63: a bounded pipeline wait of a tensor-core kernel
// ran out (the number says which); kStatusBadLabel: the softmax loss met a class label above the number of classes.
constexpr int kStatusBadLabel = 64;

namespace vlb {

int set_error(vlb_ctx* ctx, int code, char const* msg);
int pass_error(vlb_ctx* ctx, int code, char const* where);
// Scratch of at least `bytes`; contents belong to whichever op asked last
// (reference Context::getWorkspace, bits/data.cu:395-404).  nullptr on failure.
void* workspace(vlb_ctx* ctx, size_t bytes);
// cudaPeekAtLastError after a launch, as the reference does (bits/datacu.cu:356-371).
int check_launch(vlb_ctx* ctx, char const* where);

// Kinds of tensor-core contraction the profile tells apart (vlb_ctx_profile_kind).
enum { kProfFprop = 0, kProfDgrad = 1, kProfWgrad = 2, kProfFc = 3 };

// While profiling, brackets everything a contraction enqueues -- operand tile images, the contraction, the reduction of
// split partial results -- with one pair of events on the context's stream.  Records only when `flops` was set.
struct ProfScope {
  vlb_ctx* ctx;
  vlb_ctx::ProfRec rec;
  bool on;
  ProfScope(vlb_ctx* c, int kind) : ctx(c), on(c->profiling && c->profDepth == 0)
  {
    rec.flops = 0; rec.kind = kind;
    ++ctx->profDepth;
    if (on) { cudaEventCreate(&rec.start); cudaEventCreate(&rec.stop); cudaEventRecord(rec.start, ctx->stream); }
  }
  ~ProfScope()
  {
    --ctx->profDepth;
    if (!on) return;
    if (rec.flops > 0) { cudaEventRecord(rec.stop, ctx->stream); ctx->prof.push_back(rec); }
    else { cudaEventDestroy(rec.start); cudaEventDestroy(rec.stop); }
  }
};

// The opt-in to more than 48 KB of dynamic shared memory: everything the SM offers one block (227 KB) minus what the
// kernel declares statically.  Called once per kernel and device by the launch sites.
template <class Kernel>
inline cudaError_t allow_max_dynamic_smem(Kernel kernel)
{
  cudaFuncAttributes attr;
  cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - (int)attr.sharedSizeBytes);
}

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }
inline unsigned grid_for(size_t n, int threads, int maxBlocks = 148 * 16)
{
  size_t b = (n + threads - 1) / threads;
  if (b > (size_t)maxBlocks) b = maxBlocks;
  if (b == 0) b = 1;
  return (unsigned)b;
}

}  // namespace vlb

#ifdef __CUDACC__
namespace vlb {
// Exclusive prefix sum of v[0..n) in place by a whole block of kThreads threads (a multiple of 32, at most 1024);
// warpSums: 32 ints of shared memory.  Ends with a block barrier.
template <int kThreads>
__device__ inline void block_exclusive_scan(int* v, int n, int* warpSums)
{
  int const tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int const per = (n + kThreads - 1) / kThreads;
  int const beg = min(tid * per, n), end = min(beg + per, n);
  int sum = 0;
  for (int i = beg; i < end; ++i) sum += v[i];
  int incl = sum;
  for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
  if (lane == 31) warpSums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int const w = lane < kThreads / 32 ? warpSums[lane] : 0;
    int wi = w;
    for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, wi, o); if (lane >= o) wi += t; }
    warpSums[lane] = wi - w;      // exclusive over the warps
  }
  __syncthreads();
  int run = warpSums[warp] + incl - sum;
  for (int i = beg; i < end; ++i) { int c = v[i]; v[i] = run; run += c; }
  __syncthreads();
}
}  // namespace vlb
#endif

#define VLB_REQUIRE(ctx, cond, msg) \
  do { if (!(cond)) return vlb::set_error((ctx), VLB_IllegalArgument, (msg)); } while (0)

#define VLB_LAUNCHED(ctx, n) do { (ctx)->launches += (n); } while (0)
