// Direct CUDA-core convolutions for the two shapes at the image end of a network that a 128 x N
// tensor-core tile serves badly (reference bits/nnconv.cu:71-317 computes them with the same im2row +
// GEMM as every other layer):
//   * few input values per output pixel (R = FH*FW*C <= 64, e.g. a 3x3 filter on an RGB image): the
//     tensor-core kernel would run one k-block per CTA and be all prologue and epilogue;
//   * few output channels (<= 4, e.g. the data gradient of that first layer): 125 of the tile's 128
//     columns would be padding.
// Both are one thread per output pixel, so that loads and stores are coalesced along H (the fastest
// dimension of the MATLAB layout), with the filters in shared memory read as broadcasts.  Exact fp32 FMAs:
// the results are at least as accurate as the 3xTF32 arithmetic of the tensor-core path.
#include "conv_internal.cuh"
#include <stdint.h>
#include <algorithm>

namespace {

using vlb::ConvGeom;

constexpr int kThreads = 256;

struct SmallParams {
  float const* x;       // input (or dY for a data gradient), H x W x Cin x N
  float const* f;       // filter bank as stored, FH x FW x FC x K
  float* out;           // Ho x Wo x Kout x N
  float const* bias;    // per output channel or nullptr
  float inMult, outMult;
  int H, W, Cin, N, Ho, Wo, Kout;
  int FH, FW, sy, sx, pt, pl, dy, dx;
  int relu;             // apply max(., 0) to the stored value
  int flip;             // 0: forward filters F[fh,fw,c,k]; 1: data gradient, F[FH-1-fh, FW-1-fw, k(out), c(in)]
  int Cf;               // the filter bank's third extent (channels of the forward input)
};

// Pixel of this thread, element offset of its window origin and which tap rows / columns are inside the image.
struct Pix { long long base; uint32_t hm, wm; bool valid; long long outBase; };

__device__ __forceinline__ Pix pixel_of(SmallParams const& p, long long m)
{
  Pix q = {0, 0u, 0u, false, 0};
  long long const M = (long long)p.Ho * p.Wo * p.N;
  if (m >= M) return q;
  int const ho = (int)(m % p.Ho);
  long long const t = m / p.Ho;
  int const wo = (int)(t % p.Wo), n = (int)(t / p.Wo);
  q.valid = true;
  q.base = (long long)n * p.H * p.W * p.Cin + (long long)(wo * p.sx - p.pl) * p.H + (ho * p.sy - p.pt);
  for (int fh = 0; fh < p.FH; ++fh) { int h = ho * p.sy + fh * p.dy - p.pt; if (h >= 0 && h < p.H) q.hm |= 1u << fh; }
  for (int fw = 0; fw < p.FW; ++fw) { int w = wo * p.sx + fw * p.dx - p.pl; if (w >= 0 && w < p.W) q.wm |= 1u << fw; }
  q.outBase = (long long)n * p.Kout * p.Ho * p.Wo + (long long)wo * p.Ho + ho;
  return q;
}

__device__ __forceinline__ float filter_at(SmallParams const& p, int fh, int fw, int cin, int kout)
{
  if (!p.flip) return p.f[fh + (size_t)p.FH * (fw + (size_t)p.FW * (cin + (size_t)p.Cf * kout))];
  // data gradient: "input channel" cin is a filter index, "output channel" kout an image channel
  return p.f[(p.FH - 1 - fh) + (size_t)p.FH * ((p.FW - 1 - fw) + (size_t)p.FW * (kout + (size_t)p.Cf * cin))];
}

// ---- few inputs per pixel: KC accumulators per thread, filters [r][KC] in shared memory
template <int KC>
__global__ void __launch_bounds__(kThreads) conv_small_r_kernel(SmallParams p)
{
  extern __shared__ float4 smem4[];
  float* fs = reinterpret_cast<float*>(smem4);                 // [R][KC]
  int const taps = p.FH * p.FW, R = taps * p.Cin;
  int2* lut = reinterpret_cast<int2*>(fs + (size_t)R * KC);     // per r: {element offset, fh | fw << 5}
  int const k0 = blockIdx.y * KC;
  for (int i = threadIdx.x; i < R * KC; i += kThreads) {
    int const r = i / KC, k = i % KC;
    int const fh = r % p.FH, fw = (r / p.FH) % p.FW, c = r / taps;
    fs[i] = (k0 + k < p.Kout) ? filter_at(p, fh, fw, c, k0 + k) : 0.f;
  }
  for (int r = threadIdx.x; r < R; r += kThreads) {
    int const fh = r % p.FH, fw = (r / p.FH) % p.FW, c = r / taps;
    lut[r] = make_int2(c * p.H * p.W + fw * p.dx * p.H + fh * p.dy, fh | (fw << 5));
  }
  __syncthreads();
  long long const m = (long long)blockIdx.x * kThreads + threadIdx.x;
  Pix const q = pixel_of(p, m);
  float acc[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) acc[k] = 0.f;
  float const* xq = p.x + q.base;
  for (int r = 0; r < R; ++r) {
    int2 const te = lut[r];
    bool const on = ((q.hm >> (te.y & 31)) & (q.wm >> (te.y >> 5)) & 1u) != 0;
    float const xv = on ? __ldg(xq + te.x) : 0.f;
    float4 const* f4 = reinterpret_cast<float4 const*>(fs + (size_t)r * KC);
#pragma unroll
    for (int k4 = 0; k4 < KC / 4; ++k4) {
      float4 const w = f4[k4];
      acc[4 * k4 + 0] = fmaf(xv, w.x, acc[4 * k4 + 0]);
      acc[4 * k4 + 1] = fmaf(xv, w.y, acc[4 * k4 + 1]);
      acc[4 * k4 + 2] = fmaf(xv, w.z, acc[4 * k4 + 2]);
      acc[4 * k4 + 3] = fmaf(xv, w.w, acc[4 * k4 + 3]);
    }
  }
  if (!q.valid) return;
  long long const P = (long long)p.Ho * p.Wo;
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    if (k0 + k < p.Kout) {
      float* dst = p.out + q.outBase + (long long)(k0 + k) * P;
      float o = p.inMult * acc[k];
      if (p.bias) o += p.bias[k0 + k];
      if (p.outMult != 0.f) o += p.outMult * *dst;
      if (p.relu) o = o > 0.f ? o : 0.f;
      *dst = o;
    }
  }
}

// ---- few inputs per pixel, unit stride and dilation, output columns a multiple of four pixels high: four vertically adjacent
// pixels x KC filters per thread.  The FH + 3 input values of a (channel, filter column) serve all FH filter rows of the four
// pixels, and a filter value read from shared memory (a broadcast) feeds four FMAs instead of one: the kernel above spends as
// many shared-memory wavefronts as FMA issue slots, this one a quarter.  Stores are 16 bytes per thread and filter.
template <int KC, int FH>
__global__ void __launch_bounds__(kThreads) conv_small_r4_kernel(SmallParams p)
{
  extern __shared__ float4 smem4[];
  float* fs = reinterpret_cast<float*>(smem4);                 // [R][KC], r = fh + FH*(fw + FW*c)
  int const taps = FH * p.FW, R = taps * p.Cin;
  int const k0 = blockIdx.y * KC;
  for (int i = threadIdx.x; i < R * KC; i += kThreads) {
    int const r = i / KC, k = i % KC;
    int const fh = r % FH, fw = (r / FH) % p.FW, c = r / taps;
    fs[i] = (k0 + k < p.Kout) ? filter_at(p, fh, fw, c, k0 + k) : 0.f;
  }
  __syncthreads();
  int const quadsPerCol = p.Ho >> 2;
  long long const Q = (long long)quadsPerCol * p.Wo * p.N;
  // a block takes several groups of 256 quads, so that the staging of the filters above is paid once for all of them
  for (long long m4 = (long long)blockIdx.x * kThreads + threadIdx.x; m4 < Q; m4 += (long long)gridDim.x * kThreads) {
  int const ho0 = (int)(m4 % quadsPerCol) * 4;
  long long const t = m4 / quadsPerCol;
  int const wo = (int)(t % p.Wo), n = (int)(t / p.Wo);
  float acc[4][KC];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int k = 0; k < KC; ++k) acc[j][k] = 0.f;
  int const h0 = ho0 - p.pt;                                   // input row of window element 0
  float const* const xn = p.x + (long long)n * p.H * p.W * p.Cin;
  for (int c = 0; c < p.Cin; ++c) {
    for (int fw = 0; fw < p.FW; ++fw) {
      int const w = wo + fw - p.pl;
      bool const wOk = w >= 0 && w < p.W;
      float const* const col = xn + ((long long)c * p.W + (wOk ? w : 0)) * p.H;
      float xs[FH + 3];
#pragma unroll
      for (int i = 0; i < FH + 3; ++i) {
        int const h = h0 + i;
        bool const ok = wOk && h >= 0 && h < p.H;
        xs[i] = ok ? __ldg(col + h) : 0.f;
      }
      float4 const* f4 = reinterpret_cast<float4 const*>(fs + (size_t)(FH * (fw + p.FW * c)) * KC);
#pragma unroll
      for (int fh = 0; fh < FH; ++fh) {
#pragma unroll
        for (int k4 = 0; k4 < KC / 4; ++k4) {
          float4 const wv = f4[fh * (KC / 4) + k4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float const xv = xs[j + fh];
            acc[j][4 * k4 + 0] = fmaf(xv, wv.x, acc[j][4 * k4 + 0]);
            acc[j][4 * k4 + 1] = fmaf(xv, wv.y, acc[j][4 * k4 + 1]);
            acc[j][4 * k4 + 2] = fmaf(xv, wv.z, acc[j][4 * k4 + 2]);
            acc[j][4 * k4 + 3] = fmaf(xv, wv.w, acc[j][4 * k4 + 3]);
          }
        }
      }
    }
  }
  long long const P = (long long)p.Ho * p.Wo;
  float* const dst0 = p.out + (long long)n * p.Kout * P + (long long)wo * p.Ho + ho0;
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    if (k0 + k < p.Kout) {
      float4* dst = reinterpret_cast<float4*>(dst0 + (long long)(k0 + k) * P);
      float const b = p.bias ? p.bias[k0 + k] : 0.f;
      float4 o = make_float4(p.inMult * acc[0][k] + b, p.inMult * acc[1][k] + b, p.inMult * acc[2][k] + b, p.inMult * acc[3][k] + b);
      if (p.outMult != 0.f) { float4 const old = *dst; o.x += p.outMult * old.x; o.y += p.outMult * old.y; o.z += p.outMult * old.z; o.w += p.outMult * old.w; }
      if (p.relu) { o.x = o.x > 0.f ? o.x : 0.f; o.y = o.y > 0.f ? o.y : 0.f; o.z = o.z > 0.f ? o.z : 0.f; o.w = o.w > 0.f ? o.w : 0.f; }
      *dst = o;
    }
  }
  }
}

// ---- few output channels: NC accumulators per thread, filters [tap][cin][NC] in shared memory
template <int NC>
__global__ void __launch_bounds__(kThreads) conv_small_n_kernel(SmallParams p)
{
  extern __shared__ float4 smem4[];
  float* fs = reinterpret_cast<float*>(smem4);                 // [taps][Cin][NC]
  int const taps = p.FH * p.FW;
  int2* lut = reinterpret_cast<int2*>(fs + (size_t)taps * p.Cin * NC);      // per tap: {element offset, fh | fw << 5}
  for (int i = threadIdx.x; i < taps * p.Cin * NC; i += kThreads) {
    int const k = i % NC, c = (i / NC) % p.Cin, tap = i / (NC * p.Cin);
    fs[i] = k < p.Kout ? filter_at(p, tap % p.FH, tap / p.FH, c, k) : 0.f;
  }
  for (int t = threadIdx.x; t < taps; t += kThreads) {
    int const fh = t % p.FH, fw = t / p.FH;
    lut[t] = make_int2(fw * p.dx * p.H + fh * p.dy, fh | (fw << 5));
  }
  __syncthreads();
  long long const m = (long long)blockIdx.x * kThreads + threadIdx.x;
  Pix const q = pixel_of(p, m);
  float acc[NC];
#pragma unroll
  for (int k = 0; k < NC; ++k) acc[k] = 0.f;
  int const HW = p.H * p.W;
  for (int tap = 0; tap < taps; ++tap) {
    int2 const te = lut[tap];
    bool const on = ((q.hm >> (te.y & 31)) & (q.wm >> (te.y >> 5)) & 1u) != 0;
    if (!on) continue;
    float const* xq = p.x + q.base + te.x;
    float const* ft = fs + (size_t)tap * p.Cin * NC;
#pragma unroll 8
    for (int c = 0; c < p.Cin; ++c) {
      float const xv = __ldg(xq + (long long)c * HW);
      if (NC == 4) {
        float4 const w = *reinterpret_cast<float4 const*>(ft + 4 * c);
        acc[0] = fmaf(xv, w.x, acc[0]); acc[1] = fmaf(xv, w.y, acc[1]);
        acc[2] = fmaf(xv, w.z, acc[2]); acc[3] = fmaf(xv, w.w, acc[3]);
      } else {
#pragma unroll
        for (int k = 0; k < NC; ++k) acc[k] = fmaf(xv, ft[NC * c + k], acc[k]);
      }
    }
  }
  if (!q.valid) return;
  long long const P = (long long)p.Ho * p.Wo;
#pragma unroll
  for (int k = 0; k < NC; ++k) {
    if (k < p.Kout) {
      float* dst = p.out + q.outBase + (long long)k * P;
      float o = p.inMult * acc[k];
      if (p.bias) o += p.bias[k];
      if (p.outMult != 0.f) o += p.outMult * *dst;
      if (p.relu) o = o > 0.f ? o : 0.f;
      *dst = o;
    }
  }
}

// ---- few output channels, 3-row filters with one row of padding above, unit stride and dilation, columns a multiple of four
// pixels high: four vertically adjacent output pixels per thread.  The six input rows h0-1 .. h0+4 of a (filter column, input
// channel) -- one 16-byte load and two scalars -- serve all three filter rows of the four pixels, and a filter value read from
// shared memory feeds four FMAs: 2.3 times fewer load instructions per FMA than one pixel per thread.
template <int NC>
__global__ void __launch_bounds__(kThreads) conv_small_n4_kernel(SmallParams p)
{
  extern __shared__ float4 smem4[];
  float* fs = reinterpret_cast<float*>(smem4);                 // [tap][cin][4]
  int const taps = 3 * p.FW;
  for (int i = threadIdx.x; i < taps * p.Cin * 4; i += kThreads) {
    int const k = i & 3, c = (i >> 2) % p.Cin, tap = (i >> 2) / p.Cin;
    fs[i] = k < p.Kout ? filter_at(p, tap % 3, tap / 3, c, k) : 0.f;
  }
  __syncthreads();
  int const quadsPerCol = p.Ho >> 2;
  long long const Q = (long long)quadsPerCol * p.Wo * p.N;
  for (long long m4 = (long long)blockIdx.x * kThreads + threadIdx.x; m4 < Q; m4 += (long long)gridDim.x * kThreads) {
  int const ho0 = (int)(m4 % quadsPerCol) * 4;
  long long const t = m4 / quadsPerCol;
  int const wo = (int)(t % p.Wo), n = (int)(t / p.Wo);
  float acc[4][NC];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int k = 0; k < NC; ++k) acc[j][k] = 0.f;
  long long const HW = (long long)p.H * p.W;
  float const* const xn = p.x + (long long)n * HW * p.Cin;
  bool const up = ho0 - 1 >= 0, down = ho0 + 4 < p.H, mid = ho0 + 3 < p.H;      // (input and output have the same height here)
  for (int fw = 0; fw < p.FW; ++fw) {
    int const w = wo + fw - p.pl;
    if (w < 0 || w >= p.W) continue;
    float const* col = xn + (long long)w * p.H + ho0;
    float4 const* ft = reinterpret_cast<float4 const*>(fs) + (size_t)(3 * fw) * p.Cin;
#pragma unroll 4
    for (int c = 0; c < p.Cin; ++c, col += HW) {
      float xs[6];
      float4 const v = mid ? __ldg(reinterpret_cast<float4 const*>(col)) : make_float4(0.f, 0.f, 0.f, 0.f);
      xs[0] = up ? __ldg(col - 1) : 0.f;
      xs[1] = v.x; xs[2] = v.y; xs[3] = v.z; xs[4] = v.w;
      xs[5] = down ? __ldg(col + 4) : 0.f;
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        float4 const wv = ft[(size_t)fh * p.Cin + c];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float const xv = xs[j + fh];
          acc[j][0] = fmaf(xv, wv.x, acc[j][0]);
          if (NC > 1) acc[j][1] = fmaf(xv, wv.y, acc[j][1]);
          if (NC > 2) acc[j][2] = fmaf(xv, wv.z, acc[j][2]);
          if (NC > 3) acc[j][3] = fmaf(xv, wv.w, acc[j][3]);
        }
      }
    }
  }
  long long const P = (long long)p.Ho * p.Wo;
  float* const dst0 = p.out + (long long)n * p.Kout * P + (long long)wo * p.Ho + ho0;
#pragma unroll
  for (int k = 0; k < NC; ++k) {
    if (k < p.Kout) {
      float4* dst = reinterpret_cast<float4*>(dst0 + (long long)k * P);
      float const b = p.bias ? p.bias[k] : 0.f;
      float4 o = make_float4(p.inMult * acc[0][k] + b, p.inMult * acc[1][k] + b, p.inMult * acc[2][k] + b, p.inMult * acc[3][k] + b);
      if (p.outMult != 0.f) { float4 const old = *dst; o.x += p.outMult * old.x; o.y += p.outMult * old.y; o.z += p.outMult * old.z; o.w += p.outMult * old.w; }
      if (p.relu) { o.x = o.x > 0.f ? o.x : 0.f; o.y = o.y > 0.f ? o.y : 0.f; o.z = o.z > 0.f ? o.z : 0.f; o.w = o.w > 0.f ? o.w : 0.f; }
      *dst = o;
    }
  }
  }
}

// ---- filter (and bias) gradient with few inputs per pixel (R = FH*FW*C <= 27): dF[r][k] = sum over output pixels of
// x(pixel, r) * dY(pixel, k).  A block walks chunks of 256 consecutive output pixels: it stages the chunk's input windows
// (256 x R values, gathered once and then shared by all filters) and its 64 x 256 tile of dY in shared memory, both loaded
// coalesced along the pixels (runs of 1 KB per filter: with runs of 256 bytes the kernel ran at a seventh of the DRAM
// bandwidth); a lane owns the two filters `lane` and `lane + 32` and keeps their R x 2 sums in registers, a warp takes 32
// pixels of the chunk: per pixel seven broadcast 16-byte reads of the window, two conflict-free reads of dY and 54 FMAs.  Sums over a block's warps (shared memory, in warp order) and over the blocks (a second kernel, in block
// order): deterministic, no atomics.  The tensor-core kernels would use 27 of a tile's 128 rows for this shape.
constexpr int kWsR = 27, kWsRP = 28, kWsChunk = 256, kWsK = 64, kWsThreads = 256;

// 4-byte asynchronous copy global -> shared; srcBytes = 0 writes a zero instead (the source is not read)
__device__ __forceinline__ void ws_cp_async4(float* dst, float const* src, bool on)
{
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(on ? 4 : 0) : "memory");
}
__device__ __forceinline__ void ws_cp_async_wait() { asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(kWsThreads)
conv_wgrad_small_kernel(SmallParams p, float const* __restrict__ dy, float* __restrict__ part, long long M, int chunksPerBlock)
{
  extern __shared__ __align__(16) float wsSmem[];
  float (*xs)[kWsRP] = reinterpret_cast<float (*)[kWsRP]>(wsSmem);                                  // [chunk][28]: the chunk's windows
  float (*dys)[kWsChunk + 1] = reinterpret_cast<float (*)[kWsChunk + 1]>(wsSmem + kWsChunk * kWsRP); // [filter][chunk + 1]: dY of the chunk
  __shared__ int2 lut[kWsRP];                                 // per r: {element offset, fh | fw << 5}; unused r: never inside
  __shared__ float red[kWsRP][kWsK];
  int const taps = p.FH * p.FW, R = taps * p.Cin;
  int const tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kWsRP) {
    int const r = tid, fh = r % p.FH, fw = (r / p.FH) % p.FW, c = r / taps;
    lut[r] = r < R ? make_int2(c * p.H * p.W + fw * p.dx * p.H + fh * p.dy, fh | (fw << 5)) : make_int2(0, 31 | (31 << 5));
  }
  for (int i = tid; i < kWsRP * kWsK; i += kWsThreads) (&red[0][0])[i] = 0.f;
  __syncthreads();
  int const k0 = blockIdx.y * kWsK;
  long long const P = (long long)p.Ho * p.Wo;
  float acc[kWsR][2], accb[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < kWsR; ++r) { acc[r][0] = 0.f; acc[r][1] = 0.f; }
  int const sp = tid, sq = 0;                                  // staging: this thread's pixel of the chunk; it fills every row
  long long const chunk0 = (long long)blockIdx.x * chunksPerBlock;
  // this thread's staging pixel: decoded once, then advanced by a chunk at a time (no divisions in the loop)
  long long m = chunk0 * kWsChunk + sp;
  int ho = (int)(m % p.Ho), wo = (int)((m / p.Ho) % p.Wo), n = (int)(m / P);
  for (int ci = 0; ci < chunksPerBlock; ++ci, m += kWsChunk) {
    if (m - sp >= M) break;
    bool const valid = m < M;
    uint32_t hm = 0, wm = 0;
    for (int fh = 0; fh < p.FH; ++fh) { int h = ho * p.sy + fh * p.dy - p.pt; if (h >= 0 && h < p.H) hm |= 1u << fh; }
    for (int fw = 0; fw < p.FW; ++fw) { int w = wo * p.sx + fw * p.dx - p.pl; if (w >= 0 && w < p.W) wm |= 1u << fw; }
    float const* const xq = p.x + ((long long)n * p.H * p.W * p.Cin + (long long)(wo * p.sx - p.pl) * p.H + (ho * p.sy - p.pt));
    for (int r = sq; r < kWsRP; ++r) {
      int2 const te = lut[r];
      bool const on = valid && ((hm >> (te.y & 31)) & (wm >> (te.y >> 5)) & 1u) != 0;
      ws_cp_async4(&xs[sp][r], on ? xq + te.x : p.x, on);
    }
    {
      float const* const dq = dy + (long long)n * p.Kout * P + ((long long)wo * p.Ho + ho);
      // (asynchronous copies: all of a thread's 92 values are in flight together, none passes through a register)
#pragma unroll 8
      for (int k = sq; k < kWsK; ++k) {
        bool const on = valid && k0 + k < p.Kout;
        ws_cp_async4(&dys[k][sp], on ? dq + (long long)(k0 + k) * P : dy, on);
      }
    }
    ws_cp_async_wait();
    ho += kWsChunk;
    while (ho >= p.Ho) { ho -= p.Ho; if (++wo == p.Wo) { wo = 0; ++n; } }
    __syncthreads();
#pragma unroll 2
    for (int j = 0; j < kWsChunk / (kWsThreads / 32); ++j) {
      int const pp = warp * (kWsChunk / (kWsThreads / 32)) + j;
      float const d0 = dys[lane][pp], d1 = dys[lane + 32][pp];
      accb[0] += d0; accb[1] += d1;
      float4 const* const xr = reinterpret_cast<float4 const*>(&xs[pp][0]);
#pragma unroll
      for (int r4 = 0; r4 < kWsRP / 4; ++r4) {
        float4 const xv = xr[r4];
        float const x4[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int const r = 4 * r4 + e;
          if (r < kWsR) { acc[r][0] = fmaf(x4[e], d0, acc[r][0]); acc[r][1] = fmaf(x4[e], d1, acc[r][1]); }
        }
      }
    }
    __syncthreads();
  }
  // warps -> block, in warp order
  for (int w = 0; w < kWsThreads / 32; ++w) {
    if (warp == w) {
#pragma unroll
      for (int r = 0; r < kWsR; ++r) { red[r][lane] += acc[r][0]; red[r][lane + 32] += acc[r][1]; }
      red[kWsR][lane] += accb[0]; red[kWsR][lane + 32] += accb[1];
    }
    __syncthreads();
  }
  // part[blockIdx.x][k][r], r = kWsR holds the bias gradient's share
  for (int i = tid; i < kWsRP * kWsK; i += kWsThreads) {
    int const k = i / kWsRP, r = i % kWsRP;
    if (k0 + k < p.Kout) part[((size_t)blockIdx.x * p.Kout + k0 + k) * kWsRP + r] = red[r][k];
  }
}

// dF[r + R*k] = sum over blocks (ascending) of part[b][k][r]; db[k] likewise from row kWsR
__global__ void conv_wgrad_small_finish_kernel(float* __restrict__ dF, float* __restrict__ db, float const* __restrict__ part,
                                               int R, int K, int blocks)
{
  int const i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= K * kWsRP) return;
  int const k = i / kWsRP, r = i % kWsRP;
  float v = 0.f;
  for (int b = 0; b < blocks; ++b) v += part[((size_t)b * K + k) * kWsRP + r];
  if (r < R) dF[r + (size_t)R * k] = v;
  else if (r == kWsR && db) db[k] = v;
}

bool fits32(ConvGeom const& g)
{
  return (long long)g.H * g.W * g.C * g.N < (1LL << 31) - 256 && (long long)g.Ho * g.Wo * g.K * g.N < (1LL << 31) - 256;
}

}  // namespace

namespace vlb {

// Forward convolution with at most 64 input values per output pixel.
int conv_fprop_small(vlb_ctx* ctx, ConvGeom const& g, float* Y, float outMult, float const* X, float inMult,
                     float const* F, float const* b)
{
  int const R = g.FH * g.FW * g.FC;
  long long const pixels = (long long)g.Ho * g.Wo * g.N;
  if (g.G != 1 || R > 64 || pixels < 4096 || g.FH > 31 || g.FW > 26 || !fits32(g)) return VLB_Unsupported;
  SmallParams p = {};
  p.x = X; p.f = F; p.out = Y; p.bias = b; p.inMult = inMult; p.outMult = outMult;
  p.H = g.H; p.W = g.W; p.Cin = g.C; p.N = g.N; p.Ho = g.Ho; p.Wo = g.Wo; p.Kout = g.K;
  p.FH = g.FH; p.FW = g.FW; p.sy = g.sy; p.sx = g.sx; p.pt = g.pt; p.pl = g.pl; p.dy = g.dy; p.dx = g.dx;
  p.flip = 0; p.Cf = g.FC;
  p.relu = ctx->fuseRelu; ctx->reluDone = ctx->fuseRelu;
  long long const M = (long long)g.Ho * g.Wo * g.N;
  if (g.sy == 1 && g.sx == 1 && g.dy == 1 && g.dx == 1 && g.Ho % 4 == 0 && (g.FH == 3 || g.FH == 5) && g.K % 4 == 0 &&
      (((uintptr_t)Y) & 15) == 0) {
    constexpr int KC = 16;
    dim3 grid4((unsigned)std::min<long long>(ceil_div(M / 4, kThreads), (long long)ctx->smCount * 8), (unsigned)ceil_div(g.K, KC));
    size_t const smem4 = sizeof(float) * (size_t)R * KC;
    if (g.FH == 3) conv_small_r4_kernel<KC, 3><<<grid4, kThreads, smem4, ctx->stream>>>(p);
    else           conv_small_r4_kernel<KC, 5><<<grid4, kThreads, smem4, ctx->stream>>>(p);
    VLB_LAUNCHED(ctx, 1);
    return check_launch(ctx, "conv_fprop_small");
  }
  int const KC = g.K > 32 ? 64 : (g.K > 16 ? 32 : 16);
  dim3 grid((unsigned)ceil_div(M, kThreads), (unsigned)ceil_div(g.K, KC));
  size_t const smem = sizeof(float) * (size_t)R * KC + sizeof(int2) * (size_t)R;
  if (KC == 64) conv_small_r_kernel<64><<<grid, kThreads, smem, ctx->stream>>>(p);
  else if (KC == 32) conv_small_r_kernel<32><<<grid, kThreads, smem, ctx->stream>>>(p);
  else conv_small_r_kernel<16><<<grid, kThreads, smem, ctx->stream>>>(p);
  VLB_LAUNCHED(ctx, 1);
  return check_launch(ctx, "conv_fprop_small");
}

// Filter and bias gradients of a convolution with at most 27 input values per output pixel.
int conv_wgrad_small(vlb_ctx* ctx, ConvGeom const& g, float* dF, float* db, float const* X, float const* dY, bool* dbDone)
{
  *dbDone = false;
  int const R = g.FH * g.FW * g.FC;
  long long const M = (long long)g.Ho * g.Wo * g.N;
  if (g.G != 1 || R > kWsR || M < 4096 || g.FH > 30 || g.FW > 26 || !fits32(g)) return VLB_Unsupported;
  SmallParams p = {};
  p.x = X; p.H = g.H; p.W = g.W; p.Cin = g.C; p.N = g.N; p.Ho = g.Ho; p.Wo = g.Wo; p.Kout = g.K;
  p.FH = g.FH; p.FW = g.FW; p.sy = g.sy; p.sx = g.sx; p.pt = g.pt; p.pl = g.pl; p.dy = g.dy; p.dx = g.dx;
  int const kGroups = ceil_div(g.K, kWsK);
  long long const chunks = (M + kWsChunk - 1) / kWsChunk;
  int blocksX = (int)std::min<long long>(chunks, std::max(1, (2 * ctx->smCount) / kGroups));     // two blocks per SM
  int const chunksPerBlock = (int)((chunks + blocksX - 1) / blocksX);
  blocksX = (int)((chunks + chunksPerBlock - 1) / chunksPerBlock);
  float* part = (float*)workspace(ctx, sizeof(float) * (size_t)blocksX * g.K * kWsRP);
  if (!part) return ctx->lastError;
  size_t const smem = sizeof(float) * ((size_t)kWsChunk * kWsRP + (size_t)kWsK * (kWsChunk + 1));
  static bool attrDone[64] = {};
  if (ctx->device < 0 || ctx->device >= 64 || !attrDone[ctx->device]) {
    cudaError_t e = cudaFuncSetAttribute(conv_wgrad_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { cudaGetLastError(); return set_error(ctx, VLB_Cuda, cudaGetErrorString(e)); }
    if (ctx->device >= 0 && ctx->device < 64) attrDone[ctx->device] = true;
  }
  conv_wgrad_small_kernel<<<dim3((unsigned)blocksX, (unsigned)kGroups), kWsThreads, smem, ctx->stream>>>(p, dY, part, M, chunksPerBlock);
  int const n = g.K * kWsRP;
  conv_wgrad_small_finish_kernel<<<ceil_div(n, 256), 256, 0, ctx->stream>>>(dF, db, part, R, g.K, blocksX);
  VLB_LAUNCHED(ctx, 2);
  *dbDone = db != nullptr;
  return check_launch(ctx, "conv_wgrad_small");
}

// Data gradient of a stride-1 convolution whose input has at most 4 channels: a forward convolution of dY
// with the flipped, transposed filters and padding (F-1)*dilate - pad.
int conv_dgrad_small(vlb_ctx* ctx, ConvGeom const& g, float* dX, float const* F, float const* dY)
{
  if (g.G != 1 || g.C > 4 || g.sy != 1 || g.sx != 1 || (long long)g.H * g.W * g.N < 4096 || g.FH > 31 || g.FW > 26 || !fits32(g))
    return VLB_Unsupported;
  int const taps = g.FH * g.FW;
  size_t const smem = sizeof(float) * (size_t)taps * g.K * 4 + sizeof(int2) * (size_t)taps;
  if (smem > 48 * 1024) return VLB_Unsupported;
  SmallParams p = {};
  p.x = dY; p.f = F; p.out = dX; p.bias = nullptr; p.inMult = 1.f; p.outMult = 0.f;
  p.H = g.Ho; p.W = g.Wo; p.Cin = g.K; p.N = g.N; p.Ho = g.H; p.Wo = g.W; p.Kout = g.C;
  p.FH = g.FH; p.FW = g.FW; p.sy = 1; p.sx = 1; p.dy = g.dy; p.dx = g.dx;
  p.pt = (g.FH - 1) * g.dy - g.pt; p.pl = (g.FW - 1) * g.dx - g.pl;
  p.flip = 1; p.Cf = g.FC;
  long long const M = (long long)g.H * g.W * g.N;
  // filter rows: fh' = 0..2 with pt' = 1 row of padding above; the input (dY) and the output (dX) have the same height
  if (g.FH == 3 && p.pt == 1 && g.dy == 1 && g.dx == 1 && g.Ho == g.H && g.H % 4 == 0 && g.C <= 3 &&
      (((uintptr_t)dX) & 15) == 0 && (((uintptr_t)dY) & 15) == 0) {
    conv_small_n4_kernel<3><<<(unsigned)ceil_div(M / 4, kThreads), kThreads, smem, ctx->stream>>>(p);      // (one group of quads per block measured faster here than a bounded grid)
    VLB_LAUNCHED(ctx, 1);
    return check_launch(ctx, "conv_dgrad_small");
  }
  conv_small_n_kernel<4><<<(unsigned)ceil_div(M, kThreads), kThreads, smem, ctx->stream>>>(p);
  VLB_LAUNCHED(ctx, 1);
  return check_launch(ctx, "conv_dgrad_small");
}

}  // namespace vlb
