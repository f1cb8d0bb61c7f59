// Bilinear sampler (vl::nn::BilinearSampler, reference bits/nnbilinearsampler.hpp:21-36;
// CPU definition bits/nnbilinearsampler.cu:32-149).
//
// Forward and backward-to-grid: one thread per output pixel (q = ho + Ho*wo, grid n) walks the C
// channels: the grid entry and the four tap weights are computed once and reused for every
// channel; reads of dy and writes of y are contiguous across the warp; x taps of neighbouring
// output pixels fall in the same or adjacent 32-byte sectors.  Backward-to-grid accumulates the
// channels in ascending order in a register, the order of the CPU loop, and writes each grid
// entry once.
//
// Backward-to-data is a gather, not the reference GPU code's four atomicAdds per output element
// (bits/impl/nnbilinearsampler_gpu.cu:38-118).  Which output pixels touch an input pixel depends
// on the grid alone, not on the channel, so one CTA per image first inverts the grid in shared
// memory: it counts the taps that land on every input pixel, prefix-sums the counts, fills one
// list (output pixel, tap) per input pixel and sorts each list by output pixel.  Then every
// input pixel adds up its list in ascending output-pixel order -- the order in which the CPU loop
// reaches that element (bits/nnbilinearsampler.cu:72-131) -- for four channels per walk of the
// list (the dY planes of four channels wait in shared memory, the next four travel meanwhile;
// decoding an entry and forming its weight is paid once for the four), and writes dX once: no
// atomics, no zero fill, the CPU's result bit for bit, identical from run to run.  The grid
// derivative is a second sweep of the same CTA over the channels, two at a time, with the x
// planes staged beside the dY planes (dY is read a second time), every output pixel adding its
// channels' terms in ascending channel order.  A grid that sends more than kMaxList taps to one
// input pixel, and planes too large for the lists, take the atomic scatter instead.
//
// Boundary rule of the CPU reference, kept as it is: the taps are guarded by
// `-1 <= sy && sy < inHeight` with inHeight a size_t (bits/nnbilinearsampler.cu:92), so
// sy == -1 is compared as a huge unsigned number and fails: samples whose floor is -1
// in either coordinate contribute nothing.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int kThreads = 128;

struct Taps {
  int sx, sy;
  float wx, wy;
  bool inside;
};

__device__ __forceinline__ Taps make_taps(float gy, float gx, int H, int W)
{
  Taps t;
  float py = __fmul_rn(__fmul_rn(0.5f, __fadd_rn(gy, 1.f)), (float)(H - 1));
  float px = __fmul_rn(__fmul_rn(0.5f, __fadd_rn(gx, 1.f)), (float)(W - 1));
  float fx = floorf(px), fy = floorf(py);
  // keep the int conversion defined for wild grid values
  fx = fminf(fmaxf(fx, -2.f), (float)W + 1.f);
  fy = fminf(fmaxf(fy, -2.f), (float)H + 1.f);
  t.sx = (int)fx; t.sy = (int)fy;
  t.inside = (t.sy >= 0 && t.sy < H && t.sx >= 0 && t.sx < W);
  t.wx = __fadd_rn(px, -(float)t.sx);
  t.wy = __fadd_rn(py, -(float)t.sy);
  return t;
}

// mode 0: forward.  mode 1: backward (dx and/or dgrid).
template <int kMode>
__global__ void sampler_kernel(float* __restrict__ y, float* __restrict__ dx, float* __restrict__ dgrid,
                               float const* __restrict__ x, float const* __restrict__ grid,
                               float const* __restrict__ dy, int H, int W, int C, int N, int Q, int Ng)
{
  int group = Ng / N;
  size_t total = (size_t)Q * Ng;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int q = (int)(i % Q);
    int n = (int)(i / Q);
    float2 gv = reinterpret_cast<float2 const*>(grid)[i];
    Taps t = make_taps(gv.x, gv.y, H, W);
    // tap (i = row offset, j = column offset); weights as in bits/nnbilinearsampler.cu:108-110
    float wwx[2] = {__fadd_rn(1.f, -t.wx), t.wx};
    float wwy[2] = {__fadd_rn(1.f, -t.wy), t.wy};
    bool ok[2][2];
    int idx[2][2];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        int ssy = t.sy + ii, ssx = t.sx + j;
        ok[j][ii] = t.inside && ssy >= 0 && ssy < H && ssx >= 0 && ssx < W;
        idx[j][ii] = ssy + ssx * H;
      }
    size_t imgOff = (size_t)H * W * C * (size_t)(n / group);
    float const* xz = x + imgOff;
    float* dxz = (kMode == 1 && dx) ? dx + imgOff : nullptr;
    size_t outOff = (size_t)q + (size_t)Q * C * (size_t)n;
    float accGy = 0.f, accGx = 0.f;
    for (int c = 0; c < C; ++c) {
      if (kMode == 0) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int ii = 0; ii < 2; ++ii)
            if (ok[j][ii]) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(wwx[j], wwy[ii]), xz[idx[j][ii]]));
        y[outOff] = acc;
      } else {
        float d = dy[outOff];
        float dgx = 0.f, dgy = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int ii = 0; ii < 2; ++ii)
            if (ok[j][ii]) {
              if (dxz) atomicAdd(dxz + idx[j][ii], __fmul_rn(__fmul_rn(wwx[j], wwy[ii]), d));
              if (dgrid) {
                float xv = xz[idx[j][ii]];
                float sj = j ? 1.f : -1.f, si = ii ? 1.f : -1.f;
                dgx = __fadd_rn(dgx, __fmul_rn(__fmul_rn(__fmul_rn(sj, wwy[ii]), d), xv));
                dgy = __fadd_rn(dgy, __fmul_rn(__fmul_rn(__fmul_rn(si, wwx[j]), d), xv));
              }
            }
        if (dgrid) {
          accGy = __fadd_rn(accGy, __fmul_rn(__fmul_rn(0.5f, (float)(H - 1)), dgy));
          accGx = __fadd_rn(accGx, __fmul_rn(__fmul_rn(0.5f, (float)(W - 1)), dgx));
        }
      }
      xz += (size_t)H * W;
      if (dxz) dxz += (size_t)H * W;
      outOff += Q;
    }
    if (kMode == 1 && dgrid) reinterpret_cast<float2*>(dgrid)[i] = make_float2(accGy, accGx);
  }
}

// ---- backward-to-data as a gather (see the header comment) ----
constexpr int kGatherThreads = 1024;
constexpr int kMaxList = 48;          // taps of one grid on one input pixel beyond which the scatter path is used
constexpr int kMaxQPerThread = 4;     // output pixels per thread whose taps and grid derivative are kept in registers
constexpr int kCB = 4;                // channels per stage: one walk of a pixel's list serves four channels

// Shared memory (bytes): the stage buffers -- float[2][4][Q] (dY planes of four channels, double buffered) for the data gradient,
// float[2][2 x HW + 2 x Q] (x and dY planes of two channels, double buffered) for the grid derivative -- | wq float2[Q] (the two
// fractions of every output pixel) | cur int[HW] | ent uint16[4Q] (list entries: output pixel << 2 | tap)
__host__ __device__ inline size_t gather_smem(int HW, int Q)
{
  size_t const stageFloats = 8 * (size_t)Q > 4 * ((size_t)HW + Q) ? 8 * (size_t)Q : 4 * ((size_t)HW + Q);
  return sizeof(float) * stageFloats + sizeof(int) * (size_t)HW + (sizeof(float2) + 4 * sizeof(uint16_t)) * (size_t)Q + 64;
}

__device__ __forceinline__ void cp_async4(uint32_t dst, void const* src)
{ asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void cp_async16(uint32_t dst, void const* src)
{ asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }

// n floats global -> shared by the whole block, asynchronously (16-byte pieces when both sides allow; copies of four bytes
// keep the load/store unit busy four times as long and were measured to slow the whole stage down)
__device__ __forceinline__ void stage_plane(float* dst, float const* src, int n)
{
  uint32_t const d = (uint32_t)__cvta_generic_to_shared(dst);
  if ((n & 3) == 0 && ((((uintptr_t)src) | d) & 15) == 0) {
    for (int i = threadIdx.x; i < n / 4; i += kGatherThreads) cp_async16(d + 16u * i, src + 4 * i);
  } else {
    for (int i = threadIdx.x; i < n; i += kGatherThreads) cp_async4(d + 4u * i, src + i);
  }
}

// dY of the channels c .. c + nst - 1 (nst <= 4) of one grid, Q floats per channel, as nst planes of Q floats
__device__ __forceinline__ void stage_dy4(float* dst, float const* src, int Q, int nst)
{
  for (int j = 0; j < nst; ++j) stage_plane(dst + (size_t)Q * j, src + (size_t)Q * j, Q);
}

template <bool kWantGrid>
__global__ void __launch_bounds__(kGatherThreads, 1)
sampler_bwd_gather_kernel(float* __restrict__ dx, float* __restrict__ dgrid, float const* __restrict__ x,
                          float const* __restrict__ grid, float const* __restrict__ dy, int H, int W, int C, int N, int Q, int Ng,
                          int chunks, int CH)
{
  extern __shared__ __align__(16) uint8_t sm[];
  __shared__ int warpSums[32];
  int const HW = H * W, tid = threadIdx.x;
  float* dy4 = reinterpret_cast<float*>(sm);                              // [2][4][Q]
  float2* wq = reinterpret_cast<float2*>(dy4 + (2 * kCB * (size_t)Q > 4 * ((size_t)HW + Q) ? 2 * kCB * (size_t)Q : 4 * ((size_t)HW + Q)));            // [Q]   (wx, wy) of every output pixel
  int* cur = reinterpret_cast<int*>(wq + Q);                              // [HW]  list ends (starts before the fill)
  uint16_t* ent = reinterpret_cast<uint16_t*>(cur + HW);                  // [4Q]  output pixel << 2 | tap (tap = 2*column offset + row offset)
  int const group = Ng / N;
  int const img = blockIdx.x / chunks, c0 = (blockIdx.x % chunks) * CH, nch = min(CH, C - c0);
  int const nStages = (nch + kCB - 1) / kCB;
  size_t const imgOff = (size_t)HW * C * (size_t)img;

  for (int gi = 0; gi < group; ++gi) {
    int const n = img * group + gi;
    float2 const* gr = reinterpret_cast<float2 const*>(grid) + (size_t)Q * n;
    float const* const dyn = dy + (size_t)Q * C * (size_t)n;
    // the first stage's dY starts travelling while the grid is inverted
    stage_dy4(dy4, dyn + (size_t)Q * c0, Q, min(kCB, nch));
    // ---- invert the grid: count, scan, fill, sort
    for (int i = tid; i < HW; i += kGatherThreads) cur[i] = 0;
    __syncthreads();
    for (int q = tid; q < Q; q += kGatherThreads) {
      float2 const gv = gr[q];
      Taps t = make_taps(gv.x, gv.y, H, W);
      wq[q] = make_float2(t.wx, t.wy);
      if (t.inside) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int ii = 0; ii < 2; ++ii) {
            int const ssy = t.sy + ii, ssx = t.sx + j;
            if (ssy < H && ssx < W) atomicAdd(&cur[ssy + ssx * H], 1);
          }
      }
    }
    __syncthreads();
    bool tooLong = false;
    for (int i = tid; i < HW; i += kGatherThreads) tooLong |= cur[i] > kMaxList;
    bool const scatter = __syncthreads_or(tooLong) != 0;
    if (!scatter) {
      vlb::block_exclusive_scan<kGatherThreads>(cur, HW, warpSums);
      for (int q = tid; q < Q; q += kGatherThreads) {
        float2 const gv = gr[q];
        Taps t = make_taps(gv.x, gv.y, H, W);
        if (t.inside) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int ii = 0; ii < 2; ++ii) {
              int const ssy = t.sy + ii, ssx = t.sx + j;
              if (ssy < H && ssx < W) {
                int const pos = atomicAdd(&cur[ssy + ssx * H], 1);
                ent[pos] = (uint16_t)((q << 2) | (2 * j + ii));
              }
            }
        }
      }
      __syncthreads();
      // every input pixel sorts its list by output pixel (an output pixel reaches an input pixel with one tap at most)
      for (int pix = tid; pix < HW; pix += kGatherThreads) {
        int const beg = pix == 0 ? 0 : cur[pix - 1], end = cur[pix];
        for (int a = beg + 1; a < end; ++a) {
          uint16_t const kq = ent[a];
          int b = a - 1;
          while (b >= beg && ent[b] > kq) { ent[b + 1] = ent[b]; --b; }
          ent[b + 1] = kq;
        }
      }
      // ---- data gradient, four channels at a time from shared memory: the dY of stage s + 1 travels while stage s is computed
      for (int st = 0; st < nStages; ++st) {
        int const cs = c0 + st * kCB, nst = min(kCB, c0 + nch - cs);
        float const* const ds = dy4 + (size_t)(st & 1) * kCB * Q;
        cp_async_wait_all();
        __syncthreads();                    // this stage's dY has landed (and the lists are sorted); the other buffer is no longer read
        if (st + 1 < nStages) stage_dy4(dy4 + (size_t)((st + 1) & 1) * kCB * Q, dyn + (size_t)Q * (cs + kCB), Q, min(kCB, c0 + nch - cs - kCB));
        // every input pixel adds up its list in output-pixel order, four channels per walk.  The weight of an entry
        // is wwx[j] * wwy[i] as the CPU loop forms it (bits/nnbilinearsampler.cu:108-110), from the output pixel's two fractions.
        float* const dxc = dx + imgOff + (size_t)HW * cs;
        for (int pix = tid; pix < HW; pix += kGatherThreads) {
          int const beg = pix == 0 ? 0 : cur[pix - 1], end = cur[pix];
          float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
          if (gi > 0) {
            a0 = dxc[pix];
            if (nst > 1) a1 = dxc[pix + (size_t)HW];
            if (nst > 2) a2 = dxc[pix + 2 * (size_t)HW];
            if (nst > 3) a3 = dxc[pix + 3 * (size_t)HW];
          }
          for (int e = beg; e < end; ++e) {
            unsigned const en = ent[e];
            unsigned const q = en >> 2;
            float2 const f = wq[q];
            float const wx = (en & 2u) ? f.x : __fadd_rn(1.f, -f.x), wy = (en & 1u) ? f.y : __fadd_rn(1.f, -f.y);
            float const w = __fmul_rn(wx, wy);
            float const* const d = ds + q;
            a0 = __fadd_rn(a0, __fmul_rn(w, d[0])); a1 = __fadd_rn(a1, __fmul_rn(w, d[Q]));
            a2 = __fadd_rn(a2, __fmul_rn(w, d[2 * Q])); a3 = __fadd_rn(a3, __fmul_rn(w, d[3 * Q]));
          }
          dxc[pix] = a0;
          if (nst > 1) dxc[pix + (size_t)HW] = a1;
          if (nst > 2) dxc[pix + 2 * (size_t)HW] = a2;
          if (nst > 3) dxc[pix + 3 * (size_t)HW] = a3;
        }
      }
      // ---- grid derivative: a second sweep over the channels, two at a time, with the x planes beside the dY planes in the
      // stage buffers (dY is read a second time).  Every output pixel adds its channels' terms in ascending channel order, the
      // taps in the CPU loop's order (column offset j outer, row offset i inner; bits/nnbilinearsampler.cu:98-128).
      // (2j-1)*wwy*dy*x is evaluated left to right there; a negation is exact, so the two magnitudes wwy0*dy and wwy1*dy serve
      // all four taps.
      if (kWantGrid) {
        float accGy[kMaxQPerThread], accGx[kMaxQPerThread];
        // this thread's output pixels: first tap's offset in the plane | which of the four taps exist << 28, the two fractions
        int tapInfo[kMaxQPerThread];
        float tapWx[kMaxQPerThread], tapWy[kMaxQPerThread];
#pragma unroll
        for (int k = 0; k < kMaxQPerThread; ++k) {
          accGy[k] = 0.f; accGx[k] = 0.f;
          tapInfo[k] = 0; tapWx[k] = 0.f; tapWy[k] = 0.f;
          int const q = tid + k * kGatherThreads;
          if (q < Q) {
            float2 const gv = gr[q];
            Taps t = make_taps(gv.x, gv.y, H, W);
            tapWx[k] = t.wx; tapWy[k] = t.wy;
            if (t.inside)
              tapInfo[k] = (t.sy + t.sx * H) |
                           ((1 | (t.sy + 1 < H ? 2 : 0) | (t.sx + 1 < W ? 4 : 0) | ((t.sy + 1 < H && t.sx + 1 < W) ? 8 : 0)) << 28);   // bit ii + 2*j
          }
        }
        float const sclY = __fmul_rn(0.5f, (float)(H - 1)), sclX = __fmul_rn(0.5f, (float)(W - 1));
        // buffer b: x planes of two channels, then their dY planes
        size_t const bufFloats = 2 * ((size_t)HW + Q);
        auto stage2 = [&](int b, int cs, int n2) {
          float* const base = dy4 + (size_t)b * bufFloats;
          for (int j = 0; j < n2; ++j) {
            stage_plane(base + (size_t)HW * j, x + imgOff + (size_t)HW * (cs + j), HW);
            stage_plane(base + 2 * (size_t)HW + (size_t)Q * j, dyn + (size_t)Q * (cs + j), Q);
          }
        };
        int const nStages2 = (nch + 1) / 2;
        __syncthreads();                    // the last stage's dY is no longer read
        stage2(0, c0, min(2, nch));
        for (int st = 0; st < nStages2; ++st) {
          int const cs = c0 + 2 * st, n2 = min(2, c0 + nch - cs);
          float const* const xs = dy4 + (size_t)(st & 1) * bufFloats;
          float const* const ds = xs + 2 * (size_t)HW;
          cp_async_wait_all();
          __syncthreads();
          if (st + 1 < nStages2) stage2((st + 1) & 1, cs + 2, min(2, c0 + nch - cs - 2));
#pragma unroll
          for (int k = 0; k < kMaxQPerThread; ++k) {
            int const q = tid + k * kGatherThreads;
            int const ok = (int)((unsigned)tapInfo[k] >> 28);
            if (q < Q && ok) {
              float const wx1 = tapWx[k], wy1 = tapWy[k], wx0 = __fadd_rn(1.f, -wx1), wy0 = __fadd_rn(1.f, -wy1);
              float const* p0 = xs + (tapInfo[k] & 0x0fffffff);      // taps (i = 0, 1; j = 0), and H further on (j = 1)
              float const* dq = ds + q;
              for (int j = 0; j < n2; ++j) {
                float const d = dq[0];
                float const ty0 = __fmul_rn(wy0, d), ty1 = __fmul_rn(wy1, d), tx0 = __fmul_rn(wx0, d), tx1 = __fmul_rn(wx1, d);
                float dgx, dgy;
                if (ok == 15) {
                  float const x00 = p0[0], x10 = p0[1], x01 = p0[H], x11 = p0[H + 1];
                  dgx = __fsub_rn(0.f, __fmul_rn(ty0, x00)); dgy = __fsub_rn(0.f, __fmul_rn(tx0, x00));
                  dgx = __fsub_rn(dgx, __fmul_rn(ty1, x10)); dgy = __fadd_rn(dgy, __fmul_rn(tx0, x10));
                  dgx = __fadd_rn(dgx, __fmul_rn(ty0, x01)); dgy = __fsub_rn(dgy, __fmul_rn(tx1, x01));
                  dgx = __fadd_rn(dgx, __fmul_rn(ty1, x11)); dgy = __fadd_rn(dgy, __fmul_rn(tx1, x11));
                } else {
                  {                                         // j = 0, i = 0: dgx -= wwy0*d*x, dgy -= wwx0*d*x
                    float const xv = p0[0];
                    dgx = __fsub_rn(0.f, __fmul_rn(ty0, xv)); dgy = __fsub_rn(0.f, __fmul_rn(tx0, xv));
                  }
                  if (ok & 2) {                             // j = 0, i = 1: dgx -= wwy1*d*x, dgy += wwx0*d*x
                    float const xv = p0[1];
                    dgx = __fsub_rn(dgx, __fmul_rn(ty1, xv)); dgy = __fadd_rn(dgy, __fmul_rn(tx0, xv));
                  }
                  if (ok & 4) {                             // j = 1, i = 0: dgx += wwy0*d*x, dgy -= wwx1*d*x
                    float const xv = p0[H];
                    dgx = __fadd_rn(dgx, __fmul_rn(ty0, xv)); dgy = __fsub_rn(dgy, __fmul_rn(tx1, xv));
                  }
                  if (ok & 8) {                             // j = 1, i = 1: dgx += wwy1*d*x, dgy += wwx1*d*x
                    float const xv = p0[H + 1];
                    dgx = __fadd_rn(dgx, __fmul_rn(ty1, xv)); dgy = __fadd_rn(dgy, __fmul_rn(tx1, xv));
                  }
                }
                accGy[k] = __fadd_rn(accGy[k], __fmul_rn(sclY, dgy));
                accGx[k] = __fadd_rn(accGx[k], __fmul_rn(sclX, dgx));
                p0 += HW; dq += Q;
              }
            }
          }
        }
#pragma unroll
        for (int k = 0; k < kMaxQPerThread; ++k) {
          int const q = tid + k * kGatherThreads;
          if (q < Q) reinterpret_cast<float2*>(dgrid)[(size_t)Q * n + q] = make_float2(accGy[k], accGx[k]);
        }
      }
    } else {
      // a grid that piles its taps on a few input pixels: zero (first grid of the image) and scatter with atomics, from
      // global memory
      cp_async_wait_all();
      if (gi == 0) {
        for (size_t i = tid; i < (size_t)HW * nch; i += kGatherThreads) dx[imgOff + (size_t)HW * c0 + i] = 0.f;
      }
      __syncthreads();
      for (int q = tid; q < Q; q += kGatherThreads) {
        float2 const gv = gr[q];
        Taps t = make_taps(gv.x, gv.y, H, W);
        float const wwx[2] = {__fadd_rn(1.f, -t.wx), t.wx};
        float const wwy[2] = {__fadd_rn(1.f, -t.wy), t.wy};
        float accGy = 0.f, accGx = 0.f;
        for (int c = 0; c < (kWantGrid ? C : nch); ++c) {
          int const ch = kWantGrid ? c : c0 + c;
          float const d = dyn[q + (size_t)Q * ch];
          float* const dxz = dx + imgOff + (size_t)HW * ch;
          float const* const xz = x + imgOff + (size_t)HW * ch;
          bool const mine = ch >= c0 && ch < c0 + nch;
          float dgx = 0.f, dgy = 0.f;
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int ii = 0; ii < 2; ++ii) {
              int const ssy = t.sy + ii, ssx = t.sx + j;
              if (t.inside && ssy < H && ssx < W) {
                if (mine) atomicAdd(dxz + ssy + ssx * H, __fmul_rn(__fmul_rn(wwx[j], wwy[ii]), d));
                if (kWantGrid) {
                  float const xv = __ldg(xz + ssy + ssx * H);
                  float const sj = j ? 1.f : -1.f, si = ii ? 1.f : -1.f;
                  dgx = __fadd_rn(dgx, __fmul_rn(__fmul_rn(__fmul_rn(sj, wwy[ii]), d), xv));
                  dgy = __fadd_rn(dgy, __fmul_rn(__fmul_rn(__fmul_rn(si, wwx[j]), d), xv));
                }
              }
            }
          if (kWantGrid) {
            accGy = __fadd_rn(accGy, __fmul_rn(__fmul_rn(0.5f, (float)(H - 1)), dgy));
            accGx = __fadd_rn(accGx, __fmul_rn(__fmul_rn(0.5f, (float)(W - 1)), dgx));
          }
        }
        if (kWantGrid) reinterpret_cast<float2*>(dgrid)[(size_t)Q * n + q] = make_float2(accGy, accGx);
      }
    }
    __syncthreads();       // this grid's additions to dX are visible to the block, and the lists free, before the next grid
  }
}

int validate(vlb_ctx* ctx, int H, int W, int C, int N, int Ho, int Wo, int Ng)
{
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0 && Ho > 0 && Wo > 0 && Ng > 0, "bilinearsampler: empty tensor");
  // GRID must hold a whole number of grids per image (matlab/src/vl_nnbilinearsampler.cu:141-146)
  VLB_REQUIRE(ctx, Ng % N == 0, "bilinearsampler: the number of grids is not a multiple of the number of images");
  VLB_REQUIRE(ctx, (long long)H * W < (1LL << 31) && (long long)Ho * Wo < (1LL << 31), "bilinearsampler: plane too large");
  return VLB_Success;
}

}  // namespace

extern "C" {

int vlb_sampler_forward(vlb_ctx* ctx, float* Y, float const* X, float const* grid, int H, int W, int C, int N,
                        int Ho, int Wo, int Ng)
{
  if (!ctx) return VLB_IllegalArgument;
  int rc = validate(ctx, H, W, C, N, Ho, Wo, Ng);
  if (rc) return rc;
  VLB_REQUIRE(ctx, Y && X && grid, "sampler_forward: null tensor");
  VLB_REQUIRE(ctx, (((uintptr_t)grid) & 7) == 0, "sampler_forward: grid must be 8-byte aligned");
  size_t total = (size_t)Ho * Wo * Ng;
  sampler_kernel<0><<<vlb::grid_for(total, kThreads, ctx->smCount * 32), kThreads, 0, ctx->stream>>>(
      Y, nullptr, nullptr, X, grid, nullptr, H, W, C, N, Ho * Wo, Ng);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_sampler_forward");
}

int vlb_sampler_backward(vlb_ctx* ctx, float* dX, float* dGrid, float const* X, float const* grid, float const* dY,
                         int H, int W, int C, int N, int Ho, int Wo, int Ng)
{
  if (!ctx) return VLB_IllegalArgument;
  int rc = validate(ctx, H, W, C, N, Ho, Wo, Ng);
  if (rc) return rc;
  VLB_REQUIRE(ctx, grid && dY, "sampler_backward: null tensor");
  VLB_REQUIRE(ctx, !dGrid || X, "sampler_backward: the grid derivative needs the input");
  VLB_REQUIRE(ctx, ((((uintptr_t)grid) | ((uintptr_t)dGrid)) & 7) == 0, "sampler_backward: grid must be 8-byte aligned");
  if (!dX && !dGrid) return VLB_Success;
  int const Qo = Ho * Wo, HWi = H * W;
  if (dX && Qo <= kMaxQPerThread * kGatherThreads && HWi < (1 << 28) && gather_smem(HWi, Qo) <= 226 * 1024) {
    // gather: one CTA per image; with fewer images than SMs the channels are shared out among several CTAs per image,
    // and the grid derivative (which runs over all channels of an output pixel in order) is left to the other kernel
    int chunks = 1;
    if (N < ctx->smCount) chunks = vlb::ceil_div(ctx->smCount, N);
    int CH = vlb::ceil_div(C, chunks);
    chunks = vlb::ceil_div(C, CH);
    bool const fusedGrid = dGrid != nullptr && chunks == 1;
    static bool attrDone[64] = {};
    if (!(ctx->device < 64 && attrDone[ctx->device])) {
      cudaError_t ea = vlb::allow_max_dynamic_smem(sampler_bwd_gather_kernel<true>);
      if (ea == cudaSuccess) ea = vlb::allow_max_dynamic_smem(sampler_bwd_gather_kernel<false>);
      if (ea != cudaSuccess) { cudaGetLastError(); return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(ea)); }
      if (ctx->device < 64) attrDone[ctx->device] = true;
    }
    size_t const smem = gather_smem(HWi, Qo);
    unsigned const blocks = (unsigned)(N * chunks);
    if (fusedGrid) sampler_bwd_gather_kernel<true><<<blocks, kGatherThreads, smem, ctx->stream>>>(dX, dGrid, X, grid, dY, H, W, C, N, Qo, Ng, chunks, CH);
    else           sampler_bwd_gather_kernel<false><<<blocks, kGatherThreads, smem, ctx->stream>>>(dX, nullptr, X, grid, dY, H, W, C, N, Qo, Ng, chunks, CH);
    VLB_LAUNCHED(ctx, 1);
    if (dGrid && !fusedGrid) {
      size_t total = (size_t)Qo * Ng;
      sampler_kernel<1><<<vlb::grid_for(total, kThreads, ctx->smCount * 32), kThreads, 0, ctx->stream>>>(
          nullptr, nullptr, dGrid, X, grid, dY, H, W, C, N, Qo, Ng);
      VLB_LAUNCHED(ctx, 1);
    }
    return vlb::check_launch(ctx, "vlb_sampler_backward");
  }
  if (dX) {
    cudaError_t e = cudaMemsetAsync(dX, 0, sizeof(float) * (size_t)H * W * C * N, ctx->stream);
    if (e != cudaSuccess) return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e));
  }
  size_t total = (size_t)Ho * Wo * Ng;
  sampler_kernel<1><<<vlb::grid_for(total, kThreads, ctx->smCount * 32), kThreads, 0, ctx->stream>>>(
      nullptr, dX, dGrid, X, grid, dY, H, W, C, N, Ho * Wo, Ng);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_sampler_backward");
}

}  // extern "C"
