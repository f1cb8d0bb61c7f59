// ROI pooling (vl::nn::ROIPooling, reference bits/nnroipooling.hpp:23-45; CPU definition
// bits/nnroipooling.cu:102-189 forward, :217-305 backward).
//
// The bin geometry follows the CPU reference's arithmetic exactly -- affine map in
// double rounded to float, round-half-away, bin size as a double quotient rounded to
// float, float products with floor/ceil (bits/nnroipooling.cu:129-165) -- using the
// _rn intrinsics so that no multiply-add is contracted; the reference's own GPU code
// does the same maths in float throughout and can differ in the last place.
// Forward: one thread per output bin; adjacent threads take adjacent ph, so reads of a bin
// column are contiguous.  The scan order for the arg-max is the CPU's (w outer, h inner,
// first strictly greater).
//
// Backward (max) does not scatter with atomics as the reference GPU code does
// (bits/impl/nnroipooling_gpu.cu:114-246).  One CTA takes one image and a few channels.  All its
// threads first find, from the input plane in shared memory, the arg-max pixel of every bin of every
// ROI of the image; then one warp per channel walks the bins in the order of the CPU loop (ROI, bin
// column, bin row; bits/nnroipooling.cu:239-300), 32 at a time, and adds their derivatives to a copy
// of the channel's dX plane in shared memory -- lanes whose bins routed to the same pixel one after
// the other in lane order (__match_any_sync), all others at once.  The work is proportional to the
// number of bins, the sums are the CPU's bit for bit and identical from run to run, dX is written
// exactly once (no zero fill), and nothing but x, dY and dX crosses HBM.  Backward (avg), where every
// pixel of a bin receives a share, is a gather: every pixel of a channel slab walks the ROIs that
// cover it, in the same order.  Maps too large for shared memory take a zero fill and an atomic
// scatter.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int kThreads = 256;

struct RoiParams {
  int H, W, C, N, numROIs, S0, S1;
  double tf[6];
};

struct RoiGeom { int image, start_h, start_w; float bin_h, bin_w; };

__device__ __forceinline__ RoiGeom roi_geom(float const* r, RoiParams const& p)
{
  RoiGeom g;
  double u1_ = (double)r[1], v1_ = (double)r[2], u2_ = (double)r[3], v2_ = (double)r[4];
  // (tf0*u + tf2*v) + tf4, each step rounded to double: no fused multiply-add
  float u1 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[0], u1_), __dmul_rn(p.tf[2], v1_)), p.tf[4]);
  float v1 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[1], u1_), __dmul_rn(p.tf[3], v1_)), p.tf[5]);
  float u2 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[0], u2_), __dmul_rn(p.tf[2], v2_)), p.tf[4]);
  float v2 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[1], u2_), __dmul_rn(p.tf[3], v2_)), p.tf[5]);
  int image = (int)r[0];
  // ::round on the float promoted to double (bits/nnroipooling.cu:137-140)
  g.start_h = (int)round((double)v1) - 1;
  g.start_w = (int)round((double)u1) - 1;
  int end_h = (int)round((double)v2) - 1, end_w = (int)round((double)u2) - 1;
  int rh = max(end_h - g.start_h + 1, 1), rw = max(end_w - g.start_w + 1, 1);
  g.image = min(max(image - 1, 0), p.N - 1);
  g.bin_h = (float)((double)rh / (double)p.S0);
  g.bin_w = (float)((double)rw / (double)p.S1);
  return g;
}

__device__ __forceinline__ void roi_bin(int q, float bin, int start, int extent, int& lo, int& hi)
{
  int a = (int)floorf(__fmul_rn((float)q, bin));
  int b = (int)ceilf(__fmul_rn((float)(q + 1), bin));
  lo = min(max(a + start, 0), extent);
  hi = min(max(b + start, 0), extent);
}

__global__ void roipool_bounds_kernel(int* __restrict__ bounds, int* __restrict__ images,
                                      float const* __restrict__ rois, RoiParams p)
{
  int total = p.S0 * p.S1 * p.numROIs;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    int ph = i % p.S0, pw = (i / p.S0) % p.S1, r = i / (p.S0 * p.S1);
    RoiGeom g = roi_geom(rois + 5 * (size_t)r, p);
    int hs, he, ws, we;
    roi_bin(ph, g.bin_h, g.start_h, p.H, hs, he);
    roi_bin(pw, g.bin_w, g.start_w, p.W, ws, we);
    bounds[4 * (size_t)i + 0] = hs; bounds[4 * (size_t)i + 1] = he;
    bounds[4 * (size_t)i + 2] = ws; bounds[4 * (size_t)i + 3] = we;
    if (images && ph == 0 && pw == 0) images[r] = g.image;
  }
}

// kBackward = false: y[bin] = max / mean.  kBackward = true: dx += routed dy.
template <bool kMax, bool kBackward>
__global__ void roipool_kernel(float* __restrict__ out, float const* __restrict__ x,
                               float const* __restrict__ rois, float const* __restrict__ dy, RoiParams p)
{
  size_t total = (size_t)p.S0 * p.S1 * p.C * p.numROIs;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int ph = (int)(i % p.S0);
    size_t t = i / p.S0;
    int pw = (int)(t % p.S1); t /= p.S1;
    int c = (int)(t % p.C);
    int r = (int)(t / p.C);
    RoiGeom g = roi_geom(rois + 5 * (size_t)r, p);
    int hs, he, ws, we;
    roi_bin(ph, g.bin_h, g.start_h, p.H, hs, he);
    roi_bin(pw, g.bin_w, g.start_w, p.W, ws, we);
    size_t off = (size_t)p.H * p.W * ((size_t)c + (size_t)p.C * g.image);
    float const* xz = x + off;
    bool empty = (he <= hs) || (we <= ws);
    if (!kBackward) {
      float o = 0.f;
      if (!empty) {
        if (kMax) {
          float best = -INFINITY;
          for (int w = ws; w < we; ++w)
            for (int h = hs; h < he; ++h) { float a = xz[(size_t)w * p.H + h]; best = (best < a) ? a : best; }
          o = best;
        } else {
          float s = 0.f;
          for (int w = ws; w < we; ++w)
            for (int h = hs; h < he; ++h) s = __fadd_rn(s, xz[(size_t)w * p.H + h]);
          o = __fmul_rn(s, __fdiv_rn(1.f, (float)((he - hs) * (we - ws))));
        }
      }
      out[i] = o;
    } else {
      if (empty) continue;
      float d = dy[i];
      float* dxz = out + off;
      if (kMax) {
        float best = -INFINITY;
        long where = -1;
        for (int w = ws; w < we; ++w)
          for (int h = hs; h < he; ++h) {
            float a = xz[(size_t)w * p.H + h];
            if (a > best) { best = a; where = (long)w * p.H + h; }
          }
        if (where >= 0) atomicAdd(dxz + where, d);
      } else {
        float g2 = __fmul_rn(d, __fdiv_rn(1.f, (float)((he - hs) * (we - ws))));
        for (int w = ws; w < we; ++w)
          for (int h = hs; h < he; ++h) atomicAdd(dxz + (size_t)w * p.H + h, g2);
      }
    }
  }
}

// ---- backward as a gather (see the header comment) ----
constexpr int kGatherThreads = 1024;
constexpr uint32_t kNoBin = 0xFFFFu;

// Shared-memory layout (bytes): slab float[CH*HW] (max only) | argmax uint16[RB*CH*S0*S1] (max only) |
// binRow uint32[RB*S0], binCol uint32[RB*S1]: start | end << 16 of every bin row / column of every ROI of the batch |
// rowMask uint32[H*words], colMask uint32[W*words]: bit j of word k set when ROI 32k+j of the batch covers that map row /
// column | rowTab uint16[RB*H], colTab uint16[RB*W]: lo | hi << 8, the bin rows / columns covering it, or kNoBin | roiIdx int[RB].
__host__ __device__ inline size_t gather_smem(int CH, int RB, int H, int W, int S0, int S1, bool isMax)
{
  int const words = (RB + 31) / 32;
  size_t b = isMax ? sizeof(float) * (size_t)CH * H * W : 0;
  b += isMax ? ((sizeof(uint16_t) * (size_t)RB * CH * S0 * S1 + 15) & ~(size_t)15) : 0;
  b += sizeof(uint32_t) * (size_t)RB * (S0 + S1);
  b += sizeof(uint32_t) * (size_t)words * (H + W);
  b += (sizeof(uint16_t) * (size_t)RB * (H + W) + 15) & ~(size_t)15;
  b += sizeof(int) * (size_t)RB;
  return b + 64;
}

template <bool kMax>
__global__ void __launch_bounds__(kGatherThreads, 1)
roipool_bwd_gather_kernel(float* __restrict__ dx, float const* __restrict__ x, float const* __restrict__ rois,
                          float const* __restrict__ dy, RoiParams p, int CH, int RB, int chunks)
{
  extern __shared__ __align__(16) uint8_t sm[];
  __shared__ int sCount, sNext;
  int const HW = p.H * p.W, bins = p.S0 * p.S1, words = (RB + 31) / 32;
  int const img = blockIdx.x / chunks, c0 = (blockIdx.x % chunks) * CH;
  int const nch = min(CH, p.C - c0);
  int const tid = threadIdx.x, lane = tid & 31;
  uint8_t* q = sm;
  float* slab = reinterpret_cast<float*>(q);
  if (kMax) q += sizeof(float) * (size_t)CH * HW;
  uint16_t* am = reinterpret_cast<uint16_t*>(q);
  if (kMax) q += (sizeof(uint16_t) * (size_t)RB * CH * bins + 15) & ~(size_t)15;
  uint32_t* binRow = reinterpret_cast<uint32_t*>(q);
  uint32_t* binCol = binRow + (size_t)RB * p.S0;
  uint32_t* rowMask = binCol + (size_t)RB * p.S1;
  uint32_t* colMask = rowMask + (size_t)words * p.H;
  uint16_t* rowTab = reinterpret_cast<uint16_t*>(colMask + (size_t)words * p.W);
  uint16_t* colTab = rowTab + (size_t)RB * p.H;
  q = reinterpret_cast<uint8_t*>(rowTab) + ((sizeof(uint16_t) * (size_t)RB * (p.H + p.W) + 15) & ~(size_t)15);
  int* roiIdx = reinterpret_cast<int*>(q);

  size_t const slabOff = (size_t)HW * ((size_t)c0 + (size_t)p.C * img);
  if (kMax) {
    for (int i = tid; i < nch * HW; i += kGatherThreads) slab[i] = x[slabOff + i];
  }
  bool first = true;
  int base = 0;
  while (true) {
    __syncthreads();                                  // the previous batch's tables are no longer read
    if (tid < 32) {
      // the next RB ROIs of this image, in ascending order
      int cnt = 0, r = base;
      while (r < p.numROIs && cnt < RB) {
        int const rr = r + lane;
        bool mine = false;
        if (rr < p.numROIs) {
          int image = (int)rois[5 * (size_t)rr];
          mine = min(max(image - 1, 0), p.N - 1) == img;
        }
        unsigned const m = __ballot_sync(0xffffffffu, mine);
        int const pos = cnt + __popc(m & ((1u << lane) - 1u));
        if (mine && pos < RB) roiIdx[pos] = rr;
        int const tot = __popc(m);
        if (cnt + tot > RB) {                           // the batch is full inside this group of 32: resume behind its last member
          r += (int)__fns(m, 0, RB - cnt) + 1;
          cnt = RB;
          break;
        }
        cnt += tot; r += 32;
      }
      if (lane == 0) { sCount = cnt; sNext = min(r, p.numROIs); }
    }
    __syncthreads();
    int const nb = sCount;
    base = sNext;
    if (nb == 0) break;
    // bin geometry of every ROI of the batch, once (the double-precision part of the arithmetic)
    for (int i = tid; i < nb * (p.S0 + p.S1); i += kGatherThreads) {
      bool const isRow = i < nb * p.S0;
      int const k = isRow ? i : i - nb * p.S0;
      int const S = isRow ? p.S0 : p.S1;
      int const j = k / S, b = k - j * S;
      RoiGeom g = roi_geom(rois + 5 * (size_t)roiIdx[j], p);
      int s, e;
      roi_bin(b, isRow ? g.bin_h : g.bin_w, isRow ? g.start_h : g.start_w, isRow ? p.H : p.W, s, e);
      (isRow ? binRow : binCol)[k] = (uint32_t)s | ((uint32_t)e << 16);
    }
    __syncthreads();
    // which bin rows cover map row h, which bin columns cover map column w
    for (int i = tid; i < nb * (p.H + p.W); i += kGatherThreads) {
      bool const isRow = i < nb * p.H;
      int const k = isRow ? i : i - nb * p.H;
      int const ext = isRow ? p.H : p.W, S = isRow ? p.S0 : p.S1;
      int const j = k / ext, pos = k - j * ext;
      uint32_t const* tab = (isRow ? binRow : binCol) + (size_t)j * S;
      uint32_t lo = kNoBin, hi = 0;
      for (int b = 0; b < S; ++b) {
        uint32_t const se = tab[b];
        if ((int)(se & 0xFFFFu) <= pos && pos < (int)(se >> 16)) { if (lo == kNoBin) lo = (uint32_t)b; hi = (uint32_t)b; }
      }
      (isRow ? rowTab : colTab)[k] = (uint16_t)(lo == kNoBin ? kNoBin : (lo | (hi << 8)));
    }
    if (kMax) {
      // arg-max of every bin: CPU scan order, first strictly greater, none for an empty or all -inf / NaN bin
      for (int b = tid; b < nb * nch * bins; b += kGatherThreads) {
        int const ph = b % p.S0;
        int t = b / p.S0;
        int const pw = t % p.S1; t /= p.S1;
        int const cc = t % nch, j = t / nch;
        uint32_t const rs = binRow[j * p.S0 + ph], cs = binCol[j * p.S1 + pw];
        int const hs = (int)(rs & 0xFFFFu), he = (int)(rs >> 16), ws = (int)(cs & 0xFFFFu), we = (int)(cs >> 16);
        float const* xz = slab + (size_t)cc * HW;
        float best = -INFINITY;
        uint32_t where = kNoBin;
        for (int w = ws; w < we; ++w)
          for (int h = hs; h < he; ++h) {
            float a = xz[w * p.H + h];
            if (a > best) { best = a; where = (uint32_t)(w * p.H + h); }
          }
        am[b] = (uint16_t)where;
      }
    }
    __syncthreads();
    // bit masks: the ROIs of the batch that cover a map row / column, so that a pixel visits only ROIs that contain it
    for (int i = tid; i < words * (p.H + p.W); i += kGatherThreads) {
      bool const isRow = i < words * p.H;
      int const k = isRow ? i : i - words * p.H;
      int const ext = isRow ? p.H : p.W;
      int const pos = k / words, wd = k - pos * words;
      uint16_t const* tab = isRow ? rowTab : colTab;
      uint32_t m = 0;
      for (int j = wd * 32; j < min(nb, wd * 32 + 32); ++j)
        if (tab[j * ext + pos] != kNoBin) m |= 1u << (j & 31);
      (isRow ? rowMask : colMask)[k] = m;
    }
    __syncthreads();
    for (int item = tid; item < nch * HW; item += kGatherThreads) {
      int const cc = item / HW, pix = item - cc * HW;
      int const w = pix / p.H, h = pix - w * p.H;
      float* const dst = dx + slabOff + item;
      float acc = first ? 0.f : *dst;
      for (int wd = 0; wd < words; ++wd) {
        uint32_t m = rowMask[h * words + wd] & colMask[w * words + wd];
        while (m) {
          int const j = wd * 32 + __ffs(m) - 1;          // ascending: the order of the CPU loop over the ROIs
          m &= m - 1;
          uint32_t const rt = rowTab[j * p.H + h], ct = colTab[j * p.W + w];
          float const* dyr = dy + (size_t)bins * ((size_t)(c0 + cc) + (size_t)p.C * roiIdx[j]);
          if (kMax) {
            uint16_t const* amr = am + (size_t)bins * (cc + (size_t)nch * j);
            for (uint32_t pw = ct & 255u; pw <= (ct >> 8); ++pw)
              for (uint32_t ph = rt & 255u; ph <= (rt >> 8); ++ph) {
                int const b = (int)(ph + p.S0 * pw);
                if (amr[b] == (uint32_t)pix) acc = __fadd_rn(acc, dyr[b]);
              }
          } else {
            // every bin that covers the pixel contributes dy / area (bits/nnroipooling.cu:74-90, acc_sum)
            for (uint32_t pw = ct & 255u; pw <= (ct >> 8); ++pw) {
              uint32_t const cs = binCol[j * p.S1 + pw];
              for (uint32_t ph = rt & 255u; ph <= (rt >> 8); ++ph) {
                uint32_t const rs = binRow[j * p.S0 + ph];
                int const area = (int)((rs >> 16) - (rs & 0xFFFFu)) * (int)((cs >> 16) - (cs & 0xFFFFu));
                acc = __fadd_rn(acc, __fmul_rn(dyr[ph + p.S0 * pw], __fdiv_rn(1.f, (float)area)));
              }
            }
          }
        }
      }
      *dst = acc;
    }
    first = false;
    if (base >= p.numROIs) break;
  }
  if (first) {
    // no ROI of this image: the slab of dX is zero
    for (int i = tid; i < nch * HW; i += kGatherThreads) dx[slabOff + i] = 0.f;
  }
}

// ---- backward (max): arg-max of every bin in parallel, then one warp per channel adds the bins' derivatives to their
// pixels in bin order (see the header comment) ----
constexpr int kOrdThreads = 256;

// Shared memory (bytes): plane float[HW] | dxs float[G*HW] | binRow uint32[RB*S0] | binCol uint32[RB*S1] | roiIdx int[RB] |
// am uint16[G*RB*bins]
__host__ __device__ inline size_t ordered_smem(int G, int RB, int HW, int S0, int S1)
{
  return 4 * (size_t)HW * (1 + G) + 4 * (size_t)RB * (S0 + S1) + 4 * (size_t)RB + 2 * (size_t)G * RB * S0 * S1 + 64;
}

__global__ void __launch_bounds__(kOrdThreads)
roipool_bwd_ordered_kernel(float* __restrict__ dx, float const* __restrict__ x, float const* __restrict__ rois,
                           float const* __restrict__ dy, RoiParams p, int G, int RB, int groups)
{
  extern __shared__ __align__(16) uint8_t sm[];
  __shared__ int sCount, sNext;
  int const HW = p.H * p.W, bins = p.S0 * p.S1;
  int const img = blockIdx.x / groups, c0 = (blockIdx.x % groups) * G;
  int const nch = min(G, p.C - c0);
  int const tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* plane = reinterpret_cast<float*>(sm);
  float* dxs = plane + HW;
  uint32_t* binRow = reinterpret_cast<uint32_t*>(dxs + (size_t)G * HW);
  uint32_t* binCol = binRow + (size_t)RB * p.S0;
  int* roiIdx = reinterpret_cast<int*>(binCol + (size_t)RB * p.S1);
  uint16_t* am = reinterpret_cast<uint16_t*>(roiIdx + RB);
  float const invBins = 1.f / (float)bins, invS0 = 1.f / (float)p.S0;

  for (int i = tid; i < nch * HW; i += kOrdThreads) dxs[i] = 0.f;
  int base = 0;
  while (true) {
    __syncthreads();
    if (tid < 32) {
      // the next RB ROIs of this image, in ascending order
      int cnt = 0, r = base;
      while (r < p.numROIs && cnt < RB) {
        int const rr = r + lane;
        bool mine = false;
        if (rr < p.numROIs) {
          int image = (int)rois[5 * (size_t)rr];
          mine = min(max(image - 1, 0), p.N - 1) == img;
        }
        unsigned const m = __ballot_sync(0xffffffffu, mine);
        int const pos = cnt + __popc(m & ((1u << lane) - 1u));
        if (mine && pos < RB) roiIdx[pos] = rr;
        int const tot = __popc(m);
        if (cnt + tot > RB) {                           // the batch is full inside this group of 32: resume behind its last member
          r += (int)__fns(m, 0, RB - cnt) + 1;
          cnt = RB;
          break;
        }
        cnt += tot; r += 32;
      }
      if (lane == 0) { sCount = cnt; sNext = min(r, p.numROIs); }
    }
    __syncthreads();
    int const nb = sCount;
    base = sNext;
    if (nb == 0) break;
    // bin geometry of every ROI of the batch, once (the double-precision part of the arithmetic)
    for (int i = tid; i < nb * (p.S0 + p.S1); i += kOrdThreads) {
      bool const isRow = i < nb * p.S0;
      int const k = isRow ? i : i - nb * p.S0;
      int const S = isRow ? p.S0 : p.S1;
      int const j = k / S, b = k - j * S;
      RoiGeom g = roi_geom(rois + 5 * (size_t)roiIdx[j], p);
      int s, e;
      roi_bin(b, isRow ? g.bin_h : g.bin_w, isRow ? g.start_h : g.start_w, isRow ? p.H : p.W, s, e);
      (isRow ? binRow : binCol)[k] = (uint32_t)s | ((uint32_t)e << 16);
    }
    int const total = nb * bins;
    // arg-max of every bin of every channel of the group, all threads: CPU scan order, first strictly greater, none for
    // an empty or all -inf / NaN bin
    for (int cc = 0; cc < nch; ++cc) {
      __syncthreads();                                 // geometry written; the plane is no longer read
      float const* const src = x + (size_t)HW * ((size_t)(c0 + cc) + (size_t)p.C * img);
      for (int i = tid; i < HW; i += kOrdThreads) plane[i] = src[i];
      __syncthreads();
      uint16_t* const amc = am + (size_t)cc * RB * bins;
      for (int b = tid; b < total; b += kOrdThreads) {
        // quotients by way of a float reciprocal: exact for these small operands, a fraction of the cost of integer division
        int const j = (int)(((float)b + 0.5f) * invBins), t = b - j * bins;
        int const pw = (int)(((float)t + 0.5f) * invS0), ph = t - pw * p.S0;
        uint32_t const rs = binRow[j * p.S0 + ph], cs = binCol[j * p.S1 + pw];
        int const hs = (int)(rs & 0xFFFFu), he = (int)(rs >> 16), ws = (int)(cs & 0xFFFFu), we = (int)(cs >> 16);
        float best = -INFINITY;
        uint32_t where = kNoBin;
        for (int w = ws; w < we; ++w)
          for (int h = hs; h < he; ++h) {
            float a = plane[w * p.H + h];
            if (a > best) { best = a; where = (uint32_t)(w * p.H + h); }
          }
        amc[b] = (uint16_t)where;
      }
    }
    __syncthreads();
    // One warp per channel walks the bins in order -- ROI, bin column, bin row: the order of the CPU loop -- 32 at a time.
    // Lanes whose bins routed to the same pixel add one after the other, in lane order; all others add at once.
    for (int cc = warp; cc < nch; cc += kOrdThreads / 32) {
      uint16_t const* const amc = am + (size_t)cc * RB * bins;
      float* const acc = dxs + (size_t)cc * HW;
      // eight steps' derivatives are fetched together, so that their latency passes once per eight steps
      for (int b0 = 0; b0 < total; b0 += 32 * 8) {
        uint32_t wh[8];
        float vv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          int const b = b0 + 32 * u + lane;
          wh[u] = b < total ? amc[b] : kNoBin;
          vv[u] = 0.f;
          if (wh[u] != kNoBin) {
            int const j = (int)(((float)b + 0.5f) * invBins);
            vv[u] = __ldg(dy + (size_t)(b - j * bins) + (size_t)bins * ((size_t)(c0 + cc) + (size_t)p.C * roiIdx[j]));
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (b0 + 32 * u >= total) break;
          uint32_t const where = wh[u];
          unsigned const peers = __match_any_sync(0xffffffffu, where);
          int const rank = where != kNoBin ? __popc(peers & ((1u << lane) - 1u)) : -1;
          int const rounds = __reduce_max_sync(0xffffffffu, rank);
          for (int r = 0; r <= rounds; ++r) {
            if (rank == r) acc[where] = __fadd_rn(acc[where], vv[u]);
            __syncwarp();
          }
        }
      }
    }
    if (base >= p.numROIs) break;
  }
  __syncthreads();
  // dX is written once: the sums, or zeros where no bin routed (and for an image that no ROI names)
  for (int i = tid; i < nch * HW; i += kOrdThreads) dx[(size_t)HW * ((size_t)c0 + (size_t)p.C * img) + i] = dxs[i];
}

int make_params(vlb_ctx* ctx, RoiParams* p, int H, int W, int C, int N, int numROIs, int S0, int S1,
                double const* tf, int method)
{
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0, "roipool: empty input");
  VLB_REQUIRE(ctx, numROIs >= 0, "roipool: negative ROI count");
  VLB_REQUIRE(ctx, S0 >= 1 && S1 >= 1, "roipool: SUBDIVISIONS has a dimension smaller than 1");
  VLB_REQUIRE(ctx, tf != nullptr, "roipool: null transform");
  VLB_REQUIRE(ctx, method == VLB_POOL_MAX || method == VLB_POOL_AVG, "roipool: unknown method");
  p->H = H; p->W = W; p->C = C; p->N = N; p->numROIs = numROIs; p->S0 = S0; p->S1 = S1;
  for (int i = 0; i < 6; ++i) p->tf[i] = tf[i];
  return VLB_Success;
}

}  // namespace

extern "C" {

int vlb_roipool_bounds(vlb_ctx* ctx, int* bounds, int* images, float const* rois, int H, int W, int N,
                       int numROIs, int S0, int S1, double const* transform)
{
  if (!ctx) return VLB_IllegalArgument;
  RoiParams p;
  int rc = make_params(ctx, &p, H, W, 1, N, numROIs, S0, S1, transform, VLB_POOL_MAX);
  if (rc) return rc;
  VLB_REQUIRE(ctx, bounds && rois, "roipool_bounds: null tensor");
  if (numROIs == 0) return VLB_Success;
  roipool_bounds_kernel<<<vlb::grid_for((size_t)S0 * S1 * numROIs, kThreads), kThreads, 0, ctx->stream>>>(bounds, images, rois, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_roipool_bounds");
}

int vlb_roipool_forward(vlb_ctx* ctx, float* Y, float const* X, float const* rois, int H, int W, int C, int N,
                        int numROIs, int S0, int S1, double const* transform, int method)
{
  if (!ctx) return VLB_IllegalArgument;
  RoiParams p;
  int rc = make_params(ctx, &p, H, W, C, N, numROIs, S0, S1, transform, method);
  if (rc) return rc;
  VLB_REQUIRE(ctx, Y && X && rois, "roipool_forward: null tensor");
  if (numROIs == 0) return VLB_Success;
  size_t total = (size_t)S0 * S1 * C * numROIs;
  unsigned grid = vlb::grid_for(total, kThreads, ctx->smCount * 16);
  if (method == VLB_POOL_MAX) roipool_kernel<true, false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, rois, nullptr, p);
  else                        roipool_kernel<false, false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, rois, nullptr, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_roipool_forward");
}

int vlb_roipool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* rois, float const* dY, int H, int W,
                         int C, int N, int numROIs, int S0, int S1, double const* transform, int method)
{
  if (!ctx) return VLB_IllegalArgument;
  RoiParams p;
  int rc = make_params(ctx, &p, H, W, C, N, numROIs, S0, S1, transform, method);
  if (rc) return rc;
  VLB_REQUIRE(ctx, dX && X && rois && dY, "roipool_backward: null tensor");
  {
    // the gather: slabs of about 64 KB per CTA, at least as many CTAs as SMs where the channels allow, and as many ROIs
    // per batch as the rest of the shared memory holds
    bool const isMax = method == VLB_POOL_MAX;
    long long const HW = (long long)H * W;
    size_t const budget = 200 * 1024;
    if (isMax && HW < 65535 && S0 <= 255 && S1 <= 255 && numROIs > 0) {
      // channel groups so that about four CTAs come to every SM; as many ROIs per batch as the rest of 56 KB of shared
      // memory per CTA holds (four CTAs resident per SM)
      long long const planes = (long long)N * C;
      int G = (int)((planes + 4LL * ctx->smCount - 1) / (4LL * ctx->smCount));
      if (G < 1) G = 1;
      if (G > kOrdThreads / 32) G = kOrdThreads / 32;
      if (G > C) G = C;
      size_t const budget = 56 * 1024;
      size_t const fixed = ordered_smem(G, 0, (int)HW, S0, S1), perRoi = ordered_smem(G, 1, (int)HW, S0, S1) - fixed;
      long long RB = fixed < budget ? (long long)((budget - fixed) / perRoi) : 0;
      if (RB > numROIs) RB = numROIs;
      if (RB >= 8 || RB == numROIs) {
        int const groups = vlb::ceil_div(C, G);
        size_t const smem = ordered_smem(G, (int)RB, (int)HW, S0, S1);
        static bool attrDone[64] = {};
        if (!(ctx->device < 64 && attrDone[ctx->device])) {
          cudaError_t ea = vlb::allow_max_dynamic_smem(roipool_bwd_ordered_kernel);
          if (ea != cudaSuccess) { cudaGetLastError(); return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(ea)); }
          if (ctx->device < 64) attrDone[ctx->device] = true;
        }
        roipool_bwd_ordered_kernel<<<(unsigned)(N * groups), kOrdThreads, smem, ctx->stream>>>(dX, X, rois, dY, p, G, (int)RB, groups);
        VLB_LAUNCHED(ctx, 1);
        return vlb::check_launch(ctx, "vlb_roipool_backward");
      }
    }
    if (HW < 65535 && S0 <= 255 && S1 <= 255 && numROIs > 0) {
      int CH = (int)((64 * 1024) / (4 * HW));
      if (CH > C) CH = C;
      while (CH > 1 && (long long)N * vlb::ceil_div(C, CH) < ctx->smCount) --CH;
      if (CH >= 1) {
        size_t const fixed = gather_smem(CH, 0, H, W, S0, S1, isMax);
        size_t const perRoi = gather_smem(CH, 1, H, W, S0, S1, isMax) - fixed + 32;
        long long RB = fixed < budget ? (long long)((budget - fixed) / perRoi) : 0;
        if (RB > numROIs) RB = numROIs;
        if (RB >= 8 || RB == numROIs) {
          int const chunks = vlb::ceil_div(C, CH);
          size_t const smem = gather_smem(CH, (int)RB, H, W, S0, S1, isMax) + 64;
          static bool attrDone[2][64] = {};
          if (!(ctx->device < 64 && attrDone[isMax][ctx->device])) {
            cudaError_t ea = isMax ? vlb::allow_max_dynamic_smem(roipool_bwd_gather_kernel<true>)
                                   : vlb::allow_max_dynamic_smem(roipool_bwd_gather_kernel<false>);
            if (ea != cudaSuccess) { cudaGetLastError(); return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(ea)); }
            if (ctx->device < 64) attrDone[isMax][ctx->device] = true;
          }
          unsigned const grid = (unsigned)(N * chunks);
          if (isMax) roipool_bwd_gather_kernel<true><<<grid, kGatherThreads, smem, ctx->stream>>>(dX, X, rois, dY, p, CH, (int)RB, chunks);
          else       roipool_bwd_gather_kernel<false><<<grid, kGatherThreads, smem, ctx->stream>>>(dX, X, rois, dY, p, CH, (int)RB, chunks);
          VLB_LAUNCHED(ctx, 1);
          return vlb::check_launch(ctx, "vlb_roipool_backward");
        }
      }
    }
  }
  // maps too large for a shared-memory slab: zero fill and scatter with atomics
  cudaError_t e = cudaMemsetAsync(dX, 0, sizeof(float) * (size_t)H * W * C * N, ctx->stream);
  if (e != cudaSuccess) return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e));
  if (numROIs == 0) return VLB_Success;
  size_t total = (size_t)S0 * S1 * C * numROIs;
  unsigned grid = vlb::grid_for(total, kThreads, ctx->smCount * 16);
  if (method == VLB_POOL_MAX) roipool_kernel<true, true><<<grid, kThreads, 0, ctx->stream>>>(dX, X, rois, dY, p);
  else                        roipool_kernel<false, true><<<grid, kThreads, 0, ctx->stream>>>(dX, X, rois, dY, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_roipool_backward");
}

}  // extern "C"
