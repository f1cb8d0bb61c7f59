// Tensor-core contractions for vl::nn::Convolution and vl::nn::FullyConnected
// (reference bits/nnconv.cu:71-317, bits/nnfullyconnected.cu:30-185) on tcgen05 / TMEM.
//
// Every contraction on the path is D[m][n] = sum_r A(m,r) * B(n,r) with fp32 accumulation
// in tensor memory, 128 x BN output tile, reduction in blocks of 32.  Two kernels:
//
//   conv_ts_kernel   convolution forward and stride-1 data gradient: the gathered operand goes to
//                    tensor memory, only the filter tiles to shared memory (further down).
//   tc_gemm_kernel   filter gradient, fully connected layers, and convolutions whose filter support
//                    exceeds the tap table: both operands in shared memory, warp-specialised:
//     warps 0-3   fp32 drain of the accumulation chains, then epilogue: tcgen05.ld the accumulator
//                 (one TMEM lane = one output row per thread), store to global memory, coalesced along m;
//     warp  4     allocates TMEM and issues tcgen05.mma (kind::tf32, cta_group::1) from one
//                 lane; tcgen05.commit releases a stage / hands a chain to the drain warps;
//     warps 5-16  producers: gather the operand tiles from the MATLAB-order tensors
//                 (no patch matrix: the reference writes one per image, bits/nnconv.cu:109-117),
//                 split every value into a TF32 "hi" part and an exactly representable
//                 remainder "lo", and write both as 128-byte-swizzled UMMA tiles.
// The split is what makes the result fp32-faithful: x*y ~ hi*hi + hi*lo + lo*hi, three
// MMAs per product ("3xTF32"); the dropped lo*lo term is below 2^-22 relative.  The
// single-pass TF32 mode issues only hi*hi.
// Stages are handed over with mbarriers; every wait is bounded (about a tenth of a second) and on
// expiry records a status word and unwinds, releasing TMEM, instead of spinning forever.
//
// Operand layouts in shared memory (canonical UMMA layouts, 128-byte swizzle):
//   K-major  tile[rows][32]: row r at r*128 bytes, 16-byte chunk c stored at chunk c ^ (r & 7);
//            descriptor SBO = 1024 (8 rows), advance 32 bytes per MMA (K = 8).
//   MN-major tile[32][cols]: 32-bit operands that are contiguous along the row index must use the
//            "128-byte swizzle with 32-byte base" layout (type 1): atoms of 4 k x 32 cols (512 bytes),
//            row k & 3 at 128 bytes, 32-byte chunk q of a row stored at chunk q ^ (k & 3); atom
//            (ci, kq) at (kq * cols/32 + ci) * 512; LBO = 512 between column atoms, SBO =
//            cols/32 * 512 between k quads, advance 2 * SBO per MMA.
#include "conv_internal.cuh"
#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <type_traits>

namespace {

using vlb::ConvGeom;
using vlb::ProfScope;
using vlb::kProfFprop; using vlb::kProfDgrad; using vlb::kProfWgrad; using vlb::kProfFc;

constexpr int BM = 128;          // output rows per CTA (TMEM lanes)
constexpr int BK = 32;           // reduction elements per stage (one 128-byte swizzle row)
constexpr int kEpilogueWarps = 4;
constexpr int kProducerWarps = 12;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kThreads = (kEpilogueWarps + 1 + kProducerWarps) * 32;   // 544
constexpr int kGenericWarps = 8;                   // the general-purpose producer loop uses the first 8 producer warps
constexpr int kGenericThreads = kGenericWarps * 32;
constexpr int CH = (BM * 8) / kGenericThreads;    // 16-byte chunks per thread per 128 x 32 operand tile in that loop (4)
constexpr int KSTEP = 32 / CH;                    // MN-major tiles: k rows between a thread's consecutive chunks
constexpr int RSTEP = BM / CH;                    // K-major tiles: rows between a thread's consecutive chunks
constexpr int kMaxStages = 8;
constexpr int kDrainEvery = 8;                    // 3xTF32: k-blocks (of 32) accumulated by the tensor core before the fp32 drain
constexpr long long kWaitCycles = 200000000LL;    // default bound on any single barrier wait (about 0.1 s)
__constant__ long long gWaitCycles = kWaitCycles; // the bound in force on this device (vlb_ctx_set_wait_limit)

enum OperandMode {
  OP_DENSE_K = 0,    // addr(i, r) = (r / P) * bs + i * ld + (r % P)      (reduction contiguous)
  OP_DENSE_MN = 1,   // addr(i, r) = r * ld + i                           (row index contiguous)
  OP_IM2COL = 2,     // i = output pixel (ho,wo,n), r = (fh,fw,c): shifted input, MN-major
  OP_WGATHER = 3     // i = (fh,fw,c), r = output pixel (ho,wo,n): shifted input, K-major
};

enum EpilogueMode {
  EPI_PLAIN = 0,     // out[m + n*ldd] (+ bias[m]); with splits: out + split*splitStride
  EPI_CONV = 1       // m = (pixel, image): out[(image*Ktot + n)*P + pixel] = inMult*acc + bias[n] + outMult*old
};

struct Operand {
  float const* ptr;
  long long ld, bs;
  int P;               // run length of contiguous reduction indices (DENSE_K, batched); 0 = unbatched
  int rows;            // valid extent of the row (M or N) index
  int vec;             // 1 when 16-byte loads are legal for this operand
  int fast;            // pipelined gather: 1 aligned windows, 2 element-wise (any geometry), 0 none (IM2COL, WGATHER)
  // convolution geometry (IM2COL, WGATHER)
  int H, W, C, FH, FW, Ho, Wo, sy, sx, pt, pl, dy, dx;
  long long imgStride;   // H*W*Ctotal
};

struct Epilogue {
  float* out;
  float const* bias;
  long long ldd;
  long long splitStride;
  float inMult, outMult;
  int P, Ktot;
  int relu;            // apply max(., 0) to the stored value (forward convolution followed by a ReLU layer)
  float const* mask;   // conv_ts_kernel, when non-null: laid out like out; the stored value is zeroed where mask is not positive
};

struct Params {
  Operand a, b;
  Epilogue e;
  int M, N, R;
  int BN;                 // tile columns: 16, 32, 64 or 128
  int numKb, kbPerSplit;
  int stages;
  int drainEvery;         // 3xTF32: k-blocks per tensor-core accumulation chain
  int tilesM, tilesN;     // conv_ts_kernel: the grid of output tiles its persistent CTAs walk
  int chanFast;           // conv_ts_kernel: reduction in blocks of 32 channels, r = c%32 + 32*(tap + taps*(c/32)); needs C % 32 == 0
  int pipelined;          // 1: producers prefetch one stage ahead in registers (aligned gathers only)
  float const* bTiles;    // when non-null: B pre-split into shared-memory tile images, fetched with bulk copies
  int* status;
  int testSwitch;         // vlb_ctx_set_test_switch: bit 0 = conv_ts_kernel's filter-tile loader stays idle
  // conv_ts_kernel fed by tensor-map copies (tma != 0): an output tile is a box of bh x bw pixels of one image (tilesH x
  // tilesW boxes per image); its input window -- boxH rows (rowOff spare rows in front, so that the copy starts on a
  // 16-byte boundary) x boxW columns x 32 channels -- arrives in shared memory by one cp.async.bulk.tensor per channel block
  int tma, bh, bw, tilesH, tilesW, boxH, boxW, rowOff;
  int bStages;            // conv_ts_kernel: filter-tile stages in shared memory (4, or 3 where the input windows need the room)
  // conv_ts_kernel computing a filter gradient (wg != 0): D[(tap, c)][k] = sum over output pixels of x(pixel + tap, c) * dY(pixel, k).
  // A tile row is one channel of one filter tap: tapsPerTile taps x cPer channels = 128 rows, tapGroups x C/cPer row tiles; the
  // reduction (output pixels of the whole batch, kbTot k-blocks in the dY tile images) is cut into `splits` ranges of kbPerSplit
  // k-blocks, one work item per (range, row tile, column tile); the x runs arrive by tensor-map copies, xStages buffers.
  int wg, cPer, tapsPerTile, tapGroups, kbTot, splits, xStages;
  int smemSum;            // conv_ts_kernel, kMode 0 / 1: keep the running sum of a tile in shared memory even for the tile widths that fit the
                          // drain warps' registers (tiles of a few k-blocks, where the stores dominate; test switch bit 3)
  int plane;              // row mode: reduction indices per image in the tile images -- the plane's pixels rounded up to whole k-blocks
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(void const* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{ asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{ asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(bar) : "memory"); }

// Bounded wait: false when the phase did not complete within gWaitCycles.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
  long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    // the thread is suspended by the hardware until the phase completes or the time hint (ns) runs out
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(100000u) : "memory");
    if (ok) return true;
    if ((it & 15u) == 15u) {
      long long now = clock64();
      if (t0 == 0) t0 = now;
      else if (now - t0 > gWaitCycles) return false;
    }
  }
}

// One try_wait: true when the phase has completed; otherwise the thread was suspended for about `ns` nanoseconds at most.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity, uint32_t ns)
{
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}

// Has the phase completed?  No waiting.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{ asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }

// Bulk asynchronous copy global -> shared (both 16-byte aligned, size a multiple of 16); completion is
// signalled on the mbarrier as transaction bytes.  Source is always this GPU's own memory.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dstSmem, void const* src, uint32_t bytes, uint32_t bar)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dstSmem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dstSmem, uint32_t cols)
{
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dstSmem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{ asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory"); }

__device__ __forceinline__ void umma_tf32(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t iDesc, uint32_t accumulate)
{
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
               ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{ asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }

__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16])
{
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, uint32_t const (&r)[16])
{
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, LBO, SBO in 16-byte
// units, version 1 at bit 46, layout type at bits 61-63: 2 = 128-byte swizzle (K-major tiles),
// 1 = 128-byte swizzle with 32-byte base (MN-major tiles of 32-bit elements).
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lboBytes, uint32_t sboBytes, uint32_t layoutType = 2)
{
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lboBytes >> 4) << 16) | ((uint64_t)(sboBytes >> 4) << 32) |
         (1ull << 46) | ((uint64_t)layoutType << 61);
}

// kind::tf32 instruction descriptor: D = F32 (bits 4-5 = 1), A and B = TF32 (bits 7-9, 10-12 = 2),
// major-ness bits 15 / 16 (1 = MN-major), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__device__ __forceinline__ uint32_t make_idesc(bool aMN, bool bMN, int n)
{
  return (1u << 4) | (2u << 7) | (2u << 10) | ((aMN ? 1u : 0u) << 15) | ((bMN ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ------------------------------------------------------------------ hi / lo split and tile stores
__device__ __forceinline__ float tf32_hi(float x)
{
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

template <bool kSplit>
__device__ __forceinline__ void store_chunk(uint8_t* hiTile, uint8_t* loTile, uint32_t off, float const (&v)[4])
{
  if (kSplit) {
    float4 h, l;
    h.x = tf32_hi(v[0]); h.y = tf32_hi(v[1]); h.z = tf32_hi(v[2]); h.w = tf32_hi(v[3]);
    l.x = v[0] - h.x; l.y = v[1] - h.y; l.z = v[2] - h.z; l.w = v[3] - h.w;
    *reinterpret_cast<float4*>(hiTile + off) = h;
    *reinterpret_cast<float4*>(loTile + off) = l;
  } else {
    *reinterpret_cast<float4*>(hiTile + off) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

__device__ __forceinline__ uint32_t kmajor_off(int row, int kc) { return (uint32_t)row * 128u + (uint32_t)((kc ^ (row & 7)) << 4); }
__device__ __forceinline__ uint32_t mnmajor_off(int chunk, int k, int atomsPerRow)
{
  // chunk = 16-byte chunk along the row index (4 values); 32-byte chunk index (chunk & 7) >> 1 is swizzled with k & 3
  return (uint32_t)(((k >> 2) * atomsPerRow + (chunk >> 3)) * 512 + (k & 3) * 128 +
                    (((((chunk & 7) >> 1) ^ (k & 3)) << 5) | ((chunk & 1) << 4)));
}

// ------------------------------------------------------------------ operand gathers
// Each returns four values: for MN-major modes the row indices i..i+3 at reduction index r,
// for K-major modes row i at reduction indices r..r+3.  Out-of-range positions read as zero.

__device__ __forceinline__ void load_dense_k(Operand const& o, int i, int r, int R, float (&v)[4])
{
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (i >= o.rows || r >= R) return;
  if (o.vec && r + 3 < R) {
    long long a = o.P ? (long long)(r / o.P) * o.bs + (long long)i * o.ld + (r % o.P) : (long long)i * o.ld + r;
    float4 t = *reinterpret_cast<float4 const*>(o.ptr + a);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    return;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    int rr = r + e;
    if (rr < R) {
      long long a = o.P ? (long long)(rr / o.P) * o.bs + (long long)i * o.ld + (rr % o.P) : (long long)i * o.ld + rr;
      v[e] = o.ptr[a];
    }
  }
}

__device__ __forceinline__ void load_dense_mn(Operand const& o, int i, int r, int R, float (&v)[4])
{
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (i >= o.rows || r >= R) return;
  long long a = (long long)r * o.ld + i;
  if (o.vec && i + 3 < o.rows) {
    float4 t = *reinterpret_cast<float4 const*>(o.ptr + a);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    return;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (i + e < o.rows) v[e] = o.ptr[a + e];
}

// Pixel context of one output position, fixed for a producer thread in IM2COL mode.
struct PixCtx { int hs, ws; long long base; bool valid; };

__device__ __forceinline__ PixCtx pix_ctx(Operand const& o, int m)
{
  PixCtx c;
  c.valid = m < o.rows;
  int ho = m % o.Ho, t = m / o.Ho, wo = t % o.Wo, n = t / o.Wo;
  c.hs = ho * o.sy - o.pt; c.ws = wo * o.sx - o.pl;
  c.base = (long long)n * o.imgStride;
  return c;
}

__device__ __forceinline__ void load_im2col(Operand const& o, PixCtx const (&px)[4], int r, int R, float (&v)[4])
{
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (r >= R) return;
  int fh = r % o.FH, t = r / o.FH, fw = t % o.FW, c = t / o.FW;
  int dh = fh * o.dy, dw = fw * o.dx;
  long long coff = (long long)c * o.H * o.W;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    int h = px[e].hs + dh, w = px[e].ws + dw;
    if (px[e].valid && h >= 0 && h < o.H && w >= 0 && w < o.W) v[e] = o.ptr[px[e].base + coff + (long long)w * o.H + h];
  }
}

// Filter-tap context of one row (fh,fw,c), fixed for a producer thread in WGATHER mode.
struct TapCtx { int dh, dw; long long coff; bool valid; };

__device__ __forceinline__ TapCtx tap_ctx(Operand const& o, int i)
{
  TapCtx c;
  c.valid = i < o.rows;
  int fh = i % o.FH, t = i / o.FH, fw = t % o.FW, ch = t / o.FW;
  c.dh = fh * o.dy - o.pt; c.dw = fw * o.dx - o.pl;
  c.coff = (long long)ch * o.H * o.W;
  return c;
}

__device__ __forceinline__ void load_wgather(Operand const& o, TapCtx const& tc, int r, int R, float (&v)[4])
{
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (!tc.valid || r >= R) return;
  int ho = r % o.Ho, t = r / o.Ho, wo = t % o.Wo, n = t / o.Wo;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (r + e < R) {
      int h = ho * o.sy + tc.dh, w = wo * o.sx + tc.dw;
      if (h >= 0 && h < o.H && w >= 0 && w < o.W) v[e] = o.ptr[(long long)n * o.imgStride + tc.coff + (long long)w * o.H + h];
    }
    if (++ho == o.Ho) { ho = 0; if (++wo == o.Wo) { wo = 0; ++n; } }
  }
}

// ---- fast gathers.  Preconditions (Operand::fast): stride 1, H % 4 == 0, Ho % 4 == 0, base 16-byte
// aligned, fewer than 2^31 elements.  Then four consecutive output pixels lie in one column, and
// every 16-byte-aligned group of four input rows is wholly inside the image or wholly padding, so a
// shifted window of four rows is two aligned 128-bit loads and a funnel shift.
struct FastPix { int base, ho0, wo; bool valid; };   // base = image*imgStride + wo*H + ho0, in elements

__device__ __forceinline__ FastPix fast_pix(Operand const& o, int m, int limit)
{
  FastPix c;
  c.valid = m < limit;
  int ho = m % o.Ho, t = m / o.Ho;
  c.wo = t % o.Wo;
  c.ho0 = ho;
  c.base = (t / o.Wo) * (int)o.imgStride + c.wo * o.H + ho;
  return c;
}

// v[e] = x[row ho0 + s + e, column wo + dw, plane offset coff] (zero outside the image), e = 0..3
__device__ __forceinline__ void load_shifted(float const* __restrict__ ptr, int H, int W, FastPix const& px, int s, int dw,
                                             int coff, bool on, float (&v)[4])
{
  int const o = s & 3;
  int const h0 = px.ho0 + s - o;
  int const w = px.wo + dw;
  bool const wok = on && px.valid && w >= 0 && w < W;
  float const* a0 = ptr + (px.base + coff + dw * H + (s - o));
  float4 c0 = make_float4(0.f, 0.f, 0.f, 0.f), c1 = c0;
  if (wok && h0 >= 0 && h0 < H) c0 = *reinterpret_cast<float4 const*>(a0);
  if (wok && o != 0 && h0 + 4 >= 0 && h0 + 4 < H) c1 = *reinterpret_cast<float4 const*>(a0 + 4);
  bool const s2 = (o & 2) != 0, s1 = (o & 1) != 0;
  float t0 = s2 ? c0.z : c0.x, t1 = s2 ? c0.w : c0.y, t2 = s2 ? c1.x : c0.z, t3 = s2 ? c1.y : c0.w, t4 = s2 ? c1.z : c1.x;
  v[0] = s1 ? t1 : t0; v[1] = s1 ? t2 : t1; v[2] = s1 ? t3 : t2; v[3] = s1 ? t4 : t3;
}

// One row of a reduction-contiguous operand whose 16-byte loads are legal: p points at (row, batch) start.
__device__ __forceinline__ void load_row4(float const* __restrict__ p, int r, int R, bool ok, float (&v)[4])
{
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (!ok || r >= R) return;
  if (r + 3 < R) {
    float4 t = *reinterpret_cast<float4 const*>(p + r);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (r + e < R) v[e] = p[r + e];
  }
}

// ------------------------------------------------------------------ pipelined producer
// Pipelined producers work in kGroups independent groups of warps; group g fills the stages
// it = g, g + kGroups, ...  A warp stalls for the full latency of its own stage's global loads, but
// the other groups are then busy with other stages, so kGroups stages of loads are in flight per SM
// without relying on how the compiler tracks outstanding loads inside one thread.
// A group must not lap the MMA warp by more than the number of shared-memory stages, or the parity
// test of an mbarrier wait would alias: kGroups <= stages (at least 3) is required.
constexpr int kGroups = 3;
constexpr int kGroupThreads = kProducerThreads / kGroups;       // 128
constexpr int CHG = (BM * 8) / kGroupThreads;                    // chunks per thread per stage (8)
constexpr int KSTEPG = 32 / CHG;                                 // MN-major: k rows between a thread's chunks (4)
constexpr int RSTEPG = BM / CHG;                                 // K-major: rows between a thread's chunks (16)

// Four consecutive rows ho0+s .. ho0+s+3 of one input column, loaded straight into their final
// registers.  The window straddles at most two aligned groups of four rows, each wholly inside the
// image or wholly padding, so every load has a single predicate; the load widths follow the
// alignment of the window start (s & 3): 128 | 32+64+32 | 64+64 | 32+64+32 bits.
__device__ __forceinline__ void issue_window(float const* __restrict__ ptr, int H, int W, FastPix const& px, int s, int dw,
                                             int coff, bool on, float4& v)
{
  int const o = s & 3;
  int const h0 = px.ho0 + s - o;            // first row of the aligned group that holds the window start
  int const w = px.wo + dw;
  bool const wok = on && px.valid && w >= 0 && w < W;
  bool const g0 = wok && h0 >= 0 && h0 < H;
  bool const g1 = wok && h0 + 4 >= 0 && h0 + 4 < H;
  float const* a = ptr + (px.base + coff + dw * H + s);
  v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (o == 0) {
    if (g0) v = *reinterpret_cast<float4 const*>(a);
  } else if (o == 2) {
    if (g0) { float2 t = *reinterpret_cast<float2 const*>(a); v.x = t.x; v.y = t.y; }
    if (g1) { float2 t = *reinterpret_cast<float2 const*>(a + 2); v.z = t.x; v.w = t.y; }
  } else {
    // o == 1: rows 0..2 lie in the first group, row 3 in the second; o == 3: row 0 | rows 1..3
    bool const gm = (o == 1) ? g0 : g1;
    if (g0) v.x = a[0];
    if (gm) { float2 t = *reinterpret_cast<float2 const*>(a + 1); v.y = t.x; v.z = t.y; }
    if (g1) v.w = a[3];
  }
}

// The same window load with everything precomputed: a = address of the window start, o = its
// alignment (s & 3), g0 / g1 = whether the first / second aligned group of rows is inside the image.
// The window start is aligned to o = s & 3 elements only, so the four rows are fetched as four
// independent predicated 32-bit loads: straight-line code (a load inside a branch makes the compiler
// wait for it before the paths rejoin) and one destination register per load (two loads that may
// write the same register are serialised by the scoreboard even when one is predicated off).  Both
// effects were measured at about 5000 cycles per stage; this form keeps a stage's 32 loads in flight.
__device__ __forceinline__ void ldg32_if(float& x, float const* a, bool pred)
{
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %2, 0;\n @p ld.global.nc.f32 %0, [%1];\n}" : "+f"(x) : "l"(a), "r"((int)pred));
}

// a = address of the window start, o = its alignment (s & 3), g0 / g1 = whether the first / second
// aligned group of four rows is inside the image; row e of the window lies in the first group iff e < 4 - o.
__device__ __forceinline__ void issue_window2(float const* __restrict__ a, int o, bool g0, bool g1, float4& v)
{
  v = make_float4(0.f, 0.f, 0.f, 0.f);
  ldg32_if(v.x, a, g0);
  ldg32_if(v.y, a + 1, o < 3 ? g0 : g1);
  ldg32_if(v.z, a + 2, o < 2 ? g0 : g1);
  ldg32_if(v.w, a + 3, o < 1 ? g0 : g1);
}

// ------------------------------------------------------------------ the kernel
template <int kAMode, int kBMode, int kEpi, bool kSplit>
__global__ void __launch_bounds__(kThreads, 1) tc_gemm_kernel(Params p)
{
  extern __shared__ uint8_t smemRaw[];
  __shared__ __align__(8) uint64_t fullBar[kMaxStages];
  __shared__ __align__(8) uint64_t emptyBar[kMaxStages];
  __shared__ __align__(8) uint64_t accumBar;
  __shared__ __align__(8) uint64_t drainFull[2], drainEmpty[2], sumBar;   // T0/T1 hand-over; P complete
  __shared__ uint32_t tmemBase;
  __shared__ int2 tapLut[64];       // IM2COL, pipelined: per filter tap fh + FH*fw {element offset of the tap, fh | fw<<5 | (s&3)<<10}
  __shared__ int4 tapTab[BM];       // WGATHER, pipelined: per tile row (fh,fw,c) {element offset, row shift s, column shift dw, valid}

  constexpr bool kAMN = (kAMode == OP_DENSE_MN || kAMode == OP_IM2COL);
  constexpr bool kBMN = (kBMode == OP_DENSE_MN);

  uint8_t* smem = smemRaw + ((1024u - (smem_u32(smemRaw) & 1023u)) & 1023u);   // swizzle atoms need 1024-byte alignment
  int const BN = p.BN;
  uint32_t const aTileBytes = BM * BK * 4;                  // 16 KB
  uint32_t const bTileBytes = (uint32_t)BN * BK * 4;
  uint32_t const stageBytes = (kSplit ? 2u : 1u) * (aTileBytes + bTileBytes);
  // Accumulators.  The tensor core adds each MMA's result to the fp32 accumulator with truncation,
  // so the error of an accumulation chain is a bias that grows linearly with its length (3e-5
  // relative after a few thousand steps).  In the split mode the chain is therefore kept short:
  //   T0, T1  hi*hi products of p.drainEvery consecutive k-blocks (8: 32 MMAs), used alternately;
  //   P       the running sum: warps 0-3 add a finished T to it in fp32 with round-to-nearest
  //           (tcgen05.ld, add, tcgen05.st) while the tensor core fills the other T;
  //   S       the small terms lo*hi + hi*lo (about 2^-11 of the result, where the bias no longer
  //           matters) of the whole reduction.
  // The epilogue returns P + T(last) + S.  Columns: T0 | T1 | P | S, BN each.
  uint32_t const tmemCols = kSplit ? (uint32_t)(4 * BN) : (BN < 32 ? 32u : (uint32_t)BN);

  int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int const m0 = blockIdx.x * BM, n0 = blockIdx.y * BN, split = blockIdx.z;
  int const kbBeg = split * p.kbPerSplit;
  int const kbEnd = min(p.numKb, kbBeg + p.kbPerSplit);
  int const numIter = max(kbEnd - kbBeg, 0);
  int const numChunks = kSplit ? (numIter + p.drainEvery - 1) / p.drainEvery : 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(smem_u32(&fullBar[s]), p.pipelined ? kProducerWarps / kGroups : kGenericWarps); mbar_init(smem_u32(&emptyBar[s]), 1); }
    mbar_init(smem_u32(&accumBar), 1);
    for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&drainFull[b]), 1); mbar_init(smem_u32(&drainEmpty[b]), kEpilogueWarps); }
    mbar_init(smem_u32(&sumBar), kEpilogueWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kEpilogueWarps) tmem_alloc(smem_u32(&tmemBase), tmemCols);
  if (kAMode == OP_IM2COL && p.pipelined && (int)threadIdx.x < p.a.FH * p.a.FW) {
    int const fh = (int)threadIdx.x % p.a.FH, fw = (int)threadIdx.x / p.a.FH;
    int const sft = fh * p.a.dy - p.a.pt;
    tapLut[threadIdx.x] = make_int2((fw * p.a.dx - p.a.pl) * p.a.H + sft, fh | (fw << 5) | ((sft & 3) << 10));
  }
  if (kAMode == OP_WGATHER && p.pipelined && threadIdx.x < BM) {
    TapCtx tc = tap_ctx(p.a, m0 + (int)threadIdx.x);
    tapTab[threadIdx.x] = make_int4((int)tc.coff + tc.dw * p.a.H + tc.dh, tc.dh, tc.dw, tc.valid ? 1 : 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmemAcc = tmemBase;

  if (warp < kEpilogueWarps) {
    // ============================== fp32 drain (3xTF32 only) ==============================
    // Chunk c (k-blocks c*p.drainEvery ...) was accumulated in T[c & 1]; all chunks but the last are
    // added to P here.  Warp w owns TMEM lanes 32w .. 32w+31.
    if (kSplit) {
      uint32_t const lanes = tmemAcc + ((uint32_t)(warp * 32) << 16);
      bool ok = true;
      for (int c = 0; c + 1 < numChunks && ok; ++c) {
        int const b = c & 1;
        ok = mbar_wait(smem_u32(&drainFull[b]), (uint32_t)((c >> 1) & 1));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { if (lane == 0) atomicExch(p.status, 5); break; }
        tc_fence_after();
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t t0[16], t1[16], p0[16], p1[16];
          bool const two = c0 + 16 < BN;
          tmem_ld16_issue(lanes + (uint32_t)(b * BN + c0), t0);
          if (two) tmem_ld16_issue(lanes + (uint32_t)(b * BN + c0 + 16), t1);
          if (c > 0) {
            tmem_ld16_issue(lanes + (uint32_t)(2 * BN + c0), p0);
            if (two) tmem_ld16_issue(lanes + (uint32_t)(2 * BN + c0 + 16), p1);
          }
          tmem_ld_wait();
          if (c > 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              t0[j] = __float_as_uint(__uint_as_float(t0[j]) + __uint_as_float(p0[j]));
              if (two) t1[j] = __float_as_uint(__uint_as_float(t1[j]) + __uint_as_float(p1[j]));
            }
          }
          tmem_st16(lanes + (uint32_t)(2 * BN + c0), t0);
          if (two) tmem_st16(lanes + (uint32_t)(2 * BN + c0 + 16), t1);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&drainEmpty[b]));     // T[b] may be overwritten
      }
      // P is complete (its stores have been waited for): publish it to the warps of the epilogue
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sumBar));
    }
  } else if (warp == kEpilogueWarps) {
    // ============================== MMA issue ==============================
    if (lane == 0) {
      uint32_t const idesc = make_idesc(kAMN, kBMN, BN);
      uint32_t aLbo = 512, aSbo = (BM / 32) * 512, bLbo = 512, bSbo = (uint32_t)(BN / 32) * 512;
      // The issuing thread is the critical resource (the tensor core's queue is about one MMA deep, and the
      // thread shares its scheduler with busy producer warps): running counters instead of divisions, and
      // descriptors derived from one per-stage base with 64-bit adds.
      uint64_t const dA0 = kAMN ? make_desc(smem_u32(smem), aLbo, aSbo, 1) : make_desc(smem_u32(smem), 16, 1024);
      uint64_t const dB0 = kBMN ? make_desc(smem_u32(smem) + (kSplit ? 2u : 1u) * aTileBytes, bLbo, bSbo, 1)
                                : make_desc(smem_u32(smem) + (kSplit ? 2u : 1u) * aTileBytes, 16, 1024);
      uint32_t const aAdv = (kAMN ? (uint32_t)(BM / 32) * 1024u : 32u) >> 4, bAdv = (kBMN ? (uint32_t)(BN / 32) * 1024u : 32u) >> 4;
      uint32_t const stageStep = stageBytes >> 4, aLoStep = aTileBytes >> 4, bLoStep = bTileBytes >> 4;
      bool ok = true;
      int s = 0, inChunk = 0, chunk = 0;
      uint32_t ph = 0;
      for (int it = 0; it < numIter && ok; ++it) {
        int const tb = kSplit ? (chunk & 1) : 0;
        bool const chunkStart = inChunk == 0;
        if (kSplit && chunkStart && chunk >= 2) {      // T[tb] is reused: its previous contents must have been added to P
          ok = mbar_wait(smem_u32(&drainEmpty[tb]), (uint32_t)(((chunk >> 1) - 1) & 1));
          if (!ok) { atomicExch(p.status, 6); break; }
        }
        ok = mbar_wait(smem_u32(&fullBar[s]), ph);
        if (!ok) { atomicExch(p.status, 2); break; }
        tc_fence_after();
        uint64_t const dAh0 = dA0 + (uint64_t)((uint32_t)s * stageStep), dBh0 = dB0 + (uint64_t)((uint32_t)s * stageStep);
        uint32_t const tmemBig = tmemAcc + (uint32_t)(tb * BN), tmemSmall = tmemAcc + (uint32_t)(3 * BN);
#pragma unroll
        for (int k4 = 0; k4 < BK / 8; ++k4) {
          uint64_t const dAh = dAh0 + (uint64_t)(aAdv * k4), dBh = dBh0 + (uint64_t)(bAdv * k4);
          if (kSplit) {
            umma_tf32(tmemSmall, dAh + aLoStep, dBh, idesc, (it > 0 || k4 > 0) ? 1u : 0u);     // 0 = overwrite
            umma_tf32(tmemSmall, dAh, dBh + bLoStep, idesc, 1u);
            umma_tf32(tmemBig, dAh, dBh, idesc, (!chunkStart || k4 > 0) ? 1u : 0u);
          } else {
            umma_tf32(tmemAcc, dAh, dBh, idesc, (it > 0 || k4 > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&emptyBar[s]));    // frees the stage once these MMAs have read it
        if (++s == p.stages) { s = 0; ph ^= 1u; }
        if (++inChunk == p.drainEvery) {
          if (kSplit && chunk + 1 < numChunks) umma_commit(smem_u32(&drainFull[tb]));   // this chain's T is complete: hand it to the drain warps
          inChunk = 0; ++chunk;
        }
      }
      umma_commit(smem_u32(&accumBar));         // accumulator complete (or nothing was issued)
    }
    __syncwarp();
    tc_fence_before();
  } else {
    // ============================== producers ==============================
    int const t = threadIdx.x - (kEpilogueWarps + 1) * 32;      // 0..kProducerThreads-1
    // MN-major tiles: chunk column t % 32, k rows t / 32 + KSTEP j.  K-major tiles: chunk t % 8, rows t / 8 + RSTEP j.
    int const mnChunk = t & 31, mnK = t >> 5, kmChunk = t & 7, kmRow = t >> 3;
    bool const aFast = p.a.fast == 1;
    PixCtx px[4];
    TapCtx tap[CH];
    // fast IM2COL: this thread's four pixels, and its reduction index (fh,fw,c), which advances by KSTEP per step
    FastPix fpx = {0, 0, 0, false};
    int fFh = 0, fFw = 0, fC = 0, fR = 0, d8fh = 0, d8fw = 0, d8c = 0;
    uint32_t g0mask = 0, g1mask = 0, wmask = 0;    // per tap row fh / column fw: is the aligned row group / the column inside the image
    // fast WGATHER: this thread's four filter taps
    int tapS[CH], tapDw[CH], tapCoff[CH];
    bool tapOk[CH];
    int const HW = p.a.H * p.a.W;
    if (kAMode == OP_IM2COL) {
      if (aFast) {
        fpx = fast_pix(p.a, m0 + 4 * mnChunk, p.a.rows);
        fR = kbBeg * BK + mnK;
        fFh = fR % p.a.FH; int q = fR / p.a.FH; fFw = q % p.a.FW; fC = q / p.a.FW;
        d8fh = KSTEP % p.a.FH; q = KSTEP / p.a.FH; d8fw = q % p.a.FW; d8c = q / p.a.FW;
        if (fpx.valid) {
          for (int fh = 0; fh < p.a.FH; ++fh) {
            int sft = fh * p.a.dy - p.a.pt, h0 = fpx.ho0 + sft - (sft & 3);
            if (h0 >= 0 && h0 < p.a.H) g0mask |= 1u << fh;
            if (h0 + 4 >= 0 && h0 + 4 < p.a.H) g1mask |= 1u << fh;
          }
          for (int fw = 0; fw < p.a.FW; ++fw) {
            int w = fpx.wo + fw * p.a.dx - p.a.pl;
            if (w >= 0 && w < p.a.W) wmask |= 1u << fw;
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) px[e] = pix_ctx(p.a, m0 + 4 * mnChunk + e);
      }
    }
    if (kAMode == OP_WGATHER) {
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        tap[j] = tap_ctx(p.a, m0 + kmRow + RSTEP * j);
        tapS[j] = tap[j].dh; tapDw[j] = tap[j].dw; tapCoff[j] = (int)tap[j].coff; tapOk[j] = tap[j].valid;
      }
    }
    // reduction-contiguous dense operands: row pointers are fixed for the thread
    float const* aRow[CH];
    float const* bRow[CH];
    bool aRowOk[CH], bRowOk[CH];
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      int ia = m0 + kmRow + RSTEP * j, ib = n0 + kmRow + RSTEP * j;
      aRowOk[j] = (kAMode == OP_DENSE_K) && ia < p.a.rows;
      aRow[j] = p.a.ptr + (aRowOk[j] ? (long long)ia * p.a.ld : 0);
      bRowOk[j] = (kBMode == OP_DENSE_K) && ib < p.b.rows && kmRow + RSTEP * j < BN;
      bRow[j] = p.b.ptr + (bRowOk[j] ? (long long)ib * p.b.ld : 0);
    }
    if (p.pipelined && p.bTiles != nullptr && (kAMode == OP_IM2COL || kAMode == OP_WGATHER)) {
      // ---- pipelined: group-per-stage producers; B arrives as a ready-made tile image through one
      // bulk copy per stage.
      int const grp = t / kGroupThreads, tg = t % kGroupThreads;
      int const gChunk = tg & 31, gK = tg >> 5;          // MN-major: chunk column, first k row
      int const gKc = tg & 7, gRow = tg >> 3;            // K-major: 16-byte chunk within the row, first row
      uint32_t const bBytes = (kSplit ? 2u : 1u) * bTileBytes;
      FastPix gpx = {0, 0, 0, false};
      uint32_t g0m = 0, g1m = 0, wm = 0;
      if (kAMode == OP_IM2COL) {
        if (p.a.fast == 1) gpx = fast_pix(p.a, m0 + 4 * gChunk, p.a.rows);
        if (gpx.valid) {
          for (int fh = 0; fh < p.a.FH; ++fh) {
            int sft = fh * p.a.dy - p.a.pt, h0 = gpx.ho0 + sft - (sft & 3);
            if (h0 >= 0 && h0 < p.a.H) g0m |= 1u << fh;
            if (h0 + 4 >= 0 && h0 + 4 < p.a.H) g1m |= 1u << fh;
          }
          for (int fw = 0; fw < p.a.FW; ++fw) {
            int w = gpx.wo + fw * p.a.dx - p.a.pl;
            if (w >= 0 && w < p.a.W) wm |= 1u << fw;
          }
        }
      }
      // general gather (p.a.fast == 2: any extent, stride or dilation): the four pixels of a chunk are
      // tracked one by one -- element offset of the pixel's window origin, and which tap rows / columns
      // fall inside the image
      bool const aligned = p.a.fast == 1;
      int eBase[4] = {0, 0, 0, 0};
      uint32_t eHm[4] = {0, 0, 0, 0}, eWm[4] = {0, 0, 0, 0};
      if (kAMode == OP_IM2COL && !aligned) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int const m = m0 + 4 * gChunk + e;
          if (m < p.a.rows) {
            int ho = m % p.a.Ho, q = m / p.a.Ho, wo = q % p.a.Wo, n = q / p.a.Wo;
            eBase[e] = n * (int)p.a.imgStride + wo * p.a.sx * p.a.H + ho * p.a.sy;
            for (int fh = 0; fh < p.a.FH; ++fh) { int h = ho * p.a.sy + fh * p.a.dy - p.a.pt; if (h >= 0 && h < p.a.H) eHm[e] |= 1u << fh; }
            for (int fw = 0; fw < p.a.FW; ++fw) { int w = wo * p.a.sx + fw * p.a.dx - p.a.pl; if (w >= 0 && w < p.a.W) eWm[e] |= 1u << fw; }
          }
        }
      }
      float const* const xb = p.a.ptr + gpx.base;
      // reduction index of this thread's first chunk in its group's current stage, as (tap, channel);
      // it advances by KSTEPG per chunk and by kGroups * BK per stage, with carries instead of divisions
      int const taps = p.a.FH * p.a.FW;
      int tap0 = 0, ch0 = 0;
      if (kAMode == OP_IM2COL) { int r = (kbBeg + grp) * BK + gK; tap0 = r % taps; ch0 = r / taps; }
      int const dTapJ = KSTEPG % taps, dChJ = KSTEPG / taps, dTapIt = (kGroups * BK) % taps, dChIt = (kGroups * BK) / taps;
      uint32_t aOff[CHG];
#pragma unroll
      for (int j = 0; j < CHG; ++j) aOff[j] = kAMN ? mnmajor_off(gChunk, gK + KSTEPG * j, BM / 32) : kmajor_off(gRow + RSTEPG * j, gKc);
      for (int it = grp; it < numIter; it += kGroups) {
        float4 R[CHG];
        if (kAMode == OP_IM2COL) {
          int tap = tap0, ch = ch0, r = (kbBeg + it) * BK + gK;
#pragma unroll
          for (int j = 0; j < CHG; ++j) {
            int2 const te = tapLut[tap];
            uint32_t const e = (uint32_t)te.y;
            uint32_t const wv = (r < p.R ? 1u : 0u) & (wm >> ((e >> 5) & 31u));
            if (aligned) {
              bool const g0 = (wv & (g0m >> (e & 31u)) & 1u) != 0, g1 = (wv & (g1m >> (e & 31u)) & 1u) != 0;
              issue_window2(xb + (ch * HW + te.x), (int)((e >> 10) & 3u), g0, g1, R[j]);
            } else {
              uint32_t const rv = r < p.R ? 1u : 0u, fh = e & 31u, fw = (e >> 5) & 31u;
              float const* const q = p.a.ptr + (ch * HW + te.x);
              R[j] = make_float4(0.f, 0.f, 0.f, 0.f);
              ldg32_if(R[j].x, q + eBase[0], (rv & (eHm[0] >> fh) & (eWm[0] >> fw) & 1u) != 0);
              ldg32_if(R[j].y, q + eBase[1], (rv & (eHm[1] >> fh) & (eWm[1] >> fw) & 1u) != 0);
              ldg32_if(R[j].z, q + eBase[2], (rv & (eHm[2] >> fh) & (eWm[2] >> fw) & 1u) != 0);
              ldg32_if(R[j].w, q + eBase[3], (rv & (eHm[3] >> fh) & (eWm[3] >> fw) & 1u) != 0);
            }
            r += KSTEPG; tap += dTapJ; ch += dChJ;
            if (tap >= taps) { tap -= taps; ++ch; }
          }
          tap0 += dTapIt; ch0 += dChIt;
          if (tap0 >= taps) { tap0 -= taps; ++ch0; }
        } else {
          if (aligned) {
            FastPix rp = fast_pix(p.a, (kbBeg + it) * BK + 4 * gKc, p.R);
            float const* const rb = p.a.ptr + rp.base;
#pragma unroll
            for (int j = 0; j < CHG; ++j) {
              int4 const e = tapTab[gRow + RSTEPG * j];
              int const o = e.y & 3, h0 = rp.ho0 + e.y - o, w = rp.wo + e.z;
              bool const wv = rp.valid && e.w != 0 && w >= 0 && w < p.a.W;
              bool const g0 = wv && h0 >= 0 && h0 < p.a.H, g1 = wv && h0 + 4 >= 0 && h0 + 4 < p.a.H;
              issue_window2(rb + e.x, o, g0, g1, R[j]);
            }
          } else {
            // the four reduction pixels of this thread's chunk, one by one
            int const r = (kbBeg + it) * BK + 4 * gKc;
            int ho = r % p.a.Ho, q = r / p.a.Ho, wo = q % p.a.Wo, n = q / p.a.Wo;
            int pb[4], ph[4], pw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              ph[e] = (r + e < p.R) ? ho * p.a.sy : -(1 << 28);      // an invalid pixel fails every row test
              pw[e] = wo * p.a.sx;
              pb[e] = n * (int)p.a.imgStride + pw[e] * p.a.H + ho * p.a.sy;
              if (++ho == p.a.Ho) { ho = 0; if (++wo == p.a.Wo) { wo = 0; ++n; } }
            }
#pragma unroll
            for (int j = 0; j < CHG; ++j) {
              int4 const e = tapTab[gRow + RSTEPG * j];
              float const* const qp = p.a.ptr + e.x;
              bool const on = e.w != 0;
              R[j] = make_float4(0.f, 0.f, 0.f, 0.f);
              ldg32_if(R[j].x, qp + pb[0], on && (unsigned)(ph[0] + e.y) < (unsigned)p.a.H && (unsigned)(pw[0] + e.z) < (unsigned)p.a.W);
              ldg32_if(R[j].y, qp + pb[1], on && (unsigned)(ph[1] + e.y) < (unsigned)p.a.H && (unsigned)(pw[1] + e.z) < (unsigned)p.a.W);
              ldg32_if(R[j].z, qp + pb[2], on && (unsigned)(ph[2] + e.y) < (unsigned)p.a.H && (unsigned)(pw[2] + e.z) < (unsigned)p.a.W);
              ldg32_if(R[j].w, qp + pb[3], on && (unsigned)(ph[3] + e.y) < (unsigned)p.a.H && (unsigned)(pw[3] + e.z) < (unsigned)p.a.W);
            }
          }
        }
        int const s = it % p.stages;
        if (!mbar_wait(smem_u32(&emptyBar[s]), (uint32_t)(((it / p.stages) & 1) ^ 1))) { atomicExch(p.status, 1); break; }
        uint8_t* base = smem + (size_t)s * stageBytes;
        uint8_t* aHi = base;
        uint8_t* aLo = base + aTileBytes;
        if (tg == 0) {
          mbar_expect_tx(smem_u32(&fullBar[s]), bBytes);
          bulk_copy_g2s(smem_u32(base + (kSplit ? 2u : 1u) * aTileBytes),
                        p.bTiles + ((size_t)blockIdx.y * p.numKb + (size_t)(kbBeg + it)) * (bBytes / 4), bBytes, smem_u32(&fullBar[s]));
        }
#pragma unroll
        for (int j = 0; j < CHG; ++j) {
          float v[4] = {R[j].x, R[j].y, R[j].z, R[j].w};
          store_chunk<kSplit>(aHi, aLo, aOff[j], v);
        }
        fence_async_smem();
        __syncwarp();                         // every lane's stores and proxy fence precede the warp's single arrival
        if (lane == 0) mbar_arrive(smem_u32(&fullBar[s]));
      }
    } else if (t < kGenericThreads) {
    bool ok = true;
    for (int it = 0; it < numIter && ok; ++it) {
      int s = it % p.stages;
      int const r0 = (kbBeg + it) * BK;
      float va[CH][4], vb[CH][4];
      // global loads first, so that all of them are in flight before the first use
      if (kAMode == OP_IM2COL && aFast) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          load_shifted(p.a.ptr, p.a.H, p.a.W, fpx, fFh * p.a.dy - p.a.pt, fFw * p.a.dx - p.a.pl, fC * HW, fR < p.R, va[j]);
          fR += KSTEP; fFh += d8fh; fFw += d8fw; fC += d8c;
          if (fFh >= p.a.FH) { fFh -= p.a.FH; ++fFw; }
          if (fFw >= p.a.FW) { fFw -= p.a.FW; ++fC; }
        }
      } else if (kAMode == OP_WGATHER && aFast) {
        FastPix rp = fast_pix(p.a, r0 + 4 * kmChunk, p.R);
#pragma unroll
        for (int j = 0; j < CH; ++j) load_shifted(p.a.ptr, p.a.H, p.a.W, rp, tapS[j], tapDw[j], tapCoff[j], tapOk[j], va[j]);
      } else if (kAMode == OP_DENSE_K && p.a.vec) {
        int const r = r0 + 4 * kmChunk;
        long long boff = 0;
        if (p.a.P) { int nb = r / p.a.P; boff = (long long)nb * p.a.bs - (long long)nb * p.a.P; }
#pragma unroll
        for (int j = 0; j < CH; ++j) load_row4(aRow[j] + boff, r, p.R, aRowOk[j], va[j]);
      } else {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          if (kAMode == OP_IM2COL) load_im2col(p.a, px, r0 + mnK + KSTEP * j, p.R, va[j]);
          else if (kAMode == OP_DENSE_MN) load_dense_mn(p.a, m0 + 4 * mnChunk, r0 + mnK + KSTEP * j, p.R, va[j]);
          else if (kAMode == OP_WGATHER) load_wgather(p.a, tap[j], r0 + 4 * kmChunk, p.R, va[j]);
          else load_dense_k(p.a, m0 + kmRow + RSTEP * j, r0 + 4 * kmChunk, p.R, va[j]);
        }
      }
      if (kBMode == OP_DENSE_K && p.b.vec) {
        int const r = r0 + 4 * kmChunk;
        long long boff = 0;
        if (p.b.P) { int nb = r / p.b.P; boff = (long long)nb * p.b.bs - (long long)nb * p.b.P; }
#pragma unroll
        for (int j = 0; j < CH; ++j)
          if (kmRow + RSTEP * j < BN) load_row4(bRow[j] + boff, r, p.R, bRowOk[j], vb[j]);
      } else {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          if (kBMN) {
            if (4 * mnChunk < BN) load_dense_mn(p.b, n0 + 4 * mnChunk, r0 + mnK + KSTEP * j, p.R, vb[j]);
          } else {
            if (kmRow + RSTEP * j < BN) load_dense_k(p.b, n0 + kmRow + RSTEP * j, r0 + 4 * kmChunk, p.R, vb[j]);
          }
        }
      }
      ok = mbar_wait(smem_u32(&emptyBar[s]), (uint32_t)(((it / p.stages) & 1) ^ 1));
      if (!ok) { atomicExch(p.status, 1); break; }
      uint8_t* base = smem + (size_t)s * stageBytes;
      uint8_t* aHi = base;
      uint8_t* aLo = base + aTileBytes;
      uint8_t* bHi = base + (kSplit ? 2u : 1u) * aTileBytes;
      uint8_t* bLo = bHi + bTileBytes;
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        uint32_t off = kAMN ? mnmajor_off(mnChunk, mnK + KSTEP * j, BM / 32) : kmajor_off(kmRow + RSTEP * j, kmChunk);
        store_chunk<kSplit>(aHi, aLo, off, va[j]);
      }
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        if (kBMN) {
          if (4 * mnChunk < BN) store_chunk<kSplit>(bHi, bLo, mnmajor_off(mnChunk, mnK + KSTEP * j, BN / 32), vb[j]);
        } else {
          if (kmRow + RSTEP * j < BN) store_chunk<kSplit>(bHi, bLo, kmajor_off(kmRow + RSTEP * j, kmChunk), vb[j]);
        }
      }
      fence_async_smem();                     // generic-proxy writes -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&fullBar[s]));
    }
    }
  }

  // ============================== epilogue ==============================
  // Every warp but the MMA issuer drains the accumulator: a warp may read only the TMEM lanes of its
  // quarter (warp % 4), so the five warps of a quarter (one of warps 0-3 and four producers, which
  // have finished by now) share that quarter's 32 output rows and split the columns in chunks of 16.
  if (warp != kEpilogueWarps) {
    bool ok = mbar_wait(smem_u32(&accumBar), 0);
    if (kSplit && ok) ok = mbar_wait(smem_u32(&sumBar), 0);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (!ok) { if (lane == 0) atomicExch(p.status, 3); }
    else if (numIter > 0) {
      int const quarter = warp & 3;
      int const rank = warp < kEpilogueWarps ? 0 : 1 + (warp - (kEpilogueWarps + 1)) / 4;
      int const group = 1 + kProducerWarps / 4;
      int const m = m0 + quarter * 32 + lane;
      long long rowBase = 0;
      if (kEpi == EPI_CONV) { int pix = m % p.e.P, img = m / p.e.P; rowBase = (long long)img * p.e.Ktot * p.e.P + pix; }
      else rowBase = m + (long long)split * p.e.splitStride;
      uint32_t const lastT = (uint32_t)(((numChunks - 1) & 1) * BN);
      for (int c0 = 16 * rank; c0 < BN; c0 += 16 * group) {
        uint32_t const laneBase = tmemAcc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
        float big[16], small[16];
        {
          uint32_t t0[16], t1[16], t2[16];
          tmem_ld16_issue(laneBase + lastT, t0);
          if (kSplit) tmem_ld16_issue(laneBase + (uint32_t)(3 * BN), t1);
          if (kSplit && numChunks > 1) tmem_ld16_issue(laneBase + (uint32_t)(2 * BN), t2);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            big[j] = __uint_as_float(t0[j]);
            small[j] = kSplit ? __uint_as_float(t1[j]) : 0.f;
            if (kSplit && numChunks > 1) big[j] += __uint_as_float(t2[j]);
          }
        }
        if (m < p.M) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            int n = n0 + c0 + j;
            if (n < p.N) {
              float acc = big[j] + small[j];
              if (kEpi == EPI_CONV) {
                float* dst = p.e.out + rowBase + (long long)n * p.e.P;
                float o = p.e.inMult * acc;
                if (p.e.bias) o += p.e.bias[n];
                if (p.e.outMult != 0.f) o += p.e.outMult * *dst;
                if (p.e.relu) o = o > 0.f ? o : 0.f;
                *dst = o;
              } else {
                float o = acc;
                if (p.e.bias) o += p.e.bias[m];
                if (p.e.relu) o = o > 0.f ? o : 0.f;
                p.e.out[rowBase + (long long)n * p.e.ldd] = o;
              }
            }
          }
        }
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  tc_fence_after();
  if (warp == kEpilogueWarps) tmem_dealloc(tmemAcc, tmemCols);
}

// ------------------------------------------------------------------ convolution with the gathered operand in tensor memory
// fprop and stride-1 dgrad: D[m][n] = sum_r A(m,r) B(n,r), m = output pixel (ho,wo,image), r = (fh,fw,c).
// In tc_gemm_kernel both operands are read from shared memory by every MMA, and the shared-memory
// banks (MMA reads + producer stores + bulk-copy writes) are the unit that saturates first.  Here the
// gathered operand A never touches shared memory: one producer thread per output pixel (= TMEM lane)
// loads its 32 window elements of a k-block -- for a warp, 32 neighbouring pixels of one (tap,
// channel), i.e. one coalesced line per k -- splits them into hi / lo and writes them to tensor
// memory with tcgen05.st; the MMA takes A from tensor memory and only the filter tiles from shared
// memory (bulk copies of the ready-made tile images).  Any stride, padding and dilation.
//   warps 0-3   fp32 drain of the short accumulation chains (3xTF32), then epilogue
//   warps 4, 5  MMA issue (one lane each; warp 4 also allocates TMEM): issuer q takes every other k-block
//   warp  6     filter-tile loader (one lane): bulk copies into kTsBStages shared-memory stages
//   warp  7     forwarder (one lane): when the filter tile of a k-block has landed it arrives on that
//               k-block's A-stage barrier, so that an MMA thread waits on a single barrier per k-block
//   warps 8-15  producers: two groups of four warps (one warp per TMEM lane quarter); group g owns
//               A stage g and fills it for the k-blocks g, g+2, ...; a producer that finds its A stage
//               free again also knows that the filter stage of the same k-block is free and says so
//               to the loader, so that the MMA thread commits to a single barrier per k-block.
// The MMA thread is the critical resource: the tensor core's queue is about one MMA deep, so every
// cycle that thread spends on anything but issuing (each barrier wait costs it about 100 cycles even
// when the barrier is already complete, each commit about 50) is a cycle the tensor core idles.
// Tensor memory columns: T0 | T1 | T2 (BN each: chain accumulators, used round-robin by the two issuers; the small
// terms lo*hi + hi*lo go to T as well) | A stage g at 3*BN + 64*g: 32 columns hi, 32 columns lo.  The fp32 running
// sum P of a tile lives in shared memory, P[column][row], behind the filter stages.
constexpr int kTsGroups = 2;
constexpr int kTsLoaderWarp = kEpilogueWarps + 2;
constexpr int kTsForwardWarp = kEpilogueWarps + 3;
constexpr int kTsFirstProducer = kEpilogueWarps + 4;
constexpr int kTsThreads = (kTsFirstProducer + 4 * kTsGroups) * 32;      // 512: four warpgroups, 128 registers per thread at launch
constexpr int kTsRunWarp = kTsFirstProducer + 4 * kTsGroups;             // row mode only: warp 16 issues the runs (tensor-map copies)
constexpr int kTsThreadsRows = (kTsRunWarp + 4) * 32;                    // 640: warp 16's warpgroup is launched whole (warps 17-19 idle), so that it can hand its registers over
constexpr int kTsBStages = 6;           // at most; Params::bStages are in use
constexpr int kTsDrainEvery = 4;        // own k-blocks per accumulation chain: 4 x 4 k-steps x 3 MMAs.  Measured relative error of one layer
                                        // at the full VGG sizes: 4 -> 9e-7, 8 -> 1.7e-6, 16 -> 3.3e-6 (8 is 5-8% faster, 16 another 0-7%), but with 8
                                        // the end-to-end gradients of the LeNet and ResNet configurations no longer stay within 1e-5

__device__ __forceinline__ void umma_tf32_ts(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc, uint32_t iDesc, uint32_t accumulate)
{
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}"
               ::"r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(iDesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, uint32_t const (&r)[32])
{
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
               "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                 "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                 "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{ asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(bar), "r"(bytes) : "memory"); }

// Chains of one issuer in a tile of numIter k-blocks: the issuer that owns the tile's first k-block (second = 0) takes
// the k-blocks 0, 2, ..., the other one (second = 1) the k-blocks 1, 3, ...; a chain is kTsDrainEvery own k-blocks (3xTF32)
// or all of them (plain TF32).
template <bool kSplit>
__device__ __forceinline__ int ts_chains(int numIter, int second)
{
  int const nOwn = numIter > second ? (numIter - second + 1) / 2 : 0;
  return kSplit ? (nOwn + kTsDrainEvery - 1) / kTsDrainEvery : (nOwn > 0 ? 1 : 0);
}

// 4-D tensor-map copy global -> shared (tile mode, one destination CTA; the map covers this GPU's own memory only); completion
// is signalled on the mbarrier as transaction bytes.  The innermost coordinate c0 must be a multiple of four elements.
__device__ __forceinline__ void tma_load_4d(uint32_t dstSmem, void const* map, int c0, int c1, int c2, int c3, uint32_t bar)
{
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
               ::"r"(dstSmem), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dstSmem, void const* map, int c0, int c1, int c2, uint32_t bar)
{
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dstSmem), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

__device__ __forceinline__ void lds128(uint32_t addr, float (&v)[4])
{
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(addr));
}

__device__ __forceinline__ float lds32(uint32_t addr)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// Where row `row` (0..127, = TMEM lane) of row tile `tm` lies in the output: image, pixel ho + Ho*wo, and whether it exists.
// Linear mode: the tile is 128 consecutive output pixels (ho fastest, images following one another).  Box mode (p.tma):
// the tile is a box of bh x bw pixels of one image, row = dh + bh*dw.
struct RowPos { int img, pix, split; bool valid; };

__device__ __forceinline__ RowPos row_pos(Params const& p, int tm, int row)
{
  RowPos r;
  if (p.wg) {
    // tm = row tile + tilesM * reduction range; row tile = tap group + tapGroups * channel block; row = local tap * cPer + channel.
    // The "pixel" is the element of dF the row belongs to, fh + FH*(fw + FW*c), plus the offset of the range's partial result.
    int const split = tm / p.tilesM, t = tm - split * p.tilesM, cb = t / p.tapGroups, tg = t - cb * p.tapGroups;
    int const tl = row / p.cPer, c = cb * p.cPer + (row - tl * p.cPer), tap = tg * p.tapsPerTile + tl, taps = p.a.FH * p.a.FW;
    r.valid = tap < taps && c < p.a.C;
    r.img = 0; r.pix = r.valid ? tap + taps * c : 0; r.split = split;
    return r;
  }
  // tm = row tile + tilesM * reduction range (one range unless the caller cut the reduction)
  r.split = tm / p.tilesM; tm -= r.split * p.tilesM;
  if (!p.tma) {
    int const m = tm * BM + row;
    r.valid = m < p.M;
    int const mm = min(m, p.M - 1);
    r.img = mm / p.e.P; r.pix = mm - r.img * p.e.P;
  } else {
    int const per = p.tilesH * p.tilesW;
    int const n = tm / per, t = tm - n * per, wb = t / p.tilesH, hb = t - wb * p.tilesH;
    int const dw = row / p.bh, dh = row - dw * p.bh;
    int const h = hb * p.bh + dh, w = wb * p.bw + dw;
    r.valid = dw < p.bw && h < p.a.Ho && w < p.a.Wo;
    r.img = n; r.pix = r.valid ? h + p.a.Ho * w : 0;
  }
  return r;
}

// Epilogue of conv_ts_kernel: the finished tile sits in shared memory, P[column][row]; this warp stores the rows of its
// TMEM lane quarter for the columns rank, rank + nranks, ...: out[(image*Ktot + n)*P + pixel] = inMult*acc + bias[n] + outMult*old.
// P holds the columns cBeg .. cBeg + cCnt - 1 of the tile (cCnt = BN: all of it).
__device__ __forceinline__ void ts_store_tile(Params const& p, float const* P, int quarter, int lane, int rank, int nranks, int tm, int n0,
                                              uint32_t const* maskBits = nullptr, int cBeg = 0, int cCnt = 1 << 20)
{
  int const row = quarter * 32 + lane;
  RowPos const rp = row_pos(p, tm, row);
  if (!rp.valid) return;
  int const pix = rp.pix, img = rp.img;
  float* const dst0 = p.e.out + ((long long)rp.split * p.e.splitStride + (long long)img * p.e.Ktot * p.e.P + pix);
  int const nEnd = min(min(p.BN, cBeg + cCnt), p.N - n0);
  P -= (size_t)cBeg * BM;                              // column c of the tile sits at P[(c - cBeg) * BM + row]
  if (maskBits) {
    // the mask of this row was fetched while the tile was being computed: bit c = the mask is positive in column c
    uint32_t const b0 = maskBits[0], b1 = maskBits[1], b2 = maskBits[2], b3 = maskBits[3];
    for (int c = cBeg + rank; c < nEnd; c += nranks) {
      float* dst = dst0 + (long long)(n0 + c) * p.e.P;
      float o = p.e.inMult * P[c * BM + row];
      if (p.e.bias) o += p.e.bias[n0 + c];
      if (p.e.outMult != 0.f) o += p.e.outMult * *dst;
      if (p.e.relu) o = o > 0.f ? o : 0.f;
      uint32_t const w = c < 64 ? (c < 32 ? b0 : b1) : (c < 96 ? b2 : b3);
      *dst = ((w >> (c & 31)) & 1u) ? o : 0.f;
    }
    return;
  }
  if (p.e.mask) {
    // sixteen columns at a time, so that the mask loads of a batch are in flight together (one load per store in a plain
    // loop leaves the warp waiting for memory once per column)
    float const* const mk0 = p.e.mask + (dst0 - p.e.out);
    for (int c0 = cBeg + rank; c0 < nEnd; c0 += 16 * nranks) {
      float mk[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int const c = c0 + j * nranks;
        mk[j] = c < nEnd ? __ldg(mk0 + (long long)(n0 + c) * p.e.P) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int const c = c0 + j * nranks;
        if (c < nEnd) {
          float* dst = dst0 + (long long)(n0 + c) * p.e.P;
          float o = p.e.inMult * P[c * BM + row];
          if (p.e.bias) o += p.e.bias[n0 + c];
          if (p.e.outMult != 0.f) o += p.e.outMult * *dst;
          if (p.e.relu) o = o > 0.f ? o : 0.f;
          *dst = mk[j] > 0.f ? o : 0.f;
        }
      }
    }
    return;
  }
  for (int c = cBeg + rank; c < nEnd; c += nranks) {
    float* dst = dst0 + (long long)(n0 + c) * p.e.P;
    float o = p.e.inMult * P[c * BM + row];
    if (p.e.bias) o += p.e.bias[n0 + c];
    if (p.e.outMult != 0.f) o += p.e.outMult * *dst;
    if (p.e.relu) o = o > 0.f ? o : 0.f;
    *dst = o;
  }
}

// kTma: the producers take the input windows from shared memory, where the loader thread has them delivered by tensor-map copies
// (one box of boxH x boxW pixels x 32 channels per channel block and tile, zero-filled outside the image by the copy
// engine, two buffers), instead of gathering them from global memory with per-thread loads.  xmap: the 4-D tensor map
// (H, W, C, N) of the gathered tensor; unused otherwise.
// kMode 2 (filter gradient): rows are (tap, channel), the reduction runs over the output pixels; the loader thread has the run of 32
// pixels (plus up to three in front, so that the copy starts on a 16-byte boundary) of every row delivered per k-block.
constexpr int kWgRowWords = 36;                         // words per row of an x run in shared memory (144 bytes: 16-byte loads of 8 rows hit 32 banks)
constexpr int kWgRowBytes = kWgRowWords * 4;
constexpr int kWgStageBytes = BM * kWgRowBytes;         // 18432
constexpr int kTsXStages = 6;                           // at most
// "The MMAs of k-block j (numbered over the CTA's life) are through" is reported on barrier j % kTsDoneRing, phase j / kTsDoneRing,
// by the issuer's one commit per k-block.  Two parties wait for it: the producers of the A stage (for k-block j + kNA) and, in the
// forward / data-gradient modes, the filter-tile loader (for k-block j + bStages) -- the filter stage is free at the same moment,
// so the issuer needs no second commit and the producers need not tell the loader.  The ring is longer than either party can
// fall behind (at most bStages - 1 <= 5 k-blocks can complete before the loader has looked, at most kNA - 1 before a producer
// has), so a waiter never meets a barrier that is already a phase further.  (Waiting on the barriers of the kNA A stages instead
// was tried first: with six filter stages and four A stages the loader fell a whole phase behind on conv1_2 at batch 64 and then
// waited for a completion that needed its own copies -- the bounded wait ran out.)
constexpr int kTsDoneRing = 8;
static_assert(kTsBStages < kTsDoneRing, "the loader must not be able to fall a whole ring behind");

// Registers (kMode 0, 1): 128 per thread at launch (512 threads: the whole register file, one CTA per SM); then the warps 4-7
// keep 56 and the drain warps 0-3 take 200 (setmaxnreg: 128 of them hold the running sum of a tile).
// kMode 2 runs with a seventeenth warp for its per-k-block tensor-map copies -- such a copy keeps the issuing warp busy for about
// a microsecond, so it cannot share a warp with the forwarding, the filter tiles or a producer (measured: 35-50% slower each way).
// Registers are handed over by whole warpgroups, so the kernel is launched with five of them (640 threads, 96 registers each; the
// warps 17-19 have nothing to do): the warps 4-7 and 16-19 keep 40, the producers their 96, and the drain warps take 200 here
// too -- what the two groups give up (2 x 128 x 56) covers what the drain warps take (128 x 104), so the hand-over stays inside
// the registers the block was launched with and never waits.  With the running sum in shared memory this mode was
// bound by shared-memory bandwidth (per k-block about 150 KB of tile copies, operand reads by the tensor core, runs read by the
// producers and 32 KB of running sum read and rewritten, against 128 bytes per clock).
// kNarrow: tiles of 64 columns or fewer (kMode 0, 1), which get more accumulators and A stages (below).
template <bool kSplit, int kMode, bool kNarrow>
__global__ void __launch_bounds__(kMode == 2 ? kTsThreadsRows : kTsThreads, 1) conv_ts_kernel(Params p, const __grid_constant__ CUtensorMap xmap)
{
  constexpr bool kTma = kMode == 1, kWg = kMode == 2;
  extern __shared__ uint8_t smemRaw[];
  __shared__ __align__(8) uint64_t fullA[4], doneK[kTsDoneRing], fullB[kTsBStages], emptyB[kTsBStages];
  __shared__ __align__(8) uint64_t tFull[4], tFree[4], tileDone, turn[2], fullX[kTsXStages], emptyX[kTsXStages];
  __shared__ uint32_t tmemBase;
  __shared__ int2 tapLut[64];       // per filter tap fh + FH*fw: {element offset of the tap (in the input window when kTma), fh | fw << 5}

  uint8_t* smem = smemRaw + ((1024u - (smem_u32(smemRaw) & 1023u)) & 1023u);
  int const BN = p.BN;
  int const nB = p.bStages;
  uint32_t const bTileBytes = (uint32_t)BN * BK * 4;
  uint32_t const bBytes = (kSplit ? 2u : 1u) * bTileBytes;
  uint32_t const tmemCols = 512;
  // Tensor memory: kNT chain accumulators of BN columns (T[g % kNT] for chain g), then kNA A stages of 64 columns (32 hi, 32 lo).
  // 128-column tiles: three accumulators (two chains being accumulated while the third is drained and, at the end of a tile,
  // stored) and one A stage per issuer -- 512 columns.  Tiles of 64 columns or fewer have room for four accumulators and two
  // A stages per issuer: a stage is refilled while the MMAs of the issuer's other stage run, which is what these tiles, whose
  // MMAs are short, gain most from.  (Measured on 128-column tiles, same GPU, whole VGG-16 step: two accumulators + four stages is
  // level with three + two -- the refill of an A stage is not what bounds those tiles.)
  constexpr int kNA = kNarrow ? 4 : 2, kAPer = kNA / 2, kAShift = kNA == 4 ? 1 : 0;      // kAPer = 1 << kAShift
  constexpr int kNT = kNarrow ? 4 : 3;
  // Who tells the loader that a filter stage is free: the k-block's completion barrier (doneK, above) in the forward and
  // data-gradient modes (against a second commit per k-block on the narrow tiles and an arrival by the producers on the wide
  // ones: 3-4% faster on the 64-column layers, 1-3% on the 128-column layers); the row mode keeps a second commit by the issuer
  // on a barrier per filter stage (it lost 8% on its 64-column tiles without it and was level elsewhere).
  constexpr bool issuerFreesB = kWg;
  constexpr int kRing = kWg ? kNA : kTsDoneRing;      // (row mode: only the producers wait, a barrier per A stage is enough)
  uint32_t const colA = (uint32_t)(kNT * BN);
  float* const Psm = reinterpret_cast<float*>(smem + (size_t)nB * bBytes);      // [BN][BM]
  // input windows (kTma): two buffers of boxH*boxW*32 floats behind P
  uint32_t const xPlane = (uint32_t)(p.boxH * p.boxW), xTileBytes = kWg ? (uint32_t)kWgStageBytes : xPlane * 32u * 4u;
  bool const regsP = (kWg ? (BN == 128 || BN == 64) : (kNarrow ? BN == 64 : BN == 128)) && !p.smemSum;      // the running sum of a tile lives in the drain warps' registers
  uint32_t const xTile0 = smem_u32(Psm) + (regsP ? 32u : (uint32_t)BN) * BM * 4u;      // (registers: a patch of 32 columns for the stores)

  int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int const numIter = p.kbPerSplit;                      // k-blocks per tile (work item: one range of the reduction of one output tile)
  int const chunksPerTile = kSplit ? (numIter + kTsDrainEvery - 1) / kTsDrainEvery : 1;
  int const numTiles = p.tilesM * p.tilesN * p.splits;
  // this CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...; tile t = (row tile t / tilesN, column tile t % tilesN)
  int const myTiles = (int)blockIdx.x < numTiles ? (numTiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  bool const singleTile = (int)gridDim.x == numTiles;      // launched with one CTA per tile (long reductions)

  if (threadIdx.x == 0) {
    // an A stage is full when its four producer warps and the forwarder (filter tile landed) have arrived
    for (int s = 0; s < 4; ++s) mbar_init(smem_u32(&fullA[s]), 5);
    for (int s = 0; s < kTsDoneRing; ++s) mbar_init(smem_u32(&doneK[s]), 1);
    for (int s = 0; s < kTsBStages; ++s) { mbar_init(smem_u32(&fullB[s]), 1); mbar_init(smem_u32(&emptyB[s]), 1); }
    for (int b = 0; b < 4; ++b) { mbar_init(smem_u32(&tFull[b]), 1); mbar_init(smem_u32(&tFree[b]), kEpilogueWarps); }
    mbar_init(smem_u32(&tileDone), kEpilogueWarps);
    mbar_init(smem_u32(&turn[0]), 1); mbar_init(smem_u32(&turn[1]), 1);
    // an input window is full when its copy has landed (one arrival with the byte count), empty when all eight producer warps are done with it
    // (filter gradient: a run belongs to one k-block, so only the four warps of the group that owns it let go of it)
    for (int b = 0; b < kTsXStages; ++b) { mbar_init(smem_u32(&fullX[b]), 1); mbar_init(smem_u32(&emptyX[b]), kWg ? 4 : 4 * kTsGroups); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kEpilogueWarps) tmem_alloc(smem_u32(&tmemBase), tmemCols);
  if ((int)threadIdx.x < p.a.FH * p.a.FW) {
    int const fh = (int)threadIdx.x % p.a.FH, fw = (int)threadIdx.x / p.a.FH;
    if (kWg)       tapLut[threadIdx.x] = make_int2((fw * p.a.dx - p.a.pl) * p.a.H + fh * p.a.dy - p.a.pt, fh * p.a.dy - p.a.pt);   // {shift of the tap in the flattened plane, its row offset}
    else if (kTma) tapLut[threadIdx.x] = make_int2(fw * p.a.dx * p.boxH + fh * p.a.dy, fh | (fw << 5));
    else           tapLut[threadIdx.x] = make_int2((fw * p.a.dx - p.a.pl) * p.a.H + fh * p.a.dy - p.a.pt, fh | (fw << 5));
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmemAcc = tmemBase;

  if (warp < kEpilogueWarps) {
    // ============================== fp32 drain and epilogue ==============================
    // Chains are numbered over the whole life of the CTA: chain g was accumulated in T[g % 3].  Every chain of a tile is
    // added to the tile's running sum and its T released at once.  The running sum lives in this thread's registers (one
    // TMEM lane = one output row per thread, BN columns): the four drain warps take the registers the issuing / loading
    // warps give up (setmaxnreg).  After the tile's last chain the sum goes to shared memory once, P[column][row], and is
    // stored from there (coalesced along the rows) while the tensor core is already two chains into the next tile.  Tiles
    // of other widths than 128 and 64 columns keep the running sum in shared memory.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;" ::: "memory");
    uint32_t const lanes = tmemAcc + ((uint32_t)(warp * 32) << 16);
    float* const Prow = Psm + warp * 32 + lane;       // this thread's row of P: Prow[column * BM]
    bool const preMask = p.e.mask != nullptr && !singleTile;
    auto drain = [&](auto kRegsTag) {
      constexpr int kRegs = decltype(kRegsTag)::value;          // columns of the running sum held in registers (0: none, shared memory)
      float Pr[kRegs > 0 ? kRegs : 1];
      int g = 0;                                        // chains in the order they are drained, over the CTA's life: chain g sits in T[g % 3]
      bool ok = true;
      for (int ts = 0; ts < myTiles && ok; ++ts) {
        int const tile = (int)blockIdx.x + ts * (int)gridDim.x;
        int const tm = tile / p.tilesN, n0 = (tile % p.tilesN) * BN;
        int const chainsF = ts_chains<kSplit>(numIter, 0), chainsS = ts_chains<kSplit>(numIter, 1);   // of the issuer that owns the tile's first k-block, of the other
        bool fresh = true;                              // P holds nothing of this tile yet
        if (kRegs > 0) {
#pragma unroll
          for (int j = 0; j < kRegs; ++j) Pr[j] = 0.f;
        }
        // ReLU mask of this thread's output row (persistent mode): sixteen columns are fetched before each of the tile's
        // first chain waits, so that their latency passes while the chain is being computed, and kept as one bit each
        uint32_t mbits[4] = {0u, 0u, 0u, 0u};
        int const nEndT = min(BN, p.N - n0);
        float const* mkRow = p.e.mask;
        if (preMask) {
          RowPos const rp = row_pos(p, tm, warp * 32 + lane);     // a row that does not exist reads (and discards) the mask of a pixel that does
          mkRow += ((long long)rp.img * p.e.Ktot + n0) * p.e.P + rp.pix;      // (a masked data gradient is never cut into ranges)
        }
        int lc = 0;                                     // batches of sixteen mask columns fetched so far
        for (int c = 0; c < chainsF && ok; ++c) {
          for (int h = 0; h < 2 && ok; ++h) {
            if (h == 1 && c >= chainsS) continue;
            int const t = g % kNT;
            float mk[16];
            bool const fetch = preMask && 16 * lc < nEndT;
            if (fetch) {
#pragma unroll
              for (int j = 0; j < 16; ++j) mk[j] = __ldg(mkRow + (long long)min(16 * lc + j, nEndT - 1) * p.e.P);
            }
            ok = mbar_wait(smem_u32(&tFull[t]), (uint32_t)((g / kNT) & 1));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) atomicExch(p.status, 5); break; }
            ++g;
            tc_fence_after();
            if (kRegs > 0) {
              // P += T in fp32, in registers
#pragma unroll
              for (int c0 = 0; c0 < kRegs; c0 += 32) {
                uint32_t t0[16], t1[16];
                tmem_ld16_issue(lanes + (uint32_t)(t * kRegs + c0), t0);
                tmem_ld16_issue(lanes + (uint32_t)(t * kRegs + c0 + 16), t1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) { Pr[c0 + j] += __uint_as_float(t0[j]); Pr[c0 + 16 + j] += __uint_as_float(t1[j]); }
              }
            } else {
              // P = T (first chain of the tile) or P += T in fp32, in shared memory
              for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t t0[16], t1[16];
                bool const two = c0 + 16 < BN;
                tmem_ld16_issue(lanes + (uint32_t)(t * BN + c0), t0);
                if (two) tmem_ld16_issue(lanes + (uint32_t)(t * BN + c0 + 16), t1);
                tmem_ld_wait();
                float* pc = Prow + (size_t)c0 * BM;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  float v0 = __uint_as_float(t0[j]), v1 = __uint_as_float(t1[j]);
                  if (!fresh) { v0 += pc[j * BM]; if (two) v1 += pc[(16 + j) * BM]; }
                  pc[j * BM] = v0;
                  if (two) pc[(16 + j) * BM] = v1;
                }
              }
            }
            fresh = false;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tFree[t]));     // T[t] may be overwritten
            if (fetch) {
              uint32_t b = 0;
#pragma unroll
              for (int j = 0; j < 16; ++j) b |= (mk[j] > 0.f ? 1u : 0u) << j;
              b <<= 16 * (lc & 1);
              if (lc < 2) mbits[0] |= b; else if (lc < 4) mbits[1] |= b; else if (lc < 6) mbits[2] |= b; else mbits[3] |= b;
              ++lc;
            }
          }
        }
        if (!ok) break;
        for (; preMask && 16 * lc < nEndT; ++lc) {        // a tile of fewer chains than batches: the rest of the mask
          uint32_t b = 0;
#pragma unroll
          for (int j = 0; j < 16; ++j) b |= (__ldg(mkRow + (long long)min(16 * lc + j, nEndT - 1) * p.e.P) > 0.f ? 1u : 0u) << j;
          b <<= 16 * (lc & 1);
          if (lc < 2) mbits[0] |= b; else if (lc < 4) mbits[1] |= b; else if (lc < 6) mbits[2] |= b; else mbits[3] |= b;
        }
        if (kRegs > 0) {
          // The finished tile, 32 columns at a time: registers -> P[column][row] (a 16 KB patch of shared memory; every thread
          // writes and reads back its own row only, so no barrier) -> global memory, coalesced along the rows, while the tensor
          // core works on the next tile.  (The loop over the columns has to run over shared memory: registers cannot be indexed.)
#pragma unroll
          for (int c0 = 0; c0 < kRegs; c0 += 32) {
            if (c0 < nEndT) {
#pragma unroll
              for (int j = 0; j < 32; ++j) Prow[j * BM] = Pr[c0 + j];
              ts_store_tile(p, Psm, warp, lane, 0, 1, tm, n0, preMask ? mbits : nullptr, c0, 32);
            }
          }
        } else if (singleTile) {
          // one tile per CTA: the producers have nothing left to do and share the stores
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tileDone));
          ts_store_tile(p, Psm, warp, lane, 0, 1 + kTsGroups, tm, n0);
        } else {
          // the tile is complete in P: store it while the tensor core works on the next tile (its chains wait in
          // their T buffers until this is through)
          ts_store_tile(p, Psm, warp, lane, 0, 1, tm, n0, preMask ? mbits : nullptr);
        }
      }
    };
    // (each variant is compiled with the drain loops it can need only: the kernel's code has to stay small -- the variants for
    // 64-column tiles lost 10-30% whenever a few instructions were added to their roles)
    if constexpr (kWg) {
      if (regsP && BN == 128) drain(std::integral_constant<int, 128>{});
      else if (regsP) drain(std::integral_constant<int, 64>{});
      else drain(std::integral_constant<int, 0>{});
    } else if constexpr (kNarrow) {
      if (regsP && BN == 64) drain(std::integral_constant<int, 64>{});
      else drain(std::integral_constant<int, 0>{});
    } else {
      if (regsP && BN == 128) drain(std::integral_constant<int, 128>{});
      else drain(std::integral_constant<int, 0>{});
    }
  } else if (warp < 2 * kEpilogueWarps) {
    // warps 4-7 (issuers, filter-tile loader, forwarder) work with one thread each and a handful of registers: the rest goes
    // to the drain warps.  All four warps of the group execute this before anything else.
    if (kWg) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    else     asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == kEpilogueWarps || warp == kEpilogueWarps + 1) {
    // ============================== MMA issue ==============================
    // Two issuing threads (in two warps, on two schedulers).  The tensor core's queue is about one MMA deep, so
    // while a thread waits on a barrier or commits, nothing of its own is in flight; with two threads the other
    // one's MMAs fill the gap.  Issuer q takes the k-blocks gi = q, q+2, ... (numbered over the CTA's life), which
    // live in A stage q.  Chains (kTsDrainEvery own k-blocks) take the three T buffers in turn, in the order the
    // drain warps will add them to P, so two chains are being accumulated while the third is drained; the two
    // issuers never touch the same tensor-memory columns, so no ordering between the two streams is needed.
    // Per k-block: one barrier wait (A written and B landed), twelve MMAs, one commit; per chain: a wait for the T
    // buffer and a commit that hands the chain to the drain warps.  (An issuer cannot wait for its next k-block
    // ahead of time: that k-block goes into the A stage the current one still occupies.)
    if (lane == 0) {
      int const q = warp - kEpilogueWarps;
      uint32_t const idesc = make_idesc(false, false, BN);
      uint64_t const descB0 = make_desc(smem_u32(smem), 16, 1024);
      uint32_t const stageStep = bBytes >> 4, loStep = bTileBytes >> 4;
      bool ok = true;
      int sb = q, gBase = 0, g = 0;
      uint32_t tAcc = tmemAcc;
      uint32_t own = 0;                              // this issuer's k-blocks so far: k-block `own` sits in A stage q + 2*(own % kAPer)
      uint32_t phTurn = q == 0 ? 1u : 0u;            // issuer 0 has the first turn (nothing to wait for)
      // measured: +5-13% on 128-column tiles, -5% on 64-column tiles (their MMAs are short and the extra wait shows), -1-5% in the
      // row mode (whose producers read shared memory and are never late)
      bool const takeTurns = BN > 64 && !kWg;
      for (int ts = 0; ts < myTiles && ok; ++ts) {
        int const first = (int)((((long long)ts * numIter) ^ q) & 1);      // 0: this issuer owns the tile's first k-block
        int const chainsF = ts_chains<kSplit>(numIter, 0), chainsS = ts_chains<kSplit>(numIter, 1);
        for (int it = first, j = 0; it < numIter; it += 2, ++j) {
          int const inChunk = kSplit ? j % kTsDrainEvery : j;
          bool const chunkStart = inChunk == 0;
          bool const chunkEnd = it + 2 >= numIter || (kSplit && inChunk + 1 == kTsDrainEvery);
          if (chunkStart) {
            // this chain's place in the drain order (first issuer's chain c, second issuer's chain c, first's c+1, ...)
            int const c = kSplit ? j / kTsDrainEvery : 0;
            g = gBase + min(c, chainsF) + min(c, chainsS) + (first == 1 && c < chainsF ? 1 : 0);
            tAcc = tmemAcc + (uint32_t)((g % kNT) * BN);
            if (g >= kNT) {                           // the chain that sat in this T before must have been added to P
              ok = mbar_wait(smem_u32(&tFree[g % kNT]), (uint32_t)(((g / kNT) - 1) & 1));
              if (!ok) { atomicExch(p.status, 6); break; }
            }
          }
          int const sa = q + 2 * (int)(own & (uint32_t)(kAPer - 1));
          uint32_t const aHi = tmemAcc + colA + (uint32_t)(sa * 64), aLo = aHi + 32u;
          ok = mbar_wait(smem_u32(&fullA[sa]), (own >> kAShift) & 1u);
          if (!ok) { atomicExch(p.status, 2); break; }

          // The issuers take turns: left to themselves they interleave their MMAs one by one, both k-blocks finish
          // together, both A stages are refilled together and the tensor core idles meanwhile.  In turns, the MMAs of
          // one k-block run while the other issuer's A stage (freed a whole k-block earlier) is being refilled.
          if (takeTurns) {
            ok = mbar_wait(smem_u32(&turn[q]), phTurn);
            if (!ok) { atomicExch(p.status, 10); break; }
            phTurn ^= 1u;
          }
          tc_fence_after();
          uint64_t const dBh = descB0 + (uint64_t)((uint32_t)sb * stageStep), dBl = dBh + loStep;
#pragma unroll
          for (int k8 = 0; k8 < BK / 8; ++k8) {
            uint32_t const acc = (chunkStart && k8 == 0) ? 0u : 1u;      // 0 = overwrite: first MMA of a chain
            if (kSplit) {
              asm volatile(
                  "{\n .reg .pred p0, p1;\n setp.ne.b32 p0, %6, 0;\n setp.eq.b32 p1, %6, %6;\n"
                  " tcgen05.mma.cta_group::1.kind::tf32 [%0], [%2], %3, %5, p0;\n"
                  " tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %4, %5, p1;\n"
                  " tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %3, %5, p1;\n}"
                  ::"r"(tAcc), "r"(aHi + 8u * k8), "r"(aLo + 8u * k8), "l"(dBh + 2u * k8), "l"(dBl + 2u * k8), "r"(idesc), "r"(acc) : "memory");
            } else {
              umma_tf32_ts(tAcc, aHi + 8u * k8, dBh + 2u * k8, idesc, acc);
            }
            // The turn goes to the other issuer before the last MMAs of this k-block are queued: it needs about 200 cycles
            // (three MMAs) to wake up from its wait, and its MMAs, which use another A stage and another accumulator, may
            // queue up behind or between the remaining ones in any order.
            if (takeTurns && k8 == BK / 8 - 2) mbar_arrive(smem_u32(&turn[q ^ 1]));
          }
          if (!ok) break;
          umma_commit(smem_u32(&doneK[(2u * own + (uint32_t)q) & (uint32_t)(kRing - 1)]));     // when these MMAs are through: the A stage goes back to its producers and (forward, data gradient) the filter stage to the loader
          if (issuerFreesB) umma_commit(smem_u32(&emptyB[sb]));     // (row mode) the filter stage to the loader
          ++own;
          sb += 2; if (sb >= nB) sb -= nB;
          if (chunkEnd) umma_commit(smem_u32(&tFull[g % kNT]));   // chain complete: hand it to the drain warps
        }
        gBase += chainsF + chainsS;
      }
    }
    __syncwarp();
    tc_fence_before();
  } else if (warp == kTsLoaderWarp) {
    // ============================== filter tiles: bulk copies ==============================
    if (lane == 0 && !(p.testSwitch & 1)) {
      int sb = 0; uint32_t ph = 1;                       // first use of a stage: nothing to wait for
      bool ok = true;
      long long gk = 0;                                  // k-blocks numbered over the CTA's life
      for (int ts = 0; ts < myTiles && ok; ++ts) {
        int const tile = (int)blockIdx.x + ts * (int)gridDim.x;
        int const nt = tile % p.tilesN;
        float const* src = p.bTiles + ((size_t)nt * p.kbTot + (size_t)(tile / p.tilesN / p.tilesM) * numIter) * (bBytes / 4);
        for (int it = 0; it < numIter; ++it, ++gk) {
          if (!issuerFreesB) {
            // the stage held the filter tile of k-block gk - nB
            long long const j = gk - nB;
            if (j >= 0 && !mbar_wait(smem_u32(&doneK[j & (kRing - 1)]), (uint32_t)((j / kRing) & 1))) { atomicExch(p.status, 8); ok = false; break; }
          } else
          if (!mbar_wait(smem_u32(&emptyB[sb]), ph)) { atomicExch(p.status, 8); ok = false; break; }
          mbar_arrive_expect_tx(smem_u32(&fullB[sb]), bBytes);
          bulk_copy_g2s(smem_u32(smem + (size_t)sb * bBytes), src + (size_t)it * (bBytes / 4), bBytes, smem_u32(&fullB[sb]));
          if (++sb == nB) { sb = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == kTsForwardWarp) {
    // ============================== forwarder; input windows / runs: tensor-map copies ==============================
    // Forwarding: k-block gi (numbered over the CTA's life) uses A stage gi & 1 in that barrier's phase gi >> 1.  The arrival
    // for gi must fall into that phase, so the phase of gi - 2 has to be complete first (this thread arrived in it as well).
    // The windows of kTma (one per tile and block of 32 channels, xStages buffers) are numbered over the CTA's life and issued by
    // the same thread.
    if (lane == 0) {
      bool ok = true;
      int const taps = p.a.FH * p.a.FW;
      int const perTile = kTma ? numIter / taps : 0;                         // windows per tile
      int const nXb = p.xStages;
      long long const wTotal = (long long)myTiles * perTile;
      long long wxs = 0;                                  // next window to issue
      int wts = 0, wsub = 0;                              // its tile (in this CTA's sequence) and its index inside the tile
      int wbuf = 0; uint32_t wph = 1;                     // its buffer; first use of a buffer: nothing to wait for
      // Window w is issued when this thread has come to k-block wpos(w) (numbered over the CTA's life), after a wait for its buffer
      // (the window nXb before it).  That buffer is let go of at the end of a hand-over whose arrival on the A-stage barrier this
      // thread has already seen at wpos(w) -- the hand-over of k-block wpos(w) - 2 -- so the wait is short and depends on nothing
      // that this thread has yet to do.  The first nXb at once.
      auto windows = [&](long long gpos) -> bool {
        while (wxs < wTotal) {
          long long const wpos = wxs < nXb ? 0 : (wxs - nXb + 1) * taps + 1;
          if (wpos > gpos) break;
          if (!mbar_wait(smem_u32(&emptyX[wbuf]), wph)) { atomicExch(p.status, 12); return false; }
          int const tmf = ((int)blockIdx.x + wts * (int)gridDim.x) / p.tilesN;
          int const split = tmf / p.tilesM, tm = tmf - split * p.tilesM;
          {
            int const per = p.tilesH * p.tilesW;
            int const n = tm / per, t = tm - n * per, wb = t / p.tilesH, hb = t - wb * p.tilesH;
            int const c0 = hb * p.bh - p.a.pt - p.rowOff, c1 = wb * p.bw - p.a.pl;      // c0 is a multiple of four: bh and pt + rowOff are
            mbar_arrive_expect_tx(smem_u32(&fullX[wbuf]), xTileBytes);
            tma_load_4d(xTile0 + (uint32_t)wbuf * xTileBytes, &xmap, c0, c1, (split * perTile + wsub) * 32, n, smem_u32(&fullX[wbuf]));   // a range of the reduction is whole channel blocks
          }
          ++wxs;
          if (++wbuf == nXb) { wbuf = 0; wph ^= 1u; }
          if (++wsub == perTile) { wsub = 0; ++wts; }
        }
        return true;
      };
      int sb = 0; uint32_t phB = 0;
      long long const total = (long long)myTiles * numIter;
      for (long long gi = 0; gi < total && ok; ++gi) {
        int const sa = (int)(gi & (kNA - 1));
        if (gi >= kNA && !mbar_wait(smem_u32(&fullA[sa]), (uint32_t)(((gi >> (kAShift + 1)) - 1) & 1))) { atomicExch(p.status, 9); break; }
        if (kTma && !windows(gi)) break;
        if (!mbar_wait(smem_u32(&fullB[sb]), phB)) { atomicExch(p.status, 7); break; }
        mbar_arrive(smem_u32(&fullA[sa]));
        if (++sb == nB) { sb = 0; phB ^= 1u; }
      }
    }
    __syncwarp();
    }
  } else if (warp >= kTsRunWarp) {
    // ============================== row mode: runs by tensor-map copies ==============================
    // (the warpgroup of warps 16-19 exists in the row mode only and keeps a handful of registers, like the warps 4-7)
    if (kWg) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    if (kWg && warp == kTsRunWarp && lane == 0) {
      // The run of k-block j (numbered over the CTA's life) -- 36 pixels x cPer channels per
      // tap of the tile, from the plane of image r / P starting at pixel r % P + shift of the tap, rounded down to four pixels (P:
      // the plane rounded up to whole k-blocks; the tile images hold zeros for the pixels added; pixels before the plane's first
      // or past its last one -- a tap that leaves the image to the left or right, a k-block past the end of the batch -- arrive as
      // zeros) -- goes into buffer j % xStages as soon as the producers have let go of the run of k-block j - xStages.
      int const taps = p.a.FH * p.a.FW, P = p.plane, nX = p.xStages;
      int buf = 0; uint32_t ph = 1;                        // first use of a buffer: nothing to wait for
      bool ok = true;
      for (int ts = 0; ts < myTiles && ok; ++ts) {
        int const tmf = ((int)blockIdx.x + ts * (int)gridDim.x) / p.tilesN;
        int const split = tmf / p.tilesM, t = tmf - split * p.tilesM, cb = t / p.tapGroups, tg = t - cb * p.tapGroups;
        int const tap0 = tg * p.tapsPerTile, nTaps = min(p.tapsPerTile, taps - tap0);
        long long const r0 = (long long)split * numIter * BK;
        int img = (int)(r0 / P), pix0 = (int)(r0 - (long long)img * P);
        for (int it = 0; it < numIter; ++it) {
          if (!mbar_wait(smem_u32(&emptyX[buf]), ph)) { atomicExch(p.status, 12); ok = false; break; }
          mbar_arrive_expect_tx(smem_u32(&fullX[buf]), (uint32_t)(nTaps * p.cPer * kWgRowBytes));
          for (int tl = 0; tl < nTaps; ++tl)
            tma_load_3d(xTile0 + (uint32_t)buf * xTileBytes + (uint32_t)(tl * p.cPer * kWgRowBytes), &xmap,
                        pix0 + (tapLut[tap0 + tl].x & ~3), cb * p.cPer, img, smem_u32(&fullX[buf]));
          if (++buf == nX) { buf = 0; ph ^= 1u; }
          pix0 += BK; if (pix0 >= P) { pix0 -= P; ++img; }
        }
      }
    }
    __syncwarp();
  } else {
    // ============================== producers ==============================
    int const grp = (warp - kTsFirstProducer) >> 2;
    int const quarter = warp & 3;                       // the TMEM lanes this warp may access
    int const HW = p.a.H * p.a.W, taps = p.a.FH * p.a.FW;
    uint32_t const aBase = tmemAcc + ((uint32_t)(quarter * 32) << 16) + colA;
    uint32_t own = 0;                                   // this group's k-blocks so far: k-block `own` goes into A stage grp + 2*(own % kAPer)
    long long gi = 0;                                   // k-blocks numbered over the CTA's life; this group takes gi % 2 == grp
    bool ok = true;

    // One k-block, from the 32 gathered values of this thread's pixel to the arrival on the A-stage barrier.
    auto hand_over = [&](float const (&v)[32], int it) -> bool {
      // both parts are ready in registers before the wait, so that the stage is refilled as soon as it is free
      uint32_t hi[32], lo[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        hi[k] = __float_as_uint(tf32_hi(v[k]));
        if (kSplit) lo[k] = __float_as_uint(v[k] - __uint_as_float(hi[k]));
      }
      int const sa = grp + 2 * (int)(own & (uint32_t)(kAPer - 1));
      uint32_t const aAddr = aBase + (uint32_t)(sa * 64);
      if (own >= (uint32_t)kAPer) {      // (first use of a stage: nothing to wait for) the stage's previous k-block, kNA before this one, must be through
        uint32_t const jp = 2u * (own - (uint32_t)kAPer) + (uint32_t)grp;
        if (!mbar_wait(smem_u32(&doneK[jp & (uint32_t)(kRing - 1)]), (jp / (uint32_t)kRing) & 1u)) { atomicExch(p.status, 1); return false; }
      }
      ++own;
      tc_fence_after();
      tmem_st32(aAddr, hi);
      if (kSplit) tmem_st32(aAddr + 32u, lo);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&fullA[sa]));
      return true;
    };

    if (kWg) {
      // This thread's row: channel (row % cPer) of the tile's local tap row / cPer -- the same tap for the whole warp.  A k-block
      // is 32 consecutive output pixels; the row's 36-pixel run lies in shared memory, the wanted 32 start `s` pixels in.
      int const row = quarter * 32 + lane;
      int const tl = (quarter * 32) / p.cPer;
      int const H = p.a.H, P = p.plane, nX = p.xStages;
      for (int ts = 0; ts < myTiles && ok; ++ts) {
        int const tmf = ((int)blockIdx.x + ts * (int)gridDim.x) / p.tilesN;
        int const split = tmf / p.tilesM, t = tmf - split * p.tilesM, tg = t % p.tapGroups;
        int const tap = tg * p.tapsPerTile + tl;
        bool const active = tap < taps;                                   // a tap the filter does not have: rows of zeros, never stored
        int2 const te = tapLut[active ? tap : 0];
        int const s = te.x & 3, dh = te.y;
        int const itFirst = (int)((gi ^ grp) & 1);
        int pb = (int)(((long long)split * numIter + itFirst) * BK % P);      // first pixel of the k-block inside its image
        for (int it = itFirst; it < numIter; it += kTsGroups) {
          uint32_t const xs = (uint32_t)(gi + it);
          int const buf = (int)(xs % (uint32_t)nX);
          if (!mbar_wait(smem_u32(&fullX[buf]), (xs / (uint32_t)nX) & 1u)) { atomicExch(p.status, 11); ok = false; break; }
          uint32_t const src = xTile0 + (uint32_t)buf * xTileBytes + (uint32_t)(row * kWgRowBytes);
          float w[kWgRowWords];
#pragma unroll
          for (int j = 0; j < kWgRowWords / 4; ++j) lds128(src + 16u * j, *reinterpret_cast<float(*)[4]>(&w[4 * j]));
          // pixels whose tap row leaves the image above or below: output row ho + dh outside [0, H) -- the same for every lane's row
          int const ho = (pb + lane) % H;
          pb += kTsGroups * BK; while (pb >= P) pb -= P;
          uint32_t const zm = active ? __ballot_sync(0xffffffffu, (unsigned)(ho + dh) >= (unsigned)H) : 0xffffffffu;
          float v[32];
          switch (s) {
            case 0:
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = w[k];
              break;
            case 1:
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = w[k + 1];
              break;
            case 2:
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = w[k + 2];
              break;
            default:
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = w[k + 3];
              break;
          }
          if (zm) {
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = ((zm >> k) & 1u) ? 0.f : v[k];
          }
          if (!hand_over(v, it)) { ok = false; break; }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&emptyX[buf]));     // this warp's loads from the run have completed (their values were used above)
        }
        gi += numIter;
      }
    } else if (kTma) {
      // This thread's pixel inside the input window: row dh + rowOff, column dw (a lane beyond the box reads the window's
      // first element; its row is never stored).  A k-block is one filter tap and 32 channels: 32 loads from shared memory
      // one channel plane apart.
      int const row = quarter * 32 + lane;
      int const dw = row / p.bh, dh = row - dw * p.bh;
      uint32_t const laneOff = dw < p.bw ? (uint32_t)(dw * p.boxH + dh + p.rowOff) * 4u : 0u;
      uint32_t const planeBytes = xPlane * 4u;
      int const numCb = numIter / taps;
      long long xs = 0;
      for (int ts = 0; ts < myTiles && ok; ++ts) {
        int const par = (int)((gi ^ grp) & 1);              // this group's k-blocks of the tile: it % 2 == par
        for (int cb = 0; cb < numCb && ok; ++cb, ++xs) {
          int const buf = (int)(xs % p.xStages);
          // every producer warp waits for and lets go of every window, whether or not one of its k-blocks falls into it:
          // a warp can then never arrive twice in one phase of the window's barrier
          if (!mbar_wait(smem_u32(&fullX[buf]), (uint32_t)((xs / p.xStages) & 1))) { atomicExch(p.status, 11); ok = false; break; }
          uint32_t const base = xTile0 + (uint32_t)buf * xTileBytes + laneOff;
          int const itBeg = cb * taps;
          for (int it = itBeg + ((itBeg ^ par) & 1); it < itBeg + taps; it += kTsGroups) {
            uint32_t const src = base + (uint32_t)tapLut[it - itBeg].x * 4u;
            float v[32];
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = lds32(src + (uint32_t)k * planeBytes);
            if (!hand_over(v, it)) { ok = false; break; }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&emptyX[buf]));     // this warp's loads from the window have completed (their values were used above)
        }
        gi += numIter;
      }
    } else {
      for (int ts = 0; ts < myTiles && ok; ++ts) {
        int const tile = (int)blockIdx.x + ts * (int)gridDim.x;
        int const tmf = tile / p.tilesN, split = tmf / p.tilesM, kb0 = split * numIter;     // this item's range starts at k-block kb0
        int const m = (tmf - split * p.tilesM) * BM + quarter * 32 + lane;
        uint32_t hm = 0, wm = 0;                          // tap rows / columns inside the image for this pixel
        float const* xq = p.a.ptr;
        if (m < p.M) {
          int const ho = m % p.a.Ho, q = m / p.a.Ho, wo = q % p.a.Wo, n = q / p.a.Wo;
          xq += (long long)n * p.a.imgStride + (long long)wo * p.a.sx * p.a.H + ho * p.a.sy;
          for (int fh = 0; fh < p.a.FH; ++fh) { int h = ho * p.a.sy + fh * p.a.dy - p.a.pt; if (h >= 0 && h < p.a.H) hm |= 1u << fh; }
          for (int fw = 0; fw < p.a.FW; ++fw) { int w = wo * p.a.sx + fw * p.a.dx - p.a.pl; if (w >= 0 && w < p.a.W) wm |= 1u << fw; }
        }
        for (int it = (int)((gi ^ grp) & 1); it < numIter; it += kTsGroups) {
          int const r = (kb0 + it) * BK;
          float v[32];
          if (p.chanFast) {
            // the whole k-block is one filter tap and 32 consecutive channels: one validity test, constant stride.  The taps
            // of a channel block follow one another, so that the lines fetched for one tap are still in L1 for the next.
            int const tp = (kb0 + it) % taps, c0 = ((kb0 + it) / taps) * 32;
            int2 const te = tapLut[tp];
            uint32_t const e = (uint32_t)te.y;
            bool const on = ((hm >> (e & 31u)) & (wm >> (e >> 5)) & 1u) != 0 && c0 < p.a.C;      // (c0 >= C: padding of the last range)
            // unconditional loads (a pixel outside the image reads the start of the tensor instead and discards it):
            // nothing for the compiler to predicate or branch around, all 32 in flight together
            float const* const q = on ? xq + ((long long)c0 * HW + te.x) : p.a.ptr;
            long long const step = on ? (long long)HW : 0;
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = __ldg(q + k * step);
            if (!on) {
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = 0.f;
            }
          } else {
            int tap = r % taps, ch = r / taps;
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              int2 const te = tapLut[tap];
              uint32_t const e = (uint32_t)te.y;
              bool const on = ((r + k < p.R ? 1u : 0u) & (hm >> (e & 31u)) & (wm >> (e >> 5))) != 0;
              v[k] = 0.f;
              ldg32_if(v[k], xq + (ch * HW + te.x), on);
              if (++tap == taps) { tap = 0; ++ch; }
            }
          }
          if (!hand_over(v, it)) { ok = false; break; }
        }
        gi += numIter;
      }
    }
    if (singleTile && !regsP && ok && myTiles > 0) {
      bool done = mbar_wait(smem_u32(&tileDone), 0);
      done = __all_sync(0xffffffffu, done);
      tc_fence_after();
      if (!done) { if (lane == 0) atomicExch(p.status, 3); }
      else {
        int const tile = (int)blockIdx.x;
        ts_store_tile(p, Psm, quarter, lane, 1 + grp, 1 + kTsGroups, tile / p.tilesN, (tile % p.tilesN) * BN);
      }
      tc_fence_before();
    }
  }

  __syncthreads();
  tc_fence_after();
  if (warp == kEpilogueWarps) tmem_dealloc(tmemAcc, tmemCols);
}

// out[e] = sum over splits (ascending) of part[s*stride + e]
__global__ void tc_splitk_reduce_kernel(float* __restrict__ out, float const* __restrict__ part, size_t n, size_t stride, int splits)
{
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += step) {
    float s = part[e];
    for (int k = 1; k < splits; ++k) s += part[(size_t)k * stride + e];
    out[e] = s;
  }
}

// Ft[fh', fw', k, c] = F[FH-1-fh', FW-1-fw', c, k]: the filter bank whose forward convolution
// over dY is the data gradient of a stride-1 convolution.
__global__ void flip_filters_kernel(float* __restrict__ ft, float const* __restrict__ f, int FH, int FW, int C, int K)
{
  size_t total = (size_t)FH * FW * C * K;
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += step) {
    int fh = (int)(o % FH); size_t t = o / FH;
    int fw = (int)(t % FW); t /= FW;
    int k = (int)(t % K); int c = (int)(t / K);
    ft[o] = f[(FH - 1 - fh) + (size_t)FH * ((FW - 1 - fw) + (size_t)FW * (c + (size_t)C * k))];
  }
}

// The B operand of fprop / dgrad is the filter bank: small, and the same for every CTA.  It is split
// into hi / lo once and laid out as ready-made shared-memory tile images -- for n-tile t and k-block
// kb: [hi tile BN x 32][lo tile BN x 32], K-major with the 128-byte swizzle -- so that a producer
// fetches a whole stage of B with one bulk copy.
// modes 3 / 4: as 0 / 1 with the reduction index in blocks of 32 channels, all filter taps of a block one after the other.
// mode 5: B(n, r) = F[n + N*r].
// mode 0: B(n, r) = F[n*R + r].  mode 2: B(n, r) = dY[pixel, n, image] with r = pixel + P*image.  mode 1 (data gradient of a stride-1 convolution): n = channel c,
// r = fh' + FH*(fw' + FW*k), B = F[FH-1-fh', FW-1-fw', c, k].
template <bool kSplit>
__global__ void prep_b_tiles_kernel(float* __restrict__ out, float const* __restrict__ f, int N, int R, int BN, int numKb,
                                    int mode, int FH, int FW, int C, int K)
{
  size_t const Rp = (size_t)numKb * 32;
  size_t const total = (size_t)((N + BN - 1) / BN) * BN * Rp;
  size_t const step = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    int const r = (int)(idx % Rp), n = (int)(idx / Rp);
    float val = 0.f;
    if (n < N && r < R) {
      if (mode == 0) val = f[(size_t)n * R + r];
      else if (mode == 2) {
        // filter gradient: n = filter, r = pixel + P*image of dY (FH carries P here)
        int img = r / FH, pix = r - img * FH;
        val = f[((size_t)img * N + n) * FH + pix];
      } else if (mode == 5) {
        // B(n, r) = f[n + N*r]: rows contiguous (dY of a fully connected layer as the filters of its weight gradient)
        val = f[(size_t)r * N + n];
      } else if (mode == 3) {
        // forward filters, reduction in blocks of 32 channels: r = c%32 + 32*(tap + taps*(c/32))
        int taps = FH * FW, t = r >> 5, tap = t % taps, c = (t / taps) * 32 + (r & 31);
        val = f[(size_t)n * R + tap + (size_t)taps * c];
      } else if (mode == 4) {
        // data gradient, reduction in blocks of 32 filters: r = k%32 + 32*(tap' + taps*(k/32)), tap' = fh' + FH*fw'
        int taps = FH * FW, t = r >> 5, tap = t % taps, k = (t / taps) * 32 + (r & 31), fh = tap % FH, fw = tap / FH;
        val = f[(FH - 1 - fh) + (size_t)FH * ((FW - 1 - fw) + (size_t)FW * (n + (size_t)C * k))];
      } else {
        int fh = r % FH, t = r / FH, fw = t % FW, k = t / FW;
        val = f[(FH - 1 - fh) + (size_t)FH * ((FW - 1 - fw) + (size_t)FW * (n + (size_t)C * k))];
      }
    }
    int const tile = n / BN, row = n % BN, kb = r >> 5, kk = r & 31;
    size_t const base = ((size_t)tile * numKb + kb) * (kSplit ? 2 : 1) * (size_t)BN * 32;
    size_t const off = (size_t)row * 32 + ((((kk >> 2) ^ (row & 7)) << 2) | (kk & 3));
    if (kSplit) {
      float hi = tf32_hi(val);
      out[base + off] = hi;
      out[base + (size_t)BN * 32 + off] = val - hi;
    } else {
      out[base + off] = val;
    }
  }
}

// dY of a filter gradient as tile images (mode 2 of prep_b_tiles_kernel) for planes that are a multiple of
// four pixels: 16-byte loads along the pixels, 16-byte stores of the swizzled chunks, and -- dY being read
// anyway -- the bias gradient db[n] = sum of dY over pixels and images (reference bits/nnconv.cu:141-149) on
// the way: per-block partial sums, and the block that takes a channel's last ticket adds them in block order,
// so the result does not depend on the scheduling.
// grid (blocks per channel, channels rounded up to the tile), kPrepThreads threads, kPrepIters float4 per thread.
constexpr int kPrepThreads = 256, kPrepIters = 4;

template <bool kSplit>
__global__ void __launch_bounds__(kPrepThreads)
prep_dy_tiles_kernel(float* __restrict__ out, float const* __restrict__ dy, int N, int R, int P, int Pp, int BN, int numKb,
                     float* __restrict__ db, float* __restrict__ dbPart, unsigned* __restrict__ tickets)
{
  __shared__ float red[kPrepThreads / 32];
  __shared__ bool last;
  int const n = blockIdx.y, tile = n / BN, row = n % BN;
  int const Rp = numKb * 32;
  float sum = 0.f;
#pragma unroll
  for (int u = 0; u < kPrepIters; ++u) {
    int const r = ((int)blockIdx.x * kPrepIters + u) * (kPrepThreads * 4) + (int)threadIdx.x * 4;
    if (r < Rp) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      // reduction index r = pixel + Pp * image (Pp >= P: planes padded to whole k-blocks read as zeros); R = P * images
      int const img = r / Pp, pix = r - img * Pp;
      if (n < N && pix < P && img * P + pix < R) v = *reinterpret_cast<float4 const*>(dy + ((size_t)img * N + n) * P + pix);
      sum += (v.x + v.y) + (v.z + v.w);
      int const kb = r >> 5, kk = r & 31;
      size_t const base = ((size_t)tile * numKb + kb) * (kSplit ? 2 : 1) * (size_t)BN * 32;
      size_t const off = (size_t)row * 32 + (size_t)((((kk >> 2) ^ (row & 7)) << 2));
      if (kSplit) {
        float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
        *reinterpret_cast<float4*>(out + base + off) = h;
        *reinterpret_cast<float4*>(out + base + (size_t)BN * 32 + off) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
      } else {
        *reinterpret_cast<float4*>(out + base + off) = v;
      }
    }
  }
  if (db == nullptr || n >= N) return;
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < kPrepThreads / 32; ++w) s += red[w];
    dbPart[(size_t)n * gridDim.x + blockIdx.x] = s;
    __threadfence();
    last = atomicAdd(&tickets[n], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // the channel's partials in block order: strided per-thread sums, then a fixed tree
  float s = 0.f;
  for (unsigned i = threadIdx.x; i < gridDim.x; i += kPrepThreads) s += __ldcg(dbPart + (size_t)n * gridDim.x + i);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kPrepThreads / 32; ++w) t += red[w];
    db[n] = t;
    tickets[n] = 0;      // ready for the next call
  }
}

// Builds the tile images in the context's scratch; returns nullptr (error set) on failure.
size_t b_tiles_bytes(vlb_ctx* ctx, int N, int BN, int numKb)
{
  bool split3 = ctx->precision == VLB_PRECISION_3XTF32;
  size_t bytes = sizeof(float) * (size_t)vlb::ceil_div(N, BN) * BN * (size_t)numKb * 32 * (split3 ? 2 : 1);
  return (bytes + 255) & ~(size_t)255;
}

// `extraBytes` of scratch are reserved behind the tiles for the caller (split-K partials).
float const* prep_b_tiles(vlb_ctx* ctx, float const* f, int N, int R, int BN, int numKb, int mode, vlb::ConvGeom const& g,
                          size_t extraBytes = 0, int P = 0)
{
  bool split3 = ctx->precision == VLB_PRECISION_3XTF32;
  size_t total = (size_t)vlb::ceil_div(N, BN) * BN * (size_t)numKb * 32;
  float* tiles = (float*)vlb::workspace(ctx, b_tiles_bytes(ctx, N, BN, numKb) + extraBytes);
  if (!tiles) return nullptr;
  if (mode == 2) {
    unsigned grid2 = vlb::grid_for(total, 256, ctx->smCount * 16);
    if (split3) prep_b_tiles_kernel<true><<<grid2, 256, 0, ctx->stream>>>(tiles, f, N, R, BN, numKb, 2, P, 0, 0, 0);
    else        prep_b_tiles_kernel<false><<<grid2, 256, 0, ctx->stream>>>(tiles, f, N, R, BN, numKb, 2, P, 0, 0, 0);
    VLB_LAUNCHED(ctx, 1);
    return tiles;
  }
  unsigned grid = vlb::grid_for(total, 256, ctx->smCount * 8);
  if (split3) prep_b_tiles_kernel<true><<<grid, 256, 0, ctx->stream>>>(tiles, f, N, R, BN, numKb, mode, g.FH, g.FW, g.C, g.K);
  else        prep_b_tiles_kernel<false><<<grid, 256, 0, ctx->stream>>>(tiles, f, N, R, BN, numKb, mode, g.FH, g.FW, g.C, g.K);
  VLB_LAUNCHED(ctx, 1);
  return tiles;
}

// dY tile images with 16-byte accesses and, when db is given, the bias gradient from the same sweep.
// Scratch layout: [tiles][extraBytes for the caller][per-block partial sums of db].
float const* prep_dy_tiles(vlb_ctx* ctx, float const* dY, int K, int R, int P, int BN, int numKb, size_t extraBytes, float* db, int Pp = 0)
{
  if (Pp == 0) Pp = P;
  bool split3 = ctx->precision == VLB_PRECISION_3XTF32;
  size_t const tileBytes = b_tiles_bytes(ctx, K, BN, numKb);
  int const perBlock = kPrepThreads * 4 * kPrepIters;
  unsigned const bx = (unsigned)vlb::ceil_div((long long)numKb * 32, perBlock);
  size_t const partBytes = db ? sizeof(float) * (size_t)K * bx : 0;
  extraBytes = (extraBytes + 255) & ~(size_t)255;
  char* ws = (char*)vlb::workspace(ctx, tileBytes + extraBytes + partBytes);
  if (!ws) return nullptr;
  float* tiles = (float*)ws;
  float* dbPart = db ? (float*)(ws + tileBytes + extraBytes) : nullptr;
  unsigned* tickets = (unsigned*)((char*)ctx->deviceStatus + 256);
  dim3 grid(bx, (unsigned)(vlb::ceil_div(K, BN) * BN));
  if (split3) prep_dy_tiles_kernel<true><<<grid, kPrepThreads, 0, ctx->stream>>>(tiles, dY, K, R, P, Pp, BN, numKb, db, dbPart, tickets);
  else        prep_dy_tiles_kernel<false><<<grid, kPrepThreads, 0, ctx->stream>>>(tiles, dY, K, R, P, Pp, BN, numKb, db, dbPart, tickets);
  VLB_LAUNCHED(ctx, 1);
  return tiles;
}

// ------------------------------------------------------------------ host side
int pick_bn(int N) { return N > 64 ? 128 : (N > 32 ? 64 : (N > 16 ? 32 : 16)); }

bool aligned16(void const* p) { return (((uintptr_t)p) & 15) == 0; }

// Registers per thread a kernel must have been compiled with (0: no requirement).
template <auto kKernel> constexpr int kRegsAtLaunch() { return 0; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<true, 0, true>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<true, 0, false>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<true, 1, true>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<true, 1, false>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<false, 0, true>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<false, 0, false>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<false, 1, true>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<false, 1, false>>() { return 128; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<true, 2, false>>() { return 96; }
template <> constexpr int kRegsAtLaunch<conv_ts_kernel<false, 2, false>>() { return 96; }

// The opt-in to more than 48 KB of dynamic shared memory, once per kernel and device instead of before every launch.
template <auto kKernel>
cudaError_t allow_large_smem(int device)
{
  static bool done[64] = {};
  if (device >= 0 && device < 64 && done[device]) return cudaSuccess;
  cudaError_t e = vlb::allow_max_dynamic_smem(kKernel);
  if (e == cudaSuccess && kRegsAtLaunch<kKernel>() > 0) {
    // conv_ts_kernel redistributes registers between its warps (setmaxnreg) on the premise that every thread starts with
    // exactly this many; a build that gave it another count must not run (the hand-over would wait for registers for ever)
    cudaFuncAttributes attr;
    e = cudaFuncGetAttributes(&attr, kKernel);
    if (e == cudaSuccess && attr.numRegs != kRegsAtLaunch<kKernel>()) e = cudaErrorInvalidDeviceFunction;
  }
  if (e == cudaSuccess && device >= 0 && device < 64) done[device] = true;
  return e;
}

template <int kAMode, int kBMode, int kEpi>
int launch(vlb_ctx* ctx, Params& p, int splits, char const* where)
{
  bool split3 = ctx->precision == VLB_PRECISION_3XTF32;
  uint32_t stageBytes = (split3 ? 2u : 1u) * (BM * BK * 4 + (uint32_t)p.BN * BK * 4);
  int stages = (int)((200u * 1024u) / stageBytes);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > 6) stages = 6;
  p.stages = stages;
  p.status = ctx->deviceStatus;
  p.drainEvery = kDrainEvery;
  size_t smemBytes = (size_t)stages * stageBytes + 1024;
  dim3 grid(vlb::ceil_div(p.M, BM), vlb::ceil_div(p.N, p.BN), splits);
  if (grid.y > 65535u || grid.z > 65535u) return VLB_Unsupported;
  cudaError_t e;
  vlb_ctx::ProfRec rec;
  bool const record = ctx->profiling && ctx->profDepth == 0;
  if (record) {
    cudaEventCreate(&rec.start); cudaEventCreate(&rec.stop);
    rec.flops = 2.0 * (double)p.M * (double)p.N * (double)p.R; rec.kind = -1;
    cudaEventRecord(rec.start, ctx->stream);
  }
  if (split3) {
    e = allow_large_smem<tc_gemm_kernel<kAMode, kBMode, kEpi, true>>(ctx->device);
    if (e == cudaSuccess) tc_gemm_kernel<kAMode, kBMode, kEpi, true><<<grid, kThreads, smemBytes, ctx->stream>>>(p);
  } else {
    e = allow_large_smem<tc_gemm_kernel<kAMode, kBMode, kEpi, false>>(ctx->device);
    if (e == cudaSuccess) tc_gemm_kernel<kAMode, kBMode, kEpi, false><<<grid, kThreads, smemBytes, ctx->stream>>>(p);
  }
  if (record) { cudaEventRecord(rec.stop, ctx->stream); ctx->prof.push_back(rec); }
  if (e != cudaSuccess) { cudaGetLastError(); return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e)); }
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, where);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point query (the library does not link libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, cuuint64_t const*, cuuint64_t const*,
                                  cuuint32_t const*, cuuint32_t const*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled()
{
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)f;
    else
      cudaGetLastError();
  }
  return fn;
}

// Decides whether conv_ts_kernel can take its input windows from tensor-map copies and, if so, fills the box geometry in p,
// the tensor map and the shared-memory size.  Needs: reduction in blocks of 32 channels, unit stride, input rows a multiple
// of four elements (every global stride of a tensor map is a multiple of 16 bytes) on a 16-byte aligned base, an output
// map that boxes of bh x bw <= 128 pixels (bh a multiple of four, so that every box's window starts on a 16-byte boundary)
// cover with at least 95% of the tile rows in use (measured: with 112 of 128 rows in use, as on 56 x 56 and 28 x 28 maps,
// the per-thread gather is the faster route by 10-15%; on 224 x 224 and 112 x 112 maps the copies win by up to 20% on
// 64-column tiles and draw level on 128-column tiles), and room in shared memory for two windows.
// Shared memory of conv_ts_kernel for the running sum of a tile: a patch of 32 columns for the tile widths whose sum lives in registers.
size_t p_bytes(int BN, int smemSum) { return sizeof(float) * (size_t)(((BN == 128 || BN == 64) && !smemSum) ? 32 : BN) * BM; }

bool plan_windows(vlb_ctx* ctx, Params& p, CUtensorMap* map, size_t* smemBytes, bool split3)
{
  Operand const& a = p.a;
  if (ctx->testSwitch & 2) return false;
  if (!p.chanFast || a.sy != 1 || a.sx != 1 || a.H % 4 != 0 || !aligned16(a.ptr)) return false;
  if (p.splits > 1 && p.kbPerSplit % (a.FH * a.FW) != 0) return false;      // a range of the reduction must be whole channel blocks
  EncodeTiledFn const encode = encode_tiled();
  if (!encode) return false;
  int const Ho = a.Ho, Wo = a.Wo;
  int bestBh = 0, bestBw = 0;
  double bestUtil = 0.0;
  for (int bh = 4; bh <= 128 && bh < Ho + 4; bh += 4) {
    int const bw = std::min(128 / bh, Wo);
    // share of the 128 tile rows that are output pixels, over all boxes of an image
    double const util = (double)Ho * Wo / ((double)vlb::ceil_div(Ho, bh) * (double)vlb::ceil_div(Wo, bw) * 128.0);
    if (util >= bestUtil - 1e-9) { bestUtil = util; bestBh = bh; bestBw = bw; }      // on a tie the taller box: longer contiguous runs
  }
  if (bestBh == 0 || bestUtil < 0.95) return false;
  int const rowOff = (4 - a.pt % 4) % 4;
  int const boxH = (rowOff + bestBh + (a.FH - 1) * a.dy + 3) / 4 * 4, boxW = bestBw + (a.FW - 1) * a.dx;
  if (boxH > 256 || boxW > 256) return false;
  size_t const xTileBytes = (size_t)boxH * boxW * 32 * 4;
  size_t const bBytes = (size_t)(split3 ? 2 : 1) * p.BN * BK * 4, pBytes = p_bytes(p.BN, p.smemSum);
  size_t const limit = 227 * 1024 - 1536;      // what one block may have, less the kernel's static shared memory
  // window buffers: two where a window serves a whole channel block of several taps; four for 1 x 1 filters, whose windows are
  // single k-blocks and must be on their way well before their turn.  Filter-tile stages: what is left, at least three.
  int const nX = a.FH * a.FW == 1 ? 4 : 2;
  int nB = 0;
  for (int n = kTsBStages; n >= 3 && !nB; --n)
    if ((size_t)n * bBytes + pBytes + nX * xTileBytes + 1024 <= limit) nB = n;
  if (!nB) return false;
  long long const images = (long long)p.M / ((long long)Ho * Wo);
  cuuint64_t const dims[4] = {(cuuint64_t)a.H, (cuuint64_t)a.W, (cuuint64_t)a.C, (cuuint64_t)images};
  cuuint64_t const strides[3] = {(cuuint64_t)a.H * 4, (cuuint64_t)a.H * a.W * 4, (cuuint64_t)a.imgStride * 4};
  cuuint32_t const box[4] = {(cuuint32_t)boxH, (cuuint32_t)boxW, 32u, 1u};
  cuuint32_t const estr[4] = {1u, 1u, 1u, 1u};
  CUresult const r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(a.ptr), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  p.tma = 1; p.bh = bestBh; p.bw = bestBw; p.tilesH = vlb::ceil_div(Ho, bestBh); p.tilesW = vlb::ceil_div(Wo, bestBw);
  p.boxH = boxH; p.boxW = boxW; p.rowOff = rowOff; p.bStages = nB; p.xStages = nX;
  p.tilesM = (int)(images * p.tilesH * p.tilesW);
  *smemBytes = (size_t)nB * bBytes + pBytes + nX * xTileBytes + 1024;
  return true;
}

// fprop / stride-1 dgrad with the gathered operand in tensor memory (p.bTiles set, p.a a convolution operand).
int launch_ts(vlb_ctx* ctx, Params& p, char const* where)
{
  bool split3 = ctx->precision == VLB_PRECISION_3XTF32;
  p.status = ctx->deviceStatus;
  p.testSwitch = ctx->testSwitch;
  // at least 120 KB, so that two CTAs (each allocating all 512 TMEM columns) never share an SM
  // filter-tile stages: as many as fit beside the running sum's patch, six at most
  if (p.splits < 1) { p.splits = 1; p.kbPerSplit = p.numKb; }
  p.smemSum = ((ctx->testSwitch & 8) || p.kbPerSplit < 8) ? 1 : 0;
  size_t const stageBytes = (split3 ? 2u : 1u) * (size_t)p.BN * BK * 4, sumBytes = p_bytes(p.BN, p.smemSum);
  p.bStages = (int)std::min<size_t>(kTsBStages, (227 * 1024 - 1536 - 1024 - sumBytes) / stageBytes);
  size_t smemBytes = (size_t)p.bStages * stageBytes + sumBytes + 1024;
  p.tilesM = vlb::ceil_div(p.M, BM); p.tilesN = vlb::ceil_div(p.N, p.BN);
  p.kbTot = p.splits * p.kbPerSplit;       // what the tile images hold per column tile
  CUtensorMap map;
  memset(&map, 0, sizeof(map));
  bool const windows = plan_windows(ctx, p, &map, &smemBytes, split3);
  if (smemBytes < 120u * 1024u) smemBytes = 120u * 1024u;
  long long const numTiles = (long long)p.tilesM * p.tilesN * p.splits;
  if (numTiles >= (1LL << 31)) return VLB_Unsupported;
  // Persistent: one CTA per SM walks the tiles, so that the pipeline never drains between tiles and a tile is stored
  // while the next one is computed.  With fewer tiles than SMs every CTA has one tile and all its warps share the stores.
  bool const persistent = true;
  dim3 grid((unsigned)(persistent && numTiles > ctx->smCount ? ctx->smCount : numTiles), 1, 1);
  cudaError_t e;
  vlb_ctx::ProfRec rec;
  bool const record = ctx->profiling && ctx->profDepth == 0;
  if (record) {
    cudaEventCreate(&rec.start); cudaEventCreate(&rec.stop);
    rec.flops = 2.0 * (double)p.M * (double)p.N * (double)p.R; rec.kind = -1;
    cudaEventRecord(rec.start, ctx->stream);
  }
  bool const narrow = p.BN <= 64;
  auto go = [&](auto kernel) {
    e = allow_large_smem<decltype(kernel)::value>(ctx->device);
    if (e == cudaSuccess) decltype(kernel)::value<<<grid, kTsThreads, smemBytes, ctx->stream>>>(p, map);
  };
#define VLB_TS(split, mode, nar) go(std::integral_constant<decltype(&conv_ts_kernel<split, mode, nar>), &conv_ts_kernel<split, mode, nar>>{})
  if (split3) {
    if (windows) { if (narrow) VLB_TS(true, 1, true); else VLB_TS(true, 1, false); }
    else         { if (narrow) VLB_TS(true, 0, true); else VLB_TS(true, 0, false); }
  } else {
    if (windows) { if (narrow) VLB_TS(false, 1, true); else VLB_TS(false, 1, false); }
    else         { if (narrow) VLB_TS(false, 0, true); else VLB_TS(false, 0, false); }
  }
#undef VLB_TS
  if (record) { cudaEventRecord(rec.stop, ctx->stream); ctx->prof.push_back(rec); }
  if (e != cudaSuccess) { cudaGetLastError(); return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e)); }
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, where);
}

// Splits of the reduction so that the grid fills the machine; each split gets whole k-blocks.
int pick_splits(vlb_ctx* ctx, int tiles, int numKb, int minKbPerSplit)
{
  int target = 2 * ctx->smCount;
  if (tiles >= target || numKb < 2 * minKbPerSplit) return 1;
  int s = target / tiles;           // tiles * s <= two full waves
  int maxS = numKb / minKbPerSplit;
  if (s > maxS) s = maxS;
  if (s > 512) s = 512;
  return s < 1 ? 1 : s;
}

// The cut of a filter gradient's reduction (numKb k-blocks, `tiles` output tiles) into ranges: the work items -- tiles x
// ranges -- should fill whole waves of the persistent CTAs, with ranges long enough that a tile's fixed cost stays small.
int pick_wg_splits(int smCount, int tiles, int numKb, int* kbPerSplit, int minKb = 48)
{
  int best = 1; double bestEff = 0.0;
  for (int w = 1; w <= 6; ++w) {
    int s = std::max(1, (w * smCount) / tiles);
    s = std::min(s, std::max(1, numKb / minKb));
    int const per = vlb::ceil_div(numKb, s);
    s = vlb::ceil_div(numKb, per);
    long long const items = (long long)tiles * s;
    long long const perCta = (items + smCount - 1) / smCount;          // items of the busiest CTA
    // useful k-blocks per SM over the k-block slots the busiest CTA spends, a dozen k-blocks' worth of fixed cost per item
    double const eff = ((double)tiles * numKb / smCount) / ((double)perCta * (per + 12));
    if (eff > bestEff * 1.01) { bestEff = eff; best = s; }
  }
  *kbPerSplit = vlb::ceil_div(numKb, best);
  return vlb::ceil_div(numKb, *kbPerSplit);
}

void conv_operand(Operand& o, ConvGeom const& g, float const* ptr, int channels)
{
  o.ptr = ptr;
  o.H = g.H; o.W = g.W; o.C = channels; o.FH = g.FH; o.FW = g.FW; o.Ho = g.Ho; o.Wo = g.Wo;
  o.sy = g.sy; o.sx = g.sx; o.pt = g.pt; o.pl = g.pl; o.dy = g.dy; o.dx = g.dx;
  o.imgStride = (long long)g.H * g.W * channels;
  o.ld = 0; o.bs = 0; o.P = 0; o.vec = 0;
  // 1: aligned windows (stride 1, extents multiples of 4); 2: element-wise gather, any geometry; 0: no pipelined path
  bool const lut = g.FH <= 32 && g.FW <= 32 && g.FH * g.FW <= 64;
  o.fast = !lut ? 0 : ((g.sy == 1 && g.sx == 1 && g.H % 4 == 0 && g.Ho % 4 == 0 && aligned16(ptr)) ? 1 : 2);
}

bool fits32(ConvGeom const& g)
{
  long long in = (long long)g.H * g.W * g.C * g.N, out = (long long)g.Ho * g.Wo * g.K * g.N;
  return in < (1LL << 31) - 256 && out < (1LL << 31) - 256 && (long long)g.FH * g.FW * g.FC * g.K < (1LL << 31);
}

// conv_ts_kernel in its row mode (kMode 2): rows whose reduction index is contiguous in memory, delivered by the 3-D tensor map `map`
// (run of 36 elements x cPer rows x 1).  p holds the tiling (cPer, tapsPerTile, tapGroups, tilesM, tilesN, splits, kbPerSplit,
// kbTot), the operand geometry, the tile images and the epilogue.
int launch_rows(vlb_ctx* ctx, Params& p, CUtensorMap const& map, char const* where)
{
  bool const split3 = ctx->precision == VLB_PRECISION_3XTF32;
  // shared memory: filter-tile stages, the running sum, the runs
  p.smemSum = ((ctx->testSwitch & 8) || p.kbPerSplit < 8) ? 1 : 0;
  size_t const bBytes = (size_t)(split3 ? 2 : 1) * p.BN * BK * 4, pBytes = p_bytes(p.BN, p.smemSum);
  size_t const limit = 227 * 1024 - 1536;
  p.bStages = 0;
  for (int nb = kTsBStages; nb >= 3 && !p.bStages; --nb)
    for (int nx = kTsXStages; nx >= 3 && !p.bStages; --nx)
      if ((size_t)nb * bBytes + pBytes + (size_t)nx * kWgStageBytes + 1024 <= limit) { p.bStages = nb; p.xStages = nx; }
  if (!p.bStages) return vlb::set_error(ctx, VLB_Unsupported, where);
  size_t smemBytes = (size_t)p.bStages * bBytes + pBytes + (size_t)p.xStages * kWgStageBytes + 1024;
  if (smemBytes < 120u * 1024u) smemBytes = 120u * 1024u;      // two CTAs (each allocating all 512 TMEM columns) never share an SM
  p.wg = 1;
  p.status = ctx->deviceStatus;
  p.testSwitch = ctx->testSwitch;
  p.chanFast = 1;
  long long const numTiles = (long long)p.tilesM * p.tilesN * p.splits;
  if (numTiles >= (1LL << 31)) return VLB_Unsupported;
  dim3 grid((unsigned)std::min<long long>(numTiles, ctx->smCount), 1, 1);
  cudaError_t e;
  if (split3) {
    e = allow_large_smem<conv_ts_kernel<true, 2, false>>(ctx->device);
    if (e == cudaSuccess) conv_ts_kernel<true, 2, false><<<grid, kTsThreadsRows, smemBytes, ctx->stream>>>(p, map);
  } else {
    e = allow_large_smem<conv_ts_kernel<false, 2, false>>(ctx->device);
    if (e == cudaSuccess) conv_ts_kernel<false, 2, false><<<grid, kTsThreadsRows, smemBytes, ctx->stream>>>(p, map);
  }
  if (e != cudaSuccess) { cudaGetLastError(); return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e)); }
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, where);
}

// The 3-D tensor map (run, rows, planes) of launch_rows; false when the driver refuses it.
bool rows_map(CUtensorMap* map, float const* ptr, long long run, long long rows, long long planes, int cPer)
{
  EncodeTiledFn const encode = encode_tiled();
  if (!encode) return false;
  memset(map, 0, sizeof(*map));
  cuuint64_t const dims[3] = {(cuuint64_t)run, (cuuint64_t)rows, (cuuint64_t)planes};
  cuuint64_t const strides[2] = {(cuuint64_t)run * 4, (cuuint64_t)run * rows * 4};
  cuuint32_t const box[3] = {(cuuint32_t)kWgRowWords, (cuuint32_t)cPer, 1u};
  cuuint32_t const estr[3] = {1u, 1u, 1u};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Filter gradient of a stride-1 convolution whose output has the input's height (every VGG / ResNet 3x3 layer), through
// conv_ts_kernel: rows (tap, channel) in tensor memory, dY as tile images.  Returns -1 when the layer is not eligible (the
// caller then takes tc_gemm_kernel), else an error code.
//   needs: Ho == H (a tap is then a constant shift of the flattened plane), planes of a multiple of four pixels (the 16-byte
//   strides the tensor map wants) that whole k-blocks cover with at most 1/8 to spare, channels in blocks of 32.
int conv_wgrad_ts(vlb_ctx* ctx, ConvGeom const& g, float* dF, float* db, float const* X, float const* dY, bool* dbDone)
{
  int const taps = g.FH * g.FW, P = g.Ho * g.Wo, HW = g.H * g.W;
  if (ctx->testSwitch & 4) return -1;
  int const Pp = (P + BK - 1) / BK * BK;             // planes are padded to whole k-blocks (at most 1/8 more work: 14 x 14 planes still gain 3% over the other kernel), so that no k-block straddles two images
  if (g.sy != 1 || g.sx != 1 || g.Ho != g.H || P % 4 != 0 || (Pp - P) * 8 > Pp || HW % 4 != 0 || taps > 64 || g.FH > 32 || g.FW > 32) return -1;
  if (g.C % 32 != 0 || (g.C > 128 && g.C % 128 != 0) || (g.C < 128 && 128 % g.C != 0)) return -1;
  if (g.K > 4096 || !aligned16(X) || !aligned16(dY)) return -1;
  if ((g.FH - 1) * g.dy - g.pt >= g.H || g.pt >= g.H) return -1;
  int const V = taps * g.C;
  long long const R = (long long)P * g.N;
  Params p = {};
  p.cPer = std::min(g.C, 128); p.tapsPerTile = 128 / p.cPer; p.tapGroups = vlb::ceil_div(taps, p.tapsPerTile);
  p.M = V; p.N = g.K; p.R = (int)R;
  p.BN = pick_bn(p.N);
  p.tilesM = p.tapGroups * (g.C / p.cPer); p.tilesN = vlb::ceil_div(p.N, p.BN);
  if (vlb::ceil_div(g.K, p.BN) * p.BN > 65535) return -1;
  if ((long long)Pp * g.N >= (1LL << 31) - 4096) return -1;
  int const numKb = (int)((long long)Pp * g.N / BK);
  p.plane = Pp;
  p.splits = pick_wg_splits(ctx->smCount, p.tilesM * p.tilesN, numKb, &p.kbPerSplit);
  p.kbTot = p.splits * p.kbPerSplit;               // the tile images are padded with zeros to whole ranges
  p.numKb = p.kbTot;
  conv_operand(p.a, g, X, g.C);
  p.a.rows = V;
  size_t const nF = (size_t)V * g.K;
  if ((long long)nF * p.splits >= (1LL << 31)) return -1;
  size_t const partBytes = p.splits > 1 ? ((sizeof(float) * nF * p.splits + 255) & ~(size_t)255) : 0;
  size_t const tileBytes = b_tiles_bytes(ctx, g.K, p.BN, p.kbTot);
  CUtensorMap map;
  if (!rows_map(&map, X, HW, g.C, g.N, p.cPer)) return -1;

  ProfScope prof(ctx, kProfWgrad);      // includes the dY tile images (with the bias gradient) and the sum of the partial results
  prof.rec.flops = 2.0 * (double)V * (double)g.K * (double)R;
  p.bTiles = prep_dy_tiles(ctx, dY, g.K, (int)R, P, p.BN, p.kbTot, partBytes, db, Pp);
  if (!p.bTiles) return ctx->lastError;
  *dbDone = db != nullptr;
  float* const part = p.splits > 1 ? (float*)((char*)p.bTiles + tileBytes) : nullptr;
  p.e = Epilogue{};
  p.e.out = part ? part : dF; p.e.splitStride = part ? (long long)nF : 0; p.e.inMult = 1.f; p.e.P = V; p.e.Ktot = g.K;
  int const rc = launch_rows(ctx, p, map, "conv_wgrad_ts");
  if (rc) return rc;
  if (part) {
    tc_splitk_reduce_kernel<<<vlb::grid_for(nF, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(dF, part, nF, nF, p.splits);
    VLB_LAUNCHED(ctx, 1);
  }
  return vlb::check_launch(ctx, "conv_wgrad_ts");
}

// The geometry of a 1 x 1 convolution over a "plane" of `pixels` elements with `channels` channels (channel stride = pixels).
ConvGeom plane_geom(int pixels, int channels, int filters)
{
  ConvGeom t = {};
  t.H = pixels; t.W = 1; t.C = channels; t.N = 1; t.FH = 1; t.FW = 1; t.FC = channels; t.K = filters; t.Ho = pixels; t.Wo = 1;
  t.sy = 1; t.sx = 1; t.dy = 1; t.dx = 1; t.G = 1;
  return t;
}

// Fully connected layers at small batch are bound by the one pass over the weights (fc6 of VGG-16: 411 MB against 13 GFLOP at
// batch 64).  All three passes run through conv_ts_kernel, whose A operand goes from global memory to tensor memory without a
// shared-memory tile of its own, each with the weights (or their gradient) as the operand that is read or written exactly once:
//   forward   Y(K x N) = F'(K x V) X(V x N): rows = filters, the reduction index v is contiguous in a row -> row mode, X as tile images;
//   data      dX(V x N) = F(V x K) dY(K x N): a 1 x 1 convolution over the "plane" of V elements with K channels, dY as its N filters;
//   weights   dF(V x K) = X(V x N) dY'(N x K): a 1 x 1 convolution over the plane X (N channels) with the K rows of dY as filters.
// Each returns -1 when the shape is not eligible (the caller then takes tc_gemm_kernel).
int fc_fprop_ts(vlb_ctx* ctx, ConvGeom const& g, float* Y, float const* X, float const* F, float const* b)
{
  int const V = g.FH * g.FW * g.FC;
  if ((ctx->testSwitch & 4) || V % 32 != 0 || V < 128 * 64 || g.K % 128 != 0 || g.N > 4096 || !aligned16(X) || !aligned16(F)) return -1;
  Params p = {};
  p.cPer = 128; p.tapsPerTile = 1; p.tapGroups = 1;
  p.M = g.K; p.N = g.N; p.R = V;
  p.BN = pick_bn(p.N);
  p.tilesM = g.K / 128; p.tilesN = vlb::ceil_div(p.N, p.BN);
  p.splits = pick_wg_splits(ctx->smCount, p.tilesM * p.tilesN, V / BK, &p.kbPerSplit);
  p.kbTot = p.splits * p.kbPerSplit; p.numKb = p.kbTot;
  p.plane = V;
  conv_operand(p.a, plane_geom(V, g.K, g.N), F, g.K);
  p.a.rows = g.K;
  size_t const nOut = (size_t)g.K * g.N;
  size_t const partBytes = p.splits > 1 ? ((sizeof(float) * nOut * p.splits + 255) & ~(size_t)255) : 0;
  CUtensorMap map;
  if (!rows_map(&map, F, V, g.K, 1, 128)) return -1;
  ProfScope prof(ctx, kProfFc);
  prof.rec.flops = 2.0 * (double)g.K * (double)g.N * (double)V;
  p.bTiles = prep_dy_tiles(ctx, X, g.N, V, V, p.BN, p.kbTot, partBytes, nullptr);      // B(n, v) = X[v + V n]
  if (!p.bTiles) return ctx->lastError;
  float* const part = p.splits > 1 ? (float*)((char*)p.bTiles + b_tiles_bytes(ctx, g.N, p.BN, p.kbTot)) : nullptr;
  p.e = Epilogue{};
  p.e.out = part ? part : Y; p.e.splitStride = part ? (long long)nOut : 0; p.e.inMult = 1.f; p.e.P = g.K; p.e.Ktot = g.N;
  int rc = launch_rows(ctx, p, map, "fc_fprop_ts");
  if (rc) return rc;
  if (part) {
    tc_splitk_reduce_kernel<<<vlb::grid_for(nOut, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(Y, part, nOut, nOut, p.splits);
    VLB_LAUNCHED(ctx, 1);
  }
  if (b) return vlb_bias_forward(ctx, Y, 1.0, nullptr, 0.0, b, 1.0, 1, 1, g.K, g.N);
  return vlb::check_launch(ctx, "fc_fprop_ts");
}

int fc_dgrad_ts(vlb_ctx* ctx, ConvGeom const& g, float* dX, float const* F, float const* dY)
{
  int const V = g.FH * g.FW * g.FC;
  if ((ctx->testSwitch & 4) || V % 4 != 0 || g.K % 32 != 0 || !aligned16(F) || !aligned16(dY) || V < 128 * 16) return -1;
  Params p = {};
  p.M = V; p.N = g.N; p.R = g.K;
  ConvGeom const t = plane_geom(V, g.K, g.N);
  conv_operand(p.a, t, F, g.K);
  p.a.rows = V;
  p.BN = pick_bn(p.N);
  int const numKb = vlb::ceil_div(g.K, BK);
  p.splits = pick_wg_splits(ctx->smCount, vlb::ceil_div(V, BM) * vlb::ceil_div(p.N, p.BN), numKb, &p.kbPerSplit, 16);
  p.numKb = p.splits * p.kbPerSplit;
  p.chanFast = 1; p.pipelined = 1;
  size_t const nOut = (size_t)V * g.N;
  size_t const partBytes = p.splits > 1 ? sizeof(float) * nOut * p.splits : 0;
  ProfScope prof(ctx, kProfFc);
  prof.rec.flops = 2.0 * (double)V * (double)g.N * (double)g.K;
  p.bTiles = prep_b_tiles(ctx, dY, g.N, g.K, p.BN, p.numKb, 0, t, partBytes);            // B(n, k) = dY[k + K n]
  if (!p.bTiles) return ctx->lastError;
  float* const part = p.splits > 1 ? (float*)((char*)p.bTiles + b_tiles_bytes(ctx, g.N, p.BN, p.numKb)) : nullptr;
  p.e = Epilogue{};
  p.e.out = part ? part : dX; p.e.splitStride = part ? (long long)nOut : 0; p.e.inMult = 1.f; p.e.P = V; p.e.Ktot = g.N;
  int rc = launch_ts(ctx, p, "fc_dgrad_ts");
  if (rc || !part) return rc;
  tc_splitk_reduce_kernel<<<vlb::grid_for(nOut, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(dX, part, nOut, nOut, p.splits);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "fc_dgrad_ts");
}

int fc_wgrad_ts(vlb_ctx* ctx, ConvGeom const& g, float* dF, float const* X, float const* dY)
{
  int const V = g.FH * g.FW * g.FC;
  if ((ctx->testSwitch & 4) || V % 4 != 0 || g.N % 32 != 0 || !aligned16(X) || !aligned16(dY) || V < 128 * 64) return -1;
  Params p = {};
  p.M = V; p.N = g.K; p.R = g.N;
  ConvGeom const t = plane_geom(V, g.N, g.K);
  conv_operand(p.a, t, X, g.N);
  p.a.rows = V;
  p.BN = pick_bn(p.N);
  p.numKb = vlb::ceil_div(g.N, BK); p.kbPerSplit = p.numKb; p.splits = 1;
  p.chanFast = 1; p.pipelined = 1;
  ProfScope prof(ctx, kProfFc);
  prof.rec.flops = 2.0 * (double)V * (double)g.K * (double)g.N;
  p.bTiles = prep_b_tiles(ctx, dY, g.K, g.N, p.BN, p.numKb, 5, t);                       // B(k, n) = dY[k + K n]
  if (!p.bTiles) return ctx->lastError;
  p.e = Epilogue{};
  p.e.out = dF; p.e.inMult = 1.f; p.e.P = V; p.e.Ktot = g.K;
  return launch_ts(ctx, p, "fc_wgrad_ts");
}

bool is_fc(ConvGeom const& g)
{
  return g.Ho == 1 && g.Wo == 1 && g.FH == g.H && g.FW == g.W && g.FC == g.C && g.sy == 1 && g.sx == 1 && g.pt == 0 &&
         g.pb == 0 && g.pl == 0 && g.pr == 0 && g.dy == 1 && g.dx == 1;
}

}  // namespace

namespace vlb {

int conv_fprop_tc(vlb_ctx* ctx, ConvGeom const& g, float* Y, float outMult, float const* X, float inMult,
                  float const* F, float const* b)
{
  if (g.G != 1 || !fits32(g)) return VLB_Unsupported;
  int const V = g.FH * g.FW * g.FC;
  Params p = {};
  if (is_fc(g)) {
    // Y(K x N) = F'(K x V) X(V x N) + b 1'  (reference bits/nnfullyconnected.cu:45-70): rows = filters
    if (outMult != 0.f || inMult != 1.f) return VLB_Unsupported;
    {
      int const rc = fc_fprop_ts(ctx, g, Y, X, F, b);
      if (rc >= 0) return rc;
    }
    ProfScope prof(ctx, kProfFc);
    prof.rec.flops = 2.0 * (double)g.K * (double)g.N * (double)V;
    p.M = g.K; p.N = g.N; p.R = V;
    p.a = Operand{}; p.a.ptr = F; p.a.ld = V; p.a.rows = g.K; p.a.vec = (V % 4 == 0) && aligned16(F);
    p.b = Operand{}; p.b.ptr = X; p.b.ld = V; p.b.rows = g.N; p.b.vec = (V % 4 == 0) && aligned16(X);
    p.BN = pick_bn(p.N);
    p.numKb = ceil_div(p.R, BK);
    int tiles = ceil_div(p.M, BM) * ceil_div(p.N, p.BN);
    int splits = pick_splits(ctx, tiles, p.numKb, 8);
    p.kbPerSplit = ceil_div(p.numKb, splits);
    splits = ceil_div(p.numKb, p.kbPerSplit);
    p.e = Epilogue{}; p.e.ldd = g.K;
    if (splits == 1) {
      p.e.out = Y; p.e.bias = b;
      p.e.relu = ctx->fuseRelu; ctx->reluDone = ctx->fuseRelu;
      return launch<OP_DENSE_K, OP_DENSE_K, EPI_PLAIN>(ctx, p, 1, "fc_fprop_tc");
    }
    size_t nOut = (size_t)g.K * g.N;
    float* part = (float*)workspace(ctx, sizeof(float) * nOut * splits);
    if (!part) return ctx->lastError;
    p.e.out = part; p.e.splitStride = (long long)nOut;
    int rc = launch<OP_DENSE_K, OP_DENSE_K, EPI_PLAIN>(ctx, p, splits, "fc_fprop_tc");
    if (rc) return rc;
    tc_splitk_reduce_kernel<<<grid_for(nOut, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(Y, part, nOut, nOut, splits);
    VLB_LAUNCHED(ctx, 1);
    if (b) return vlb_bias_forward(ctx, Y, 1.0, nullptr, 0.0, b, 1.0, 1, 1, g.K, g.N);
    return check_launch(ctx, "fc_fprop_tc");
  }
  long long M = (long long)g.Ho * g.Wo * g.N;
  ProfScope prof(ctx, kProfFprop);
  prof.rec.flops = 2.0 * (double)M * (double)g.K * (double)V;
  p.M = (int)M; p.N = g.K; p.R = V;
  conv_operand(p.a, g, X, g.C);
  p.a.rows = p.M;
  p.b = Operand{}; p.b.ptr = F; p.b.ld = V; p.b.rows = g.K; p.b.vec = (V % 4 == 0) && aligned16(F);
  p.BN = pick_bn(p.N);
  p.numKb = ceil_div(p.R, BK); p.kbPerSplit = p.numKb;
  p.e = Epilogue{}; p.e.out = Y; p.e.bias = b; p.e.inMult = inMult; p.e.outMult = outMult; p.e.P = g.Ho * g.Wo; p.e.Ktot = g.K;
  p.e.relu = ctx->fuseRelu; ctx->reluDone = ctx->fuseRelu;
  if (p.a.fast) {
    p.chanFast = g.C % 32 == 0;
    p.bTiles = prep_b_tiles(ctx, F, g.K, V, p.BN, p.numKb, p.chanFast ? 3 : 0, g);
    if (!p.bTiles) return ctx->lastError;
    p.pipelined = 1;
    return launch_ts(ctx, p, "conv_fprop_ts");
  }
  return launch<OP_IM2COL, OP_DENSE_K, EPI_CONV>(ctx, p, 1, "conv_fprop_tc");
}

int conv_dgrad_tc(vlb_ctx* ctx, ConvGeom const& g, float* dX, float const* F, float const* dY)
{
  if (g.G != 1 || !fits32(g)) return VLB_Unsupported;
  Params p = {};
  if (is_fc(g)) {
    // dX(V x N) = F(V x K) dY(K x N)  (reference bits/nnfullyconnected.cu:139-151): rows = input elements
    int const V = g.FH * g.FW * g.FC;
    {
      int const rc = fc_dgrad_ts(ctx, g, dX, F, dY);
      if (rc >= 0) return rc;
    }
    ProfScope prof(ctx, kProfFc);
    prof.rec.flops = 2.0 * (double)V * (double)g.N * (double)g.K;
    p.M = V; p.N = g.N; p.R = g.K;
    p.a = Operand{}; p.a.ptr = F; p.a.ld = V; p.a.rows = V; p.a.vec = (V % 4 == 0) && aligned16(F);
    p.b = Operand{}; p.b.ptr = dY; p.b.ld = g.K; p.b.rows = g.N; p.b.vec = (g.K % 4 == 0) && aligned16(dY);
    p.BN = pick_bn(p.N);
    p.numKb = ceil_div(p.R, BK); p.kbPerSplit = p.numKb;
    p.e = Epilogue{}; p.e.out = dX; p.e.ldd = V;
    return launch<OP_DENSE_MN, OP_DENSE_K, EPI_PLAIN>(ctx, p, 1, "fc_dgrad_tc");
  }
  if (g.sy != 1 || g.sx != 1) return VLB_Unsupported;
  // dX = conv(dY, flipped and transposed filters) with padding (F-1)*dilate - pad
  ConvGeom t = g;
  t.H = g.Ho; t.W = g.Wo; t.C = g.K; t.FC = g.K; t.K = g.C; t.Ho = g.H; t.Wo = g.W;
  t.pt = (g.FH - 1) * g.dy - g.pt; t.pl = (g.FW - 1) * g.dx - g.pl;
  long long M = (long long)g.H * g.W * g.N;
  int const V = g.FH * g.FW * g.K;
  ProfScope prof(ctx, kProfDgrad);
  prof.rec.flops = 2.0 * (double)M * (double)g.C * (double)V;
  p.M = (int)M; p.N = g.C; p.R = V;
  conv_operand(p.a, t, dY, g.K);
  p.a.rows = p.M;
  p.BN = pick_bn(p.N);
  p.numKb = ceil_div(p.R, BK); p.kbPerSplit = p.numKb;
  p.b = Operand{}; p.b.ld = V; p.b.rows = g.C;
  if (p.a.fast) {
    p.chanFast = g.K % 32 == 0;
    p.bTiles = prep_b_tiles(ctx, F, g.C, V, p.BN, p.numKb, p.chanFast ? 4 : 1, g);
    if (!p.bTiles) return ctx->lastError;
    p.b.ptr = p.bTiles;          // not read by the pipelined producers
    p.pipelined = 1;
  } else {
    size_t nF = (size_t)g.FH * g.FW * g.FC * g.K;
    float* ft = (float*)workspace(ctx, sizeof(float) * nF);
    if (!ft) return ctx->lastError;
    flip_filters_kernel<<<grid_for(nF, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(ft, F, g.FH, g.FW, g.C, g.K);
    VLB_LAUNCHED(ctx, 1);
    p.b.ptr = ft; p.b.vec = (V % 4 == 0);
  }
  p.e = Epilogue{}; p.e.out = dX; p.e.inMult = 1.f; p.e.P = g.H * g.W; p.e.Ktot = g.C;
  if (p.pipelined) {
    p.e.mask = ctx->reluMask; ctx->maskDone = ctx->reluMask != nullptr;
    return launch_ts(ctx, p, "conv_dgrad_ts");
  }
  return launch<OP_IM2COL, OP_DENSE_K, EPI_CONV>(ctx, p, 1, "conv_dgrad_tc");
}

int conv_wgrad_tc(vlb_ctx* ctx, ConvGeom const& g, float* dF, float* db, float const* X, float const* dY, bool* dbDone)
{
  *dbDone = false;
  if (g.G != 1 || !fits32(g)) return VLB_Unsupported;
  int const V = g.FH * g.FW * g.FC;
  Params p = {};
  if (is_fc(g)) {
    // dF(V x K) = X(V x N) dY'(N x K)  (reference bits/nnfullyconnected.cu:126-137): reduction over the batch
    {
      int const rc = fc_wgrad_ts(ctx, g, dF, X, dY);
      if (rc >= 0) return rc;
    }
    ProfScope prof(ctx, kProfFc);
    prof.rec.flops = 2.0 * (double)V * (double)g.K * (double)g.N;
    p.M = V; p.N = g.K; p.R = g.N;
    p.a = Operand{}; p.a.ptr = X; p.a.ld = V; p.a.rows = V; p.a.vec = (V % 4 == 0) && aligned16(X);
    p.b = Operand{}; p.b.ptr = dY; p.b.ld = g.K; p.b.rows = g.K; p.b.vec = (g.K % 4 == 0) && aligned16(dY);
    p.BN = p.N > 64 ? 128 : (p.N > 32 ? 64 : 32);     // MN-major tiles are built from 32-column atoms
    p.numKb = ceil_div(p.R, BK); p.kbPerSplit = p.numKb;
    p.e = Epilogue{}; p.e.out = dF; p.e.ldd = V;
    return launch<OP_DENSE_MN, OP_DENSE_MN, EPI_PLAIN>(ctx, p, 1, "fc_wgrad_tc");
  }
  {
    int const rc = conv_wgrad_ts(ctx, g, dF, db, X, dY, dbDone);
    if (rc >= 0) return rc;
  }
  long long R = (long long)g.Ho * g.Wo * g.N;
  ProfScope prof(ctx, kProfWgrad);      // includes the dY tile images (with the bias gradient) and the sum of the split partial results
  prof.rec.flops = 2.0 * (double)V * (double)g.K * (double)R;
  p.M = V; p.N = g.K; p.R = (int)R;
  conv_operand(p.a, g, X, g.C);
  p.a.rows = V;
  int const P = g.Ho * g.Wo;
  p.b = Operand{}; p.b.ptr = dY; p.b.ld = P; p.b.bs = (long long)P * g.K; p.b.P = P; p.b.rows = g.K;
  p.b.vec = (P % 4 == 0) && aligned16(dY);
  p.BN = pick_bn(p.N);
  p.numKb = ceil_div(p.R, BK);
  int tiles = ceil_div(p.M, BM) * ceil_div(p.N, p.BN);
  int splits = pick_splits(ctx, tiles, p.numKb, 8);
  p.kbPerSplit = ceil_div(p.numKb, splits);
  splits = ceil_div(p.numKb, p.kbPerSplit);
  p.e = Epilogue{}; p.e.ldd = V;
  size_t nF = (size_t)V * g.K;
  size_t partBytes = splits > 1 ? sizeof(float) * nF * splits : 0;
  size_t tileBytes = 0;
  if (p.a.fast) {
    // dY is split into hi / lo once and laid out as tile images, like the filters of fprop
    tileBytes = b_tiles_bytes(ctx, g.K, p.BN, p.numKb);
    partBytes = (partBytes + 255) & ~(size_t)255;
    if (P % 4 == 0 && aligned16(dY) && g.K <= 4096 && vlb::ceil_div(g.K, p.BN) * p.BN <= 65535) {
      p.bTiles = prep_dy_tiles(ctx, dY, g.K, p.R, P, p.BN, p.numKb, partBytes, db);
      *dbDone = db != nullptr;
    } else {
      p.bTiles = prep_b_tiles(ctx, dY, g.K, p.R, p.BN, p.numKb, 2, g, partBytes, P);
    }
    if (!p.bTiles) return ctx->lastError;
    p.pipelined = 1;
  }
  if (splits == 1) {
    p.e.out = dF;
    return launch<OP_WGATHER, OP_DENSE_K, EPI_PLAIN>(ctx, p, 1, "conv_wgrad_tc");
  }
  char* ws = (char*)workspace(ctx, tileBytes + partBytes);
  float* part = ws ? (float*)(ws + tileBytes) : nullptr;
  if (!part) return ctx->lastError;
  p.e.out = part; p.e.splitStride = (long long)nF;
  int rc = launch<OP_WGATHER, OP_DENSE_K, EPI_PLAIN>(ctx, p, splits, "conv_wgrad_tc");
  if (rc) return rc;
  tc_splitk_reduce_kernel<<<grid_for(nF, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(dF, part, nF, nF, splits);
  VLB_LAUNCHED(ctx, 1);
  return check_launch(ctx, "conv_wgrad_tc");
}

}  // namespace vlb

extern "C" int vlb_ctx_set_wait_limit(vlb_ctx* ctx, long long cycles)
{
  if (!ctx || cycles < 0) return VLB_IllegalArgument;
  long long const v = cycles == 0 ? kWaitCycles : cycles;
  // ordered behind the kernels already enqueued on the context's stream, which keep the limit they were launched under
  cudaError_t e = cudaMemcpyToSymbolAsync(gWaitCycles, &v, sizeof(v), 0, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) { cudaGetLastError(); return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e)); }
  return VLB_Success;
}
