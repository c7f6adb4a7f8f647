// NHWC bf16 convolutions as implicit GEMMs on the 5th-generation tensor cores.
//
// The activation tensor [N, H, W, C] is never unfolded.  An output tile is a box of up to 128 output
// pixels (tn images x th rows x tw columns); for every filter tap (r, s) the TMA unit loads the same box
// shifted by the tap's offset as a 4-D tile of 64 channels per pixel, which lands in shared memory in the
// 128-byte-swizzled K-major layout that tcgen05.mma reads: the tap loop simply extends the K loop of
// a GEMM, and out-of-image coordinates are zero-filled by the TMA unit, which is the padding.  Strided
// convolutions read through "phase" tensor maps: for stride 2 the input pixels of one parity class
// (h mod 2, w mod 2) form a dense tensor with doubled strides, and each tap belongs to exactly one class.
// The same kernel therefore serves
//   forward            y[p, co]  = sum_{tap, ci} x[p*stride + tap - pad, ci] * w[co, tap, ci]
//   data gradient      dx[q, ci] = sum_{tap, co} dy[(q + pad - tap)/stride, co] * w^T[ci, tap, co]
// (the host builds the tap list; for stride 2 one launch per parity class of dx, written through a phase map).
// The weight gradient contracts over pixels instead, so both operands are MN-major in shared memory
// (pixels are rows); it splits the pixel range over CTAs and accumulates into an fp32 buffer with
// vector reductions.
//
// Pipeline and warp roles are those of the persistent GEMM: warp 0 issues TMA loads (never multicast),
// warp 1 issues tcgen05.mma into a double-buffered TMEM accumulator, warps 2-5 drain TMEM, convert and hand
// swizzled boxes to the TMA store unit; all mbarrier waits are bounded and report through an error word.
//
// The reference has no convolution (it delegates model math to TensorFlow); these kernels serve the
// ResNet-50 benchmark model.
#include <cuda.h>

#include <algorithm>
#include <vector>

#include "kernels/common.cuh"
#include "kernels/tcgen05.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

constexpr int kMaxTaps = 9;

struct ConvTap {
  int16_t dh, dw;  // offset of the loaded box relative to the output box, in the coordinates of map `map`
  int16_t map;     // which activation tensor map
  int16_t pad_;
  int32_t kofs;    // first column of this tap in the weight matrix
};

struct ConvParams {
  int32_t* error;
  float* stat_sum;  // optional per-channel sum of the bf16 outputs
  float* stat_sq;   // optional per-channel sum of squares
  int taps, cblocks;               // filter taps, 64-channel blocks of the contraction
  int accumulate;                  // 1: add the result to what the output tensor holds (TMA reduce-add store)
  int b_resident;                  // bytes of weights kept in shared memory for the whole kernel (0: streamed per stage)
  int b_mn;                        // 1: the weight matrix is [contracted channel, tap * produced channel] (MN-major B)
  int tiles_w, tiles_h, tiles_n;   // boxes per output extent
  int tw, th, tn;                  // box extents; tw * th * tn <= 128
  int wo, ho, nb;                  // output extents (for the statistics mask)
  int cout, n_tiles;               // output channels and tiles of BN channels
  ConvTap tap[kMaxTaps];
};

struct ConvMaps {
  CUtensorMap a[4];  // activation phases
  CUtensorMap b;     // weights [Cout, taps * Cin], K-major; or [contracted, taps * produced] when b_mn
  CUtensorMap c;     // output
};

__device__ __forceinline__ void TmaLoad4D(void* smem_dst, const CUtensorMap* tmap, int c, int w, int h, int n,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(SmemAddr(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c), "r"(w), "r"(h), "r"(n),
      "r"(SmemAddr(bar))
      : "memory");
}
__device__ __forceinline__ void TmaStore4D(const CUtensorMap* tmap, int c, int w, int h, int n, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(c), "r"(w), "r"(h), "r"(n), "r"(SmemAddr(smem_src))
               : "memory");
}

// The same box added (in bf16) to the tensor in global memory instead of overwriting it.
__device__ __forceinline__ void TmaReduceAdd4D(const CUtensorMap* tmap, int c, int w, int h, int n,
                                               const void* smem_src) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(c), "r"(w), "r"(h), "r"(n), "r"(SmemAddr(smem_src))
               : "memory");
}

template <int BN>
struct ConvCfg {
  // A stage of a narrow tile carries few bytes, so it takes more stages to cover the load latency.
  static constexpr int kStages       = BN >= 256 ? 3 : BN >= 128 ? 5 : 8;
  static constexpr int kABytes       = kBM * kBK * 2;
  static constexpr int kBBytes       = BN * kBK * 2;
  static constexpr int kStageBytes   = kABytes + kBBytes;
  static constexpr int kStagingBytes = kBM * BN * 2;
  static constexpr int kTmemCols     = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kSmemBytes    = kStages * kStageBytes + kStagingBytes + 1024 + 256 + 4096 /*statistics*/;
};

constexpr int kMaxSmemBytes = 227 * 1024;  // dynamic shared memory limit per CTA
constexpr int kConvThreads = 320;  // TMA warp, MMA warp, four epilogue warps, four statistics warps

template <int BN>
__global__ void __launch_bounds__(kConvThreads, 1)
ConvTapsKernel(const __grid_constant__ ConvMaps maps, const __grid_constant__ ConvParams p) {
  using Cfg = ConvCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem    = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;
  // With a single tile of output channels and a small filter the whole weight matrix stays in shared memory
  // (one [BN x 64] block per K step) instead of being re-read from L2 for every output tile.
  uint8_t* resident    = staging + Cfg::kStagingBytes;
  uint64_t* full_bar   = reinterpret_cast<uint64_t*>(resident + p.b_resident);
  uint64_t* empty_bar  = full_bar + Cfg::kStages;
  uint64_t* tmem_full  = empty_bar + Cfg::kStages;  // [2]
  uint64_t* tmem_empty = tmem_full + 2;             // [2]
  uint64_t* b_full     = tmem_empty + 2;
  uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(b_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k     = p.taps * p.cblocks;
  const int m_tiles   = p.tiles_w * p.tiles_h * p.tiles_n;
  const int num_tiles = m_tiles * p.n_tiles;
  const int box_rows  = p.tw * p.th * p.tn;
  const bool b_res    = p.b_resident > 0;
  const uint32_t stage_tx = static_cast<uint32_t>(box_rows) * 128u + (b_res ? 0u : Cfg::kBBytes);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      MbarInit(&full_bar[s], 1);
      MbarInit(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      MbarInit(&tmem_full[b], 1);
      MbarInit(&tmem_empty[b], 4);
    }
    MbarInit(b_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(tmem_slot)),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      if (b_res) {
        MbarExpectTx(b_full, static_cast<uint32_t>(p.b_resident));
        for (int t = 0; t < p.taps; ++t)
          for (int cb = 0; cb < p.cblocks; ++cb) {
            uint8_t* dst = resident + (t * p.cblocks + cb) * Cfg::kBBytes;
            if (p.b_mn) {  // BN/64 boxes of [64 contracted rows x 64 produced channels]
              for (int j = 0; j < BN / 64; ++j) TmaLoad2D(dst + j * 8192, &maps.b, p.tap[t].kofs + j * 64, cb * kBK, b_full);
            } else {
              TmaLoad2D(dst, &maps.b, p.tap[t].kofs + cb * kBK, 0, b_full);
            }
          }
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile / p.n_tiles, nt = tile % p.n_tiles;
        const int w0 = (mt % p.tiles_w) * p.tw;
        const int h0 = ((mt / p.tiles_w) % p.tiles_h) * p.th;
        const int n0 = (mt / (p.tiles_w * p.tiles_h)) * p.tn;
        for (int t = 0; t < p.taps && ok; ++t) {
          const ConvTap tap = p.tap[t];
          for (int cb = 0; cb < p.cblocks; ++cb, ++it) {
            const int s = it % Cfg::kStages;
            if (!MbarWait(&empty_bar[s], ((it / Cfg::kStages) & 1) ^ 1)) {
              atomicExch(p.error, 1);
              ok = false;
              break;
            }
            uint8_t* a_dst = smem + s * Cfg::kStageBytes;
            MbarExpectTx(&full_bar[s], stage_tx);
            TmaLoad4D(a_dst, &maps.a[tap.map], cb * kBK, w0 + tap.dw, h0 + tap.dh, n0, &full_bar[s]);
            if (!b_res) {
              if (p.b_mn) {
                for (int j = 0; j < BN / 64; ++j)
                  TmaLoad2D(a_dst + Cfg::kABytes + j * 8192, &maps.b, tap.kofs + nt * BN + j * 64, cb * kBK, &full_bar[s]);
              } else {
                TmaLoad2D(a_dst + Cfg::kABytes, &maps.b, tap.kofs + cb * kBK, nt * BN, &full_bar[s]);
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // bit 16: B is MN-major (the weights in the layout the forward pass uses, contracted over their rows)
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (p.b_mn ? (1u << 16) : 0u) |
                             (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      const uint64_t b_kstep = p.b_mn ? 128 : 2;  // 16 contraction steps further: +2048 bytes MN-major, +32 K-major
      uint32_t it = 0;
      int local = 0;
      bool ok = true;
      if (b_res && !MbarWait(b_full, 0)) {
        atomicExch(p.error, 5);
        ok = false;
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        if (!MbarWait(&tmem_empty[buf], ((local >> 1) & 1) ^ 1)) {
          atomicExch(p.error, 4);
          break;
        }
        TcFenceAfter();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kt = 0; kt < num_k; ++kt, ++it) {
          const int s = it % Cfg::kStages;
          if (!MbarWait(&full_bar[s], (it / Cfg::kStages) & 1)) {
            atomicExch(p.error, 2);
            ok = false;
            break;
          }
          TcFenceAfter();
          const uint32_t a_addr = SmemAddr(smem + s * Cfg::kStageBytes);
          const uint64_t adesc  = SmemDescSw128(a_addr);
          const uint32_t b_addr = b_res ? SmemAddr(resident) + kt * Cfg::kBBytes : a_addr + Cfg::kABytes;
          const uint64_t bdesc  = p.b_mn ? SmemDescMnSw128(b_addr, 8192) : SmemDescSw128(b_addr);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            UmmaBf16(tmem_d, adesc + 2 * k, bdesc + b_kstep * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          UmmaCommit(&empty_bar[s]);
        }
        if (ok) UmmaCommit(&tmem_full[buf]);
      }
    }
  } else if (warp < 6) {
    // Epilogue warps.  The tile leaves through 64-channel boxes: as soon as a box is staged, one thread hands it
    // to the TMA store unit while the next box is converted; the TMEM load of the next 32 columns is in flight
    // while this one is converted.
    const int q = warp & 3;
    const int r = q * 32 + lane;  // row of the tile = pixel of the box
    constexpr int kBoxes  = BN / 64;
    constexpr int kChunks = BN / 32;
    const int bar_threads = p.stat_sum != nullptr ? 256 : 128;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int mt = tile / p.n_tiles, nt = tile % p.n_tiles;
      const int w0 = (mt % p.tiles_w) * p.tw;
      const int h0 = ((mt / p.tiles_w) % p.tiles_h) * p.th;
      const int n0 = (mt / (p.tiles_w * p.tiles_h)) * p.tn;
      const int buf = local & 1;
      if (ok && !MbarWait(&tmem_full[buf], (local >> 1) & 1)) {
        if (lane == 0) atomicExch(p.error, 3);
        ok = false;
      }
      TcFenceAfter();
      const uint32_t tsrc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * BN);
      uint32_t acc[2][32];
      if (ok) TmemLoad32Async(tsrc, acc[0]);
#pragma unroll
      for (int b = 0; b < kBoxes; ++b) {
        // the store that last read this box (one tile ago) is kBoxes - 1 groups behind the newest one
        if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kBoxes - 1) : "memory");
        NamedBarSync(1, bar_threads);
        uint8_t* box = staging + b * (kBM * 128);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c = 2 * b + half;
          if (ok) {
            TmemLoadWait(acc[c & 1]);
            if (c + 1 < kChunks) TmemLoad32Async(tsrc + static_cast<uint32_t>((c + 1) * 32), acc[(c + 1) & 1]);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              alignas(16) __nv_bfloat16 o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(__uint_as_float(acc[c & 1][g * 8 + j]));
              const int chunk = half * 4 + g;
              *reinterpret_cast<uint4*>(box + r * 128 + ((chunk ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(o);
            }
          }
        }
        if (b == kBoxes - 1 && ok) {  // the accumulator is drained: hand it back to the MMA warp
          TcFenceBefore();
          __syncwarp();
          if (lane == 0) MbarArrive(&tmem_empty[buf]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        NamedBarSync(1, bar_threads);
        if (warp == 2 && lane == 0) {
          if (ok && nt * BN + b * 64 < p.cout) {
            if (p.accumulate) TmaReduceAdd4D(&maps.c, nt * BN + b * 64, w0, h0, n0, box);
            else TmaStore4D(&maps.c, nt * BN + b * 64, w0, h0, n0, box);
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else if (p.stat_sum != nullptr) {
    // Statistics warps: per-channel sum and sum of squares of the bf16 values of every staged box (what the
    // normalisation that follows will read), over the rows that are real output pixels.  They read a box
    // between its "full" barrier and the next "free" barrier, off the epilogue warps' critical path.
    constexpr int kBoxes = BN / 64;
    float* partial   = reinterpret_cast<float*>(tmem_slot + 4);  // [2][4 warps][64 columns][2]
    const int st     = threadIdx.x - 192;  // 0..127
    const int chunk  = st & 7;             // 16-byte chunk of a box row = 8 channels
    const int rg     = st >> 3;            // rows rg, rg + 16, ...
    const int sw     = st >> 5;            // statistics warp 0..3
    uint32_t boxes_done = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int mt = tile / p.n_tiles, nt = tile % p.n_tiles;
      const int w0 = (mt % p.tiles_w) * p.tw;
      const int h0 = ((mt / p.tiles_w) % p.tiles_h) * p.th;
      const int n0 = (mt / (p.tiles_w * p.tiles_h)) * p.tn;
      uint32_t valid = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = rg + 16 * i;
        if (row < box_rows) {
          const int iw = row % p.tw, ih = (row / p.tw) % p.th, in = row / (p.tw * p.th);
          if (w0 + iw < p.wo && h0 + ih < p.ho && n0 + in < p.nb) valid |= 1u << i;
        }
      }
#pragma unroll 1
      for (int b = 0; b < kBoxes; ++b, ++boxes_done) {
        NamedBarSync(1, 256);  // "free": this warp no longer reads the box about to be overwritten
        NamedBarSync(1, 256);  // "full"
        const uint8_t* box = staging + b * (kBM * 128);
        float s1[8], s2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) s1[j] = s2[j] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (valid & (1u << i)) {
            const int row = rg + 16 * i;
            const uint4 v = *reinterpret_cast<const uint4*>(box + row * 128 + ((chunk ^ (row & 7)) << 4));
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(h[j]);
              s1[2 * j] += f.x; s2[2 * j] += f.x * f.x;
              s1[2 * j + 1] += f.y; s2[2 * j + 1] += f.y * f.y;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // lanes that share a chunk differ in bits 3 and 4
          s1[j] += __shfl_xor_sync(0xffffffffu, s1[j], 8);
          s1[j] += __shfl_xor_sync(0xffffffffu, s1[j], 16);
          s2[j] += __shfl_xor_sync(0xffffffffu, s2[j], 8);
          s2[j] += __shfl_xor_sync(0xffffffffu, s2[j], 16);
        }
        float* P = partial + (boxes_done & 1) * (4 * 64 * 2);
        if (lane < 8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            P[(sw * 64 + lane * 8 + j) * 2]     = s1[j];
            P[(sw * 64 + lane * 8 + j) * 2 + 1] = s2[j];
          }
        }
        NamedBarSync(2, 128);
        const int col = st & 63, which = st >> 6;
        const float tot = P[(0 * 64 + col) * 2 + which] + P[(1 * 64 + col) * 2 + which] +
                          P[(2 * 64 + col) * 2 + which] + P[(3 * 64 + col) * 2 + which];
        const int ch = nt * BN + b * 64 + col;
        if (ch < p.cout) atomicAdd((which ? p.stat_sq : p.stat_sum) + ch, tot);
      }
    }
  }
  TcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
  }
}

// ------------------------------------------------------------------ weight gradient
// dw[co, tap, ci] = sum over output pixels p of dy[p, co] * x[p*stride + tap - pad, ci].  The contraction runs
// over pixels, which are the ROWS of both tiles as the TMA unit delivers them, so both operands are
// MN-major: a 64-channel box is [pixels x 128 bytes], 8-pixel groups 1024 bytes apart, and the next 64
// channels start one box (16 KB) further.  One CTA owns (tap, 128 output channels, BN input channels) and
// a contiguous share of the pixel boxes; partial results are added into the fp32 gradient.

struct WgradParams {
  int32_t* error;
  float* dw;        // [Cout, taps_total * Cin] fp32, accumulated into
  int ldw;          // taps_total * Cin
  int taps;
  int cout_tiles, cin_tiles;
  int tiles_w, tiles_h, tiles_n;
  int tw, th, tn;   // tw * th * tn is a multiple of 16, at most 128
  int cout, cin;
  int a_boxes;      // 64-channel boxes of dy to load per stage: 1 when cout <= 64 (rows 64..127 are then unused)
  ConvTap tap[kMaxTaps];  // kofs = first column of the tap inside a row of dw
};

struct WgradMaps {
  CUtensorMap x[4];  // activation phases
  CUtensorMap dy;
};


// kBoxRows: pixels per K step (rows of a box).  The widest tile (256 input channels) takes 64-pixel steps so that four
// stages still fit; it moves a third fewer bytes per FLOP through L2 than the 128-channel tile.
// kMH: output-channel halves of 128 per CTA.  With two (256 x 256 tile, both accumulators filling TMEM) a K step moves
// 64 KB for 1024 tensor-core clocks, which the 64 B/clk/SM L2 path can just sustain; the 128-row tiles are load-bound.
template <int BN, int kBoxRows, int kMH = 1>
struct WgradCfg {
  static constexpr int kBoxBytes   = kBoxRows * 128;
  static constexpr int kStages     = (BN == 128 || kMH == 2) ? 3 : 4;
  static constexpr int kABytes     = 2 * kMH * kBoxBytes;
  static constexpr int kBBytes     = (BN / 64) * kBoxBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols   = BN * kMH;
  static constexpr int kSmemBytes  = kStages * kStageBytes + 1024 + 256;
};

template <int BN, int kBoxRows, int kMH = 1>
__global__ void __launch_bounds__(kGemmThreads, 1)
ConvWgradKernel(const __grid_constant__ WgradMaps maps, const __grid_constant__ WgradParams p) {
  using Cfg = WgradCfg<BN, kBoxRows, kMH>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar  = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* tmem_full = empty_bar + Cfg::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int id = blockIdx.x;
  const int cin_t  = id % p.cin_tiles;  id /= p.cin_tiles;
  const int cout_t = id % p.cout_tiles; id /= p.cout_tiles;
  const ConvTap tap = p.tap[id];
  const int box_rows = p.tw * p.th * p.tn;
  const int k_tiles  = p.tiles_w * p.tiles_h * p.tiles_n;
  const int k_begin  = static_cast<int>(static_cast<int64_t>(k_tiles) * blockIdx.y / gridDim.y);
  const int k_end    = static_cast<int>(static_cast<int64_t>(k_tiles) * (blockIdx.y + 1) / gridDim.y);
  const int num_k    = k_end - k_begin;
  const uint32_t stage_tx = static_cast<uint32_t>(box_rows) * 128u * (p.a_boxes + BN / 64);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      MbarInit(&full_bar[s], 1);
      MbarInit(&empty_bar[s], 1);
    }
    MbarInit(tmem_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(tmem_slot)),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    if (lane == 0) {
      for (int kt = 0; kt < num_k; ++kt) {
        const int s = kt % Cfg::kStages;
        if (!MbarWait(&empty_bar[s], ((kt / Cfg::kStages) & 1) ^ 1)) {
          atomicExch(p.error, 1);
          break;
        }
        const int mt = k_begin + kt;
        const int w0 = (mt % p.tiles_w) * p.tw;
        const int h0 = ((mt / p.tiles_w) % p.tiles_h) * p.th;
        const int n0 = (mt / (p.tiles_w * p.tiles_h)) * p.tn;
        uint8_t* a_dst = smem + s * Cfg::kStageBytes;
        uint8_t* b_dst = a_dst + Cfg::kABytes;
        MbarExpectTx(&full_bar[s], stage_tx);
        for (int j = 0; j < p.a_boxes; ++j)
          TmaLoad4D(a_dst + j * Cfg::kBoxBytes, &maps.dy, cout_t * kBM * kMH + j * 64, w0, h0, n0, &full_bar[s]);
#pragma unroll
        for (int j = 0; j < BN / 64; ++j)
          TmaLoad4D(b_dst + j * Cfg::kBoxBytes, &maps.x[tap.map], cin_t * BN + j * 64, w0 + tap.dw, h0 + tap.dh, n0,
                    &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // both operands MN-major: bits 15 and 16
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                 (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      const int ksteps = box_rows / 16;
      bool ok = true;
      for (int kt = 0; kt < num_k && ok; ++kt) {
        const int s = kt % Cfg::kStages;
        if (!MbarWait(&full_bar[s], (kt / Cfg::kStages) & 1)) {
          atomicExch(p.error, 2);
          ok = false;
          break;
        }
        TcFenceAfter();
        const uint32_t a_addr = SmemAddr(smem + s * Cfg::kStageBytes);
        const uint64_t bdesc  = SmemDescMnSw128(a_addr + Cfg::kABytes, Cfg::kBoxBytes);
#pragma unroll
        for (int h = 0; h < kMH; ++h) {
          const uint64_t adesc = SmemDescMnSw128(a_addr + h * 2 * Cfg::kBoxBytes, Cfg::kBoxBytes);
          for (int k = 0; k < ksteps; ++k) {
            // 16 pixels further along K = 16 rows of 128 bytes
            UmmaBf16(tmem_base + static_cast<uint32_t>(h * BN), adesc + static_cast<uint64_t>(k) * (2048 >> 4),
                     bdesc + static_cast<uint64_t>(k) * (2048 >> 4), idesc, (kt > 0 || k > 0) ? 1u : 0u);
          }
        }
        UmmaCommit(&empty_bar[s]);
      }
      UmmaCommit(tmem_full);
    }
  } else {
    const int q = warp & 3;
    const bool ok = MbarWait(tmem_full, 0);
    if (!ok && lane == 0) atomicExch(p.error, 3);
    TcFenceAfter();
    if (ok && num_k > 0) {
#pragma unroll 1
      for (int c = 0; c < kMH * (BN / 32); ++c) {
        uint32_t acc[32];
        TmemLoad32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c * 32), acc);
        const int row  = (cout_t * kMH + c / (BN / 32)) * kBM + q * 32 + lane;  // accumulator c / (BN/32) = its half
        const int col0 = cin_t * BN + (c % (BN / 32)) * 32;
        if (row < p.cout && col0 < p.cin) {
          float* dst = p.dw + static_cast<int64_t>(row) * p.ldw + tap.kofs + col0;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + g * 4),
                         "f"(__uint_as_float(acc[g * 4])), "f"(__uint_as_float(acc[g * 4 + 1])),
                         "f"(__uint_as_float(acc[g * 4 + 2])), "f"(__uint_as_float(acc[g * 4 + 3]))
                         : "memory");
          }
        }
      }
    }
  }
  TcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
  }
}

// ------------------------------------------------------------------ host side

struct Box {
  int tw, th, tn;
};

// Box of at most max_px (<= 128) pixels that covers the extents (wo, ho, nb) with the fewest tiles; `mult16` restricts the
// pixel count to multiples of 16 (one MMA K step) for the weight gradient.
Box PickBox(int wo, int ho, int nb, bool mult16, int max_px = 128) {
  Box best{1, 1, 1};
  int64_t best_tiles = INT64_MAX;
  for (int tw = 1; tw <= std::min(wo, max_px); ++tw) {
    for (int th = 1; th <= std::min(ho, max_px / tw); ++th) {
      const int tn = std::max(1, std::min(nb, max_px / (tw * th)));
      if (mult16 && (tw * th * tn) % 16 != 0) continue;
      const int64_t tiles = static_cast<int64_t>(CeilDiv(wo, tw)) * CeilDiv(ho, th) * CeilDiv(nb, tn);
      if (tiles < best_tiles || (tiles == best_tiles && tw > best.tw)) {
        best_tiles = tiles;
        best = Box{tw, th, tn};
      }
    }
  }
  if (best_tiles == INT64_MAX) {  // mult16 with tiny extents: rely on the zero fill beyond the extents
    best = Box{16, 1, 1};
  }
  return best;
}

// Tensor map over a bf16 NHWC view: extents (c, w, h, n), strides in elements, box (64, tw, th, tn), 128B swizzle.
int MakeTmap4D(CUtensorMap* out, const void* base, int64_t c, int64_t w, int64_t h, int64_t n, int64_t sw, int64_t sh,
               int64_t sn, const Box& box) {
  EncodeFn enc = GetEncodeFn();
  if (!enc) return SetError(-7, "cuTensorMapEncodeTiled is not available from the driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return SetError(-2, "conv: tensor base must be 16-byte aligned");
  if (c % 8 != 0) return SetError(-2, "conv: channel count must be a multiple of 8");
  cuuint64_t dims[4]    = {static_cast<cuuint64_t>(c), static_cast<cuuint64_t>(w), static_cast<cuuint64_t>(h),
                           static_cast<cuuint64_t>(n)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(sw) * 2, static_cast<cuuint64_t>(sh) * 2,
                           static_cast<cuuint64_t>(sn) * 2};
  cuuint32_t bx[4]      = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box.tw), static_cast<cuuint32_t>(box.th),
                           static_cast<cuuint32_t>(box.tn)};
  cuuint32_t estr[4]    = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, bx, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return SetError(-7, "cuTensorMapEncodeTiled (4-D) failed with code " + std::to_string((int)r));
  return 0;
}

int MakeTmap2D(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int box_rows) {
  EncodeFn enc = GetEncodeFn();
  if (!enc) return SetError(-7, "cuTensorMapEncodeTiled is not available from the driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return SetError(-2, "conv: weight base must be 16-byte aligned");
  cuuint64_t dims[2]    = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t bx[2]      = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2]    = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, bx, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return SetError(-7, "cuTensorMapEncodeTiled (weights) failed with code " + std::to_string((int)r));
  return 0;
}

// A view of an NHWC tensor in which (w, h) extents and strides may be those of a stride-2 parity class,
// or the pixels flattened into one axis.
struct View {
  const void* base;
  int64_t c, w, h, n;     // extents
  int64_t sw, sh, sn;     // strides in elements
};

View FullView(const void* base, int n, int h, int w, int c) {
  return View{base, c, w, h, n, c, static_cast<int64_t>(w) * c, static_cast<int64_t>(h) * w * c};
}
View FlatView(const void* base, int n, int h, int w, int c) {  // all pixels on the w axis
  const int64_t px = static_cast<int64_t>(n) * h * w;
  return View{base, c, px, 1, 1, c, px * c, px * c};
}
View PhaseView(const void* base, int n, int h, int w, int c, int bh, int bw) {
  const char* b = static_cast<const char*>(base) + (static_cast<int64_t>(bh) * w + bw) * c * 2;
  return View{b, c, (w - bw + 1) / 2, (h - bh + 1) / 2, n, 2 * static_cast<int64_t>(c), 2 * static_cast<int64_t>(w) * c,
              static_cast<int64_t>(h) * w * c};
}
int MapOf(CUtensorMap* out, const View& v, const Box& box) {
  return MakeTmap4D(out, v.base, v.c, v.w, v.h, v.n, v.sw, v.sh, v.sn, box);
}

int32_t* ConvErrorWord() {
  static int32_t* word = nullptr;
  if (!word) {
    if (cudaMalloc(reinterpret_cast<void**>(&word), sizeof(int32_t)) != cudaSuccess) return nullptr;
    cudaMemset(word, 0, sizeof(int32_t));
  }
  return word;
}

template <int BN>
int LaunchTaps(const ConvMaps& maps, const ConvParams& p, cudaStream_t s) {
  using Cfg = ConvCfg<BN>;
  static bool configured = false;
  if (!configured) {
    TIPSK_CUDA(cudaFuncSetAttribute(ConvTapsKernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes));
    configured = true;
  }
  const int64_t tiles = static_cast<int64_t>(p.tiles_w) * p.tiles_h * p.tiles_n * p.n_tiles;
  const int grid = static_cast<int>(std::min<int64_t>(tiles, NumSMs()));
  ConvTapsKernel<BN><<<grid, kConvThreads, Cfg::kSmemBytes + p.b_resident, s>>>(maps, p);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

template <int BN, int kBoxRows, int kMH = 1>
int LaunchWgrad(const WgradMaps& maps, const WgradParams& p, int splits, cudaStream_t s) {
  using Cfg = WgradCfg<BN, kBoxRows, kMH>;
  static bool configured = false;
  if (!configured) {
    TIPSK_CUDA(cudaFuncSetAttribute(ConvWgradKernel<BN, kBoxRows, kMH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes));
    configured = true;
  }
  dim3 grid(p.taps * p.cout_tiles * p.cin_tiles, splits);
  ConvWgradKernel<BN, kBoxRows, kMH><<<grid, kGemmThreads, Cfg::kSmemBytes, s>>>(maps, p);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

// Runs the tap kernel: out[view_out pixel, co] = sum over taps and 64-channel blocks.
int RunTaps(const View* in_views, int n_views, const ConvTap* taps, int n_taps, int cin, const void* weights,
            int w_rows, int64_t w_cols, const View& out, float* stat_sum, float* stat_sq, cudaStream_t s,
            int accumulate = 0, int b_mn = 0) {
  TIPSK_REQUIRE(n_taps >= 1 && n_taps <= kMaxTaps, "conv: 1..9 filter taps are supported");
  TIPSK_REQUIRE(cin % 64 == 0, "conv: the contracted channel count must be a multiple of 64");
  TIPSK_REQUIRE(w_rows % 64 == 0, "conv: the produced channel count must be a multiple of 64");
  const Box box = PickBox(static_cast<int>(out.w), static_cast<int>(out.h), static_cast<int>(out.n), false);
  ConvMaps maps;
  ConvParams p{};
  p.tiles_w = CeilDiv(out.w, box.tw);
  p.tiles_h = CeilDiv(out.h, box.th);
  p.tiles_n = CeilDiv(out.n, box.tn);
  const int64_t m_tiles = static_cast<int64_t>(p.tiles_w) * p.tiles_h * p.tiles_n;
  int bn = 128;
  if (w_rows % 128 != 0) bn = 64;
  else if (w_rows % 256 == 0 && m_tiles * (w_rows / 256) >= NumSMs()) bn = 256;
  int rc;
  for (int i = 0; i < n_views; ++i) {
    rc = MapOf(&maps.a[i], in_views[i], box);
    if (rc) return rc;
  }
  for (int i = n_views; i < 4; ++i) maps.a[i] = maps.a[0];
  // K-major: [produced channel, tap * contracted] read in boxes of bn rows; MN-major: [contracted channel,
  // tap * produced] read in boxes of 64 rows x 64 produced channels
  rc = b_mn ? MakeTmap2D(&maps.b, weights, cin, w_cols, 64) : MakeTmap2D(&maps.b, weights, w_rows, w_cols, bn);
  if (rc) return rc;
  p.b_mn = b_mn;
  rc = MapOf(&maps.c, out, box);
  if (rc) return rc;
  p.error = ConvErrorWord();
  TIPSK_REQUIRE(p.error != nullptr, "conv: cannot allocate the error word");
  p.stat_sum = stat_sum;
  p.stat_sq  = stat_sq;
  p.accumulate = accumulate;
  p.taps = n_taps;
  p.cblocks = cin / 64;
  p.tw = box.tw; p.th = box.th; p.tn = box.tn;
  p.wo = static_cast<int>(out.w); p.ho = static_cast<int>(out.h); p.nb = static_cast<int>(out.n);
  p.cout = w_rows;
  p.n_tiles = CeilDiv(w_rows, bn);
  for (int i = 0; i < n_taps; ++i) p.tap[i] = taps[i];
  {
    const int64_t weights = static_cast<int64_t>(n_taps) * p.cblocks * bn * 128;  // one [bn x 64] block per K step
    const int base_smem = bn == 64 ? ConvCfg<64>::kSmemBytes : bn == 128 ? ConvCfg<128>::kSmemBytes : ConvCfg<256>::kSmemBytes;
    static const bool no_resident = getenv("TIPS_CONV_NO_RESIDENT_WEIGHTS") != nullptr;
    p.b_resident = (!no_resident && p.n_tiles == 1 && m_tiles >= 4 * NumSMs() && base_smem + weights <= kMaxSmemBytes)
                       ? static_cast<int>(weights) : 0;
  }
  switch (bn) {
    case 64: return LaunchTaps<64>(maps, p, s);
    case 256: return LaunchTaps<256>(maps, p, s);
    default: return LaunchTaps<128>(maps, p, s);
  }
}

// Tap list of a forward-style gather: input coordinate = stride * out + (f - pad).
int ForwardTaps(int r, int s, int stride, int pad, int cin, ConvTap* taps) {
  int n = 0;
  for (int fr = 0; fr < r; ++fr) {
    for (int fs = 0; fs < s; ++fs) {
      const int oh = fr - pad, ow = fs - pad;
      ConvTap t{};
      if (stride == 1) {
        t.dh = static_cast<int16_t>(oh); t.dw = static_cast<int16_t>(ow); t.map = 0;
      } else {
        const int bh = oh & 1, bw = ow & 1;
        t.dh = static_cast<int16_t>((oh - bh) / 2); t.dw = static_cast<int16_t>((ow - bw) / 2);
        t.map = static_cast<int16_t>(bh * 2 + bw);
      }
      t.kofs = (fr * s + fs) * cin;
      taps[n++] = t;
    }
  }
  return n;
}

// Weight gradient over arbitrary activation views and taps: dw[co, tap.kofs + ci] += sum_p dy[p, co] * x_view[p + tap].
int RunWgrad(const View& dyv, const View* xv, int n_views, const ConvTap* taps, int n_taps, int cin, int cout, int ldw,
             float* dw, cudaStream_t st) {
  TIPSK_REQUIRE(n_taps >= 1 && n_taps <= kMaxTaps, "conv: 1..9 filter taps are supported");
  WgradMaps maps;
  WgradParams p{};
  p.taps = n_taps;
  for (int i = 0; i < n_taps; ++i) p.tap[i] = taps[i];
  const int bn  = cin % 256 == 0 ? 256 : cin % 128 == 0 ? 128 : 64;
  const Box box = PickBox(static_cast<int>(dyv.w), static_cast<int>(dyv.h), static_cast<int>(dyv.n), true,
                          bn == 256 ? 64 : 128);
  int rc = MapOf(&maps.dy, dyv, box);
  if (rc) return rc;
  for (int b = 0; b < 4; ++b) {
    if (b < n_views) {
      rc = MapOf(&maps.x[b], xv[b], box);
      if (rc) return rc;
    } else {
      maps.x[b] = maps.x[0];
    }
  }
  p.error = ConvErrorWord();
  TIPSK_REQUIRE(p.error != nullptr, "conv: cannot allocate the error word");
  p.dw  = dw;
  p.ldw = ldw;
  // The 256 x 256 tile pays when each CTA still runs a long K loop after the pixel range is split over two waves
  // (measured: it wins on the linear layers' 16k-row contractions, it loses on the short pixel ranges of the
  // 14x14 and 7x7 convolutions, where it leaves too few CTAs).
  static const bool no_big = getenv("TIPS_WGRAD_NO_BM256") != nullptr;
  int mh = 1;
  if (!no_big && bn == 256 && cout % 256 == 0) {
    const int64_t kt    = static_cast<int64_t>(CeilDiv(dyv.w, box.tw)) * CeilDiv(dyv.h, box.th) * CeilDiv(dyv.n, box.tn);
    const int64_t base2 = static_cast<int64_t>(n_taps) * (cout / 256) * (cin / 256);
    const int64_t sp2   = std::max<int64_t>(1, 2 * NumSMs() / base2);
    if (kt / sp2 >= 32) mh = 2;
  }
  p.cout_tiles = CeilDiv(cout, kBM * mh);
  p.cin_tiles  = CeilDiv(cin, bn);
  p.tiles_w = CeilDiv(dyv.w, box.tw);
  p.tiles_h = CeilDiv(dyv.h, box.th);
  p.tiles_n = CeilDiv(dyv.n, box.tn);
  p.tw = box.tw; p.th = box.th; p.tn = box.tn;
  p.cout = cout; p.cin = cin;
  p.a_boxes = mh == 2 ? 4 : (cout <= 64 ? 1 : 2);
  const int64_t k_tiles = static_cast<int64_t>(p.tiles_w) * p.tiles_h * p.tiles_n;
  const int base = p.taps * p.cout_tiles * p.cin_tiles;
  int splits = 2 * NumSMs() / base;  // one CTA per SM at a time: at most two full waves, no straggler wave
  if (splits > k_tiles) splits = static_cast<int>(k_tiles);
  if (splits < 1) splits = 1;
  TIPSK_CUDA(cudaMemsetAsync(dw, 0, sizeof(float) * static_cast<size_t>(cout) * ldw, st));
  if (bn == 256 && mh == 2) return LaunchWgrad<256, 64, 2>(maps, p, splits, st);
  if (bn == 256) return LaunchWgrad<256, 64>(maps, p, splits, st);
  return bn == 128 ? LaunchWgrad<128, 128>(maps, p, splits, st) : LaunchWgrad<64, 128>(maps, p, splits, st);
}

// Copies a 3-channel NHWC image into the zero-padded 8-channel buffer of the stem convolution.
__global__ void __launch_bounds__(256)
StemPadKernel(const __nv_bfloat16* __restrict__ x, uint4* __restrict__ xp, int n, int h, int w, int hp, int wp) {
  const int64_t total = static_cast<int64_t>(n) * hp * wp;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int pw = static_cast<int>(i % wp);
    const int ph = static_cast<int>((i / wp) % hp);
    const int in = static_cast<int>(i / (static_cast<int64_t>(wp) * hp));
    const int ih = ph - 3, iw = pw - 3;
    alignas(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __float2bfloat16_rn(0.f);
    if (ih >= 0 && ih < h && iw >= 0 && iw < w) {
      const __nv_bfloat16* src = x + ((static_cast<int64_t>(in) * h + ih) * w + iw) * 3;
      v[0] = src[0]; v[1] = src[1]; v[2] = src[2];
    }
    xp[i] = *reinterpret_cast<const uint4*>(v);
  }
}

// Same for an fp32 image in NCHW layout, as an input pipeline delivers it: the layout change and the cast to
// bf16 happen inside the copy that the stem needs anyway.
__global__ void __launch_bounds__(256)
StemPadNchwKernel(const float* __restrict__ x, uint4* __restrict__ xp, int n, int h, int w, int hp, int wp) {
  const int64_t total = static_cast<int64_t>(n) * hp * wp;
  const int64_t plane = static_cast<int64_t>(h) * w;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int pw = static_cast<int>(i % wp);
    const int ph = static_cast<int>((i / wp) % hp);
    const int in = static_cast<int>(i / (static_cast<int64_t>(wp) * hp));
    const int ih = ph - 3, iw = pw - 3;
    alignas(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __float2bfloat16_rn(0.f);
    if (ih >= 0 && ih < h && iw >= 0 && iw < w) {
      const float* src = x + static_cast<int64_t>(in) * 3 * plane + static_cast<int64_t>(ih) * w + iw;
      v[0] = __float2bfloat16_rn(src[0]);
      v[1] = __float2bfloat16_rn(src[plane]);
      v[2] = __float2bfloat16_rn(src[2 * plane]);
    }
    xp[i] = *reinterpret_cast<const uint4*>(v);
  }
}

// The two row-parity views of the padded stem input (windows of 8 pixels = 64 elements every 2 pixels) and the
// seven filter-row taps.
void StemViewsAndTaps(const void* xp, int n, int hp, int wp, int ho, int wo, View* views, ConvTap* taps) {
  for (int b = 0; b < 2; ++b) {
    const char* base = static_cast<const char*>(xp) + static_cast<int64_t>(b) * wp * 8 * 2;
    views[b] = View{base, 64, wo, (hp - b + 1) / 2, n, 16, 2 * static_cast<int64_t>(wp) * 8,
                    static_cast<int64_t>(hp) * wp * 8};
  }
  for (int r = 0; r < 7; ++r) {
    ConvTap t{};
    t.dh = static_cast<int16_t>(r >> 1); t.dw = 0; t.map = static_cast<int16_t>(r & 1);
    t.kofs = r * 64;
    taps[r] = t;
  }
  (void)ho;
}

}  // namespace
}  // namespace tipsk

using namespace tipsk;

extern "C" {

/* 1 when the tcgen05 convolution kernels accept the problem. */
int tipsk_conv2d_supported(int cin, int cout, int r, int s, int stride, int pad) {
  return (cin % 64 == 0 && cout % 64 == 0 && r == s && (r == 1 || r == 3) && (stride == 1 || stride == 2) &&
          pad == r / 2) ? 1 : 0;
}

/* y[n, ho, wo, cout] = conv(x[n, h, w, cin], wgt[cout, r, s, cin]); bf16 NHWC, fp32 accumulation.
 * stat_sum / stat_sq (optional, fp32 [cout], zeroed by the caller) receive the per-channel sum and sum of
 * squares of the bf16 outputs. */
int tipsk_conv2d_fwd(const void* x, const void* wgt, void* y, int n, int h, int w, int cin, int cout, int r, int s,
                     int stride, int pad, float* stat_sum, float* stat_sq, void* stream) {
  TIPSK_REQUIRE(tipsk_conv2d_supported(cin, cout, r, s, stride, pad), "conv2d_fwd: unsupported shape");
  const int ho = (h + 2 * pad - r) / stride + 1, wo = (w + 2 * pad - s) / stride + 1;
  ConvTap taps[kMaxTaps];
  const int nt = ForwardTaps(r, s, stride, pad, cin, taps);
  View views[4];
  int nv = 1;
  View out = FullView(y, n, ho, wo, cout);
  if (stride == 1) {
    if (r == 1) {
      views[0] = FlatView(x, n, h, w, cin);
      out      = FlatView(y, n, ho, wo, cout);
    } else {
      views[0] = FullView(x, n, h, w, cin);
    }
  } else {
    nv = 4;
    for (int b = 0; b < 4; ++b) views[b] = PhaseView(x, n, h, w, cin, b >> 1, b & 1);
  }
  return RunTaps(views, nv, taps, nt, cin, wgt, cout, static_cast<int64_t>(r) * s * cin, out, stat_sum, stat_sq,
                 static_cast<cudaStream_t>(stream));
}

/* dx[n, h, w, cin] = data gradient; wgt_t is the weight permuted to [cin, r, s, cout].  With `accumulate` the
 * gradient is added to what dx already holds (the gradient of another consumer of the same activation). */
static int DgradImpl(const void* dy, const void* wgt_t, void* dx, int n, int h, int w, int cin, int cout, int r, int s,
                     int stride, int pad, int accumulate, int ohwi, void* stream);

int tipsk_conv2d_dgrad(const void* dy, const void* wgt_t, void* dx, int n, int h, int w, int cin, int cout, int r,
                       int s, int stride, int pad, int accumulate, void* stream) {
  return DgradImpl(dy, wgt_t, dx, n, h, w, cin, cout, r, s, stride, pad, accumulate, 0, stream);
}

/* The same data gradient from the weights as the forward pass takes them, wgt[cout, r, s, cin]: the kernel
 * contracts over the rows of that matrix (MN-major B operand), so no transposed copy of the weights is made. */
int tipsk_conv2d_dgrad_ohwi(const void* dy, const void* wgt, void* dx, int n, int h, int w, int cin, int cout, int r,
                            int s, int stride, int pad, int accumulate, void* stream) {
  return DgradImpl(dy, wgt, dx, n, h, w, cin, cout, r, s, stride, pad, accumulate, 1, stream);
}

static int DgradImpl(const void* dy, const void* wgt_t, void* dx, int n, int h, int w, int cin, int cout, int r, int s,
                     int stride, int pad, int accumulate, int ohwi, void* stream) {
  TIPSK_REQUIRE(tipsk_conv2d_supported(cin, cout, r, s, stride, pad), "conv2d_dgrad: unsupported shape");
  const int ho = (h + 2 * pad - r) / stride + 1, wo = (w + 2 * pad - s) / stride + 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // columns of the weight matrix and the width of one tap in it
  const int tap_cols   = ohwi ? cin : cout;
  const int64_t w_cols = static_cast<int64_t>(r) * s * tap_cols;
  if (stride == 1) {
    ConvTap taps[kMaxTaps];
    int nt = 0;
    for (int fr = 0; fr < r; ++fr)
      for (int fs = 0; fs < s; ++fs) {
        ConvTap t{};
        t.dh = static_cast<int16_t>(pad - fr); t.dw = static_cast<int16_t>(pad - fs); t.map = 0;
        t.kofs = (fr * s + fs) * tap_cols;
        taps[nt++] = t;
      }
    View in  = r == 1 ? FlatView(dy, n, ho, wo, cout) : FullView(dy, n, ho, wo, cout);
    View out = r == 1 ? FlatView(dx, n, h, w, cin) : FullView(dx, n, h, w, cin);
    return RunTaps(&in, 1, taps, nt, cout, wgt_t, cin, w_cols, out, nullptr, nullptr, st, accumulate, ohwi);
  }
  // stride 2: the input pixels of parity class (bh, bw) receive the taps with (b + pad - f) even
  const View in = FullView(dy, n, ho, wo, cout);
  if (r == 1 && !accumulate) {
    // a 1x1 filter only reaches the even pixels: the other three classes receive no gradient
    TIPSK_CUDA(cudaMemsetAsync(dx, 0, static_cast<size_t>(n) * h * w * cin * 2, st));
  }
  for (int b = 0; b < 4; ++b) {
    const int bh = b >> 1, bw = b & 1;
    ConvTap taps[kMaxTaps];
    int nt = 0;
    for (int fr = 0; fr < r; ++fr) {
      if ((bh + pad - fr) & 1) continue;
      for (int fs = 0; fs < s; ++fs) {
        if ((bw + pad - fs) & 1) continue;
        ConvTap t{};
        t.dh = static_cast<int16_t>((bh + pad - fr) / 2); t.dw = static_cast<int16_t>((bw + pad - fs) / 2); t.map = 0;
        t.kofs = (fr * s + fs) * tap_cols;
        taps[nt++] = t;
      }
    }
    if (nt == 0) continue;
    const View out = PhaseView(dx, n, h, w, cin, bh, bw);
    if (out.w <= 0 || out.h <= 0) continue;
    int rc = RunTaps(&in, 1, taps, nt, cout, wgt_t, cin, w_cols, out, nullptr, nullptr, st, accumulate, ohwi);
    if (rc) return rc;
  }
  return 0;
}

/* dw[cout, r, s, cin] (fp32, overwritten) = weight gradient of the convolution. */
int tipsk_conv2d_wgrad(const void* x, const void* dy, float* dw, int n, int h, int w, int cin, int cout, int r, int s,
                       int stride, int pad, void* stream) {
  TIPSK_REQUIRE(tipsk_conv2d_supported(cin, cout, r, s, stride, pad), "conv2d_wgrad: unsupported shape");
  const int ho = (h + 2 * pad - r) / stride + 1, wo = (w + 2 * pad - s) / stride + 1;
  ConvTap taps[kMaxTaps];
  const int nt = ForwardTaps(r, s, stride, pad, cin, taps);
  const bool flat = (r == 1 && stride == 1);
  const View dyv = flat ? FlatView(dy, n, ho, wo, cout) : FullView(dy, n, ho, wo, cout);
  View xv[4];
  int nv = 1;
  if (stride == 1) {
    xv[0] = flat ? FlatView(x, n, h, w, cin) : FullView(x, n, h, w, cin);
  } else {
    nv = 4;
    for (int b = 0; b < 4; ++b) xv[b] = PhaseView(x, n, h, w, cin, b >> 1, b & 1);
  }
  return RunWgrad(dyv, xv, nv, taps, nt, cin, cout, r * s * cin, dw, static_cast<cudaStream_t>(stream));
}

/* ---- the 7x7 / stride 2 / pad 3 stem on 3-channel images ----
 * The image is first copied into a zero-padded 8-channel buffer xp[n, hp, wp, 8] (pixel (h, w) at (h+3, w+3)).
 * Eight consecutive pixels of that buffer are 64 contiguous elements, so the 7 (+1 zero) horizontal taps of one
 * filter row form one 64-element K block; the tensor map walks the output columns with a stride of two pixels
 * (overlapping windows) and the filter rows are the taps of the ordinary kernel, split by row parity as for any
 * stride-2 convolution.  Weights come as [cout, 7, 8, 8] (horizontal tap 7 and channels 3..7 zero). */
int tipsk_stem_geometry(int h, int w, int* hp, int* wp, int* ho, int* wo) {
  *ho = (h + 6 - 7) / 2 + 1;
  *wo = (w + 6 - 7) / 2 + 1;
  *hp = h + 6 > 2 * (*ho - 1) + 7 ? h + 6 : 2 * (*ho - 1) + 7;
  int need = w + 6 > 2 * (*wo - 1) + 8 ? w + 6 : 2 * (*wo - 1) + 8;
  *wp = (need + 7) / 8 * 8;
  return 0;
}

int tipsk_stem_pad(const void* x, void* xp, int n, int h, int w, void* stream) {
  int hp, wp, ho, wo;
  tipsk_stem_geometry(h, w, &hp, &wp, &ho, &wo);
  const int64_t total = static_cast<int64_t>(n) * hp * wp;
  StemPadKernel<<<static_cast<int>(std::min<int64_t>((total + 255) / 256, NumSMs() * 16)), 256, 0,
                  static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                       static_cast<uint4*>(xp), n, h, w, hp, wp);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* x: [n, 3, h, w] fp32 (NCHW, contiguous) -> xp: the padded 8-channel bf16 buffer of the stem. */
int tipsk_stem_pad_nchw_f32(const void* x, void* xp, int n, int h, int w, void* stream) {
  int hp, wp, ho, wo;
  tipsk_stem_geometry(h, w, &hp, &wp, &ho, &wo);
  const int64_t total = static_cast<int64_t>(n) * hp * wp;
  StemPadNchwKernel<<<static_cast<int>(std::min<int64_t>((total + 255) / 256, NumSMs() * 16)), 256, 0,
                      static_cast<cudaStream_t>(stream)>>>(static_cast<const float*>(x), static_cast<uint4*>(xp), n, h,
                                                           w, hp, wp);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_stem_conv_fwd(const void* xp, const void* wgt_p, void* y, int n, int h, int w, int cout, float* stat_sum,
                        float* stat_sq, void* stream) {
  TIPSK_REQUIRE(cout % 64 == 0, "stem: the output channel count must be a multiple of 64");
  int hp, wp, ho, wo;
  tipsk_stem_geometry(h, w, &hp, &wp, &ho, &wo);
  View views[2];
  ConvTap taps[kMaxTaps];
  StemViewsAndTaps(xp, n, hp, wp, ho, wo, views, taps);
  return RunTaps(views, 2, taps, 7, 64, wgt_p, cout, 7 * 64, FullView(y, n, ho, wo, cout), stat_sum, stat_sq,
                 static_cast<cudaStream_t>(stream));
}

/* dw[cout, 7, 8, 8] (fp32, overwritten). */
int tipsk_stem_conv_wgrad(const void* xp, const void* dy, float* dw, int n, int h, int w, int cout, void* stream) {
  TIPSK_REQUIRE(cout % 64 == 0, "stem: the output channel count must be a multiple of 64");
  int hp, wp, ho, wo;
  tipsk_stem_geometry(h, w, &hp, &wp, &ho, &wo);
  View views[2];
  ConvTap taps[kMaxTaps];
  StemViewsAndTaps(xp, n, hp, wp, ho, wo, views, taps);
  return RunWgrad(FullView(dy, n, ho, wo, cout), views, 2, taps, 7, 64, cout, 7 * 64, dw,
                  static_cast<cudaStream_t>(stream));
}

/* Reads and clears the convolution error word (0 ok; 1/2/3/4 = which wait ran out). Synchronises. */
int tipsk_conv_status(void) {
  int32_t* w = ConvErrorWord();
  if (!w) return -7;
  int32_t v = 0;
  if (cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -7;
  if (v) cudaMemset(w, 0, sizeof(v));
  return v;
}

}  // extern "C"
