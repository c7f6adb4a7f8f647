// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = act(A[M,K] * B[N,K]^T + bias).
//
// Both operands are K-major (row-major A and row-major B = "TN"), which is the
// layout of a linear layer's forward pass (activations [M,K], weight [N,K]).
// Pipeline inside one CTA (192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor.2d (no multicast) brings a
//               128 x 64 tile of A and a BN x 64 tile of B per stage into
//               128-byte-swizzled shared memory, signalling an mbarrier
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (kind::f16,
//               M=128, N=BN, K=16) four times per stage with shared-memory
//               descriptors, accumulating in TMEM; tcgen05.commit releases the
//               stage back to the producer and finally signals the epilogue
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator rows out of TMEM, add
//               the bias, apply the activation, convert to bf16 and store
// Every mbarrier wait is bounded; on a timeout the kernel sets an error word,
// frees its TMEM and returns.
//
// The reference contains no GEMM (its only math is an elementwise loop,
// tips/core/common/vec.h:194-216); this kernel serves the CTR model's MLP and
// the BERT-shaped encoder's linear layers.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "kernels/common.cuh"
#include "kernels/tcgen05.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

struct GemmParams {
  __nv_bfloat16* c;
  __nv_bfloat16* pre;          // optional: pre-activation output
  const __nv_bfloat16* bias;   // optional, [N]
  int32_t* error;              // device error word
  int m, n, k;
  int ldc;
  int act;                     // 0 none, 1 relu, 2 gelu
  int tma_store;               // 1: the output goes through shared memory and the TMA store unit
  int accumulate;              // 1 (TMA store path only): add to what C holds, with a reduce-add store
  int bias_vec;                // 1: bias is 16-byte aligned, so eight values can be read with one load
};

// Eight consecutive bias values as floats (zeros without a bias): one 16-byte load when the bias is 16-byte aligned
// and the eight columns exist, scalar loads at a ragged edge.
__device__ __forceinline__ void LoadBias8(const GemmParams& p, int col, float (&bv)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) bv[j] = 0.f;
  if (p.bias == nullptr) return;
  if (p.bias_vec && col + 8 <= p.n) {
    const uint4 q = *reinterpret_cast<const uint4*>(p.bias + col);
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) bv[j] = __bfloat162float(b[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (col + j < p.n) bv[j] = __bfloat162float(p.bias[col + j]);
  }
}

// Hands a staged 64-column box to the TMA store unit: a plain store, or a bf16 reduce-add into global memory.
__device__ __forceinline__ void TmaStoreOrAdd2D(const CUtensorMap* tmap, int x, int y, const void* smem_src, int add) {
  if (add) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(x), "r"(y), "r"(SmemAddr(smem_src))
                 : "memory");
  } else {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(x), "r"(y), "r"(SmemAddr(smem_src))
                 : "memory");
  }
}

template <int BN>
struct GemmCfg {
  // Up to 128 columns: three stages (<= 97 KB) so that two CTAs fit on an SM and one CTA's epilogue
  // overlaps the other's main loop; 256 columns: one CTA per SM with four stages.
  static constexpr int kStages     = BN >= 256 ? 4 : 3;
  static constexpr int kABytes     = kBM * kBK * 2;
  static constexpr int kBBytes     = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols   = BN < 32 ? 32 : BN;
  static constexpr int kSmemBytes  = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// kBMn: B is given as [K, N] row-major (the contraction runs over its rows), loaded as BN/64 boxes of
// [64 x 64] and read by the MMA as an MN-major operand; used for dx = dy * W without transposing W.
template <int BN, bool kBMn = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
GemmTnKernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const __grid_constant__ CUtensorMap tmap_c, GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar  = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* tmem_full = empty_bar + Cfg::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0   = blockIdx.y * kBM;
  const int n0   = blockIdx.x * BN;
  const int num_k = (p.k + kBK - 1) / kBK;

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
        const uint32_t parity = ((kt / Cfg::kStages) & 1) ^ 1;
        if (!MbarWait(&empty_bar[s], parity)) {
          atomicExch(p.error, 1);
          break;
        }
        uint8_t* a_dst = smem + s * Cfg::kStageBytes;
        uint8_t* b_dst = a_dst + Cfg::kABytes;
        MbarExpectTx(&full_bar[s], Cfg::kStageBytes);
        TmaLoad2D(a_dst, &tmap_a, kt * kBK, m0, &full_bar[s]);
        if (kBMn) {
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) TmaLoad2D(b_dst + j * 8192, &tmap_b, n0 + j * 64, kt * kBK, &full_bar[s]);
        } else {
          TmaLoad2D(b_dst, &tmap_b, kt * kBK, n0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (kBMn ? (1u << 16) : 0u) |
                                 (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      bool ok = true;
      for (int kt = 0; kt < num_k && ok; ++kt) {
        const int s = kt % Cfg::kStages;
        const uint32_t parity = (kt / Cfg::kStages) & 1;
        if (!MbarWait(&full_bar[s], parity)) {
          atomicExch(p.error, 2);
          ok = false;
          break;
        }
        TcFenceAfter();
        const uint32_t a_addr = SmemAddr(smem + s * Cfg::kStageBytes);
        const uint32_t b_addr = a_addr + Cfg::kABytes;
        const uint64_t adesc  = SmemDescSw128(a_addr);
        const uint64_t bdesc  = kBMn ? SmemDescMnSw128(b_addr, 8192) : SmemDescSw128(b_addr);
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) {
          // advancing 16 elements (32 bytes) along K inside the swizzle row = +2 in the address field;
          // for the MN-major B sixteen K rows = 2048 bytes = +128
          UmmaBf16(tmem_base, adesc + 2 * k, bdesc + (kBMn ? 128 : 2) * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
        }
        UmmaCommit(&empty_bar[s]);
      }
      UmmaCommit(tmem_full);  // arrives when every MMA issued so far has completed
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const bool ok = MbarWait(tmem_full, 0);
    if (!ok && lane == 0) atomicExch(p.error, 3);
    TcFenceAfter();
    const int row = m0 + q * 32 + lane;
    if (p.tma_store) {
      if (ok) {
      // Coalesced path: convert in registers, stage the tile in shared memory in the 128-byte-swizzled
      // layout of the output tensor map (the pipeline stages are free once every MMA has completed),
      // then one thread hands 64-column boxes to the TMA store unit.  Rows / columns beyond M / N are
      // clipped by the TMA unit.
      const int r = q * 32 + lane;  // row inside the tile
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t acc[32];
        TmemLoad32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c * 32), acc);
        const int col0 = n0 + c * 32;
        uint8_t* box   = smem + (c >> 1) * (kBM * 128);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          alignas(16) __nv_bfloat16 o[8];
#pragma unroll
          float bv[8];
          LoadBias8(p, col0 + g * 8, bv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float x = __uint_as_float(acc[g * 8 + j]) + bv[j];
            if (p.act == 1) x = fmaxf(x, 0.f);
            else if (p.act == 2) x = 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
            o[j] = __float2bfloat16_rn(x);
          }
          const int chunk = (c & 1) * 4 + g;  // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(box + r * 128 + ((chunk ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(o);
        }
      }
      }
      // every epilogue warp reaches this barrier, whether or not its wait succeeded
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
      if (ok && warp == 2 && lane == 0) {
#pragma unroll 1
        for (int b = 0; b < BN / 64; ++b) {
          if (n0 + b * 64 < p.n) {
            TmaStoreOrAdd2D(&tmap_c, n0 + b * 64, m0, smem + b * (kBM * 128), p.accumulate);
          }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
    } else if (ok) {
#pragma unroll 1
      for (int c = 0; c < BN / 32 + (BN % 32 ? 1 : 0); ++c) {
        uint32_t r[32];
        if (BN >= 32 || c == 0) {
          TmemLoad32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c * 32), r);
        }
        const int col0 = n0 + c * 32;
        if (row < p.m && col0 < p.n) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(r[j]);
            if (p.bias && col0 + j < p.n) v[j] += __bfloat162float(p.bias[col0 + j]);
          }
          __nv_bfloat16* crow = p.c + static_cast<int64_t>(row) * p.ldc + col0;
          __nv_bfloat16* prow = p.pre ? p.pre + static_cast<int64_t>(row) * p.ldc + col0 : nullptr;
          const bool vec_ok = (p.ldc % 8 == 0) && (col0 + 32 <= p.n) && (BN >= 32);
          if (vec_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              alignas(16) __nv_bfloat16 o[8];
              if (prow) {
                alignas(16) __nv_bfloat16 pr[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) pr[j] = __float2bfloat16_rn(v[g * 8 + j]);
                *reinterpret_cast<uint4*>(prow + g * 8) = *reinterpret_cast<uint4*>(pr);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float x = v[g * 8 + j];
                if (p.act == 1) x = fmaxf(x, 0.f);
                else if (p.act == 2) x = 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
                o[j] = __float2bfloat16_rn(x);
              }
              *reinterpret_cast<uint4*>(crow + g * 8) = *reinterpret_cast<uint4*>(o);
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.n && j < BN; ++j) {
              float x = v[j];
              if (prow) prow[j] = __float2bfloat16_rn(x);
              if (p.act == 1) x = fmaxf(x, 0.f);
              else if (p.act == 2) x = 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
              crow[j] = __float2bfloat16_rn(x);
            }
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

// ---------------------------------------------------------------- persistent variant
// One CTA per SM walks over the output tiles (tile = blockIdx.x + i * gridDim.x, N fastest).  The
// accumulator is double-buffered in TMEM, so the epilogue of tile i (TMEM -> registers -> swizzled
// shared memory -> TMA store) overlaps the TMA loads and MMAs of tile i+1.  Used when there are more
// tiles than SMs and the output qualifies for the TMA store path.
template <int BN>
struct PersistCfg {
  static constexpr int kStages     = BN >= 256 ? 3 : 5;
  static constexpr int kABytes     = kBM * kBK * 2;
  static constexpr int kBBytes     = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = kBM * BN * 2;
  static constexpr int kTmemCols   = 2 * BN;  // two accumulators
  static constexpr int kSmemBytes  = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

template <int BN, bool kBMn = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
GemmTnPersistentKernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_c, GemmParams p) {
  using Cfg = PersistCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem    = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* full_bar   = reinterpret_cast<uint64_t*>(staging + Cfg::kStagingBytes);
  uint64_t* empty_bar  = full_bar + Cfg::kStages;
  uint64_t* tmem_full  = empty_bar + Cfg::kStages;  // [2]
  uint64_t* tmem_empty = tmem_full + 2;             // [2]
  uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k   = (p.k + kBK - 1) / kBK;
  const int tiles_n = (p.n + BN - 1) / BN;
  const int tiles_m = (p.m + kBM - 1) / kBM;
  const int num_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      MbarInit(&full_bar[s], 1);
      MbarInit(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      MbarInit(&tmem_full[b], 1);
      MbarInit(&tmem_empty[b], 4);  // one arrival per epilogue warp
    }
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
      uint32_t it = 0;  // running k-stage counter over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * kBM, n0 = (tile % tiles_n) * BN;
        for (int kt = 0; kt < num_k; ++kt, ++it) {
          const int s = it % Cfg::kStages;
          if (!MbarWait(&empty_bar[s], ((it / Cfg::kStages) & 1) ^ 1)) {
            atomicExch(p.error, 1);
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * Cfg::kStageBytes;
          MbarExpectTx(&full_bar[s], Cfg::kStageBytes);
          TmaLoad2D(a_dst, &tmap_a, kt * kBK, m0, &full_bar[s]);
          if (kBMn) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              TmaLoad2D(a_dst + Cfg::kABytes + j * 8192, &tmap_b, n0 + j * 64, kt * kBK, &full_bar[s]);
          } else {
            TmaLoad2D(a_dst + Cfg::kABytes, &tmap_b, kt * kBK, n0, &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (kBMn ? (1u << 16) : 0u) |
                                 (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      uint32_t it = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        if (!MbarWait(&tmem_empty[buf], ((local >> 1) & 1) ^ 1)) {  // the epilogue has drained this accumulator
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
          const uint64_t bdesc  = kBMn ? SmemDescMnSw128(a_addr + Cfg::kABytes, 8192) : SmemDescSw128(a_addr + Cfg::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            UmmaBf16(tmem_d, adesc + 2 * k, bdesc + (kBMn ? 128 : 2) * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          UmmaCommit(&empty_bar[s]);
        }
        if (ok) UmmaCommit(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile / tiles_n) * kBM, n0 = (tile % tiles_n) * BN;
      const int buf = local & 1;
      if (ok && !MbarWait(&tmem_full[buf], (local >> 1) & 1)) {
        if (lane == 0) atomicExch(p.error, 3);
        ok = false;
      }
      TcFenceAfter();
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t acc[32];
          TmemLoad32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * BN + c * 32), acc);
          const int col0 = n0 + c * 32;
          uint8_t* box   = staging + (c >> 1) * (kBM * 128);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            alignas(16) __nv_bfloat16 o[8];
#pragma unroll
            float bv[8];
            LoadBias8(p, col0 + g * 8, bv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float x = __uint_as_float(acc[g * 8 + j]) + bv[j];
              if (p.act == 1) x = fmaxf(x, 0.f);
              else if (p.act == 2) x = 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
              o[j] = __float2bfloat16_rn(x);
            }
            const int chunk = (c & 1) * 4 + g;
            *reinterpret_cast<uint4*>(box + r * 128 + ((chunk ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(o);
          }
        }
        // this warp is done with the accumulator: hand it back to the MMA warp
        TcFenceBefore();
        __syncwarp();
        if (lane == 0) MbarArrive(&tmem_empty[buf]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        if (ok) {
#pragma unroll 1
          for (int b = 0; b < BN / 64; ++b) {
            if (n0 + b * 64 < p.n) {
              TmaStoreOrAdd2D(&tmap_c, n0 + b * 64, m0, staging + b * (kBM * 128), p.accumulate);
            }
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staging may be overwritten afterwards
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
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

// ---------------------------------------------------------------- 256 x 256 tiles
// A 128 x 256 tile streams 48 KB per K block from L2 for 512 tensor-core clocks of work, and an SM takes 64 bytes per
// clock from L2: the main loop is load-bound at two thirds of the tensor peak.  Here one CTA owns a 256 x 256 tile: two
// A blocks share one B block, 64 KB per 1024 clocks of work, so loads and MMAs balance.  The two accumulators fill all
// 512 TMEM columns, so the epilogue of a tile cannot overlap the MMAs of the next (only its loads); the variant is
// chosen for long K and grids that fill whole waves.  Persistent, one CTA per SM.
struct Big256Cfg {
  static constexpr int kBN         = 256;
  static constexpr int kStages     = 3;
  static constexpr int kABytes     = kBM * kBK * 2;          // one 128-row half
  static constexpr int kBBytes     = kBN * kBK * 2;
  static constexpr int kStageBytes = 2 * kABytes + kBBytes;  // 64 KB
  static constexpr int kStagingBytes = 2 * kBM * 128;        // two 64-column boxes, used alternately
  static constexpr int kTmemCols   = 512;
  static constexpr int kSmemBytes  = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

template <bool kBMn>
__global__ void __launch_bounds__(kGemmThreads, 1)
GemmTn256Kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_c, GemmParams p) {
  using Cfg = Big256Cfg;
  constexpr int BN = Cfg::kBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem    = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* full_bar   = reinterpret_cast<uint64_t*>(staging + Cfg::kStagingBytes);
  uint64_t* empty_bar  = full_bar + Cfg::kStages;
  uint64_t* tmem_full  = empty_bar + Cfg::kStages;
  uint64_t* tmem_empty = tmem_full + 1;
  uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(tmem_empty + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k   = (p.k + kBK - 1) / kBK;
  const int tiles_n = (p.n + BN - 1) / BN;
  const int tiles_m = (p.m + 2 * kBM - 1) / (2 * kBM);
  const int num_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      MbarInit(&full_bar[s], 1);
      MbarInit(&empty_bar[s], 1);
    }
    MbarInit(tmem_full, 1);
    MbarInit(tmem_empty, 4);  // one arrival per epilogue warp
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * 2 * kBM, n0 = (tile % tiles_n) * BN;
        for (int kt = 0; kt < num_k; ++kt, ++it) {
          const int s = it % Cfg::kStages;
          if (!MbarWait(&empty_bar[s], ((it / Cfg::kStages) & 1) ^ 1)) {
            atomicExch(p.error, 1);
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * Cfg::kStageBytes;
          uint8_t* b_dst = a_dst + 2 * Cfg::kABytes;
          MbarExpectTx(&full_bar[s], Cfg::kStageBytes);
          TmaLoad2D(a_dst, &tmap_a, kt * kBK, m0, &full_bar[s]);
          TmaLoad2D(a_dst + Cfg::kABytes, &tmap_a, kt * kBK, m0 + kBM, &full_bar[s]);
          if (kBMn) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) TmaLoad2D(b_dst + j * 8192, &tmap_b, n0 + j * 64, kt * kBK, &full_bar[s]);
          } else {
            TmaLoad2D(b_dst, &tmap_b, kt * kBK, n0, &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (kBMn ? (1u << 16) : 0u) |
                                 (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      uint32_t it = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        if (!MbarWait(tmem_empty, (local & 1) ^ 1)) {  // the epilogue has drained both accumulators
          atomicExch(p.error, 4);
          break;
        }
        TcFenceAfter();
        for (int kt = 0; kt < num_k; ++kt, ++it) {
          const int s = it % Cfg::kStages;
          if (!MbarWait(&full_bar[s], (it / Cfg::kStages) & 1)) {
            atomicExch(p.error, 2);
            ok = false;
            break;
          }
          TcFenceAfter();
          const uint32_t a_addr = SmemAddr(smem + s * Cfg::kStageBytes);
          const uint32_t b_addr = a_addr + 2 * Cfg::kABytes;
          const uint64_t bdesc  = kBMn ? SmemDescMnSw128(b_addr, 8192) : SmemDescSw128(b_addr);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint64_t adesc = SmemDescSw128(a_addr + h * Cfg::kABytes);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              UmmaBf16(tmem_base + static_cast<uint32_t>(h * BN), adesc + 2 * k, bdesc + (kBMn ? 128 : 2) * k, idesc,
                       (kt > 0 || k > 0) ? 1u : 0u);
          }
          UmmaCommit(&empty_bar[s]);
        }
        if (ok) UmmaCommit(tmem_full);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    constexpr int kBoxes = BN / 64;
    int local = 0;
    uint32_t boxes_done = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile / tiles_n) * 2 * kBM, n0 = (tile % tiles_n) * BN;
      if (ok && !MbarWait(tmem_full, local & 1)) {
        if (lane == 0) atomicExch(p.error, 3);
        ok = false;
      }
      TcFenceAfter();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const uint32_t tsrc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(h * BN);
        uint32_t acc[2][32];
        if (ok) TmemLoad32Async(tsrc, acc[0]);
#pragma unroll
        for (int b = 0; b < kBoxes; ++b, ++boxes_done) {
          uint8_t* box = staging + (boxes_done & 1) * (kBM * 128);
          // the store that read this staging box two boxes ago must have finished reading it
          if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          NamedBarSync(1, 128);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c = 2 * b + half;
            if (ok) {
              // the 32 bias values of this chunk as four 16-byte loads, in flight while the TMEM load completes
              // (N is a multiple of 256 here, so the chunk is never ragged)
              const int col0 = n0 + c * 32;
              uint4 bq[4] = {};
              if (p.bias) {
#pragma unroll
                for (int g = 0; g < 4; ++g) bq[g] = *reinterpret_cast<const uint4*>(p.bias + col0 + g * 8);
              }
              TmemLoadWait(acc[c & 1]);
              if (c + 1 < BN / 32) TmemLoad32Async(tsrc + static_cast<uint32_t>((c + 1) * 32), acc[(c + 1) & 1]);
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                alignas(16) __nv_bfloat16 o[8];
                const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&bq[g]);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float x = __uint_as_float(acc[c & 1][g * 8 + j]);
                  if (p.bias) x += __bfloat162float(bb[j]);
                  if (p.act == 1) x = fmaxf(x, 0.f);
                  else if (p.act == 2) x = 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
                  o[j] = __float2bfloat16_rn(x);
                }
                const int chunk = half * 4 + g;
                *reinterpret_cast<uint4*>(box + r * 128 + ((chunk ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(o);
              }
            }
          }
          if (h == 1 && b == kBoxes - 1 && ok) {  // both accumulators are drained
            TcFenceBefore();
            __syncwarp();
            if (lane == 0) MbarArrive(tmem_empty);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          NamedBarSync(1, 128);
          if (warp == 2 && lane == 0) {
            if (ok && n0 + b * 64 < p.n && m0 + h * kBM < p.m)
              TmaStoreOrAdd2D(&tmap_c, n0 + b * 64, m0 + h * kBM, box, p.accumulate);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
    }
    if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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

// Row-major [rows, cols] bf16 matrix with leading dimension ld (elements); box = 64 x box_rows, 128B swizzle.
int MakeTmap(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeFn enc = GetEncodeFn();
  if (!enc) return SetError(-7, "cuTensorMapEncodeTiled is not available from the driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return SetError(-2, "gemm: operand base must be 16-byte aligned");
  if ((ld * 2) % 16 != 0) return SetError(-2, "gemm: operand row stride must be a multiple of 16 bytes");
  cuuint64_t dims[2]    = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2]     = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2]    = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return SetError(-7, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return 0;
}

int32_t* GemmErrorWord() {
  static int32_t* word = nullptr;
  if (!word) {
    if (cudaMalloc(reinterpret_cast<void**>(&word), sizeof(int32_t)) != cudaSuccess) return nullptr;
    cudaMemset(word, 0, sizeof(int32_t));
  }
  return word;
}

template <int BN, bool kBMn = false>
int LaunchGemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
               cudaStream_t s) {
  using Cfg = GemmCfg<BN>;
  static bool configured = false;
  if (!configured) {
    TIPSK_CUDA(cudaFuncSetAttribute(GemmTnKernel<BN, kBMn>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    TIPSK_CUDA(cudaFuncSetAttribute(GemmTnKernel<BN, kBMn>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    cudaSharedmemCarveoutMaxShared));
    configured = true;
  }
  dim3 grid((p.n + BN - 1) / BN, (p.m + kBM - 1) / kBM);
  GemmTnKernel<BN, kBMn><<<grid, kGemmThreads, Cfg::kSmemBytes, s>>>(ta, tb, tc, p);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

template <int BN, bool kBMn = false>
int LaunchGemmPersistent(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                         cudaStream_t s) {
  using Cfg = PersistCfg<BN>;
  static bool configured = false;
  if (!configured) {
    TIPSK_CUDA(cudaFuncSetAttribute(GemmTnPersistentKernel<BN, kBMn>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes));
    configured = true;
  }
  const int tiles = ((p.n + BN - 1) / BN) * ((p.m + kBM - 1) / kBM);
  const int grid  = tiles < NumSMs() ? tiles : NumSMs();
  GemmTnPersistentKernel<BN, kBMn><<<grid, kGemmThreads, Cfg::kSmemBytes, s>>>(ta, tb, tc, p);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

template <bool kBMn>
int LaunchGemm256(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                  cudaStream_t s) {
  using Cfg = Big256Cfg;
  static bool configured = false;
  if (!configured) {
    TIPSK_CUDA(cudaFuncSetAttribute(GemmTn256Kernel<kBMn>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  const int tiles = ((p.n + 255) / 256) * ((p.m + 255) / 256);
  const int grid  = tiles < NumSMs() ? tiles : NumSMs();
  GemmTn256Kernel<kBMn><<<grid, kGemmThreads, Cfg::kSmemBytes, s>>>(ta, tb, tc, p);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

// Whether the 256 x 256 tile variant should take the problem: long enough K for the exposed epilogue to be a small
// share of a tile, and a tile count that fills its waves.
bool Prefer256(int m, int n, int k) {
  static const bool off = getenv("TIPS_GEMM_NO_BM256") != nullptr;
  if (off || n % 256 != 0 || m < 512 || k < 2048) return false;  // measured: no gain at K = 1024, +17..19 % at K = 4096
  const int64_t tiles = static_cast<int64_t>((m + 255) / 256) * (n / 256);
  const int64_t sms   = NumSMs();
  const int64_t waves = (tiles + sms - 1) / sms;
  const double fill   = static_cast<double>(tiles) / static_cast<double>(waves * sms);
  return fill >= 0.80;
}

}  // namespace
}  // namespace tipsk

using namespace tipsk;

extern "C" {

/* 1 when tipsk_gemm_bf16 accepts the problem (alignment of the leading dimensions). */
int tipsk_gemm_supported(int m, int n, int k, int lda, int ldb) {
  return (m > 0 && n > 0 && k > 0 && lda % 8 == 0 && ldb % 8 == 0) ? 1 : 0;
}

/* C[m,n] = act(A[m,k] * B[n,k]^T + bias); bf16 in, fp32 accumulate in TMEM, bf16 out.
 * lda/ldb/ldc are leading dimensions in elements; `pre` (optional) receives the value before the activation. */
int tipsk_gemm_bf16(const void* a, const void* b, void* c, const void* bias, void* pre, int m, int n, int k, int lda,
                    int ldb, int ldc, int act, void* stream) {
  TIPSK_REQUIRE(tipsk_gemm_supported(m, n, k, lda, ldb), "gemm: lda and ldb must be multiples of 8 elements");
  int bn = 128;
  if (n <= 16) bn = 16;
  else if (n <= 32) bn = 32;
  else if (n <= 64) bn = 64;
  else if (n % 256 == 0 && (static_cast<int64_t>(m) / kBM) * (n / 256) >= NumSMs()) bn = 256;
  CUtensorMap ta, tb;
  int rc = MakeTmap(&ta, a, m, k, lda, kBM);
  if (rc) return rc;
  rc = MakeTmap(&tb, b, n, k, ldb, bn);
  if (rc) return rc;
  GemmParams p;
  p.c     = static_cast<__nv_bfloat16*>(c);
  p.pre   = static_cast<__nv_bfloat16*>(pre);
  p.bias  = static_cast<const __nv_bfloat16*>(bias);
  p.error = GemmErrorWord();
  TIPSK_REQUIRE(p.error != nullptr, "gemm: cannot allocate the error word");
  p.m = m; p.n = n; p.k = k; p.ldc = ldc; p.act = act; p.accumulate = 0;
  p.bias_vec = (bias != nullptr && reinterpret_cast<uintptr_t>(bias) % 16 == 0) ? 1 : 0;
  // The coalesced store path needs 64-column boxes and a 16-byte aligned, 16-byte strided output.
  p.tma_store = (bn >= 64 && pre == nullptr && ldc % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0) ? 1 : 0;
  CUtensorMap tc = ta;
  if (p.tma_store) {
    rc = MakeTmap(&tc, c, m, n, ldc, kBM);
    if (rc) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p.tma_store && bn == 256 && Prefer256(m, n, k) && reinterpret_cast<uintptr_t>(bias) % 16 == 0)
    return LaunchGemm256<false>(ta, tb, tc, p, s);
  // More tiles than SMs and a TMA-storable output: the persistent kernel overlaps epilogue and main loop.
  static const bool no_persist = getenv("TIPS_GEMM_NO_PERSISTENT") != nullptr;
  if (!no_persist && p.tma_store && (bn == 128 || bn == 256)) {
    const int64_t tiles = static_cast<int64_t>((n + bn - 1) / bn) * ((m + kBM - 1) / kBM);
    // Measured on B200: the overlap pays when the epilogue is a visible share of a tile (K <= 2048) and
    // there are enough tiles to fill several waves; otherwise two independent CTAs per SM do better.
    if (tiles >= 3 * NumSMs() && k <= 2048) {
      if (bn == 256) return LaunchGemmPersistent<256>(ta, tb, tc, p, s);
      return LaunchGemmPersistent<128>(ta, tb, tc, p, s);
    }
  }
  switch (bn) {
    case 16: return LaunchGemm<16>(ta, tb, tc, p, s);
    case 32: return LaunchGemm<32>(ta, tb, tc, p, s);
    case 64: return LaunchGemm<64>(ta, tb, tc, p, s);
    case 256: return LaunchGemm<256>(ta, tb, tc, p, s);
    default: return LaunchGemm<128>(ta, tb, tc, p, s);
  }
}

/* C[m,n] = A[m,k] * B[k,n]: B row-major with the contraction over its rows (no transposed copy is made; the MMA
 * reads it as an MN-major operand).  Serves dx = dy * W of a linear layer with W stored [out, in].  n >= 64.
 * With `accumulate` the product is added (in bf16, by reduce-add stores) to what C already holds. */
int tipsk_gemm_bf16_nn(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb, int ldc,
                       int accumulate, void* stream) {
  TIPSK_REQUIRE(m > 0 && n >= 64 && k > 0 && lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0,
                "gemm_nn: leading dimensions must be multiples of 8 elements and n >= 64");
  TIPSK_REQUIRE(reinterpret_cast<uintptr_t>(c) % 16 == 0, "gemm_nn: output must be 16-byte aligned");
  int bn = 128;
  if (n <= 64) bn = 64;
  else if (n % 256 == 0 && (static_cast<int64_t>(m) / kBM) * (n / 256) >= NumSMs()) bn = 256;
  CUtensorMap ta, tb, tc;
  int rc = MakeTmap(&ta, a, m, k, lda, kBM);
  if (rc) return rc;
  rc = MakeTmap(&tb, b, k, n, ldb, kBK);  // boxes of 64 contraction rows x 64 columns
  if (rc) return rc;
  rc = MakeTmap(&tc, c, m, n, ldc, kBM);
  if (rc) return rc;
  GemmParams p;
  p.c = static_cast<__nv_bfloat16*>(c);
  p.pre = nullptr;
  p.bias = nullptr;
  p.error = GemmErrorWord();
  TIPSK_REQUIRE(p.error != nullptr, "gemm: cannot allocate the error word");
  p.m = m; p.n = n; p.k = k; p.ldc = ldc; p.act = 0; p.tma_store = 1; p.accumulate = accumulate ? 1 : 0;
  p.bias_vec = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 256 && Prefer256(m, n, k)) return LaunchGemm256<true>(ta, tb, tc, p, s);
  if (bn != 64) {
    const int64_t tiles = static_cast<int64_t>((n + bn - 1) / bn) * ((m + kBM - 1) / kBM);
    if (tiles >= 3 * NumSMs() && k <= 2048) {
      if (bn == 256) return LaunchGemmPersistent<256, true>(ta, tb, tc, p, s);
      return LaunchGemmPersistent<128, true>(ta, tb, tc, p, s);
    }
  }
  switch (bn) {
    case 64: return LaunchGemm<64, true>(ta, tb, tc, p, s);
    case 256: return LaunchGemm<256, true>(ta, tb, tc, p, s);
    default: return LaunchGemm<128, true>(ta, tb, tc, p, s);
  }
}

/* Reads and clears the GEMM error word (0 ok; 1/2/3 = producer / MMA / epilogue wait ran out). Synchronises. */
int tipsk_gemm_status(void) {
  int32_t* w = GemmErrorWord();
  if (!w) return -7;
  int32_t v = 0;
  if (cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -7;
  if (v) cudaMemset(w, 0, sizeof(v));
  return v;
}

}  // extern "C"
