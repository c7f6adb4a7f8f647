// Collectives over NVLink peer memory: allreduce (one-shot and two-shot, P2P and
// NVLS multimem), allgatherv and broadcast, each fused with the scale / cast /
// staging copies around it so that one launch takes a tensor from its producer
// to its consumer.
//
// These replace the reference's MPI calls on host memory: MPI_Allreduce
// (tips/core/collective/utils.h:52-67), MPI_Allgatherv (utils.h:83-128) and
// MPI_Bcast (utils.h:130-134).
//
// Work decomposition.  The tensor is cut into 16-byte vectors and the vectors
// into tiles; tile t belongs to block (t mod grid) ON EVERY RANK.  Inside a tile
// each rank owns one sub-tile (two-shot) which it reduces from all peers and
// pushes back to all peers.  Because a block only ever touches tiles of its own
// index, the only synchronisation needed is a barrier between same-index blocks
// of the ranks: no grid-wide sync, no host round trip.  Three phases:
//   A  copy the local input into this rank's window (skipped when it is there)
//   -- barrier --
//   B  reduce: own sub-tile from every peer's window -> scaled -> every peer's window
//      (one-shot: whole tile from every peer -> local output)
//   -- barrier --
//   C  copy the reduced tile from the window to the local output (skipped in place)
//
// The same kernels run with gridDim.y = number of ranks on ONE device when the
// rank windows all live there (used by the single-GPU tests); then the launch is
// cooperative so that all blocks are co-resident.
#include "kernels/comm.cuh"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "kernels/common.cuh"
#include "kernels/optim_rules.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

constexpr int kCommThreads = 512;
// Vectors per thread per sub-tile.  The in-switch reduction needs one load per vector, so it can keep
// many more in flight per thread than the peer-load path, which holds one vector per rank.
constexpr int kUnrollP2p   = 2;
constexpr int kUnrollMc    = 8;
constexpr int UnrollOf(bool multimem) { return multimem ? kUnrollMc : kUnrollP2p; }
constexpr int SubTileOf(bool multimem) { return kCommThreads * UnrollOf(multimem); }  // vectors per rank per tile
constexpr int kCopyUnroll  = 4;                       // vectors in flight per thread in the copy loops
constexpr int kCopyTile    = kCommThreads * kCopyUnroll * 2;  // vectors per tile of allgather / broadcast

struct RankArgs {
  CommCtx ctx;
  const char* src;  // local input, or null when the data already sits in the window
  char* dst;        // local output, or null to leave the result in the window
  uint64_t win_off; // byte offset of the buffer inside every rank's window
};
struct CommLaunch {
  RankArgs r[kMaxRanks];
};

template <typename T>
struct Acc;  // accumulate a 16-byte vector of T in fp32 (floats) or natively (ints / double)

template <>
struct Acc<float> {
  float a[4];
  __device__ void Zero() { a[0] = a[1] = a[2] = a[3] = 0.f; }
  __device__ void Add(const U4& v) {
    a[0] += __uint_as_float(v.x); a[1] += __uint_as_float(v.y);
    a[2] += __uint_as_float(v.z); a[3] += __uint_as_float(v.w);
  }
  __device__ void Max(const U4& v, bool first) {
    float b[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
    for (int i = 0; i < 4; ++i) a[i] = first ? b[i] : fmaxf(a[i], b[i]);
  }
  __device__ void Min(const U4& v, bool first) {
    float b[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
    for (int i = 0; i < 4; ++i) a[i] = first ? b[i] : fminf(a[i], b[i]);
  }
  __device__ void Mul(const U4& v, bool first) {
    float b[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
    for (int i = 0; i < 4; ++i) a[i] = first ? b[i] : a[i] * b[i];
  }
  __device__ void Scale(float s) { for (int i = 0; i < 4; ++i) a[i] *= s; }
  __device__ U4 Pack() const {
    return U4{__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3])};
  }
};

template <typename H>  // __nv_bfloat16 or __half
struct Acc16 {
  float a[8];
  __device__ static float Lo(uint32_t w);
  __device__ void Zero() { for (int i = 0; i < 8; ++i) a[i] = 0.f; }
  __device__ void Unpack(const U4& v, float (&b)[8]) const {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    for (int i = 0; i < 4; ++i) {
      H lo, hi;
      uint16_t l = static_cast<uint16_t>(w[i] & 0xffffu), h = static_cast<uint16_t>(w[i] >> 16);
      memcpy(&lo, &l, 2);
      memcpy(&hi, &h, 2);
      b[2 * i]     = ToFloat<H>(lo);
      b[2 * i + 1] = ToFloat<H>(hi);
    }
  }
  __device__ void Add(const U4& v) { float b[8]; Unpack(v, b); for (int i = 0; i < 8; ++i) a[i] += b[i]; }
  __device__ void Max(const U4& v, bool first) { float b[8]; Unpack(v, b); for (int i = 0; i < 8; ++i) a[i] = first ? b[i] : fmaxf(a[i], b[i]); }
  __device__ void Min(const U4& v, bool first) { float b[8]; Unpack(v, b); for (int i = 0; i < 8; ++i) a[i] = first ? b[i] : fminf(a[i], b[i]); }
  __device__ void Mul(const U4& v, bool first) { float b[8]; Unpack(v, b); for (int i = 0; i < 8; ++i) a[i] = first ? b[i] : a[i] * b[i]; }
  __device__ void Scale(float s) { for (int i = 0; i < 8; ++i) a[i] *= s; }
  __device__ U4 Pack() const {
    uint32_t w[4];
    for (int i = 0; i < 4; ++i) {
      H lo = FromFloat<H>(a[2 * i]), hi = FromFloat<H>(a[2 * i + 1]);
      uint16_t l, h;
      memcpy(&l, &lo, 2);
      memcpy(&h, &hi, 2);
      w[i] = static_cast<uint32_t>(l) | (static_cast<uint32_t>(h) << 16);
    }
    return U4{w[0], w[1], w[2], w[3]};
  }
};
template <> struct Acc<__nv_bfloat16> : Acc16<__nv_bfloat16> {};
template <> struct Acc<__half> : Acc16<__half> {};

template <typename I, int N>  // native accumulation for int32 (N=4), int64 / double (N=2)
struct AccNative {
  I a[N];
  __device__ void Zero() { for (int i = 0; i < N; ++i) a[i] = I(0); }
  __device__ void Get(const U4& v, I (&b)[N]) const { memcpy(b, &v, 16); }
  __device__ void Add(const U4& v) { I b[N]; Get(v, b); for (int i = 0; i < N; ++i) a[i] += b[i]; }
  __device__ void Max(const U4& v, bool first) { I b[N]; Get(v, b); for (int i = 0; i < N; ++i) a[i] = first ? b[i] : (a[i] > b[i] ? a[i] : b[i]); }
  __device__ void Min(const U4& v, bool first) { I b[N]; Get(v, b); for (int i = 0; i < N; ++i) a[i] = first ? b[i] : (a[i] < b[i] ? a[i] : b[i]); }
  __device__ void Mul(const U4& v, bool first) { I b[N]; Get(v, b); for (int i = 0; i < N; ++i) a[i] = first ? b[i] : a[i] * b[i]; }
  __device__ void Scale(float s) { if (s != 1.f) for (int i = 0; i < N; ++i) a[i] = static_cast<I>(static_cast<double>(a[i]) * s); }
  __device__ U4 Pack() const { U4 v; memcpy(&v, a, 16); return v; }
};
template <> struct Acc<int32_t> : AccNative<int32_t, 4> {};
template <> struct Acc<int64_t> : AccNative<int64_t, 2> {};
template <> struct Acc<double> : AccNative<double, 2> {};

template <typename T> __device__ __forceinline__ U4 MultimemLdReduce(const void* p);
template <> __device__ __forceinline__ U4 MultimemLdReduce<float>(const void* p) { return MultimemLdReduceF32(p); }
template <> __device__ __forceinline__ U4 MultimemLdReduce<__nv_bfloat16>(const void* p) { return MultimemLdReduceBf16(p); }
template <> __device__ __forceinline__ U4 MultimemLdReduce<__half>(const void* p) { return MultimemLdReduceF16(p); }
template <> __device__ __forceinline__ U4 MultimemLdReduce<int32_t>(const void* p) { return LdSys(p); }
template <> __device__ __forceinline__ U4 MultimemLdReduce<int64_t>(const void* p) { return LdSys(p); }
template <> __device__ __forceinline__ U4 MultimemLdReduce<double>(const void* p) { return LdSys(p); }

__device__ __forceinline__ uint32_t NextEpoch(const CommCtx& ctx, int channel, int block) {
  return ctx.epochs[channel * kMaxCommBlocks + block] + 1;
}
__device__ __forceinline__ void SaveEpoch(const CommCtx& ctx, int channel, int block, uint32_t last) {
  __syncthreads();
  if (threadIdx.x == 0) ctx.epochs[channel * kMaxCommBlocks + block] = last;
}

// Copies `nbytes` between local buffers for the vectors of tiles owned by this
// block; the ragged tail (nbytes % 16) is handled bytewise, and the rest of a
// partial vector in the window is zero-filled when `zero_pad`.
__device__ __forceinline__ void CopyOwnedTiles(char* dst, const char* src, uint64_t nbytes, uint64_t nvec,
                                               uint64_t tile_vecs, bool zero_pad) {
  const uint64_t ntiles = (nvec + tile_vecs - 1) / tile_vecs;
  const bool aligned    = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0;
  for (uint64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t lo = t * tile_vecs;
    const uint64_t hi = lo + tile_vecs < nvec ? lo + tile_vecs : nvec;
    if (aligned && hi * 16 <= nbytes) {
      // full vectors: four loads in flight per thread before the stores
      for (uint64_t v = lo + threadIdx.x; v < hi; v += static_cast<uint64_t>(blockDim.x) * kCopyUnroll) {
        U4 q[kCopyUnroll];
#pragma unroll
        for (int u = 0; u < kCopyUnroll; ++u) {
          const uint64_t i = v + static_cast<uint64_t>(u) * blockDim.x;
          if (i < hi) q[u] = *reinterpret_cast<const U4*>(src + i * 16);
        }
#pragma unroll
        for (int u = 0; u < kCopyUnroll; ++u) {
          const uint64_t i = v + static_cast<uint64_t>(u) * blockDim.x;
          if (i < hi) *reinterpret_cast<U4*>(dst + i * 16) = q[u];
        }
      }
      continue;
    }
    for (uint64_t v = lo + threadIdx.x; v < hi; v += blockDim.x) {
      const uint64_t off = v * 16;
      if (aligned && off + 16 <= nbytes) {
        *reinterpret_cast<U4*>(dst + off) = *reinterpret_cast<const U4*>(src + off);
      } else {
        for (uint64_t b = off; b < off + 16; ++b) {
          if (b < nbytes) dst[b] = src[b];
          else if (zero_pad) dst[b] = 0;
        }
      }
    }
  }
}

// op: 0 sum, 1 max, 2 min, 3 prod
template <typename T, bool kMultimem, bool kOneShot>
__global__ void __launch_bounds__(kCommThreads)
AllreduceKernel(CommLaunch args, int channel, uint64_t nbytes, int op, float prescale, float postscale) {
  const RankArgs& ra = args.r[blockIdx.y];
  const CommCtx& ctx = ra.ctx;
  const int n        = ctx.nranks;
  const int block    = blockIdx.x;
  constexpr int kUnroll  = UnrollOf(kMultimem);
  constexpr int kSubTile = SubTileOf(kMultimem);
  constexpr int kSrcs    = kMultimem ? 1 : kMaxRanks;  // vectors held per output vector
  const uint64_t nvec      = (nbytes + 15) / 16;
  const uint64_t tile_vecs = static_cast<uint64_t>(kSubTile) * n;
  const uint64_t ntiles    = (nvec + tile_vecs - 1) / tile_vecs;
  char* my_win = ctx.peer[ctx.rank] + ra.win_off;
  uint32_t epoch = NextEpoch(ctx, channel, block);

  if (ra.src) CopyOwnedTiles(my_win, ra.src, nbytes, nvec, tile_vecs, true);
  bool ok = BlockBarrier(ctx, channel, block, epoch, 1);

  if (ok) {
    const float sum_scale = prescale * postscale;
    for (uint64_t t = block; t < ntiles; t += gridDim.x) {
      const uint64_t tile_lo = t * tile_vecs;
      const uint64_t sub_lo  = kOneShot ? tile_lo : tile_lo + static_cast<uint64_t>(ctx.rank) * kSubTile;
      const uint64_t sub_n   = kOneShot ? tile_vecs : kSubTile;
      for (uint64_t base = threadIdx.x; base < sub_n; base += blockDim.x * kUnroll) {
        U4 in[kUnroll][kSrcs];
        uint64_t vec[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          vec[u] = sub_lo + base + static_cast<uint64_t>(u) * blockDim.x;
          if (base + static_cast<uint64_t>(u) * blockDim.x >= sub_n || vec[u] >= nvec) {
            vec[u] = ~0ull;
            continue;
          }
          const uint64_t off = ra.win_off + vec[u] * 16;
          if constexpr (kMultimem) {  // the host selects this variant for sums only
            in[u][0] = MultimemLdReduce<T>(ctx.mc + off);
          } else {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < n) in[u][r] = LdSys(ctx.peer[(ctx.rank + r) % n] + off);
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (vec[u] == ~0ull) continue;
          U4 out;
          Acc<T> acc;
          if constexpr (kMultimem) {
            acc.Zero();
            acc.Add(in[u][0]);
            acc.Scale(sum_scale);
          } else {
            acc.Zero();
#pragma unroll
            for (int r = 0; r < kSrcs; ++r) {
              if (r >= n) break;
              if (op == 0) acc.Add(in[u][r]);
              else if (op == 1) acc.Max(in[u][r], r == 0);
              else if (op == 2) acc.Min(in[u][r], r == 0);
              else acc.Mul(in[u][r], r == 0);
            }
            acc.Scale(op == 3 ? postscale : sum_scale);
          }
          out = acc.Pack();
          const uint64_t off = ra.win_off + vec[u] * 16;
          if (kOneShot) {  // the host side only selects one-shot when a local output exists
            if (vec[u] * 16 + 16 <= nbytes && (reinterpret_cast<uintptr_t>(ra.dst) & 15) == 0) {
              *reinterpret_cast<U4*>(ra.dst + vec[u] * 16) = out;
            } else {
              const char* ob = reinterpret_cast<const char*>(&out);
              for (uint64_t b = 0; b < 16 && vec[u] * 16 + b < nbytes; ++b) ra.dst[vec[u] * 16 + b] = ob[b];
            }
          } else if (kMultimem) {
            MultimemSt(ctx.mc + off, out);
          } else {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < n) StSys(ctx.peer[(ctx.rank + r) % n] + off, out);
          }
        }
      }
    }
  }
  ok = BlockBarrier(ctx, channel, block, epoch + 1, 2) && ok;
  if (ok && !kOneShot && ra.dst) CopyOwnedTiles(ra.dst, my_win, nbytes, nvec, tile_vecs, false);
  SaveEpoch(ctx, channel, block, epoch + 1);
}

// ---------------------------------------------------------------------------
// Allreduce fused with the optimizer step.  The gradient bucket and the
// parameter buffer both live in the window.  Every rank owns the same share of
// the 16-byte vectors as in the two-shot allreduce (sub-tile `rank` of every
// tile) and keeps the fp32 master weights and the optimizer state of that share
// only, packed densely: vector j of tile t sits at [t * kUpdSubTile + j].
//   -- barrier: every rank has packed its gradients --
//   reduce own share of the gradients (in the switch, or from every peer)
//   -> scale -> SGD-momentum / Adam on the master share -> cast -> store the new
//   parameters into EVERY rank's parameter buffer (multicast store, or one store per peer)
//   -- barrier: every rank's share has arrived, the parameters are complete --
// The reduced gradient is never written anywhere, the optimizer reads and
// writes 1/N of its state per rank, and no separate optimizer launch follows.
constexpr int kUpdSubTile = 2048;  // vectors per rank per tile; also the layout unit of the state shards

struct UpdateArgs {
  float* master;       // this rank's share of the fp32 weights
  float* s0;           // momentum buffer / first moment
  float* s1;           // second moment (Adam)
  uint64_t param_off;  // byte offset of the parameter buffer inside every rank's window
};
struct UpdateLaunch {
  UpdateArgs r[kMaxRanks];
  SgdParams sgd;
  AdamParams adam;
};

template <int kE>
__device__ __forceinline__ void LoadState(const float* p, float (&v)[kE]) {
#pragma unroll
  for (int i = 0; i < kE; i += 4) {
    const float4 q = *reinterpret_cast<const float4*>(p + i);
    v[i] = q.x; v[i + 1] = q.y; v[i + 2] = q.z; v[i + 3] = q.w;
  }
}
template <int kE>
__device__ __forceinline__ void StoreState(float* p, const float (&v)[kE]) {
#pragma unroll
  for (int i = 0; i < kE; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
}

template <typename T, bool kMultimem, bool kAdam>
__global__ void __launch_bounds__(kCommThreads)
AllreduceUpdateKernel(CommLaunch args, UpdateLaunch upd, int channel, uint64_t nbytes, float scale) {
  const RankArgs& ra   = args.r[blockIdx.y];
  const UpdateArgs& ua = upd.r[blockIdx.y];
  const CommCtx& ctx   = ra.ctx;
  const int n          = ctx.nranks;
  const int block      = blockIdx.x;
  constexpr int kE      = 16 / sizeof(T);
  constexpr int kUnroll = kMultimem ? 4 : 2;  // one reduced vector per load in the switch: more of them in flight
  constexpr int kSrcs   = kMultimem ? 1 : kMaxRanks;
  const uint64_t nvec      = nbytes / 16;  // the host side only accepts whole vectors
  const uint64_t tile_vecs = static_cast<uint64_t>(kUpdSubTile) * n;
  const uint64_t ntiles    = (nvec + tile_vecs - 1) / tile_vecs;
  uint32_t epoch = NextEpoch(ctx, channel, block);

  bool ok = BlockBarrier(ctx, channel, block, epoch, 1);
  if (ok) {
    for (uint64_t t = block; t < ntiles; t += gridDim.x) {
      const uint64_t sub_lo = t * tile_vecs + static_cast<uint64_t>(ctx.rank) * kUpdSubTile;
      for (uint32_t base = threadIdx.x; base < kUpdSubTile; base += kCommThreads * kUnroll) {
        U4 in[kUnroll][kSrcs];
        bool live[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const uint64_t vec = sub_lo + base + u * kCommThreads;
          live[u] = base + u * kCommThreads < kUpdSubTile && vec < nvec;
          if (!live[u]) continue;
          const uint64_t off = ra.win_off + vec * 16;
          if constexpr (kMultimem) {
            in[u][0] = MultimemLdReduce<T>(ctx.mc + off);
          } else {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < n) in[u][r] = LdSys(ctx.peer[(ctx.rank + r) % n] + off);
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (!live[u]) continue;
          const uint32_t j   = base + u * kCommThreads;
          const uint64_t vec = sub_lo + j;
          Acc<T> acc;
          acc.Zero();
#pragma unroll
          for (int r = 0; r < kSrcs; ++r)
            if (r < n) acc.Add(in[u][r]);
          acc.Scale(scale);
          const uint64_t at = (t * kUpdSubTile + j) * kE;  // element offset inside the state share
          float w[kE], m[kE], v[kE];
          LoadState<kE>(ua.master + at, w);
          if constexpr (kAdam) {
            LoadState<kE>(ua.s0 + at, m);
            LoadState<kE>(ua.s1 + at, v);
#pragma unroll
            for (int e = 0; e < kE; ++e) AdamUpdate(w[e], m[e], v[e], acc.a[e], upd.adam);
            StoreState<kE>(ua.s0 + at, m);
            StoreState<kE>(ua.s1 + at, v);
          } else {
            const bool has_m = upd.sgd.momentum != 0.f;
            if (has_m && !upd.sgd.first_step) LoadState<kE>(ua.s0 + at, m);
#pragma unroll
            for (int e = 0; e < kE; ++e) SgdUpdate(w[e], m[e], acc.a[e], upd.sgd);
            if (has_m) StoreState<kE>(ua.s0 + at, m);
          }
          StoreState<kE>(ua.master + at, w);
#pragma unroll
          for (int e = 0; e < kE; ++e) acc.a[e] = w[e];
          const U4 out       = acc.Pack();
          const uint64_t off = ua.param_off + vec * 16;
          if constexpr (kMultimem) {
            MultimemSt(ctx.mc + off, out);
          } else {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < n) StSys(ctx.peer[(ctx.rank + r) % n] + off, out);
          }
        }
      }
    }
  }
  BlockBarrier(ctx, channel, block, epoch + 1, 2);
  SaveEpoch(ctx, channel, block, epoch + 1);
}

// Allgatherv: phase A copies the local slab into the window, phase B pulls every
// rank's slab from its window into the local output at its displacement.
struct GatherSizes {
  uint64_t bytes[kMaxRanks];
  uint64_t displ[kMaxRanks];
};

__global__ void __launch_bounds__(kCommThreads)
AllgathervKernel(CommLaunch args, int channel, GatherSizes sizes) {
  const RankArgs& ra = args.r[blockIdx.y];
  const CommCtx& ctx = ra.ctx;
  const int n        = ctx.nranks;
  const int block    = blockIdx.x;
  char* my_win       = ctx.peer[ctx.rank] + ra.win_off;
  uint32_t epoch     = NextEpoch(ctx, channel, block);
  const uint64_t my_bytes = sizes.bytes[ctx.rank];
  CopyOwnedTiles(my_win, ra.src, my_bytes, (my_bytes + 15) / 16, kCopyTile, true);
  bool ok = BlockBarrier(ctx, channel, block, epoch, 1);
  if (ok) {
    for (int i = 0; i < n; ++i) {
      const int r          = (ctx.rank + i) % n;
      const uint64_t bytes = sizes.bytes[r];
      const uint64_t nvec  = (bytes + 15) / 16;
      const uint64_t ntiles = (nvec + kCopyTile - 1) / kCopyTile;
      const char* from     = ctx.peer[r] + ra.win_off;
      char* to             = ra.dst + sizes.displ[r];
      const bool aligned   = (reinterpret_cast<uintptr_t>(to) & 15) == 0;
      for (uint64_t t = block; t < ntiles; t += gridDim.x) {
        const uint64_t lo = t * kCopyTile;
        const uint64_t hi = lo + kCopyTile < nvec ? lo + kCopyTile : nvec;
        for (uint64_t v = lo + threadIdx.x; v < hi; v += static_cast<uint64_t>(blockDim.x) * kCopyUnroll) {
          U4 q[kCopyUnroll];
#pragma unroll
          for (int u = 0; u < kCopyUnroll; ++u) {  // several peer loads in flight per thread
            const uint64_t i = v + static_cast<uint64_t>(u) * blockDim.x;
            if (i < hi) q[u] = LdSys(from + i * 16);
          }
#pragma unroll
          for (int u = 0; u < kCopyUnroll; ++u) {
            const uint64_t i = v + static_cast<uint64_t>(u) * blockDim.x;
            if (i >= hi) continue;
            if (aligned && i * 16 + 16 <= bytes) {
              *reinterpret_cast<U4*>(to + i * 16) = q[u];
            } else {
              const char* qb = reinterpret_cast<const char*>(&q[u]);
              for (uint64_t b = 0; b < 16 && i * 16 + b < bytes; ++b) to[i * 16 + b] = qb[b];
            }
          }
        }
      }
    }
  }
  BlockBarrier(ctx, channel, block, epoch + 1, 2);
  SaveEpoch(ctx, channel, block, epoch + 1);
}

// One 16-byte vector of a byte buffer that may be unaligned and may end inside the vector (the rest reads as zero).
__device__ __forceinline__ U4 LoadVecBytes(const char* base, uint64_t v, uint64_t nbytes, bool aligned) {
  if (aligned && v * 16 + 16 <= nbytes) return *reinterpret_cast<const U4*>(base + v * 16);
  U4 q;
  char* qb = reinterpret_cast<char*>(&q);
  for (uint64_t b = 0; b < 16; ++b) qb[b] = v * 16 + b < nbytes ? base[v * 16 + b] : 0;
  return q;
}
__device__ __forceinline__ void StoreVecBytes(char* base, uint64_t v, uint64_t nbytes, bool aligned, const U4& q) {
  if (aligned && v * 16 + 16 <= nbytes) {
    *reinterpret_cast<U4*>(base + v * 16) = q;
    return;
  }
  const char* qb = reinterpret_cast<const char*>(&q);
  for (uint64_t b = 0; b < 16 && v * 16 + b < nbytes; ++b) base[v * 16 + b] = qb[b];
}

// Allgatherv for small slabs, by pushing: every rank stores its slab straight from its input into every rank's
// window (one multimem store per vector, or one store per peer), one barrier, and everyone copies the gathered
// slabs from its own window to its output.  Against the pulling kernel above it saves the copy of the input into
// the window and, above all, the chain of peer loads that a block walks rank after rank: with slabs of a few
// hundred KB that chain, not the bytes, is the time.  Tiles are small so that a 64 KB slab already spreads over
// several blocks.  Tile t of every slab belongs to block t % grid on every rank, for the stores and for the copy.
constexpr int kPushUnroll = 1;
constexpr int kPushTile   = kCommThreads * kPushUnroll;  // vectors (8 KB)

template <bool kMultimem>
__global__ void __launch_bounds__(kCommThreads)
AllgatherPushKernel(CommLaunch args, int channel, GatherSizes sizes) {
  const RankArgs& ra = args.r[blockIdx.y];
  const CommCtx& ctx = ra.ctx;
  const int n        = ctx.nranks;
  const int block    = blockIdx.x;
  char* my_win       = ctx.peer[ctx.rank] + ra.win_off;
  uint32_t epoch     = NextEpoch(ctx, channel, block);
  uint64_t wdispl[kMaxRanks];  // where rank r's slab starts inside the staging area (16-byte aligned)
  {
    uint64_t at = 0;
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      wdispl[r] = at;
      if (r < n) at += (sizes.bytes[r] + 15) & ~15ull;
    }
  }
  {
    const uint64_t bytes  = sizes.bytes[ctx.rank];
    const uint64_t nvec   = (bytes + 15) / 16;
    const uint64_t ntiles = (nvec + kPushTile - 1) / kPushTile;
    const bool aligned    = (reinterpret_cast<uintptr_t>(ra.src) & 15) == 0;
    const uint64_t base   = ra.win_off + wdispl[ctx.rank];
    for (uint64_t t = block; t < ntiles; t += gridDim.x) {
      const uint64_t lo = t * kPushTile;
      const uint64_t hi = lo + kPushTile < nvec ? lo + kPushTile : nvec;
      U4 q[kPushUnroll];
#pragma unroll
      for (int u = 0; u < kPushUnroll; ++u) {
        const uint64_t v = lo + threadIdx.x + static_cast<uint64_t>(u) * blockDim.x;
        if (v < hi) q[u] = LoadVecBytes(ra.src, v, bytes, aligned);
      }
#pragma unroll
      for (int u = 0; u < kPushUnroll; ++u) {
        const uint64_t v = lo + threadIdx.x + static_cast<uint64_t>(u) * blockDim.x;
        if (v >= hi) continue;
        if (kMultimem) {
          MultimemSt(ctx.mc + base + v * 16, q[u]);
        } else {
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < n) StSys(ctx.peer[(ctx.rank + r) % n] + base + v * 16, q[u]);
        }
      }
    }
  }
  const bool ok = BlockBarrier(ctx, channel, block, epoch, 1);
  if (ok && ra.dst) {
    for (int r = 0; r < n; ++r) {
      const uint64_t bytes  = sizes.bytes[r];
      const uint64_t nvec   = (bytes + 15) / 16;
      const uint64_t ntiles = (nvec + kPushTile - 1) / kPushTile;
      const char* from      = my_win + wdispl[r];
      char* to              = ra.dst + sizes.displ[r];
      const bool aligned    = (reinterpret_cast<uintptr_t>(to) & 15) == 0;
      for (uint64_t t = block; t < ntiles; t += gridDim.x) {
        const uint64_t lo = t * kPushTile;
        const uint64_t hi = lo + kPushTile < nvec ? lo + kPushTile : nvec;
        U4 q[kPushUnroll];
#pragma unroll
        for (int u = 0; u < kPushUnroll; ++u) {
          const uint64_t v = lo + threadIdx.x + static_cast<uint64_t>(u) * blockDim.x;
          if (v < hi) q[u] = *reinterpret_cast<const U4*>(from + v * 16);
        }
#pragma unroll
        for (int u = 0; u < kPushUnroll; ++u) {
          const uint64_t v = lo + threadIdx.x + static_cast<uint64_t>(u) * blockDim.x;
          if (v < hi) StoreVecBytes(to, v, bytes, aligned, q[u]);
        }
      }
    }
  }
  BlockBarrier(ctx, channel, block, epoch + 1, 2);  // nobody overwrites a window that is still being copied out
  SaveEpoch(ctx, channel, block, epoch + 1);
}

// Broadcast of a large message as scatter + allgather.  One root that stores everything to everybody is bound by
// what a single source can feed into the switch; here the root sends every tile to ONE rank, its owner (tiles
// rotate over the ranks), and the owner passes it on to the others (one multimem store, or a store per peer), so
// that all ranks feed the switch.  The message is cut into chunks and the three steps run as a pipeline with one
// barrier per step:
//   step i:  root      scatters chunk i                                  (S)
//            the rest  forward their tiles of chunk i-1 to everybody      (G)  and write them to their output,
//                      copy the other tiles of chunk i-2 from their own window to their output  (C)
// G waits on the links and C on local memory, so half of the block's threads do one and half the other.
// The root writes its output from the registers it sends; tiles the root owns itself go to everybody at once.
// A barrier drains the block's stores and waits for the slowest rank, and a block moves nothing meanwhile; blocks
// only meet the same block of the other ranks, so the blocks run in four lanes whose chunk boundaries are a
// quarter of a chunk apart: while one lane waits the other three keep the links busy.
constexpr int kBcastLanes = 4;

template <bool kMultimem>
__global__ void __launch_bounds__(kCommThreads)
BroadcastScatterKernel(CommLaunch args, int channel, uint64_t nbytes, int root, int nchunks) {
  const RankArgs& ra = args.r[blockIdx.y];
  const CommCtx& ctx = ra.ctx;
  const int n        = ctx.nranks;
  const int block    = blockIdx.x;
  const int grid     = gridDim.x;
  const int me       = ctx.rank;
  char* my_win       = ctx.peer[me] + ra.win_off;
  uint32_t epoch     = NextEpoch(ctx, channel, block);
  const uint64_t nvec   = (nbytes + 15) / 16;
  const uint64_t ntiles = (nvec + kCopyTile - 1) / kCopyTile;
  const bool src_aligned = me == root && (reinterpret_cast<uintptr_t>(ra.src) & 15) == 0;
  const bool dst_aligned = ra.dst != nullptr && (reinterpret_cast<uintptr_t>(ra.dst) & 15) == 0;
  const bool write_dst   = ra.dst != nullptr && !(me == root && ra.dst == ra.src);
  // Chunks of this block's lane: [lo(c), lo(c+1)) in tiles; the first chunk of lanes 1..3 is shorter.
  const int lane           = block % kBcastLanes;
  const uint64_t per_chunk = (ntiles + nchunks - 1) / nchunks;
  const uint64_t shift     = per_chunk * lane / kBcastLanes;
  const int my_chunks      = static_cast<int>((ntiles + shift + per_chunk - 1) / per_chunk);
  auto chunk_lo = [&](int c) {
    if (c <= 0) return static_cast<uint64_t>(0);
    const uint64_t at = per_chunk * c - shift;
    return at < ntiles ? at : ntiles;
  };
  // Tiles of [t_lo, t_hi) that belong to this block are first, first + grid, ...; tile t is owned by rank (t / grid) % n.
  auto first_of = [&](uint64_t t_lo) { return t_lo + (static_cast<uint64_t>(block) + grid - t_lo % grid) % grid; };

  // S: the root reads a tile of its input and sends it to the tile's owner.
  auto scatter = [&](uint64_t t_lo, uint64_t t_hi) {
    for (uint64_t t = first_of(t_lo); t < t_hi; t += grid) {
      const int owner   = static_cast<int>((t / grid) % n);
      const uint64_t lo = t * kCopyTile;
      const uint64_t hi = lo + kCopyTile < nvec ? lo + kCopyTile : nvec;
      for (uint64_t v0 = lo + threadIdx.x; v0 < hi; v0 += static_cast<uint64_t>(blockDim.x) * kCopyUnroll) {
        U4 q[kCopyUnroll];
#pragma unroll
        for (int u = 0; u < kCopyUnroll; ++u) {
          const uint64_t v = v0 + static_cast<uint64_t>(u) * blockDim.x;
          if (v < hi) q[u] = LoadVecBytes(ra.src, v, nbytes, src_aligned);
        }
#pragma unroll
        for (int u = 0; u < kCopyUnroll; ++u) {
          const uint64_t v = v0 + static_cast<uint64_t>(u) * blockDim.x;
          if (v >= hi) continue;
          const uint64_t off = ra.win_off + v * 16;
          if (owner != root) {
            StSys(ctx.peer[owner] + off, q[u]);
          } else if (kMultimem) {
            MultimemSt(ctx.mc + off, q[u]);
          } else {
#pragma unroll
            for (int r = 1; r < kMaxRanks; ++r)
              if (r < n) StSys(ctx.peer[(me + r) % n] + off, q[u]);
          }
          if (write_dst) StoreVecBytes(ra.dst, v, nbytes, dst_aligned, q[u]);
        }
      }
    }
  };
  // G (forward = true): my tiles go from my window to everybody and to my output.
  // C (forward = false): the others' tiles go from my window to my output.  `tid` of `nthr` threads take part.
  auto drain = [&](uint64_t t_lo, uint64_t t_hi, bool forward, int tid, int nthr) {
    for (uint64_t t = first_of(t_lo); t < t_hi; t += grid) {
      if ((static_cast<int>((t / grid) % n) == me) != forward) continue;
      const uint64_t lo = t * kCopyTile;
      const uint64_t hi = lo + kCopyTile < nvec ? lo + kCopyTile : nvec;
      for (uint64_t v0 = lo + tid; v0 < hi; v0 += static_cast<uint64_t>(nthr) * kCopyUnroll) {
        U4 q[kCopyUnroll];
#pragma unroll
        for (int u = 0; u < kCopyUnroll; ++u) {
          const uint64_t v = v0 + static_cast<uint64_t>(u) * nthr;
          if (v < hi) q[u] = *reinterpret_cast<const U4*>(my_win + v * 16);
        }
#pragma unroll
        for (int u = 0; u < kCopyUnroll; ++u) {
          const uint64_t v = v0 + static_cast<uint64_t>(u) * nthr;
          if (v >= hi) continue;
          if (forward) {
            const uint64_t off = ra.win_off + v * 16;
            if (kMultimem) {
              MultimemSt(ctx.mc + off, q[u]);  // also lands in the root's window and in mine: same bytes, unread
            } else {
#pragma unroll
              for (int r = 1; r < kMaxRanks; ++r) {
                const int to = (me + r) % n;
                if (r < n && to != root) StSys(ctx.peer[to] + off, q[u]);
              }
            }
          }
          if (write_dst) StoreVecBytes(ra.dst, v, nbytes, dst_aligned, q[u]);
        }
      }
    }
  };

  bool ok = BlockBarrier(ctx, channel, block, epoch, 1);  // the windows are free
  for (int it = 0; it < my_chunks + 2; ++it) {
    if (ok && me == root && it < my_chunks) scatter(chunk_lo(it), chunk_lo(it + 1));
    if (ok && me != root) {
      const bool has_g = it >= 1 && it <= my_chunks;
      const bool has_c = it >= 2 && write_dst;
      const int half   = blockDim.x / 2;
      if (has_g && has_c) {
        if (static_cast<int>(threadIdx.x) < half) drain(chunk_lo(it - 1), chunk_lo(it), true, threadIdx.x, half);
        else drain(chunk_lo(it - 2), chunk_lo(it - 1), false, threadIdx.x - half, blockDim.x - half);
      } else if (has_g) {
        drain(chunk_lo(it - 1), chunk_lo(it), true, threadIdx.x, blockDim.x);
      } else if (has_c) {
        drain(chunk_lo(it - 2), chunk_lo(it - 1), false, threadIdx.x, blockDim.x);
      }
    }
    ok = BlockBarrier(ctx, channel, block, epoch + 1 + it, 2) && ok;
  }
  SaveEpoch(ctx, channel, block, epoch + 2 + my_chunks);
}

// Broadcast: the root writes its data into every rank's window (one multimem store per vector, or one P2P store per
// peer), then everyone copies from its own window to its output.  The message can be cut into chunks with a barrier
// after each, so that the other ranks copy chunk c out of their windows while the root stores chunk c+1; the root
// fills its own output from the registers it is sending.
template <bool kMultimem>
__global__ void __launch_bounds__(kCommThreads)
BroadcastKernel(CommLaunch args, int channel, uint64_t nbytes, int root, int nchunks) {
  const RankArgs& ra = args.r[blockIdx.y];
  const CommCtx& ctx = ra.ctx;
  const int n        = ctx.nranks;
  const int block    = blockIdx.x;
  const int grid     = gridDim.x;
  char* my_win       = ctx.peer[ctx.rank] + ra.win_off;
  uint32_t epoch     = NextEpoch(ctx, channel, block);
  const uint64_t nvec   = (nbytes + 15) / 16;
  const uint64_t ntiles = (nvec + kCopyTile - 1) / kCopyTile;
  const bool src_aligned = ctx.rank == root && (reinterpret_cast<uintptr_t>(ra.src) & 15) == 0;
  const bool dst_aligned = ra.dst != nullptr && (reinterpret_cast<uintptr_t>(ra.dst) & 15) == 0;
  // Peers must be done with the previous contents of their windows before the root overwrites them.
  bool ok = BlockBarrier(ctx, channel, block, epoch, 1);
  for (int c = 0; c < nchunks; ++c) {
    const uint64_t t_lo = ntiles * c / nchunks, t_hi = ntiles * (c + 1) / nchunks;
    // first tile of this chunk that belongs to this block (tile t belongs to block t % grid)
    const uint64_t first = t_lo + (static_cast<uint64_t>(block) + grid - t_lo % grid) % grid;
    if (ok && ctx.rank == root) {
      for (uint64_t t = first; t < t_hi; t += grid) {
        const uint64_t lo = t * kCopyTile;
        const uint64_t hi = lo + kCopyTile < nvec ? lo + kCopyTile : nvec;
        for (uint64_t v0 = lo + threadIdx.x; v0 < hi; v0 += static_cast<uint64_t>(blockDim.x) * kCopyUnroll) {
          U4 q[kCopyUnroll];
#pragma unroll
          for (int u = 0; u < kCopyUnroll; ++u) {
            const uint64_t v = v0 + static_cast<uint64_t>(u) * blockDim.x;
            if (v >= hi) continue;
            if (src_aligned && v * 16 + 16 <= nbytes) {
              q[u] = *reinterpret_cast<const U4*>(ra.src + v * 16);
            } else {
              char* qb = reinterpret_cast<char*>(&q[u]);
              for (uint64_t b = 0; b < 16; ++b) qb[b] = v * 16 + b < nbytes ? ra.src[v * 16 + b] : 0;
            }
          }
#pragma unroll
          for (int u = 0; u < kCopyUnroll; ++u) {
            const uint64_t v = v0 + static_cast<uint64_t>(u) * blockDim.x;
            if (v >= hi) continue;
            if (kMultimem) {
              MultimemSt(ctx.mc + ra.win_off + v * 16, q[u]);
            } else {
              for (int r = 0; r < n; ++r) StSys(ctx.peer[r] + ra.win_off + v * 16, q[u]);
            }
            // the root fills its own output from the registers it is sending, so it has no copy-out pass
            if (ra.dst != nullptr && ra.dst != ra.src) {
              if (dst_aligned && v * 16 + 16 <= nbytes) {
                *reinterpret_cast<U4*>(ra.dst + v * 16) = q[u];
              } else {
                const char* qb = reinterpret_cast<const char*>(&q[u]);
                for (uint64_t b = 0; b < 16 && v * 16 + b < nbytes; ++b) ra.dst[v * 16 + b] = qb[b];
              }
            }
          }
        }
      }
    }
    ok = BlockBarrier(ctx, channel, block, epoch + 1 + c, 2) && ok;
    // the other ranks copy this chunk out of their own windows
    if (ok && ra.dst && ctx.rank != root) {
      for (uint64_t t = first; t < t_hi; t += grid) {
        const uint64_t lo = t * kCopyTile;
        const uint64_t hi = lo + kCopyTile < nvec ? lo + kCopyTile : nvec;
        for (uint64_t v0 = lo + threadIdx.x; v0 < hi; v0 += static_cast<uint64_t>(blockDim.x) * kCopyUnroll) {
          U4 q[kCopyUnroll];
#pragma unroll
          for (int u = 0; u < kCopyUnroll; ++u) {
            const uint64_t v = v0 + static_cast<uint64_t>(u) * blockDim.x;
            if (v < hi) q[u] = *reinterpret_cast<const U4*>(my_win + v * 16);
          }
#pragma unroll
          for (int u = 0; u < kCopyUnroll; ++u) {
            const uint64_t v = v0 + static_cast<uint64_t>(u) * blockDim.x;
            if (v >= hi) continue;
            if (dst_aligned && v * 16 + 16 <= nbytes) {
              *reinterpret_cast<U4*>(ra.dst + v * 16) = q[u];
            } else {
              const char* qb = reinterpret_cast<const char*>(&q[u]);
              for (uint64_t b = 0; b < 16 && v * 16 + b < nbytes; ++b) ra.dst[v * 16 + b] = qb[b];
            }
          }
        }
      }
    }
  }
  SaveEpoch(ctx, channel, block, epoch + nchunks);
}

// A kernel that waits for a flag nothing will ever set; used to test the
// bounded-wait path: it must return with a timeout status inside the budget.
__global__ void WaitNeverKernel(CommCtx ctx, int channel) {
  if (threadIdx.x == 0) {
    const uint32_t* flag = FlagAddr(ctx.peer[ctx.rank], channel, kMaxCommBlocks - 1, ctx.rank);
    const uint64_t t0    = GlobalTimerNs();
    const uint32_t want  = *flag + 0x40000000u;
    while (static_cast<int32_t>(LdAcquireSys(flag) - want) < 0) {
      if (GlobalTimerNs() - t0 > ctx.budget_ns) {
        ReportTimeout(ctx, ctx.rank, 9, kMaxCommBlocks - 1, want, channel);
        break;
      }
      __nanosleep(256);
    }
  }
}

// ------------------------------------------------------------------ host side

struct CommState {
  bool ready = false;
  int rank = 0, nranks = 1;
  int emulated = 0;  // >0: all rank windows live on this device (single-GPU tests)
  CommCtx ctx[kMaxRanks];
  size_t window_bytes = 0, staging_bytes = 0;
  cudaStream_t streams[kNumChannels] = {nullptr, nullptr};
  CommStatus* status_host = nullptr;
  int blocks = 32;
  size_t one_shot_bytes = 512 << 10;
  // kernel selection (tipsk_comm_set_option; the environment gives the initial values)
  uint64_t allgather_push_bytes = 2ull << 20;    // largest slab up to which the pushing allgather runs (0: never)
  uint64_t bcast_scatter_bytes  = 128ull << 20;   // message size from which broadcast runs as scatter + allgather (0: never)
  uint64_t bcast_scatter_chunk  = 32ull << 20;   // its pipeline chunk
  int bcast_scatter_min_ranks   = 8;
  bool use_multimem = false;
  std::vector<cudaEvent_t> event_pool;
  std::mutex mu;
  uint64_t launches = 0;
};
CommState g_comm;

int GridFor(uint64_t nbytes, uint64_t tile_bytes, int max_blocks) {
  uint64_t tiles = (nbytes + tile_bytes - 1) / tile_bytes;
  if (tiles < 1) tiles = 1;
  return static_cast<int>(tiles < static_cast<uint64_t>(max_blocks) ? tiles : max_blocks);
}

// Who takes part in a launch: all ranks of the job, or a sub-group of them with its own flags, epochs and staging
// area.  `ctx` has one entry per grid row: one (this process) or, with the ranks emulated on one GPU, one per member.
struct CommView {
  int nranks = 1;              // participants
  int nlocal = 1;              // grid rows launched here
  bool cooperative = false;    // the rows wait on one another inside one launch (emulation)
  bool multimem = false;
  uint64_t stage_off = kSignalBytes;
  uint64_t stage_bytes = 0;
  CommCtx ctx[kMaxRanks];
  int member_rank[kMaxRanks];  // world rank of participant r (identity for the world view)
};

CommView WorldView() {
  CommState& st = g_comm;
  CommView v;
  v.nranks      = st.nranks;
  v.nlocal      = st.emulated > 0 ? st.emulated : 1;
  v.cooperative = st.emulated > 0;
  v.multimem    = st.use_multimem;
  v.stage_off   = kSignalBytes;
  v.stage_bytes = st.staging_bytes;
  for (int i = 0; i < v.nlocal; ++i) v.ctx[i] = st.ctx[st.emulated > 0 ? i : st.rank];
  for (int r = 0; r < kMaxRanks; ++r) v.member_rank[r] = r;
  return v;
}

template <typename K, typename... A>
int LaunchComm(const CommView& view, K kernel, int grid_x, cudaStream_t stream, A... a) {
  CommState& st = g_comm;
  dim3 grid(grid_x, view.nlocal), block(kCommThreads);
  if (view.cooperative) {
    void* params[] = {(void*)&a...};
    TIPSK_CUDA(cudaLaunchCooperativeKernel((const void*)kernel, grid, block, params, 0, stream));
  } else {
    kernel<<<grid, block, 0, stream>>>(a...);
    TIPSK_LAUNCH_CHECK();
  }
  st.launches++;
  return 0;
}

}  // namespace

// Gives other translation units (the parameter-server kernels) the rank contexts.
// Without an initialised communicator it reports a single rank.
int CommGetContexts(CommCtx* out, int* rank, int* nranks, int* emulated) {
  CommState& st = g_comm;
  if (!st.ready) {
    memset(out, 0, sizeof(CommCtx) * kMaxRanks);
    *rank     = 0;
    *nranks   = 1;
    *emulated = 0;
    return 0;
  }
  for (int i = 0; i < kMaxRanks; ++i) out[i] = st.ctx[i];
  *rank     = st.rank;
  *nranks   = st.nranks;
  *emulated = st.emulated > 0 ? 1 : 0;
  return 0;
}

}  // namespace tipsk

using namespace tipsk;

namespace {

// Builds the per-row launch arguments: `srcs` / `dsts` hold one pointer per grid row of the view.
CommLaunch MakeLaunch(const CommView& view, const void* const* srcs, void* const* dsts, uint64_t win_off) {
  CommLaunch l;
  memset(&l, 0, sizeof(l));
  for (int i = 0; i < view.nlocal; ++i) {
    l.r[i].ctx     = view.ctx[i];
    l.r[i].src     = static_cast<const char*>(srcs ? srcs[i] : nullptr);
    l.r[i].dst     = static_cast<char*>(dsts ? dsts[i] : nullptr);
    l.r[i].win_off = win_off;
  }
  return l;
}

template <typename T>
int LaunchAllreduceT(const CommView& vw, const CommLaunch& l, int channel, uint64_t nbytes, int op, float pre, float post,
                     bool one_shot, bool multimem, int grid, cudaStream_t s) {
  if (one_shot) {
    if (multimem) return LaunchComm(vw, AllreduceKernel<T, true, true>, grid, s, l, channel, nbytes, op, pre, post);
    return LaunchComm(vw, AllreduceKernel<T, false, true>, grid, s, l, channel, nbytes, op, pre, post);
  }
  if (multimem) return LaunchComm(vw, AllreduceKernel<T, true, false>, grid, s, l, channel, nbytes, op, pre, post);
  return LaunchComm(vw, AllreduceKernel<T, false, false>, grid, s, l, channel, nbytes, op, pre, post);
}

int LaunchAllreduce(const CommView& vw, int dtype, const CommLaunch& l, int channel, uint64_t nbytes, int op, float pre,
                    float post, bool one_shot, bool multimem, int grid, cudaStream_t s) {
  switch (dtype) {
    case kF32: return LaunchAllreduceT<float>(vw, l, channel, nbytes, op, pre, post, one_shot, multimem, grid, s);
    case kBF16: return LaunchAllreduceT<__nv_bfloat16>(vw, l, channel, nbytes, op, pre, post, one_shot, multimem, grid, s);
    case kF16: return LaunchAllreduceT<__half>(vw, l, channel, nbytes, op, pre, post, one_shot, multimem, grid, s);
    case kI32: return LaunchAllreduceT<int32_t>(vw, l, channel, nbytes, op, pre, post, one_shot, false, grid, s);
    case kI64: return LaunchAllreduceT<int64_t>(vw, l, channel, nbytes, op, pre, post, one_shot, false, grid, s);
    case kF64: return LaunchAllreduceT<double>(vw, l, channel, nbytes, op, pre, post, one_shot, false, grid, s);
    default: return SetError(-2, "allreduce: unsupported dtype on the device path");
  }
}


// Optimizer updates attached to gradient buckets, keyed by the bucket's window offset.
struct AttachedUpdate {
  uint64_t nbytes = 0;
  int dtype = 0;
  int kind = 0;  // 0 SGD with momentum, 1 Adam / AdamW
  UpdateArgs r[kMaxRanks];
  float h[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t step = 0;
  uint64_t launches = 0;
};
std::map<int64_t, AttachedUpdate> g_updates;
std::mutex g_updates_mu;

template <typename T>
int LaunchUpdateT(const CommLaunch& l, const UpdateLaunch& u, bool adam, bool multimem, int channel, uint64_t nbytes,
                  float scale, int grid, cudaStream_t s) {
  const CommView vw = WorldView();
  if (adam) {
    if (multimem) return LaunchComm(vw, AllreduceUpdateKernel<T, true, true>, grid, s, l, u, channel, nbytes, scale);
    return LaunchComm(vw, AllreduceUpdateKernel<T, false, true>, grid, s, l, u, channel, nbytes, scale);
  }
  if (multimem) return LaunchComm(vw, AllreduceUpdateKernel<T, true, false>, grid, s, l, u, channel, nbytes, scale);
  return LaunchComm(vw, AllreduceUpdateKernel<T, false, false>, grid, s, l, u, channel, nbytes, scale);
}

// The three collectives on a view (all ranks, or a sub-group): see the comments of the extern "C" entry points.
int AllreduceOn(const CommView& vw, const void* const* srcs, void* const* dsts, int64_t win_off, uint64_t nbytes,
                int dtype, int op, float prescale, float postscale, int channel, cudaStream_t s) {
  CommState& st = g_comm;
  if (nbytes == 0) return 0;
  const bool mm  = vw.multimem && op == 0;
  const uint64_t tile_bytes = static_cast<uint64_t>(SubTileOf(mm)) * vw.nranks * 16;
  if (!srcs) {
    TIPSK_REQUIRE(win_off >= static_cast<int64_t>(kSignalBytes) && win_off % 16 == 0, "allreduce: bad window offset");
    TIPSK_REQUIRE(static_cast<uint64_t>(win_off) + ((nbytes + 15) & ~15ull) <= st.window_bytes,
                  "allreduce: buffer exceeds the window");
    const bool one_shot = dsts != nullptr && nbytes <= st.one_shot_bytes;
    CommLaunch l = MakeLaunch(vw, nullptr, dsts, static_cast<uint64_t>(win_off));
    return LaunchAllreduce(vw, dtype, l, channel, nbytes, op, prescale, postscale, one_shot, mm,
                           GridFor(nbytes, tile_bytes, st.blocks), s);
  }
  TIPSK_REQUIRE(dsts != nullptr, "allreduce: staged mode needs an output");
  const uint64_t chunk = vw.stage_bytes;
  TIPSK_REQUIRE(chunk >= 4096, "allreduce: no staging area configured");
  for (uint64_t done = 0; done < nbytes; done += chunk) {
    const uint64_t len = nbytes - done < chunk ? nbytes - done : chunk;
    const void* sp[kMaxRanks];
    void* dp[kMaxRanks];
    for (int i = 0; i < vw.nlocal; ++i) {
      sp[i] = static_cast<const char*>(srcs[i]) + done;
      dp[i] = static_cast<char*>(dsts[i]) + done;
    }
    CommLaunch l = MakeLaunch(vw, sp, dp, vw.stage_off);
    const bool one_shot = len <= st.one_shot_bytes;
    int rc = LaunchAllreduce(vw, dtype, l, channel, len, op, prescale, postscale, one_shot, mm,
                             GridFor(len, tile_bytes, st.blocks), s);
    if (rc) return rc;
  }
  return 0;
}

int AllgathervOn(const CommView& vw, const void* const* srcs, void* const* dsts, const uint64_t* bytes_per_rank,
                 int channel, cudaStream_t s) {
  CommState& st = g_comm;
  const int n = vw.nranks;
  uint64_t displ[kMaxRanks], largest = 0;
  uint64_t acc = 0;
  for (int r = 0; r < n; ++r) {
    displ[r] = acc;
    acc += bytes_per_rank[r];
    if (bytes_per_rank[r] > largest) largest = bytes_per_rank[r];
  }
  const uint64_t chunk = vw.stage_bytes;
  TIPSK_REQUIRE(chunk >= 4096, "allgatherv: no staging area configured");
  // Small gathers are pushed (see AllgatherPushKernel): everything has to fit the staging area at once.
  const uint64_t push_limit = st.allgather_push_bytes;
  uint64_t padded = 0;
  for (int r = 0; r < n; ++r) padded += (bytes_per_rank[r] + 15) & ~15ull;
  if (padded > 0 && largest <= push_limit && padded <= chunk) {
    GatherSizes gs;
    memset(&gs, 0, sizeof(gs));
    for (int r = 0; r < n; ++r) {
      gs.bytes[r] = bytes_per_rank[r];
      gs.displ[r] = displ[r];
    }
    CommLaunch l = MakeLaunch(vw, srcs, dsts, vw.stage_off);
    const int grid = GridFor(largest, static_cast<uint64_t>(kPushTile) * 16, st.blocks);
    return vw.multimem ? LaunchComm(vw, AllgatherPushKernel<true>, grid, s, l, channel, gs)
                       : LaunchComm(vw, AllgatherPushKernel<false>, grid, s, l, channel, gs);
  }
  for (uint64_t done = 0; done < largest; done += chunk) {
    GatherSizes gs;
    memset(&gs, 0, sizeof(gs));
    for (int r = 0; r < n; ++r) {
      uint64_t left = bytes_per_rank[r] > done ? bytes_per_rank[r] - done : 0;
      gs.bytes[r]   = left < chunk ? left : chunk;
      gs.displ[r]   = displ[r] + done;
    }
    const void* sp[kMaxRanks];
    for (int i = 0; i < vw.nlocal; ++i) {
      const int r = vw.ctx[i].rank;  // this row's rank among the participants
      sp[i] = static_cast<const char*>(srcs[i]) + (bytes_per_rank[r] > done ? done : 0);
    }
    CommLaunch l = MakeLaunch(vw, sp, dsts, vw.stage_off);
    uint64_t biggest = 0;
    for (int r = 0; r < n; ++r) if (gs.bytes[r] > biggest) biggest = gs.bytes[r];
    int rc = LaunchComm(vw, AllgathervKernel, GridFor(biggest, static_cast<uint64_t>(kCopyTile) * 16, st.blocks), s, l,
                        channel, gs);
    if (rc) return rc;
  }
  return 0;
}

int BroadcastOn(const CommView& vw, const void* const* srcs, void* const* dsts, uint64_t nbytes, int root, int channel,
                cudaStream_t s) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(root >= 0 && root < vw.nranks, "broadcast: bad root");
  const uint64_t chunk = vw.stage_bytes;
  TIPSK_REQUIRE(chunk >= 4096, "broadcast: no staging area configured");
  for (uint64_t done = 0; done < nbytes; done += chunk) {
    const uint64_t len = nbytes - done < chunk ? nbytes - done : chunk;
    const void* sp[kMaxRanks];
    void* dp[kMaxRanks];
    for (int i = 0; i < vw.nlocal; ++i) {
      sp[i] = srcs[i] ? static_cast<const char*>(srcs[i]) + done : nullptr;
      dp[i] = static_cast<char*>(dsts[i]) + done;
    }
    CommLaunch l = MakeLaunch(vw, sp, dp, vw.stage_off);
    const int grid = GridFor(len, static_cast<uint64_t>(kCopyTile) * 16, st.blocks);
    // 32 MiB chunks (TIPS_BCAST_CHUNK_BYTES overrides; the tests use small ones).  Measured on 2 GPUs at 64-256 MiB:
    // one chunk 374-411 GB/s, 16 MiB chunks 390-421 GB/s, 32 MiB chunks 410-475 GB/s; smaller chunks lose to the
    // extra barriers.
    static const uint64_t chunk_bytes = [] {
      const char* e = getenv("TIPS_BCAST_CHUNK_BYTES");
      const uint64_t v = e ? strtoull(e, nullptr, 10) : 0;
      return v >= 4096 ? v : (32ull << 20);
    }();
    // Large messages go as scatter + allgather (see BroadcastScatterKernel).  Measured: with 8 ranks it passes the
    // root-stores-everything kernel from 128 MiB on (400 against 350 GB/s at 1 GiB); with 4 ranks it stays behind.
    const uint64_t scatter_min = st.bcast_scatter_bytes, scatter_chunk = st.bcast_scatter_chunk;
    if (scatter_min > 0 && len >= scatter_min && vw.nranks >= st.bcast_scatter_min_ranks) {
      int nc = static_cast<int>(len / scatter_chunk);
      nc     = nc < 1 ? 1 : (nc > 64 ? 64 : nc);
      int rc = vw.multimem ? LaunchComm(vw, BroadcastScatterKernel<true>, grid, s, l, channel, len, root, nc)
                           : LaunchComm(vw, BroadcastScatterKernel<false>, grid, s, l, channel, len, root, nc);
      if (rc) return rc;
      continue;
    }
    int nchunks = static_cast<int>(len / chunk_bytes);
    nchunks = nchunks < 1 ? 1 : (nchunks > 16 ? 16 : nchunks);
    int rc = vw.multimem ? LaunchComm(vw, BroadcastKernel<true>, grid, s, l, channel, len, root, nchunks)
                         : LaunchComm(vw, BroadcastKernel<false>, grid, s, l, channel, len, root, nchunks);
    if (rc) return rc;
  }
  return 0;
}

// Sub-groups of ranks with device collectives of their own.
struct DeviceGroup {
  int n = 0;
  int members[kMaxRanks];        // world ranks, ascending
  uint64_t area_off = 0;         // window offset of the group's area: [kFlagBytes flags | staging]
  uint64_t stage_bytes = 0;
  uint32_t* epochs[kMaxRanks];   // per local row
};
std::map<int64_t, DeviceGroup> g_groups;
std::mutex g_groups_mu;

// View of a group for this process; fails when no local rank is a member.
int GroupView(int64_t id, CommView* out) {
  CommState& st = g_comm;
  std::lock_guard<std::mutex> lock(g_groups_mu);
  auto it = g_groups.find(id);
  TIPSK_REQUIRE(it != g_groups.end(), "comm group: unknown group");
  const DeviceGroup& g = it->second;
  CommView v;
  v.nranks      = g.n;
  v.cooperative = st.emulated > 0;
  v.multimem    = false;  // the multicast mapping spans all ranks: a sub-group uses peer loads and stores
  v.stage_off   = g.area_off + kFlagBytes;
  v.stage_bytes = g.stage_bytes;
  v.nlocal      = 0;
  for (int r = 0; r < g.n; ++r) v.member_rank[r] = g.members[r];
  for (int r = 0; r < g.n; ++r) {
    const int world = g.members[r];
    if (st.emulated == 0 && world != st.rank) continue;
    CommCtx c = st.ctx[world];
    for (int q = 0; q < kMaxRanks; ++q) c.peer[q] = q < g.n ? st.ctx[world].peer[g.members[q]] : nullptr;
    c.mc       = nullptr;
    c.rank     = r;
    c.nranks   = g.n;
    c.flag_off = g.area_off;
    c.epochs   = g.epochs[v.nlocal];
    v.ctx[v.nlocal++] = c;
  }
  TIPSK_REQUIRE(v.nlocal > 0, "comm group: this process is not a member");
  *out = v;
  return 0;
}

}  // namespace

extern "C" {

int tipsk_comm_init(int rank, int nranks, void* const* peer_windows, void* multicast_window, uint64_t window_bytes,
                    uint64_t staging_bytes, int wait_budget_ms, int blocks, uint64_t one_shot_bytes, int use_multimem,
                    int emulated) {
  CommState& st = g_comm;
  std::lock_guard<std::mutex> lock(st.mu);
  TIPSK_REQUIRE(nranks >= 1 && nranks <= kMaxRanks, "comm: 1..8 ranks are supported");
  TIPSK_REQUIRE(rank >= 0 && rank < nranks, "comm: bad rank");
  TIPSK_REQUIRE(window_bytes >= kSignalBytes + staging_bytes, "comm: window smaller than signals + staging");
  // the last two flag slots of every channel belong to the one-block fence and to the wait self-test
  TIPSK_REQUIRE(blocks >= 1 && blocks <= kMaxCommBlocks - 2, "comm: blocks out of range");
  st.rank          = rank;
  st.nranks        = nranks;
  st.emulated      = emulated ? nranks : 0;
  st.window_bytes  = window_bytes;
  st.staging_bytes = staging_bytes & ~static_cast<uint64_t>(4095);
  st.blocks        = blocks;
  if (emulated) {  // a cooperative launch needs every block of every rank resident at once
    int cap = NumSMs() / nranks;
    if (cap < 1) cap = 1;
    if (st.blocks > cap) st.blocks = cap;
  }
  st.one_shot_bytes = one_shot_bytes;
  {
    auto env_u64 = [](const char* name, uint64_t dflt) {
      const char* e = getenv(name);
      return e ? strtoull(e, nullptr, 10) : dflt;
    };
    st.allgather_push_bytes    = env_u64("TIPS_ALLGATHER_PUSH_BYTES", 2ull << 20);
    st.bcast_scatter_bytes     = env_u64("TIPS_BCAST_SCATTER_BYTES", 128ull << 20);
    st.bcast_scatter_chunk     = env_u64("TIPS_BCAST_SCATTER_CHUNK_BYTES", 32ull << 20);
    st.bcast_scatter_min_ranks = static_cast<int>(env_u64("TIPS_BCAST_SCATTER_MIN_RANKS", 8));
    if (st.bcast_scatter_chunk < 65536) st.bcast_scatter_chunk = 65536;
  }
  st.use_multimem  = use_multimem && multicast_window != nullptr && !emulated;
  if (!st.status_host) {
    TIPSK_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&st.status_host), sizeof(CommStatus) * kMaxRanks,
                             cudaHostAllocMapped));
  }
  memset(st.status_host, 0, sizeof(CommStatus) * kMaxRanks);
  CommStatus* status_dev = nullptr;
  TIPSK_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev), st.status_host, 0));
  const int local = emulated ? nranks : 1;
  for (int i = 0; i < local; ++i) {
    CommCtx& c = st.ctx[emulated ? i : rank];
    memset(&c, 0, sizeof(c));
    for (int r = 0; r < nranks; ++r) c.peer[r] = static_cast<char*>(peer_windows[r]);
    c.mc        = st.use_multimem ? static_cast<char*>(multicast_window) : nullptr;
    c.rank      = emulated ? i : rank;
    c.nranks    = nranks;
    c.budget_ns = static_cast<uint64_t>(wait_budget_ms) * 1000000ull;
    c.status    = status_dev + (emulated ? i : 0);
    TIPSK_CUDA(cudaMalloc(reinterpret_cast<void**>(&c.epochs), sizeof(uint32_t) * kNumChannels * kMaxCommBlocks));
    TIPSK_CUDA(cudaMemset(c.epochs, 0, sizeof(uint32_t) * kNumChannels * kMaxCommBlocks));
    TIPSK_CUDA(cudaMalloc(reinterpret_cast<void**>(&c.failed), sizeof(int32_t)));
    TIPSK_CUDA(cudaMemset(c.failed, 0, sizeof(int32_t)));
  }
  for (int ch = 0; ch < kNumChannels; ++ch) {
    if (!st.streams[ch]) {
      int lo = 0, hi = 0;
      cudaDeviceGetStreamPriorityRange(&lo, &hi);
      TIPSK_CUDA(cudaStreamCreateWithPriority(&st.streams[ch], cudaStreamNonBlocking, hi));
    }
  }
  TIPSK_CUDA(cudaDeviceSynchronize());
  st.ready = true;
  return 0;
}

int tipsk_comm_shutdown(void) {
  CommState& st = g_comm;
  std::lock_guard<std::mutex> lock(st.mu);
  if (!st.ready) return 0;
  cudaDeviceSynchronize();
  for (int i = 0; i < kMaxRanks; ++i) {
    if (st.ctx[i].epochs) cudaFree(st.ctx[i].epochs);
    if (st.ctx[i].failed) cudaFree(st.ctx[i].failed);
    st.ctx[i].epochs = nullptr;
    st.ctx[i].failed = nullptr;
  }
  for (cudaEvent_t e : st.event_pool) cudaEventDestroy(e);
  st.event_pool.clear();
  st.ready = false;
  {
    std::lock_guard<std::mutex> ulock(g_updates_mu);
    g_updates.clear();
  }
  {
    std::lock_guard<std::mutex> glock(g_groups_mu);
    for (auto& kv : g_groups)
      for (uint32_t* e : kv.second.epochs)
        if (e) cudaFree(e);
    g_groups.clear();
  }
  return 0;
}

/* Kernel selection at run time (every rank sets the same values, between collectives):
 *   allgather_push_bytes       largest per-rank slab up to which allgatherv pushes instead of pulling (0: never)
 *   bcast_scatter_bytes        message size from which broadcast runs as scatter + allgather (0: never)
 *   bcast_scatter_chunk_bytes  pipeline chunk of that kernel (>= 64 KiB)
 *   bcast_scatter_min_ranks    fewest ranks for which it is used (>= 2) */
int tipsk_comm_set_option(const char* name, uint64_t value) {
  CommState& st = g_comm;
  const std::string key = name ? name : "";
  if (key == "allgather_push_bytes") st.allgather_push_bytes = value;
  else if (key == "bcast_scatter_bytes") st.bcast_scatter_bytes = value;
  else if (key == "bcast_scatter_chunk_bytes") st.bcast_scatter_chunk = value < 65536 ? 65536 : value;
  else if (key == "bcast_scatter_min_ranks") st.bcast_scatter_min_ranks = value < 2 ? 2 : static_cast<int>(value);
  else return SetError(-2, "comm option: unknown name");
  return 0;
}

int tipsk_comm_ready(void) { return g_comm.ready ? 1 : 0; }
uint64_t tipsk_comm_staging_offset(void) { return kSignalBytes; }
uint64_t tipsk_comm_launches(void) { return g_comm.launches; }
void* tipsk_comm_stream(int channel) { return g_comm.streams[channel & 1]; }
int tipsk_comm_uses_multimem(void) { return g_comm.use_multimem ? 1 : 0; }
int tipsk_comm_set_budget_ms(int ms) {
  for (int i = 0; i < kMaxRanks; ++i) g_comm.ctx[i].budget_ns = static_cast<uint64_t>(ms) * 1000000ull;
  return 0;
}

/* Reads (and optionally clears) the status block of local rank slot `slot`.
 * out = {code, peer, phase, block, epoch, channel, rank}. */
int tipsk_comm_status(int slot, int32_t* out7, int clear) {
  CommState& st = g_comm;
  if (!st.status_host || slot < 0 || slot >= kMaxRanks) return -2;
  CommStatus s = st.status_host[slot];
  out7[0] = s.code; out7[1] = s.peer; out7[2] = s.phase; out7[3] = s.block;
  out7[4] = static_cast<int32_t>(s.epoch); out7[5] = s.channel; out7[6] = s.rank;
  if (clear && s.code != 0) {
    memset(&st.status_host[slot], 0, sizeof(CommStatus));
    const int idx = st.emulated > 0 ? slot : st.rank;
    if (st.ctx[idx].failed) cudaMemset(st.ctx[idx].failed, 0, sizeof(int32_t));
  }
  return s.code;
}

/* Zeroes the flags of this rank's window and the local epoch counters. Call it on every
 * rank, then synchronise the ranks on the host, before the next collective. */
int tipsk_comm_reset(void) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  TIPSK_CUDA(cudaDeviceSynchronize());
  const int local = st.emulated > 0 ? st.emulated : 1;
  for (int i = 0; i < local; ++i) {
    CommCtx& c = st.ctx[st.emulated > 0 ? i : st.rank];
    TIPSK_CUDA(cudaMemset(c.peer[c.rank], 0, kFlagBytes));
    TIPSK_CUDA(cudaMemset(c.epochs, 0, sizeof(uint32_t) * kNumChannels * kMaxCommBlocks));
    TIPSK_CUDA(cudaMemset(c.failed, 0, sizeof(int32_t)));
  }
  {  // sub-groups: the flag areas of the local members and their epoch counters
    std::lock_guard<std::mutex> lock(g_groups_mu);
    for (auto& kv : g_groups) {
      DeviceGroup& g = kv.second;
      int row = 0;
      for (int r = 0; r < g.n; ++r) {
        const int world = g.members[r];
        if (st.emulated == 0 && world != st.rank) continue;
        TIPSK_CUDA(cudaMemset(st.ctx[world].peer[world] + g.area_off, 0, kFlagBytes));
        TIPSK_CUDA(cudaMemset(g.epochs[row++], 0, sizeof(uint32_t) * kNumChannels * kMaxCommBlocks));
      }
    }
  }
  memset(st.status_host, 0, sizeof(CommStatus) * kMaxRanks);
  TIPSK_CUDA(cudaDeviceSynchronize());
  return 0;
}

/* Allreduce of `nbytes` bytes of `dtype`.
 *  win_off >= 0 and srcs == NULL : the data already sits at that offset of every rank's window
 *                                   (in place; dsts may be NULL to leave the result there)
 *  srcs != NULL                   : staged through the staging area (win_off ignored)
 * srcs / dsts are host arrays with one device pointer per LOCAL rank (1, or nranks when emulated). */
int tipsk_allreduce(const void* const* srcs, void* const* dsts, int64_t win_off, uint64_t nbytes, int dtype, int op,
                    float prescale, float postscale, int channel, void* stream) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  TIPSK_REQUIRE(channel >= 0 && channel < kNumChannels, "bad channel");
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st.streams[channel];
  return AllreduceOn(WorldView(), srcs, dsts, win_off, nbytes, dtype, op, prescale, postscale, channel, s);
}

/* ---- allreduce fused with the optimizer step ----
 * Number of 16-byte vectors of master weights / state that every rank keeps for a bucket of `nbytes` bytes. */
int tipsk_comm_update_subtile(void) { return kUpdSubTile; }
int64_t tipsk_comm_update_shard_vecs(uint64_t nbytes) {
  CommState& st = g_comm;
  const uint64_t nvec      = nbytes / 16;
  const uint64_t tile_vecs = static_cast<uint64_t>(kUpdSubTile) * st.nranks;
  return static_cast<int64_t>((nvec + tile_vecs - 1) / tile_vecs * kUpdSubTile);
}

/* Attaches an optimizer update to the gradient bucket at window offset `grad_off`: from now on
 * tipsk_allreduce_update (and the engine's in-place sum-allreduce of exactly that buffer) reduces the gradients,
 * updates this rank's share of the fp32 master weights / state and stores the new parameters, in `dtype`, into every
 * rank's window at `param_off`.  master / s0 / s1 are host arrays with one device pointer per LOCAL rank, each
 * tipsk_comm_update_shard_vecs(nbytes) * 16 / sizeof(dtype) floats (s1 only for Adam, s0 may be null for plain SGD). */
int tipsk_comm_attach_update(int64_t grad_off, uint64_t nbytes, int dtype, int64_t param_off, int kind,
                             void* const* master, void* const* s0, void* const* s1) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  TIPSK_REQUIRE(dtype == kF32 || dtype == kBF16 || dtype == kF16, "update: gradients must be fp32, bf16 or fp16");
  TIPSK_REQUIRE(nbytes > 0 && nbytes % 16 == 0, "update: the bucket must be a whole number of 16-byte vectors");
  TIPSK_REQUIRE(kind == 0 || kind == 1, "update: kind is 0 (SGD) or 1 (Adam)");
  for (int64_t off : {grad_off, param_off}) {
    TIPSK_REQUIRE(off >= static_cast<int64_t>(kSignalBytes) && off % 16 == 0, "update: bad window offset");
    TIPSK_REQUIRE(static_cast<uint64_t>(off) + nbytes <= st.window_bytes, "update: buffer exceeds the window");
  }
  TIPSK_REQUIRE(grad_off + static_cast<int64_t>(nbytes) <= param_off || param_off + static_cast<int64_t>(nbytes) <= grad_off,
                "update: gradient and parameter buffers overlap");
  AttachedUpdate a;
  a.nbytes = nbytes;
  a.dtype  = dtype;
  a.kind   = kind;
  const int local = st.emulated > 0 ? st.emulated : 1;
  for (int i = 0; i < local; ++i) {
    TIPSK_REQUIRE(master && master[i], "update: master weights missing");
    TIPSK_REQUIRE(kind == 0 || (s0 && s0[i] && s1 && s1[i]), "update: Adam needs both moment buffers");
    a.r[i].master    = static_cast<float*>(master[i]);
    a.r[i].s0        = s0 ? static_cast<float*>(s0[i]) : nullptr;
    a.r[i].s1        = s1 ? static_cast<float*>(s1[i]) : nullptr;
    a.r[i].param_off = static_cast<uint64_t>(param_off);
  }
  std::lock_guard<std::mutex> lock(g_updates_mu);
  g_updates[grad_off] = a;
  return 0;
}

int tipsk_comm_detach_update(int64_t grad_off) {
  std::lock_guard<std::mutex> lock(g_updates_mu);
  if (grad_off < 0) g_updates.clear();
  else g_updates.erase(grad_off);
  return 0;
}

int tipsk_comm_update_attached(int64_t grad_off, uint64_t nbytes) {
  std::lock_guard<std::mutex> lock(g_updates_mu);
  auto it = g_updates.find(grad_off);
  return it != g_updates.end() && it->second.nbytes == nbytes ? 1 : 0;
}

/* Hyper-parameters of the next update of that bucket.  SGD: {lr, momentum, dampening, weight_decay, nesterov};
 * Adam: {lr, beta1, beta2, eps, weight_decay, decoupled}.  `step` counts from 1 (first step of SGD seeds the
 * momentum buffer, Adam's bias correction). */
int tipsk_comm_set_update_hyper(int64_t grad_off, const float* h, int nh, int64_t step) {
  std::lock_guard<std::mutex> lock(g_updates_mu);
  auto it = g_updates.find(grad_off);
  TIPSK_REQUIRE(it != g_updates.end(), "update: no update attached at that offset");
  TIPSK_REQUIRE(nh >= 1 && nh <= 8 && step >= 1, "update: bad hyper-parameters");
  for (int i = 0; i < nh; ++i) it->second.h[i] = h[i];
  it->second.step = step;
  return 0;
}

uint64_t tipsk_comm_update_launches(int64_t grad_off) {
  std::lock_guard<std::mutex> lock(g_updates_mu);
  auto it = g_updates.find(grad_off);
  return it == g_updates.end() ? 0 : it->second.launches;
}

/* One launch: sum-allreduce of the attached gradient bucket times `scale`, optimizer step on the owned share,
 * new parameters stored to every rank. */
int tipsk_allreduce_update(int64_t grad_off, float scale, int channel, void* stream) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  TIPSK_REQUIRE(channel >= 0 && channel < kNumChannels, "bad channel");
  AttachedUpdate a;
  {
    std::lock_guard<std::mutex> lock(g_updates_mu);
    auto it = g_updates.find(grad_off);
    TIPSK_REQUIRE(it != g_updates.end(), "update: no update attached at that offset");
    TIPSK_REQUIRE(it->second.step >= 1, "update: hyper-parameters were never set");
    it->second.launches++;
    a = it->second;
  }
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st.streams[channel];
  CommLaunch l   = MakeLaunch(WorldView(), nullptr, nullptr, static_cast<uint64_t>(grad_off));
  UpdateLaunch u;
  memset(&u, 0, sizeof(u));
  for (int i = 0; i < kMaxRanks; ++i) u.r[i] = a.r[i];
  const float* h = a.h;
  if (a.kind == 0) {
    u.sgd = SgdParams{h[0], h[1], h[2], h[3], 1.f, h[4] != 0.f ? 1 : 0, a.step == 1 ? 1 : 0};
  } else {
    const float step = static_cast<float>(a.step);
    u.adam = AdamParams{h[0], h[1], h[2], h[3], h[4], 1.f, 1.f - powf(h[1], step), 1.f - powf(h[2], step),
                        h[5] != 0.f ? 1 : 0, nullptr};
  }
  const uint64_t tile_bytes = static_cast<uint64_t>(kUpdSubTile) * st.nranks * 16;
  // Most of this kernel's traffic is the optimizer state in local HBM, not the link: it wants more blocks than
  // the plain collectives (64 MB of bf16 gradients with Adam on 2 GPUs: 0.45 ms with 64 blocks, 0.27 ms with 126).
  // TIPS_UPDATE_BLOCKS overrides; a cooperative (emulated) launch keeps the co-residency cap.
  static const int env_blocks = [] {
    const char* e = getenv("TIPS_UPDATE_BLOCKS");
    return e ? atoi(e) : 0;
  }();
  int max_blocks = st.blocks;
  if (st.emulated == 0) {
    max_blocks = env_blocks > 0 ? env_blocks : kMaxCommBlocks - 2;
    if (max_blocks > kMaxCommBlocks - 2) max_blocks = kMaxCommBlocks - 2;
  }
  const int grid = GridFor(a.nbytes, tile_bytes, max_blocks);
  const bool mm  = st.use_multimem;
  switch (a.dtype) {
    case kF32: return LaunchUpdateT<float>(l, u, a.kind == 1, mm, channel, a.nbytes, scale, grid, s);
    case kBF16: return LaunchUpdateT<__nv_bfloat16>(l, u, a.kind == 1, mm, channel, a.nbytes, scale, grid, s);
    case kF16: return LaunchUpdateT<__half>(l, u, a.kind == 1, mm, channel, a.nbytes, scale, grid, s);
    default: return SetError(-2, "update: unsupported dtype");
  }
}

/* Allgatherv of per-rank byte counts; staged through the staging area, chunked when a slab is larger. */
int tipsk_allgatherv(const void* const* srcs, void* const* dsts, const uint64_t* bytes_per_rank, int channel,
                     void* stream) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st.streams[channel];
  return AllgathervOn(WorldView(), srcs, dsts, bytes_per_rank, channel, s);
}

int tipsk_broadcast(const void* const* srcs, void* const* dsts, uint64_t nbytes, int root, int channel, void* stream) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st.streams[channel];
  return BroadcastOn(WorldView(), srcs, dsts, nbytes, root, channel, s);
}

/* ---- device collectives of a sub-group of ranks ----
 * `members`: ascending world ranks.  `area_off`: offset of kFlagBytes + stage_bytes zeroed bytes inside EVERY rank's
 * window, the same offset everywhere (flags first, then the group's staging area), reserved for this group alone.
 * Called by every member (with the ranks emulated on one GPU: once).  The collectives below are launched by the
 * members only, in the same order on every member, on the stream they are given; srcs / dsts hold one pointer per
 * local member (one; with emulation one per member, in member order).  Ranks inside a group are group ranks. */
int tipsk_comm_group_create(int64_t id, const int32_t* members, int n, uint64_t area_off, uint64_t stage_bytes) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  TIPSK_REQUIRE(n >= 1 && n <= st.nranks, "comm group: bad size");
  TIPSK_REQUIRE(area_off >= kSignalBytes && area_off % 256 == 0 && area_off + kFlagBytes + stage_bytes <= st.window_bytes,
                "comm group: the area does not fit the window");
  TIPSK_REQUIRE(stage_bytes >= 4096 && stage_bytes % 4096 == 0, "comm group: the staging area must be a multiple of 4096");
  DeviceGroup g;
  g.n = n;
  for (int i = 0; i < n; ++i) {
    TIPSK_REQUIRE(members[i] >= 0 && members[i] < st.nranks && (i == 0 || members[i] > members[i - 1]),
                  "comm group: members must be ascending ranks of the job");
    g.members[i] = members[i];
  }
  g.area_off    = area_off;
  g.stage_bytes = stage_bytes;
  const int rows = st.emulated > 0 ? n : 1;
  for (int i = 0; i < kMaxRanks; ++i) g.epochs[i] = nullptr;
  for (int i = 0; i < rows; ++i) {
    TIPSK_CUDA(cudaMalloc(reinterpret_cast<void**>(&g.epochs[i]), sizeof(uint32_t) * kNumChannels * kMaxCommBlocks));
    TIPSK_CUDA(cudaMemset(g.epochs[i], 0, sizeof(uint32_t) * kNumChannels * kMaxCommBlocks));
  }
  std::lock_guard<std::mutex> lock(g_groups_mu);
  auto old = g_groups.find(id);
  if (old != g_groups.end())  // the id is being reused: release the previous group's counters
    for (uint32_t* e : old->second.epochs)
      if (e) cudaFree(e);
  g_groups[id] = g;
  return 0;
}

int tipsk_comm_group_destroy(int64_t id) {
  std::lock_guard<std::mutex> lock(g_groups_mu);
  auto it = g_groups.find(id);
  if (it == g_groups.end()) return 0;
  for (uint32_t* e : it->second.epochs)
    if (e) cudaFree(e);
  g_groups.erase(it);
  return 0;
}

int tipsk_group_allreduce(int64_t id, const void* const* srcs, void* const* dsts, uint64_t nbytes, int dtype, int op,
                          float prescale, float postscale, void* stream) {
  CommView vw;
  int rc = GroupView(id, &vw);
  if (rc) return rc;
  TIPSK_REQUIRE(srcs && dsts && stream, "group allreduce: needs inputs, outputs and a stream");
  return AllreduceOn(vw, srcs, dsts, -1, nbytes, dtype, op, prescale, postscale, 0, static_cast<cudaStream_t>(stream));
}

int tipsk_group_allgatherv(int64_t id, const void* const* srcs, void* const* dsts, const uint64_t* bytes_per_member,
                           void* stream) {
  CommView vw;
  int rc = GroupView(id, &vw);
  if (rc) return rc;
  TIPSK_REQUIRE(srcs && dsts && stream, "group allgatherv: needs inputs, outputs and a stream");
  return AllgathervOn(vw, srcs, dsts, bytes_per_member, 0, static_cast<cudaStream_t>(stream));
}

int tipsk_group_broadcast(int64_t id, const void* const* srcs, void* const* dsts, uint64_t nbytes, int root,
                          void* stream) {
  CommView vw;
  int rc = GroupView(id, &vw);
  if (rc) return rc;
  TIPSK_REQUIRE(srcs && dsts && stream, "group broadcast: needs inputs, outputs and a stream");
  return BroadcastOn(vw, srcs, dsts, nbytes, root, 0, static_cast<cudaStream_t>(stream));
}

uint64_t tipsk_comm_flag_bytes(void) { return kFlagBytes; }

/* Launches a kernel that waits (bounded) for a flag that is never set; afterwards
 * tipsk_comm_status reports a timeout. */
int tipsk_comm_wait_never(int channel, void* stream) {
  CommState& st = g_comm;
  TIPSK_REQUIRE(st.ready, "comm not initialised");
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st.streams[channel & 1];
  WaitNeverKernel<<<1, 32, 0, s>>>(st.ctx[st.emulated > 0 ? 0 : st.rank], channel & 1);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* ---- events / streams for the executor and the Python layer ---- */
void* tipsk_event_create(void) {
  CommState& st = g_comm;
  {
    std::lock_guard<std::mutex> lock(st.mu);
    if (!st.event_pool.empty()) {
      cudaEvent_t e = st.event_pool.back();
      st.event_pool.pop_back();
      return e;
    }
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  return e;
}
void tipsk_event_recycle(void* ev) {
  if (!ev) return;
  std::lock_guard<std::mutex> lock(g_comm.mu);
  g_comm.event_pool.push_back(static_cast<cudaEvent_t>(ev));
}
int tipsk_event_record(void* ev, void* stream) {
  TIPSK_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev), static_cast<cudaStream_t>(stream)));
  return 0;
}
int tipsk_stream_wait_event(void* stream, void* ev) {
  TIPSK_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(ev), 0));
  return 0;
}
int tipsk_stream_synchronize(void* stream) {
  TIPSK_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return 0;
}

}  // extern "C"
