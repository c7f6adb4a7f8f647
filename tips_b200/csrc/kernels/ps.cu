// Parameter-server data path on the GPU: sharded embedding tables that live in
// peer-mapped memory, pull fused with the embedding lookup, push fused with a
// cross-rank scatter-reduce and the server-side optimizer.
//
// Reference counterpart: PsClient::Pull / PsServer::PullTask (rows travel as
// FlatBuffers over a ZeroMQ RPC, tips/core/ps/ps_client.h:78-109,
// ps_server.h:147-192), PsClient::Push / PsServer::PushTask and the access
// method that applies the update on the server (ps_client.h:111-130,
// ps_server.h:232-265, sparse_access_method.h:41-61), and the zero
// initialisation of a row on first pull (sparse_access_method.h:23-27).
//
// Placement: row `id` of a table is owned by rank (id mod N) and stored at
// local row (id div N) of that rank's shard; pull and push use the same rule.
//
// Pull: one half-warp (or warp) per (sample, field) resolves the owner and
// loads the row straight from the owner's HBM over NVLink with 16-byte
// system-scope loads, converts and writes it into the consumer's input matrix at
// its column offset.  No request message, no staging copy.
//
// Push: three launches separated by cross-rank fences.
//   scatter  every (sample, field) gradient row is added into a slot of the
//            OWNER's accumulation table (open addressing keyed by (field,row);
//            the slot is claimed with a 64-bit CAS on peer memory, the gradient
//            is added with vector float atomics on peer memory); duplicates
//            inside a batch and across ranks end up summed in one slot
//   apply    the owner walks its slots, applies SGD or Adagrad to the row with
//            the summed gradient, and clears the slot
// so the update is exactly the synchronous one: one optimizer step per touched
// row with the gradient summed over every occurrence on every rank.
#include "kernels/comm.cuh"
#include "kernels/common.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

constexpr int kMaxFields = 64;

struct PsMeta {
  uint64_t field_off[kMaxFields];   // byte offset of the field's shard inside every rank's slab
  uint64_t state_off[kMaxFields];   // byte offset of the optimizer state shard (Adagrad), same layout
  int64_t rows_per_shard[kMaxFields];
  int32_t nfields;
  int32_t dim;                      // fp32 elements per row, multiple of 4
};

struct PsRank {
  char* slab[kMaxRanks];            // every rank's table slab as mapped here
  char* acc[kMaxRanks];             // every rank's accumulation table as mapped here
  const int64_t* ids;               // [batch, nfields]
  const void* grads;                // push: [batch, ld] rows of nfields*dim (fp32 or bf16)
  void* out;                        // pull: [batch, ld]
  int32_t* error;                   // local error word (accumulation table full, bad id)
  int32_t rank;
  int32_t nranks;
};
struct PsLaunch {
  PsRank r[kMaxRanks];
};

__device__ __forceinline__ uint64_t Mix64(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

// Counter-based uniform in [-scale, scale): depends only on (seed, field, global row, column),
// so a table has the same contents however it is sharded.
__global__ void __launch_bounds__(256)
TableInitKernel(float* shard, int64_t rows_local, int dim, int field, int rank, int nranks, int64_t rows_global,
                uint64_t seed, float scale) {
  const int64_t total  = rows_local * dim;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    if (scale == 0.f) {
      shard[i] = 0.f;
      continue;
    }
    const int64_t lrow = i / dim;
    const int col      = static_cast<int>(i % dim);
    const int64_t grow = lrow * nranks + rank;
    float v = 0.f;
    if (grow < rows_global) {
      uint64_t h = Mix64(seed ^ (static_cast<uint64_t>(field) << 48) ^ (static_cast<uint64_t>(grow) * 0x9e3779b97f4a7c15ull) ^
                         static_cast<uint64_t>(col) * 0xbf58476d1ce4e5b9ull);
      v = (static_cast<float>(h >> 40) * (1.0f / 16777216.0f) * 2.f - 1.f) * scale;
    }
    shard[i] = v;
  }
}

template <typename OutT>
__global__ void __launch_bounds__(256)
PsPullKernel(PsLaunch args, PsMeta meta, int64_t batch, int64_t out_ld, int64_t out_col0) {
  const PsRank& pr   = args.r[blockIdx.y];
  const int n        = pr.nranks;
  const int dim      = meta.dim;
  const int vecs     = dim / 4;
  int lanes_per_item = 1;
  while (lanes_per_item < vecs && lanes_per_item < 32) lanes_per_item <<= 1;
  const int items_per_warp = 32 / lanes_per_item;
  const int lane     = threadIdx.x & 31;
  const int sub      = lane / lanes_per_item;
  const int sublane  = lane % lanes_per_item;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  OutT* out = static_cast<OutT*>(pr.out);
  for (int64_t base = warp_global * items_per_warp; base < total; base += nwarps * items_per_warp) {
    const int64_t item = base + sub;
    if (item >= total) continue;
    const int f      = static_cast<int>(item % meta.nfields);
    const int64_t b  = item / meta.nfields;
    const int64_t id = pr.ids[item];
    OutT* dst        = out + b * out_ld + out_col0 + static_cast<int64_t>(f) * dim;
    const int owner  = static_cast<int>(id % n);
    const int64_t lrow = id / n;
    if (id < 0 || lrow >= meta.rows_per_shard[f]) {
      if (sublane == 0) atomicExch(pr.error, 2);
      for (int v = sublane; v < vecs; v += lanes_per_item)
        for (int k = 0; k < 4; ++k) dst[v * 4 + k] = FromFloat<OutT>(0.f);
      continue;
    }
    const char* row = pr.slab[owner] + meta.field_off[f] + static_cast<uint64_t>(lrow) * dim * 4;
    for (int v = sublane; v < vecs; v += lanes_per_item) {
      U4 q = owner == pr.rank ? *reinterpret_cast<const U4*>(row + v * 16) : LdSys(row + v * 16);
      const float fv[4] = {__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w)};
      if (sizeof(OutT) == 4) {
        *reinterpret_cast<U4*>(dst + v * 4) = q;
      } else {
        OutT o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = FromFloat<OutT>(fv[k]);
        *reinterpret_cast<uint2*>(dst + v * 4) = *reinterpret_cast<uint2*>(o);
      }
    }
  }
}

// Slot layout of the accumulation table: [slots] u64 keys, then [slots][dim] fp32 sums.
__device__ __forceinline__ uint64_t SlotKey(int field, int64_t lrow) {
  return ((static_cast<uint64_t>(field) << 44) | static_cast<uint64_t>(lrow)) + 1;  // 0 = empty
}

template <typename GradT>
__global__ void __launch_bounds__(256)
PsPushScatterKernel(PsLaunch args, PsMeta meta, int64_t batch, int64_t grad_ld, int64_t grad_col0, uint64_t slots,
                    float grad_scale) {
  const PsRank& pr   = args.r[blockIdx.y];
  const int n        = pr.nranks;
  const int dim      = meta.dim;
  const int vecs     = dim / 4;
  int lanes_per_item = 1;
  while (lanes_per_item < vecs && lanes_per_item < 32) lanes_per_item <<= 1;
  const int items_per_warp = 32 / lanes_per_item;
  const int lane     = threadIdx.x & 31;
  const int sub      = lane / lanes_per_item;
  const int sublane  = lane % lanes_per_item;
  const unsigned group_mask = lanes_per_item == 32 ? 0xffffffffu : (((1u << lanes_per_item) - 1u) << (sub * lanes_per_item));
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  const GradT* grads = static_cast<const GradT*>(pr.grads);
  for (int64_t base = warp_global * items_per_warp; base < total; base += nwarps * items_per_warp) {
    const int64_t item = base + sub;
    if (item >= total) continue;
    const int f      = static_cast<int>(item % meta.nfields);
    const int64_t b  = item / meta.nfields;
    const int64_t id = pr.ids[item];
    const int owner  = static_cast<int>(id % n);
    const int64_t lrow = id / n;
    if (id < 0 || lrow >= meta.rows_per_shard[f]) {
      if (sublane == 0) atomicExch(pr.error, 2);
      continue;
    }
    // claim / find the slot in the owner's table (one lane probes, the group follows)
    uint64_t slot = ~0ull;
    if (sublane == 0) {
      const uint64_t key = SlotKey(f, lrow);
      unsigned long long* keys = reinterpret_cast<unsigned long long*>(pr.acc[owner]);
      uint64_t h = Mix64(key) & (slots - 1);
      for (uint64_t probe = 0; probe < slots && probe < 4096; ++probe) {
        unsigned long long prev = atomicCAS_system(keys + h, 0ull, static_cast<unsigned long long>(key));
        if (prev == 0ull || prev == key) {
          slot = h;
          break;
        }
        h = (h + 1) & (slots - 1);
      }
      if (slot == ~0ull) atomicExch(pr.error, 1);  // table full: the host raises after the step
    }
    slot = __shfl_sync(group_mask, slot, sub * lanes_per_item);
    if (slot == ~0ull) continue;
    float* sums = reinterpret_cast<float*>(pr.acc[owner] + slots * 8) + slot * dim;
    const GradT* g = grads + b * grad_ld + grad_col0 + static_cast<int64_t>(f) * dim;
    for (int v = sublane; v < vecs; v += lanes_per_item) {
      float gv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) gv[k] = ToFloat<GradT>(g[v * 4 + k]) * grad_scale;
      asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(sums + v * 4), "f"(gv[0]), "f"(gv[1]),
                   "f"(gv[2]), "f"(gv[3])
                   : "memory");
    }
  }
}

// Asynchronous push: every gradient row is applied straight to the owner's row with atomics, no accumulation table,
// no fences; concurrent pulls may see a row half-way through an update and duplicate ids are applied one after the
// other.  This is the reference's own consistency model: its servers apply pushes as they arrive, shard by shard, with
// no barrier between workers (tips/core/ps/ps_server.h:248-264).  SGD: w += -lr * g (one vector reduction).  Adagrad:
// read G, then G += g^2 and w += -lr * g / (sqrt(G + g^2) + eps) as two vector reductions.
template <typename GradT>
__global__ void __launch_bounds__(256)
PsPushDirectKernel(PsLaunch args, PsMeta meta, int64_t batch, int64_t grad_ld, int64_t grad_col0, float grad_scale,
                   int rule, float lr, float eps) {
  const PsRank& pr   = args.r[blockIdx.y];
  const int n        = pr.nranks;
  const int dim      = meta.dim;
  const int vecs     = dim / 4;
  int lanes_per_item = 1;
  while (lanes_per_item < vecs && lanes_per_item < 32) lanes_per_item <<= 1;
  const int items_per_warp = 32 / lanes_per_item;
  const int lane     = threadIdx.x & 31;
  const int sub      = lane / lanes_per_item;
  const int sublane  = lane % lanes_per_item;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  const GradT* grads = static_cast<const GradT*>(pr.grads);
  for (int64_t base = warp_global * items_per_warp; base < total; base += nwarps * items_per_warp) {
    const int64_t item = base + sub;
    if (item >= total) continue;
    const int f      = static_cast<int>(item % meta.nfields);
    const int64_t b  = item / meta.nfields;
    const int64_t id = pr.ids[item];
    const int owner  = static_cast<int>(id % n);
    const int64_t lrow = id / n;
    if (id < 0 || lrow >= meta.rows_per_shard[f]) {
      if (sublane == 0) atomicExch(pr.error, 2);
      continue;
    }
    float* w  = reinterpret_cast<float*>(pr.slab[owner] + meta.field_off[f]) + lrow * dim;
    float* st = reinterpret_cast<float*>(pr.slab[owner] + meta.state_off[f]) + lrow * dim;
    const GradT* g = grads + b * grad_ld + grad_col0 + static_cast<int64_t>(f) * dim;
    for (int v = sublane; v < vecs; v += lanes_per_item) {
      float d[4], gv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) gv[k] = ToFloat<GradT>(g[v * 4 + k]) * grad_scale;
      if (rule == 1) {
        // one vector load of the accumulator (it may miss updates that are in flight: the asynchronous model),
        // then two vector reductions; no returning atomics, which would cost a round trip per element
        const U4 q = LdSys(reinterpret_cast<const char*>(st + v * 4));
        const float acc[4] = {__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w)};
        float g2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          g2[k] = gv[k] * gv[k];
          d[k]  = -lr * gv[k] / (sqrtf(acc[k] + g2[k]) + eps);
        }
        asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(st + v * 4), "f"(g2[0]), "f"(g2[1]),
                     "f"(g2[2]), "f"(g2[3])
                     : "memory");
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) d[k] = -lr * gv[k];
      }
      asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(w + v * 4), "f"(d[0]), "f"(d[1]),
                   "f"(d[2]), "f"(d[3])
                   : "memory");
    }
  }
}

// rule: 0 = SGD (w -= lr*g), 1 = Adagrad (G += g*g; w -= lr*g/(sqrt(G)+eps)),
//       2 = the reference's literal rule (w = lr*g, sparse_access_method.h:51-56)
__global__ void __launch_bounds__(256)
PsPushApplyKernel(PsLaunch args, PsMeta meta, uint64_t slots, int rule, float lr, float eps, unsigned long long* touched) {
  const PsRank& pr = args.r[blockIdx.y];
  const int dim    = meta.dim;
  const int vecs   = dim / 4;
  int lanes_per_item = 1;
  while (lanes_per_item < vecs && lanes_per_item < 32) lanes_per_item <<= 1;
  const int items_per_warp = 32 / lanes_per_item;
  const int lane    = threadIdx.x & 31;
  const int sub     = lane / lanes_per_item;
  const int sublane = lane % lanes_per_item;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  unsigned long long* keys  = reinterpret_cast<unsigned long long*>(pr.acc[pr.rank]);
  float* sums_base          = reinterpret_cast<float*>(pr.acc[pr.rank] + slots * 8);
  char* slab                = pr.slab[pr.rank];
  for (uint64_t base = warp_global * items_per_warp; base < slots; base += nwarps * items_per_warp) {
    const uint64_t slot = base + sub;
    if (slot >= slots) continue;
    const uint64_t key = keys[slot];
    if (key == 0) continue;
    const int f        = static_cast<int>((key - 1) >> 44);
    const int64_t lrow = static_cast<int64_t>((key - 1) & ((1ull << 44) - 1));
    float* w  = reinterpret_cast<float*>(slab + meta.field_off[f]) + lrow * dim;
    float* st = reinterpret_cast<float*>(slab + meta.state_off[f]) + lrow * dim;
    float* sums = sums_base + slot * dim;
    for (int v = sublane; v < vecs; v += lanes_per_item) {
      float4 g  = *reinterpret_cast<float4*>(sums + v * 4);
      float4 wv = *reinterpret_cast<float4*>(w + v * 4);
      if (rule == 1) {
        float4 s = *reinterpret_cast<float4*>(st + v * 4);
        s.x += g.x * g.x; s.y += g.y * g.y; s.z += g.z * g.z; s.w += g.w * g.w;
        wv.x -= lr * g.x / (sqrtf(s.x) + eps);
        wv.y -= lr * g.y / (sqrtf(s.y) + eps);
        wv.z -= lr * g.z / (sqrtf(s.z) + eps);
        wv.w -= lr * g.w / (sqrtf(s.w) + eps);
        *reinterpret_cast<float4*>(st + v * 4) = s;
      } else if (rule == 0) {
        wv.x -= lr * g.x; wv.y -= lr * g.y; wv.z -= lr * g.z; wv.w -= lr * g.w;
      } else {
        wv.x = lr * g.x; wv.y = lr * g.y; wv.z = lr * g.z; wv.w = lr * g.w;
      }
      *reinterpret_cast<float4*>(w + v * 4)    = wv;
      *reinterpret_cast<float4*>(sums + v * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncwarp(lanes_per_item == 32 ? 0xffffffffu : (((1u << lanes_per_item) - 1u) << (sub * lanes_per_item)));
    if (sublane == 0) {
      keys[slot] = 0;
      if (touched) atomicAdd(touched, 1ull);
    }
  }
}

// One-block cross-rank barrier: when it completes on this rank, every rank has reached the
// same point of its stream, i.e. finished all the work it enqueued before its own fence.
__global__ void FenceKernel(CommCtx c0, CommCtx c1, CommCtx c2, CommCtx c3, CommCtx c4, CommCtx c5, CommCtx c6, CommCtx c7,
                            int channel) {
  const CommCtx* all[kMaxRanks] = {&c0, &c1, &c2, &c3, &c4, &c5, &c6, &c7};
  const CommCtx& ctx = *all[blockIdx.y];
  const int slot = kMaxCommBlocks - 2;
  uint32_t epoch = ctx.epochs[channel * kMaxCommBlocks + slot] + 1;
  BlockBarrier(ctx, channel, slot, epoch, 7);
  __syncthreads();
  if (threadIdx.x == 0) ctx.epochs[channel * kMaxCommBlocks + slot] = epoch;
}

}  // namespace

// Implemented in comm.cu: gives access to the per-rank contexts.
int CommGetContexts(CommCtx* out, int* rank, int* nranks, int* emulated);

namespace {

struct PsState {
  bool ready = false;
  PsMeta meta;
  char* slab[kMaxRanks];
  char* acc[kMaxRanks];
  uint64_t slots = 0;
  int32_t* error_dev = nullptr;
  unsigned long long* touched_dev = nullptr;
};
PsState g_ps;

int MakePsLaunch(PsLaunch* l, const int64_t* const* ids, const void* const* grads, void* const* outs) {
  CommCtx ctx[kMaxRanks];
  int rank = 0, nranks = 1, emulated = 0;
  int rc = CommGetContexts(ctx, &rank, &nranks, &emulated);
  if (rc) return rc;
  memset(l, 0, sizeof(*l));
  const int local = emulated ? nranks : 1;
  for (int i = 0; i < local; ++i) {
    PsRank& r = l->r[i];
    for (int p = 0; p < nranks; ++p) {
      r.slab[p] = g_ps.slab[p];
      r.acc[p]  = g_ps.acc[p];
    }
    r.ids    = ids ? ids[i] : nullptr;
    r.grads  = grads ? grads[i] : nullptr;
    r.out    = outs ? outs[i] : nullptr;
    r.error  = g_ps.error_dev;
    r.rank   = emulated ? i : rank;
    r.nranks = nranks;
  }
  return local;
}

int PsGrid(int64_t items, int lanes_per_item) {
  int64_t warps  = (items * lanes_per_item + 31) / 32;
  int64_t blocks = (warps + 7) / 8;
  int64_t cap    = static_cast<int64_t>(NumSMs()) * 8;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

int LanesPerItem(int dim) {
  int l = 1;
  while (l < dim / 4 && l < 32) l <<= 1;
  return l;
}

}  // namespace
}  // namespace tipsk

using namespace tipsk;

extern "C" {

/* Cross-rank fence on `channel`, enqueued on `stream`. */
int tipsk_comm_fence(int channel, void* stream) {
  CommCtx ctx[kMaxRanks];
  int rank = 0, nranks = 1, emulated = 0;
  int rc = CommGetContexts(ctx, &rank, &nranks, &emulated);
  if (rc) return rc;
  if (nranks == 1) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(1, emulated ? nranks : 1), block(32);
  CommCtx a[kMaxRanks];
  for (int i = 0; i < kMaxRanks; ++i) a[i] = ctx[emulated ? (i < nranks ? i : 0) : rank];
  if (emulated) {
    void* params[] = {&a[0], &a[1], &a[2], &a[3], &a[4], &a[5], &a[6], &a[7], &channel};
    TIPSK_CUDA(cudaLaunchCooperativeKernel((const void*)FenceKernel, grid, block, params, 0, s));
  } else {
    FenceKernel<<<grid, block, 0, s>>>(a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], channel);
    TIPSK_LAUNCH_CHECK();
  }
  return 0;
}

int tipsk_table_init(float* shard, int64_t rows_local, int dim, int field, int rank, int nranks, int64_t rows_global,
                     uint64_t seed, float scale, void* stream) {
  if (rows_local <= 0) return 0;
  int64_t blocks = (rows_local * dim + 255) / 256;
  int64_t cap    = static_cast<int64_t>(NumSMs()) * 16;
  TableInitKernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      shard, rows_local, dim, field, rank, nranks, rows_global, seed, scale);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* Registers the table slabs and accumulation tables (one pointer per rank, as mapped in this
 * process) and the per-field layout.  `slots` must be a power of two; an accumulation table is
 * slots*8 + slots*dim*4 bytes and must be zero before the first push. */
int tipsk_ps_configure(void* const* slabs, void* const* accs, int nranks, const uint64_t* field_off,
                       const uint64_t* state_off, const int64_t* rows_per_shard, int nfields, int dim, uint64_t slots) {
  TIPSK_REQUIRE(nfields >= 1 && nfields <= kMaxFields, "ps: 1..64 fields are supported");
  TIPSK_REQUIRE(dim >= 4 && dim % 4 == 0, "ps: the row dimension must be a multiple of 4");
  TIPSK_REQUIRE(slots >= 2 && (slots & (slots - 1)) == 0, "ps: slots must be a power of two");
  TIPSK_REQUIRE(nranks >= 1 && nranks <= kMaxRanks, "ps: 1..8 ranks");
  PsState& st = g_ps;
  memset(&st.meta, 0, sizeof(st.meta));
  for (int f = 0; f < nfields; ++f) {
    st.meta.field_off[f]      = field_off[f];
    st.meta.state_off[f]      = state_off ? state_off[f] : 0;
    st.meta.rows_per_shard[f] = rows_per_shard[f];
  }
  st.meta.nfields = nfields;
  st.meta.dim     = dim;
  for (int r = 0; r < kMaxRanks; ++r) {
    st.slab[r] = r < nranks ? static_cast<char*>(slabs[r]) : nullptr;
    st.acc[r]  = r < nranks && accs ? static_cast<char*>(accs[r]) : nullptr;
  }
  st.slots = slots;
  if (!st.error_dev) {
    TIPSK_CUDA(cudaMalloc(reinterpret_cast<void**>(&st.error_dev), sizeof(int32_t)));
    TIPSK_CUDA(cudaMalloc(reinterpret_cast<void**>(&st.touched_dev), sizeof(unsigned long long)));
  }
  TIPSK_CUDA(cudaMemset(st.error_dev, 0, sizeof(int32_t)));
  TIPSK_CUDA(cudaMemset(st.touched_dev, 0, sizeof(unsigned long long)));
  st.ready = true;
  return 0;
}

/* Reads and clears the PS error word (0 ok, 1 accumulation table full, 2 id out of range) and the
 * count of rows updated since the last call.  Synchronises the device. */
int tipsk_ps_status(int32_t* error, uint64_t* touched) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  TIPSK_CUDA(cudaMemcpy(error, st.error_dev, sizeof(int32_t), cudaMemcpyDeviceToHost));
  unsigned long long t = 0;
  TIPSK_CUDA(cudaMemcpy(&t, st.touched_dev, sizeof(t), cudaMemcpyDeviceToHost));
  *touched = t;
  TIPSK_CUDA(cudaMemset(st.error_dev, 0, sizeof(int32_t)));
  TIPSK_CUDA(cudaMemset(st.touched_dev, 0, sizeof(unsigned long long)));
  return 0;
}

/* ids: [batch, nfields] int64 (one pointer per local rank); out: [batch, out_ld] of out_dtype (fp32/bf16),
 * field f lands at columns out_col0 + f*dim.  `fence` non-zero puts a cross-rank fence first, so that
 * rows updated by the previous push on any rank are visible. */
int tipsk_ps_pull(const int64_t* const* ids, void* const* outs, int64_t batch, int64_t out_ld, int64_t out_col0,
                  int out_dtype, int fence, void* stream) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  if (batch <= 0) return 0;
  if (fence) {
    int rc = tipsk_comm_fence(2, stream);
    if (rc) return rc;
  }
  PsLaunch l;
  int local = MakePsLaunch(&l, ids, nullptr, outs);
  if (local < 0) return local;
  const int lpi = LanesPerItem(st.meta.dim);
  dim3 grid(PsGrid(batch * st.meta.nfields, lpi), local);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == kF32)
    PsPullKernel<float><<<grid, 256, 0, s>>>(l, st.meta, batch, out_ld, out_col0);
  else if (out_dtype == kBF16)
    PsPullKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(l, st.meta, batch, out_ld, out_col0);
  else
    return SetError(-2, "ps pull: output must be fp32 or bf16");
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* grads: [batch, grad_ld] of grad_dtype, field f at columns grad_col0 + f*dim. */
int tipsk_ps_push(const int64_t* const* ids, const void* const* grads, int64_t batch, int64_t grad_ld,
                  int64_t grad_col0, int grad_dtype, float grad_scale, int rule, float lr, float eps, void* stream) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  TIPSK_REQUIRE(st.acc[0] != nullptr, "ps push: no accumulation tables configured");
  if (batch <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = tipsk_comm_fence(2, stream);  // every rank finished reading rows (its pull) and clearing slots
  if (rc) return rc;
  PsLaunch l;
  int local = MakePsLaunch(&l, ids, grads, nullptr);
  if (local < 0) return local;
  const int lpi = LanesPerItem(st.meta.dim);
  dim3 grid(PsGrid(batch * st.meta.nfields, lpi), local);
  if (grad_dtype == kF32)
    PsPushScatterKernel<float><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, st.slots, grad_scale);
  else if (grad_dtype == kBF16)
    PsPushScatterKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, st.slots, grad_scale);
  else
    return SetError(-2, "ps push: gradients must be fp32 or bf16");
  TIPSK_LAUNCH_CHECK();
  rc = tipsk_comm_fence(2, stream);  // every rank's scatter has landed
  if (rc) return rc;
  dim3 agrid(PsGrid(static_cast<int64_t>(st.slots), lpi), local);
  PsPushApplyKernel<<<agrid, 256, 0, s>>>(l, st.meta, st.slots, rule, lr, eps, st.touched_dev);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* Asynchronous push (see PsPushDirectKernel): no fences, no accumulation table; rule 0 (SGD) or 1 (Adagrad). */
int tipsk_ps_push_async(const int64_t* const* ids, const void* const* grads, int64_t batch, int64_t grad_ld,
                        int64_t grad_col0, int grad_dtype, float grad_scale, int rule, float lr, float eps,
                        void* stream) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  TIPSK_REQUIRE(rule == 0 || rule == 1, "ps async push: SGD or Adagrad only");
  if (batch <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PsLaunch l;
  int local = MakePsLaunch(&l, ids, grads, nullptr);
  if (local < 0) return local;
  const int lpi = LanesPerItem(st.meta.dim);
  dim3 grid(PsGrid(batch * st.meta.nfields, lpi), local);
  if (grad_dtype == kF32)
    PsPushDirectKernel<float><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, grad_scale, rule, lr, eps);
  else if (grad_dtype == kBF16)
    PsPushDirectKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, grad_scale, rule, lr,
                                                          eps);
  else
    return SetError(-2, "ps push: gradients must be fp32 or bf16");
  TIPSK_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
