// Parameter-server data path on the GPU: sharded embedding tables that live in
// peer-mapped memory, pull fused with the embedding lookup, push fused with a
// local segment-reduce, a cross-rank scatter and the server-side optimizer.
//
// Reference counterpart: PsClient::Pull / PsServer::PullTask (rows travel as
// FlatBuffers over a ZeroMQ RPC, tips/core/ps/ps_client.h:78-109,
// ps_server.h:147-192), PsClient::Push / PsServer::PushTask and the access
// method that applies the update on the server (ps_client.h:111-130,
// ps_server.h:232-265, sparse_access_method.h:41-61), and the zero
// initialisation of a row on first pull (sparse_access_method.h:23-27).
//
// Placement: see ps_placement.h (rotated round-robin, one rule for pull, push,
// initialisation, dump and load).
//
// Pull: one half-warp (or warp) per (sample, field) resolves the owner and
// loads the row straight from the owner's HBM over NVLink with 16-byte
// system-scope loads, converts and writes it into the consumer's input matrix at
// its column offset.  No request message, no staging copy.
//
// Indexed pull (the training path, tipsk_ps_pull with `index`): the (field, id)
// pairs of the batch are first resolved into slots of a LOCAL open-addressing
// table (device-scope CAS in this GPU's L2), which yields the list of distinct
// rows and a slot per item; every distinct row is then fetched ONCE from its
// owner into a row cache and the items are expanded from the cache.  Under a
// Zipf distribution about half of a batch is duplicates, so half of the NVLink
// traffic of the pull disappears, and the index is reused by the push of the
// same step.
//
// Synchronous push, per rank:
//   scatter   every (sample, field) gradient row is added into its slot of the
//             local table (vector float atomics in this GPU's L2): duplicate ids
//             of the batch end up summed in one slot.  With the index of the
//             pull the slot is known; otherwise the slot is found or claimed
//             here and appended to the list of distinct rows
//   send      walks the list of distinct rows: a row this rank owns stays in
//             the table and moves to the apply list; every other row goes to
//             its owner's inbox (a region per sender, so plain 16-byte stores
//             over NVLink, no remote atomics and no round trips), its sums are
//             zeroed and its key stays in place until the apply pass, so that
//             the probe chains of the table stay whole
//   fence     cross-rank barrier; the per-sender row counts travel with it
//   reduce    the owner folds the rows of its inboxes into the same table
//             (rows that several ranks touched are summed) and extends the
//             apply list
//   apply     the owner walks the apply list, applies SGD or Adagrad to the
//             row with the gradient summed over every occurrence on every rank,
//             and clears the slot; the keys of the rows that were sent away are
//             emptied in the same pass
// so the update is exactly the synchronous one: one optimizer step per touched
// row.  With one rank the scatter is followed directly by the apply.  A training
// step needs two fences: the one inside the push and the one in front of the
// next pull (every owner has applied its updates); the push only fences first
// when no fenced pull has run since the previous push.
#include "kernels/comm.cuh"
#include "kernels/common.cuh"
#include "kernels/ps_placement.h"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

constexpr int kMaxFields      = 64;
constexpr uint32_t kNoSlot    = 0xffffffffu;
constexpr unsigned kFullMask  = 0xffffffffu;
constexpr size_t kInboxHeader = 128;  // per-sender row counts, one u32 per rank

struct PsMeta {
  uint64_t field_off[kMaxFields];   // byte offset of the field's shard inside every rank's slab
  uint64_t state_off[kMaxFields];   // byte offset of the optimizer state shard (Adagrad), same layout
  int64_t rows_per_shard[kMaxFields];
  int32_t nfields;
  int32_t dim;                      // fp32 elements per row, multiple of 4
  // Optional bf16 copy of the rows that the owner keeps current (0: none): field f starts at
  // shadow_base + f * rows_per_shard[f] * dim * 2.  Pulls into bf16 read it, which halves their bytes on NVLink.
  uint64_t shadow_base;
};

__host__ __device__ __forceinline__ uint64_t ShadowOffset(const PsMeta& m, int f, int64_t lrow) {
  return m.shadow_base + (static_cast<uint64_t>(f) * m.rows_per_shard[f] + static_cast<uint64_t>(lrow)) * m.dim * 2;
}

// Per-rank control words in device memory; all zero between steps.
struct alignas(8) PsCtl {
  uint32_t ucount;                  // entries of the list of distinct rows of the batch
  uint32_t acount;                  // entries of the apply list (several ranks)
  uint32_t done;                    // blocks of the running list walker that have finished
  uint32_t send_count[kMaxRanks];   // rows sent to each owner by the running send
  uint32_t pad[5];
  unsigned long long sent_total;    // distinct rows of the batches since the last status call (own rows included)
  unsigned long long sent_remote;   // of those, rows that crossed NVLink
  unsigned long long applied;       // rows updated since the last status call
  unsigned long long fetched_remote;  // rows that the indexed pull read over NVLink
};

struct PsRank {
  char* slab[kMaxRanks];            // every server's table slab as mapped here
  char* inbox[kMaxRanks];           // every server's inbox as mapped here (null with one rank)
  char* acc;                        // local table: [slots] u64 keys, [slots][dim] fp32 sums
  uint32_t* ulist;                  // [2][slots]: list of distinct rows of the batch, then the apply list
  PsCtl* ctl;
  uint32_t* item_slot;              // [capacity] slot of every (sample, field) item of the indexed batch
  char* cache;                      // [slots][dim] rows fetched by the indexed pull, in the output dtype
  const int64_t* ids;               // [batch, nfields]
  const void* grads;                // push: [batch, ld] rows of nfields*dim (fp32 or bf16)
  void* out;                        // pull: [batch, ld]
  int32_t* error;                   // local error word (table full, bad id, inbox full)
  int32_t rank;
  int32_t nranks;                   // ranks of the job: every one of them may pull and push (a worker)
  int32_t nservers;                 // ranks that hold shards; slab[] and inbox[] are in server order
  int32_t my_server;                // this rank's index among the servers, or -1 for a pure worker
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

// Work split of a warp over rows of `dim` floats: `lpi` lanes move one row as 16-byte vectors.
struct RowLanes {
  int lpi, ipw, sub, sublane, lane;
  __device__ __forceinline__ explicit RowLanes(int dim) {
    const int vecs = dim / 4;
    lpi = 1;
    while (lpi < vecs && lpi < 32) lpi <<= 1;
    ipw     = 32 / lpi;
    lane    = threadIdx.x & 31;
    sub     = lane / lpi;
    sublane = lane % lpi;
  }
  __device__ __forceinline__ unsigned group_mask() const {
    return lpi == 32 ? kFullMask : (((1u << lpi) - 1u) << (sub * lpi));
  }
};

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
    const int64_t grow = PsGlobalId(field, lrow, rank, nranks);
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
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nservers;
  const int dim    = meta.dim;
  const int vecs   = dim / 4;
  const RowLanes L(dim);
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  OutT* out = static_cast<OutT*>(pr.out);
  for (int64_t base = warp_global * L.ipw; base < total; base += nwarps * L.ipw) {
    const int64_t item = base + L.sub;
    if (item >= total) continue;
    const int f      = static_cast<int>(item % meta.nfields);
    const int64_t b  = item / meta.nfields;
    const int64_t id = pr.ids[item];
    OutT* dst        = out + b * out_ld + out_col0 + static_cast<int64_t>(f) * dim;
    int owner;
    int64_t lrow;
    PsPlace(f, id < 0 ? 0 : id, n, &owner, &lrow);
    if (id < 0 || lrow >= meta.rows_per_shard[f]) {
      if (L.sublane == 0) atomicExch(pr.error, 2);
      for (int v = L.sublane; v < vecs; v += L.lpi)
        for (int k = 0; k < 4; ++k) dst[v * 4 + k] = FromFloat<OutT>(0.f);
      continue;
    }
    const char* row = pr.slab[owner] + meta.field_off[f] + static_cast<uint64_t>(lrow) * dim * 4;
    for (int v = L.sublane; v < vecs; v += L.lpi) {
      U4 q = owner == pr.my_server ? *reinterpret_cast<const U4*>(row + v * 16) : LdSys(row + v * 16);
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

// Key of a table slot: field and global row id; 0 = empty.
__device__ __forceinline__ uint64_t SlotKey(int field, int64_t id) {
  return ((static_cast<uint64_t>(field) << 44) | static_cast<uint64_t>(id)) + 1;
}
__device__ __forceinline__ int KeyField(uint64_t key) { return static_cast<int>((key - 1) >> 44); }
__device__ __forceinline__ int64_t KeyId(uint64_t key) { return static_cast<int64_t>((key - 1) & ((1ull << 44) - 1)); }

// Finds or claims the slot of `key` in the local table; *claimed tells whether this call created it.
__device__ __forceinline__ uint32_t ClaimSlot(unsigned long long* keys, uint64_t slots, uint64_t key, bool* claimed) {
  uint64_t h = Mix64(key) & (slots - 1);
  for (uint32_t probe = 0; probe < 4096 && probe < slots; ++probe) {
    const unsigned long long prev = atomicCAS(keys + h, 0ull, static_cast<unsigned long long>(key));
    if (prev == 0ull) {
      *claimed = true;
      return static_cast<uint32_t>(h);
    }
    if (prev == key) return static_cast<uint32_t>(h);
    h = (h + 1) & (slots - 1);
  }
  return kNoSlot;
}

// Appends the slots flagged by the lanes of this warp to a list: one atomic per warp.
// Every lane of the warp calls it.
__device__ __forceinline__ void AppendSlots(uint32_t* list, uint32_t* count, bool flagged, uint32_t slot, int lane) {
  const unsigned m = __ballot_sync(kFullMask, flagged);
  if (m == 0) return;
  const int leader = __ffs(m) - 1;
  uint32_t first   = 0;
  if (lane == leader) first = atomicAdd(count, static_cast<uint32_t>(__popc(m)));
  first = __shfl_sync(kFullMask, first, leader);
  if (flagged) list[first + __popc(m & ((1u << lane) - 1u))] = slot;
}

// No "memory" clobber: nothing in these kernels reads the sums back, so the loads of the next rows may be
// scheduled ahead of the reduction.
__device__ __forceinline__ void RedAdd4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d));
}

// System-scope 16-byte load of data that no one writes while the kernel runs (rows between two fences, inbox
// entries after the fence): not volatile and without a "memory" clobber, so several of them can be in flight.
__device__ __forceinline__ U4 LdSysFree(const void* addr) {
  U4 v;
  asm("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr));
  return v;
}

template <typename GradT, bool kVec>
__device__ __forceinline__ void LoadGrad4(const GradT* g, float* out) {
  if (kVec) {
    if (sizeof(GradT) == 4) {
      const float4 q = *reinterpret_cast<const float4*>(g);
      out[0] = q.x; out[1] = q.y; out[2] = q.z; out[3] = q.w;
    } else {
      uint2 q = *reinterpret_cast<const uint2*>(g);
      const GradT* h = reinterpret_cast<const GradT*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = ToFloat<GradT>(h[k]);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) out[k] = ToFloat<GradT>(g[k]);
  }
}

constexpr int kRowsInFlight = 8;  // rows that a lane group loads before it stores the first one

// Resolves every (sample, field) item of the batch into a slot of the local table: the distinct rows land in
// the list, item_slot[item] holds the slot (kNoSlot for a bad id or a full table).
__global__ void __launch_bounds__(256)
PsIndexKernel(PsLaunch args, PsMeta meta, int64_t batch, uint64_t slots) {
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nservers;  // placement is among the servers
  const int lane   = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  unsigned long long* keys  = reinterpret_cast<unsigned long long*>(pr.acc);
  for (int64_t base = warp_global * 32; base < total; base += nwarps * 32) {
    const int64_t mine = base + lane;
    uint32_t slot = kNoSlot;
    bool claimed  = false;
    if (mine < total) {
      const int f      = static_cast<int>(mine % meta.nfields);
      const int64_t id = pr.ids[mine];
      if (id < 0 || id / n >= meta.rows_per_shard[f]) {
        atomicExch(pr.error, 2);
      } else {
        slot = ClaimSlot(keys, slots, SlotKey(f, id), &claimed);
        if (slot == kNoSlot) atomicExch(pr.error, 1);
      }
      pr.item_slot[mine] = slot;
    }
    AppendSlots(pr.ulist, &pr.ctl->ucount, claimed, slot, lane);
  }
}

constexpr int kChunk = 256;  // list entries that a block resolves together (one per thread)

// Moves the rows that a block has resolved into shared memory (s_slot: table slot or kNoSlot, s_ptr: the other
// end of the copy): `lpi` lanes per row, kRowsInFlight rows loaded by a lane group before the first is consumed.
// load(ptr, slot, v) returns the 16 bytes of vector v of a row, store(ptr, slot, v, q) consumes them.
template <typename Load, typename Store>
__device__ __forceinline__ void MoveRows(const uint32_t* s_slot, char* const* s_ptr, int dim, Load load, Store store) {
  const int vecs = dim / 4;
  int lpi = 1;
  while (lpi < vecs && lpi < 32) lpi <<= 1;
  const int groups  = kChunk / lpi;
  const int g       = threadIdx.x / lpi;
  const int sublane = threadIdx.x % lpi;
  for (int v = sublane; v < vecs; v += lpi) {
    for (int r0 = g; r0 < kChunk; r0 += groups * kRowsInFlight) {
      U4 q[kRowsInFlight];
      uint32_t sl[kRowsInFlight];
      char* ptr[kRowsInFlight];
#pragma unroll
      for (int u = 0; u < kRowsInFlight; ++u) {
        const int r = r0 + u * groups;
        sl[u]       = r < kChunk ? s_slot[r] : kNoSlot;
        if (sl[u] == kNoSlot) continue;
        ptr[u] = s_ptr[r];
        q[u]   = load(ptr[u], sl[u], v);
      }
#pragma unroll
      for (int u = 0; u < kRowsInFlight; ++u)
        if (sl[u] != kNoSlot) store(ptr[u], sl[u], v, q[u]);
    }
  }
}

// Fetches every distinct row of the indexed batch once, from its owner's HBM, into the row cache (converted to
// the output dtype).  A block resolves 256 list entries at a time (slot -> key -> owner and address, one entry
// per thread, so the dependent loads of all of them overlap), then moves their rows.
template <typename OutT>
__global__ void __launch_bounds__(kChunk)
PsFetchKernel(PsLaunch args, PsMeta meta, uint64_t slots) {
  __shared__ uint32_t s_slot[kChunk];
  __shared__ char* s_ptr[kChunk];
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nservers;  // placement is among the servers
  const int dim    = meta.dim;
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(pr.acc);
  OutT* cache              = reinterpret_cast<OutT*>(pr.cache);
  const bool shadow        = sizeof(OutT) == 2 && meta.shadow_base != 0;
  const int64_t total      = *reinterpret_cast<volatile uint32_t*>(&pr.ctl->ucount);
  const int64_t nchunks    = (total + kChunk - 1) / kChunk;
  for (int64_t chunk = blockIdx.x; chunk < nchunks; chunk += gridDim.x) {
    const int64_t mine = chunk * kChunk + threadIdx.x;
    uint32_t slot = kNoSlot;
    char* row     = nullptr;
    int remote    = 0;
    if (mine < total) {
      slot = pr.ulist[mine];
      const unsigned long long key = keys[slot];
      const int f = KeyField(key);
      int owner;
      int64_t lrow;
      PsPlace(f, KeyId(key), n, &owner, &lrow);
      row    = shadow ? pr.slab[owner] + ShadowOffset(meta, f, lrow)
                      : pr.slab[owner] + meta.field_off[f] + static_cast<uint64_t>(lrow) * dim * 4;
      remote = owner != pr.my_server;
    }
    s_slot[threadIdx.x] = slot;
    s_ptr[threadIdx.x]  = row;
    const int nremote   = __syncthreads_count(remote);
    if (threadIdx.x == 0 && nremote) atomicAdd(&pr.ctl->fetched_remote, static_cast<unsigned long long>(nremote));
    MoveRows(
        s_slot, s_ptr, dim,
        [&](char* p, uint32_t, int v) {
          if (!shadow) return LdSysFree(p + v * 16);
          U4 q{0, 0, 0, 0};  // four bf16 values of the owner's bf16 copy: 8 bytes per lane
          asm("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(q.x), "=r"(q.y) : "l"(p + v * 8));
          return q;
        },
        [&](char*, uint32_t sl, int v, const U4& q) {
          OutT* dst = cache + static_cast<uint64_t>(sl) * dim + v * 4;
          if (sizeof(OutT) == 4) {
            *reinterpret_cast<U4*>(dst) = q;
          } else if (shadow) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(q.x, q.y);
          } else {
            OutT o[4] = {FromFloat<OutT>(__uint_as_float(q.x)), FromFloat<OutT>(__uint_as_float(q.y)),
                         FromFloat<OutT>(__uint_as_float(q.z)), FromFloat<OutT>(__uint_as_float(q.w))};
            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(o);
          }
        });
    __syncthreads();
  }
}

// Copies every item's row from the cache into the consumer's input matrix.
template <typename OutT>
__global__ void __launch_bounds__(256)
PsExpandKernel(PsLaunch args, PsMeta meta, int64_t batch, int64_t out_ld, int64_t out_col0) {
  const PsRank& pr = args.r[blockIdx.y];
  const int dim    = meta.dim;
  const int vecs   = dim / 4;
  const RowLanes L(dim);
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  const OutT* cache         = reinterpret_cast<const OutT*>(pr.cache);
  OutT* out                 = static_cast<OutT*>(pr.out);
  using V = typename std::conditional<sizeof(OutT) == 4, U4, uint2>::type;  // four elements
  for (int64_t base = warp_global * L.ipw; base < total; base += nwarps * L.ipw) {
    const int64_t item = base + L.sub;
    if (item >= total) continue;
    const int f       = static_cast<int>(item % meta.nfields);
    const int64_t b   = item / meta.nfields;
    const uint32_t sl = pr.item_slot[item];
    OutT* dst         = out + b * out_ld + out_col0 + static_cast<int64_t>(f) * dim;
    for (int v = L.sublane; v < vecs; v += L.lpi) {
      V q{};
      if (sl != kNoSlot) q = *reinterpret_cast<const V*>(cache + static_cast<uint64_t>(sl) * dim + v * 4);
      *reinterpret_cast<V*>(dst + v * 4) = q;
    }
  }
}

// Forgets an index that no push consumed: empties the slots of the list.
__global__ void __launch_bounds__(256)
PsClearIndexKernel(PsLaunch args, uint64_t slots);

// Local segment-reduce of the batch.  kIndexed: the slot of every item comes from the index of the pull.
// Otherwise phase 1 resolves one item per lane (32 probes in flight per warp) and extends the list of distinct
// rows; phase 2 adds the gradient rows with `lpi` lanes per row.
template <typename GradT, bool kVec, bool kIndexed>
__global__ void __launch_bounds__(256)
PsScatterKernel(PsLaunch args, PsMeta meta, int64_t batch, int64_t grad_ld, int64_t grad_col0, uint64_t slots,
                float grad_scale) {
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nservers;  // placement is among the servers
  const int dim    = meta.dim;
  const int vecs   = dim / 4;
  const RowLanes L(dim);
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  const GradT* grads        = static_cast<const GradT*>(pr.grads);
  unsigned long long* keys  = reinterpret_cast<unsigned long long*>(pr.acc);
  float* sums_base          = reinterpret_cast<float*>(pr.acc + slots * 8);
  for (int64_t base = warp_global * 32; base < total; base += nwarps * 32) {
    const int64_t mine = base + L.lane;
    uint32_t slot = kNoSlot;
    if (kIndexed) {
      if (mine < total) slot = pr.item_slot[mine];
    } else {
      bool claimed = false;
      if (mine < total) {
        const int f      = static_cast<int>(mine % meta.nfields);
        const int64_t id = pr.ids[mine];
        if (id < 0 || id / n >= meta.rows_per_shard[f]) {
          atomicExch(pr.error, 2);
        } else {
          slot = ClaimSlot(keys, slots, SlotKey(f, id), &claimed);
          if (slot == kNoSlot) atomicExch(pr.error, 1);  // table full: the host raises after the step
        }
      }
      AppendSlots(pr.ulist, &pr.ctl->ucount, claimed, slot, L.lane);
    }
    for (int j = 0; j < 32; j += L.ipw) {
      const int src      = j + L.sub;
      const uint32_t s   = __shfl_sync(kFullMask, slot, src);
      const int64_t item = base + src;
      if (item >= total || s == kNoSlot) continue;
      const int f     = static_cast<int>(item % meta.nfields);
      const int64_t b = item / meta.nfields;
      float* sums     = sums_base + static_cast<uint64_t>(s) * dim;
      const GradT* g  = grads + b * grad_ld + grad_col0 + static_cast<int64_t>(f) * dim;
      for (int v = L.sublane; v < vecs; v += L.lpi) {
        float gv[4];
        LoadGrad4<GradT, kVec>(g + v * 4, gv);
        RedAdd4(sums + v * 4, gv[0] * grad_scale, gv[1] * grad_scale, gv[2] * grad_scale, gv[3] * grad_scale);
      }
    }
  }
}

// Byte offsets inside an inbox: header, then per sender `cap` keys, then per sender `cap` rows.
__device__ __forceinline__ unsigned long long* InboxKeys(char* inbox, int sender, uint64_t cap) {
  return reinterpret_cast<unsigned long long*>(inbox + kInboxHeader) + static_cast<uint64_t>(sender) * cap;
}
__device__ __forceinline__ float* InboxRows(char* inbox, int nranks, int sender, uint64_t cap, int dim) {
  return reinterpret_cast<float*>(inbox + kInboxHeader + static_cast<uint64_t>(nranks) * cap * 8) +
         static_cast<uint64_t>(sender) * cap * dim;
}

// Last-block detection for the list walkers: returns true in exactly one block, after every other
// block of this rank's grid row has finished its share.
__device__ __forceinline__ bool LastBlockDone(PsCtl* ctl) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&ctl->done, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  return s_last != 0;
}

__global__ void __launch_bounds__(256)
PsClearIndexKernel(PsLaunch args, uint64_t slots) {
  const PsRank& pr = args.r[blockIdx.y];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(pr.acc);
  const int64_t total      = *reinterpret_cast<volatile uint32_t*>(&pr.ctl->ucount);
  const int64_t stride     = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    keys[pr.ulist[i]] = 0;
  if (LastBlockDone(pr.ctl) && threadIdx.x == 0) {
    pr.ctl->ucount = 0;
    pr.ctl->done   = 0;
  }
  (void)slots;
}

// Positions for the entries of a block in per-destination lists: every thread names a destination (or -1),
// gets its position inside the block with a shared-memory atomic, one thread per destination reserves the block's
// range with ONE global atomic, and the thread's final position comes back.  All threads of the block call it.
__device__ __forceinline__ uint32_t ReservePositions(int dest, int ndest, uint32_t* const* counters, uint32_t* s_cnt,
                                                     uint32_t* s_base) {
  if (threadIdx.x < ndest) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  uint32_t local = 0;
  if (dest >= 0) local = atomicAdd(&s_cnt[dest], 1u);
  __syncthreads();
  if (threadIdx.x < ndest) s_base[threadIdx.x] = s_cnt[threadIdx.x] ? atomicAdd(counters[threadIdx.x], s_cnt[threadIdx.x]) : 0;
  __syncthreads();
  return dest >= 0 ? s_base[dest] + local : 0;
}

// Walks the list of distinct rows of the batch: a row this rank owns stays in the table and joins the apply
// list; every other row goes to its owner's inbox, its sums are zeroed and its key stays until the apply pass.
// wire_bf16: the summed rows cross NVLink as bf16 (half the bytes); the inbox keeps its fp32 row pitch.
__global__ void __launch_bounds__(kChunk)
PsSendKernel(PsLaunch args, PsMeta meta, uint64_t slots, uint64_t cap, int wire_bf16) {
  __shared__ uint32_t s_slot[kChunk];
  __shared__ char* s_ptr[kChunk];
  __shared__ uint32_t s_cnt[kMaxRanks + 1], s_base[kMaxRanks + 1];
  __shared__ uint32_t* s_counter[kMaxRanks + 1];
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nranks;    // senders: every rank of the job
  const int ns     = pr.nservers;  // destinations: the ranks that hold shards
  const int dim    = meta.dim;
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(pr.acc);
  float* sums_base         = reinterpret_cast<float*>(pr.acc + slots * 8);
  uint32_t* apply_list     = pr.ulist + slots;
  const int64_t total      = *reinterpret_cast<volatile uint32_t*>(&pr.ctl->ucount);
  const int64_t nchunks    = (total + kChunk - 1) / kChunk;
  // destination d < ns: the inbox of server d; destination ns: this rank's apply list
  if (threadIdx.x <= ns) s_counter[threadIdx.x] = threadIdx.x < ns ? &pr.ctl->send_count[threadIdx.x] : &pr.ctl->acount;
  __syncthreads();
  for (int64_t chunk = blockIdx.x; chunk < nchunks; chunk += gridDim.x) {
    const int64_t mine = chunk * kChunk + threadIdx.x;
    uint32_t slot = kNoSlot;
    int owner     = -1;
    unsigned long long key = 0;
    if (mine < total) {
      slot = pr.ulist[mine];
      key  = keys[slot];
      int64_t lrow;
      PsPlace(KeyField(key), KeyId(key), ns, &owner, &lrow);
    }
    const bool own     = owner >= 0 && owner == pr.my_server;
    const uint32_t pos = ReservePositions(own ? ns : owner, ns + 1, s_counter, s_cnt, s_base);
    char* dst = nullptr;
    if (own) {
      apply_list[pos] = slot;
      slot            = kNoSlot;  // nothing to send
    } else if (owner >= 0) {
      if (pos < cap) {
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(InboxKeys(pr.inbox[owner], pr.rank, cap) + pos), "l"(key)
                     : "memory");
        dst = reinterpret_cast<char*>(InboxRows(pr.inbox[owner], n, pr.rank, cap, dim) + static_cast<uint64_t>(pos) * dim);
      } else {
        atomicExch(pr.error, 3);  // inbox full: the row is dropped, the host raises after the step
      }
      // The key stays in its slot until the apply pass: emptying it here would cut the probe chains of the
      // rows that remain, and the reduce pass would then claim a second slot for a key that is already present.
    }
    s_slot[threadIdx.x] = slot;
    s_ptr[threadIdx.x]  = dst;
    __syncthreads();
    MoveRows(
        s_slot, s_ptr, dim,
        [&](char*, uint32_t sl, int v) {
          return *reinterpret_cast<const U4*>(sums_base + static_cast<uint64_t>(sl) * dim + v * 4);
        },
        [&](char* d, uint32_t sl, int v, const U4& q) {
          if (d) {
            if (wire_bf16) {
              const __nv_bfloat162 lo = __floats2bfloat162_rn(__uint_as_float(q.x), __uint_as_float(q.y));
              const __nv_bfloat162 hi = __floats2bfloat162_rn(__uint_as_float(q.z), __uint_as_float(q.w));
              asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(d + v * 8),
                           "r"(*reinterpret_cast<const uint32_t*>(&lo)), "r"(*reinterpret_cast<const uint32_t*>(&hi))
                           : "memory");
            } else {
              StSys(d + v * 16, q);
            }
          }
          *reinterpret_cast<float4*>(sums_base + static_cast<uint64_t>(sl) * dim + v * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        });
    __syncthreads();
  }
  if (LastBlockDone(pr.ctl)) {
    __shared__ unsigned long long s_remote;
    if (threadIdx.x == 0) s_remote = 0;
    __syncthreads();
    if (threadIdx.x < ns && threadIdx.x != pr.my_server) {
      const int o = threadIdx.x;
      uint32_t c  = atomicExch(&pr.ctl->send_count[o], 0u);
      if (c > cap) c = static_cast<uint32_t>(cap);
      // the count is published by the fence that follows (system-scope release after this kernel)
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t*>(pr.inbox[o]) + pr.rank), "r"(c)
                   : "memory");
      atomicAdd(&s_remote, static_cast<unsigned long long>(c));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      pr.ctl->sent_total += static_cast<unsigned long long>(total);
      pr.ctl->sent_remote += s_remote;
      pr.ctl->done = 0;  // ucount stays: the apply pass empties the slots of the rows that were sent
    }
    __threadfence_system();
  }
}

// The owner folds the rows that arrived in its inboxes into its local table and extends the apply list.
__global__ void __launch_bounds__(kChunk)
PsOwnerReduceKernel(PsLaunch args, PsMeta meta, uint64_t slots, uint64_t cap, int wire_bf16) {
  __shared__ uint32_t s_slot[kChunk];
  __shared__ char* s_ptr[kChunk];
  __shared__ uint32_t s_cnt[1], s_base[1];
  __shared__ uint32_t* s_counter[1];
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nranks;
  const int dim    = meta.dim;
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(pr.acc);
  float* sums_base         = reinterpret_cast<float*>(pr.acc + slots * 8);
  uint32_t* apply_list     = pr.ulist + slots;
  char* inbox              = pr.inbox[pr.my_server < 0 ? 0 : pr.my_server];
  // exclusive prefix of the per-sender counts (written by the senders, published by the fence)
  uint32_t start[kMaxRanks + 1];
  start[0] = 0;
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s) {
    uint32_t c = 0;
    if (pr.my_server >= 0 && s < n && s != pr.rank) {
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(c) : "l"(reinterpret_cast<uint32_t*>(inbox) + s) : "memory");
      if (c > cap) c = static_cast<uint32_t>(cap);
    }
    start[s + 1] = start[s] + c;
  }
  const int64_t total   = start[kMaxRanks];
  const int64_t nchunks = (total + kChunk - 1) / kChunk;
  char* rows            = inbox + kInboxHeader + static_cast<uint64_t>(n) * cap * 8;
  if (threadIdx.x == 0) s_counter[0] = &pr.ctl->acount;
  __syncthreads();
  for (int64_t chunk = blockIdx.x; chunk < nchunks; chunk += gridDim.x) {
    const int64_t mine = chunk * kChunk + threadIdx.x;
    uint32_t slot = kNoSlot;
    char* row     = nullptr;
    bool claimed  = false;
    if (mine < total) {
      int s           = 0;
      uint32_t sstart = 0;
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k)
        if (mine >= start[k]) {
          s      = k;
          sstart = start[k];
        }
      const uint64_t cell = static_cast<uint64_t>(s) * cap + (mine - sstart);  // where the entry sits in the inbox
      unsigned long long key;
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];"
                   : "=l"(key)
                   : "l"(reinterpret_cast<unsigned long long*>(inbox + kInboxHeader) + cell)
                   : "memory");
      slot = ClaimSlot(keys, slots, key, &claimed);
      if (slot == kNoSlot) atomicExch(pr.error, 1);
      row = rows + cell * dim * 4;
    }
    const uint32_t pos = ReservePositions(claimed ? 0 : -1, 1, s_counter, s_cnt, s_base);
    if (claimed) apply_list[pos] = slot;
    s_slot[threadIdx.x] = slot;
    s_ptr[threadIdx.x]  = row;
    __syncthreads();
    MoveRows(
        s_slot, s_ptr, dim,
        [&](char* p, uint32_t, int v) {
          if (!wire_bf16) return LdSysFree(p + v * 16);
          uint32_t a, b;
          asm("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "l"(p + v * 8));
          U4 q;  // bf16 -> fp32: the 16 bits become the high half of the word
          q.x = a << 16; q.y = a & 0xffff0000u; q.z = b << 16; q.w = b & 0xffff0000u;
          return q;
        },
        [&](char*, uint32_t sl, int v, const U4& q) {
          RedAdd4(sums_base + static_cast<uint64_t>(sl) * dim + v * 4, __uint_as_float(q.x), __uint_as_float(q.y),
                  __uint_as_float(q.z), __uint_as_float(q.w));
        });
    __syncthreads();
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
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nservers;  // placement is among the servers
  const int dim    = meta.dim;
  const int vecs   = dim / 4;
  const RowLanes L(dim);
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total       = batch * meta.nfields;
  const GradT* grads = static_cast<const GradT*>(pr.grads);
  for (int64_t base = warp_global * L.ipw; base < total; base += nwarps * L.ipw) {
    const int64_t item = base + L.sub;
    if (item >= total) continue;
    const int f      = static_cast<int>(item % meta.nfields);
    const int64_t b  = item / meta.nfields;
    const int64_t id = pr.ids[item];
    int owner;
    int64_t lrow;
    PsPlace(f, id < 0 ? 0 : id, n, &owner, &lrow);
    if (id < 0 || lrow >= meta.rows_per_shard[f]) {
      if (L.sublane == 0) atomicExch(pr.error, 2);
      continue;
    }
    float* w  = reinterpret_cast<float*>(pr.slab[owner] + meta.field_off[f]) + lrow * dim;
    float* st = reinterpret_cast<float*>(pr.slab[owner] + meta.state_off[f]) + lrow * dim;
    const GradT* g = grads + b * grad_ld + grad_col0 + static_cast<int64_t>(f) * dim;
    for (int v = L.sublane; v < vecs; v += L.lpi) {
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
// Walks the touched list only: the cost follows the number of distinct rows, not the table size.
__global__ void __launch_bounds__(256)
PsPushApplyKernel(PsLaunch args, PsMeta meta, uint64_t slots, int rule, float lr, float eps) {
  const PsRank& pr = args.r[blockIdx.y];
  const int n      = pr.nranks;
  const int ns     = pr.nservers;
  const int dim    = meta.dim;
  const int vecs   = dim / 4;
  const RowLanes L(dim);
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  unsigned long long* keys  = reinterpret_cast<unsigned long long*>(pr.acc);
  float* sums_base          = reinterpret_cast<float*>(pr.acc + slots * 8);
  char* slab                = pr.slab[pr.my_server < 0 ? 0 : pr.my_server];
  // several ranks: the apply list that send and reduce built; one rank: the list of distinct rows of the batch
  const uint32_t* list      = n > 1 ? pr.ulist + slots : pr.ulist;
  uint32_t* count           = n > 1 ? &pr.ctl->acount : &pr.ctl->ucount;
  const int64_t total       = *reinterpret_cast<volatile uint32_t*>(count);
  for (int64_t base = warp_global * L.ipw; base < total; base += nwarps * L.ipw) {
    const int64_t e = base + L.sub;
    if (e >= total) continue;
    const uint32_t slot = list[e];
    const uint64_t key  = keys[slot];
    const int f         = KeyField(key);
    int owner;
    int64_t lrow;
    PsPlace(f, KeyId(key), ns, &owner, &lrow);
    float* w    = reinterpret_cast<float*>(slab + meta.field_off[f]) + lrow * dim;
    float* st   = reinterpret_cast<float*>(slab + meta.state_off[f]) + lrow * dim;
    float* sums = sums_base + static_cast<uint64_t>(slot) * dim;
    for (int v = L.sublane; v < vecs; v += L.lpi) {
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
      if (meta.shadow_base) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y), hi = __floats2bfloat162_rn(wv.z, wv.w);
        *reinterpret_cast<uint2*>(slab + ShadowOffset(meta, f, lrow) + v * 8) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
      }
    }
    __syncwarp(L.group_mask());
    if (L.sublane == 0) keys[slot] = 0;
  }
  if (n > 1) {
    // rows of this rank's batch that other ranks own were sent away: their sums are zero, empty their keys
    const int64_t batch_rows = *reinterpret_cast<volatile uint32_t*>(&pr.ctl->ucount);
    const int64_t stride     = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < batch_rows; i += stride) {
      const uint32_t slot = pr.ulist[i];
      const uint64_t key  = *reinterpret_cast<volatile unsigned long long*>(keys + slot);
      if (key == 0) continue;  // a row of this rank, already applied and emptied by the loop above
      int owner;
      int64_t lrow;
      PsPlace(KeyField(key), KeyId(key), ns, &owner, &lrow);
      if (owner != pr.my_server) keys[slot] = 0;
    }
  }
  if (LastBlockDone(pr.ctl)) {
    if (threadIdx.x == 0) {
      pr.ctl->applied += static_cast<unsigned long long>(total);
      if (n == 1) pr.ctl->sent_total += static_cast<unsigned long long>(total);
      pr.ctl->ucount = 0;
      pr.ctl->acount = 0;
      pr.ctl->done   = 0;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Tables keyed by arbitrary 64-bit ids: rows are created on first pull, as in the reference's sparse table
// (PullAccessAgent creates and zero-initialises a missing row, tips/core/ps/access_method.h:90-99,
// sparse_access_method.h:23-27; any hashable key, sparse_table.h:164-165).  Every rank owns an open-addressing
// table in peer-mapped memory: [cap] keys (stored as key + 1, 0 = empty), [cap][dim] fp32 rows that start at
// zero, and the Adagrad accumulators.  The owner of a key is a hash of it; a pull finds the slot or claims an
// empty one with a system-scope CAS on the owner's memory (bounded probes; a full table raises an error word),
// then reads the row.  A push finds the slot (a key that was never pulled is counted as missing, like the host
// server does) and applies SGD or Adagrad to the owner's row with vector atomics as the gradients arrive: the
// reference's consistency model, servers apply pushes in arrival order (ps_server.h:248-264).
struct HashTables {
  unsigned long long* keys[kMaxRanks];
  float* rows[kMaxRanks];
  float* state[kMaxRanks];
  uint64_t cap;   // slots per rank, power of two
  int32_t dim;
  int32_t nranks;
};
struct HashIO {
  const int64_t* ids[kMaxRanks];   // per local rank: [count] keys
  const void* grads[kMaxRanks];    // push: [count, ld]
  void* out[kMaxRanks];            // pull: [count, ld]
  int32_t* error;                  // 1 table full, 2 key not representable
  unsigned long long* missing;     // push: rows that were never pulled
};

constexpr uint32_t kHashMaxProbes = 4096;

__device__ __forceinline__ int HashOwner(uint64_t key, int n) { return static_cast<int>(Mix64(key ^ 0x9e3779b97f4a7c15ull) % n); }

// Slot of `key` in the owner's table; insert = claim an empty slot when the key is absent.
__device__ __forceinline__ uint32_t HashFind(unsigned long long* keys, uint64_t cap, uint64_t key, bool insert) {
  const unsigned long long stored = key + 1;
  uint64_t h = Mix64(key) & (cap - 1);
  for (uint32_t probe = 0; probe < kHashMaxProbes && probe < cap; ++probe) {
    unsigned long long cur;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(cur) : "l"(keys + h) : "memory");
    if (cur == stored) return static_cast<uint32_t>(h);
    if (cur == 0ull) {
      if (!insert) return kNoSlot;
      cur = atomicCAS_system(keys + h, 0ull, stored);
      if (cur == 0ull || cur == stored) return static_cast<uint32_t>(h);
    }
    h = (h + 1) & (cap - 1);
  }
  return kNoSlot - 1;  // probes exhausted: the table is (nearly) full
}

template <typename OutT>
__global__ void __launch_bounds__(256)
HashPullKernel(HashTables t, HashIO io, int64_t count, int64_t out_ld) {
  const int dim  = t.dim;
  const int vecs = dim / 4;
  const RowLanes L(dim);
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t* ids        = io.ids[blockIdx.y];
  OutT* out                 = static_cast<OutT*>(io.out[blockIdx.y]);
  for (int64_t base = warp_global * 32; base < count; base += nwarps * 32) {
    const int64_t mine = base + L.lane;
    uint32_t slot = kNoSlot;
    int owner     = 0;
    if (mine < count) {
      const uint64_t key = static_cast<uint64_t>(ids[mine]);
      if (key == ~0ull) {
        atomicExch(io.error, 2);
      } else {
        owner = HashOwner(key, t.nranks);
        slot  = HashFind(t.keys[owner], t.cap, key, true);
        if (slot == kNoSlot - 1) {
          atomicExch(io.error, 1);
          slot = kNoSlot;
        }
      }
    }
    for (int j = 0; j < 32; j += L.ipw) {
      const int src      = j + L.sub;
      const uint32_t s   = __shfl_sync(kFullMask, slot, src);
      const int o        = __shfl_sync(kFullMask, owner, src);
      const int64_t item = base + src;
      if (item >= count) continue;
      OutT* dst = out + item * out_ld;
      for (int v = L.sublane; v < vecs; v += L.lpi) {
        U4 q{0, 0, 0, 0};
        if (s != kNoSlot) q = LdSys(t.rows[o] + static_cast<uint64_t>(s) * dim + v * 4);
        if (sizeof(OutT) == 4) {
          *reinterpret_cast<U4*>(dst + v * 4) = q;
        } else {
          OutT w[4] = {FromFloat<OutT>(__uint_as_float(q.x)), FromFloat<OutT>(__uint_as_float(q.y)),
                       FromFloat<OutT>(__uint_as_float(q.z)), FromFloat<OutT>(__uint_as_float(q.w))};
          *reinterpret_cast<uint2*>(dst + v * 4) = *reinterpret_cast<uint2*>(w);
        }
      }
    }
  }
}

template <typename GradT>
__global__ void __launch_bounds__(256)
HashPushKernel(HashTables t, HashIO io, int64_t count, int64_t grad_ld, float grad_scale, int rule, float lr, float eps) {
  const int dim  = t.dim;
  const int vecs = dim / 4;
  const RowLanes L(dim);
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps      = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t* ids        = io.ids[blockIdx.y];
  const GradT* grads        = static_cast<const GradT*>(io.grads[blockIdx.y]);
  for (int64_t base = warp_global * 32; base < count; base += nwarps * 32) {
    const int64_t mine = base + L.lane;
    uint32_t slot = kNoSlot;
    int owner     = 0;
    if (mine < count) {
      const uint64_t key = static_cast<uint64_t>(ids[mine]);
      owner = HashOwner(key, t.nranks);
      slot  = key == ~0ull ? kNoSlot : HashFind(t.keys[owner], t.cap, key, false);
      if (slot >= kNoSlot - 1) {
        slot = kNoSlot;
        atomicAdd(io.missing, 1ull);
      }
    }
    for (int j = 0; j < 32; j += L.ipw) {
      const int src      = j + L.sub;
      const uint32_t s   = __shfl_sync(kFullMask, slot, src);
      const int o        = __shfl_sync(kFullMask, owner, src);
      const int64_t item = base + src;
      if (item >= count || s == kNoSlot) continue;
      float* w       = t.rows[o] + static_cast<uint64_t>(s) * dim;
      float* st      = t.state[o] ? t.state[o] + static_cast<uint64_t>(s) * dim : nullptr;
      const GradT* g = grads + item * grad_ld;
      for (int v = L.sublane; v < vecs; v += L.lpi) {
        float d[4], gv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) gv[k] = ToFloat<GradT>(g[v * 4 + k]) * grad_scale;
        if (rule == 1 && st) {
          const U4 q = LdSys(st + v * 4);
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
  char* inbox[kMaxRanks];
  char* acc[kMaxRanks];        // per local rank (one entry unless the ranks are emulated on one GPU)
  uint32_t* ulist[kMaxRanks];
  PsCtl* ctl[kMaxRanks];
  uint32_t* item_slot[kMaxRanks];
  char* cache[kMaxRanks];
  int nlocal = 0;
  int nservers = 0;
  int server_rank[kMaxRanks];  // world rank of server j
  uint64_t slots = 0;
  uint64_t inbox_cap = 0;
  uint64_t item_cap = 0;       // items (sample, field) that item_slot can hold
  int32_t* error_dev = nullptr;
  bool lead_fence = true;      // the next push must fence first (no fenced pull since the previous push)
  bool wire_follows_grads = true;  // bf16 gradients: the rows cross NVLink as bf16
  int64_t index_items = -1;    // >= 0: the table holds the index of a pulled batch of that many items
  bool timing = false;
  cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int ev_used = 0;
  cudaEvent_t pull_ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  int pull_ev_used = 0;
};
PsState g_ps;

int MakePsLaunch(PsLaunch* l, const int64_t* const* ids, const void* const* grads, void* const* outs) {
  CommCtx ctx[kMaxRanks];
  int rank = 0, nranks = 1, emulated = 0;
  int rc = CommGetContexts(ctx, &rank, &nranks, &emulated);
  if (rc) return rc;
  memset(l, 0, sizeof(*l));
  const int local = emulated ? nranks : 1;
  if (local != g_ps.nlocal) return SetError(-2, "ps: configured for another number of local ranks");
  for (int i = 0; i < local; ++i) {
    PsRank& r = l->r[i];
    for (int p = 0; p < g_ps.nservers; ++p) {
      r.slab[p]  = g_ps.slab[p];
      r.inbox[p] = g_ps.inbox[p];
    }
    r.acc    = g_ps.acc[i];
    r.ulist  = g_ps.ulist[i];
    r.ctl    = g_ps.ctl[i];
    r.item_slot = g_ps.item_slot[i];
    r.cache  = g_ps.cache[i];
    r.ids    = ids ? ids[i] : nullptr;
    r.grads  = grads ? grads[i] : nullptr;
    r.out    = outs ? outs[i] : nullptr;
    r.error  = g_ps.error_dev;
    r.rank      = emulated ? i : rank;
    r.nranks    = nranks;
    r.nservers  = g_ps.nservers;
    r.my_server = -1;
    for (int j = 0; j < g_ps.nservers; ++j)
      if (g_ps.server_rank[j] == r.rank) r.my_server = j;
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

// Grid of the list walkers (fetch, send, reduce): one block per 256 list entries, at most 3 blocks per SM (what
// their register count lets an SM hold, so the grid is one wave and blocks loop over further chunks).
int ListGrid(int64_t max_entries) {
  int64_t blocks = (max_entries + 255) / 256;
  int64_t cap    = static_cast<int64_t>(NumSMs()) * 3;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

int LanesPerItem(int dim) {
  int l = 1;
  while (l < dim / 4 && l < 32) l <<= 1;
  return l;
}

void Mark(cudaStream_t s) {
  PsState& st = g_ps;
  if (st.timing && st.ev_used < 6) cudaEventRecord(st.ev[st.ev_used++], s);
}
void MarkPull(cudaStream_t s) {
  PsState& st = g_ps;
  if (st.timing && st.pull_ev_used < 5) cudaEventRecord(st.pull_ev[st.pull_ev_used++], s);
}

// Drops an index that no push consumed, so that the table is empty again.
int DropIndex(PsLaunch& l, int local, cudaStream_t s) {
  PsState& st = g_ps;
  if (st.index_items < 0) return 0;
  dim3 grid(PsGrid(st.index_items, 1), local);
  PsClearIndexKernel<<<grid, 256, 0, s>>>(l, st.slots);
  TIPSK_LAUNCH_CHECK();
  st.index_items = -1;
  return 0;
}

template <typename GradT>
int LaunchScatter(const PsLaunch& l, dim3 grid, cudaStream_t s, bool vec, bool indexed, int64_t batch,
                         int64_t grad_ld, int64_t grad_col0, float grad_scale) {
  PsState& st = g_ps;
  if (indexed) {
    if (vec)
      PsScatterKernel<GradT, true, true><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, st.slots, grad_scale);
    else
      PsScatterKernel<GradT, false, true><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, st.slots, grad_scale);
  } else {
    if (vec)
      PsScatterKernel<GradT, true, false><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, st.slots, grad_scale);
    else
      PsScatterKernel<GradT, false, false><<<grid, 256, 0, s>>>(l, st.meta, batch, grad_ld, grad_col0, st.slots, grad_scale);
  }
  TIPSK_LAUNCH_CHECK();
  return 0;
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

/* Placement rule of the tables as the kernels compute it (ps_placement.h), for host code and tests. */
int tipsk_ps_place(int field, int64_t id, int nranks, int32_t* owner, int64_t* local_row) {
  TIPSK_REQUIRE(nranks >= 1 && id >= 0, "ps place: bad arguments");
  int o;
  int64_t l;
  PsPlace(field, id, nranks, &o, &l);
  *owner     = o;
  *local_row = l;
  return 0;
}

/* Bytes of the per-rank buffers of the push path for a given geometry. */
uint64_t tipsk_ps_acc_bytes(uint64_t slots, int dim) { return slots * 8 + slots * static_cast<uint64_t>(dim) * 4; }
uint64_t tipsk_ps_inbox_bytes(int nranks, uint64_t inbox_cap, int dim) {
  return kInboxHeader + static_cast<uint64_t>(nranks) * inbox_cap * (8 + static_cast<uint64_t>(dim) * 4);
}
uint64_t tipsk_ps_ctl_bytes() { return sizeof(PsCtl); }

/* Registers the buffers of the data path and the per-field layout.
 *   servers          world ranks that hold shards, ascending (null: every rank); rows are placed among them, every
 *                    rank of the job may pull and push
 *   slabs, inboxes   one pointer per SERVER, in the order of `servers`, as mapped in this process (inboxes may be
 *                    null with one rank)
 *   accs, ulists, ctls, item_slots, caches   one pointer per LOCAL rank (one, or `nranks` when the ranks are
 *                    emulated on one GPU): accumulation table (tipsk_ps_acc_bytes), the two lists (2 * slots u32),
 *                    control words (tipsk_ps_ctl_bytes), slot per item (item_cap u32), row cache of the indexed
 *                    pull (slots * dim * 4 bytes); the first three must be zero before the first call; item_slots
 *                    and caches may be null (no indexed pull)
 *   slots            power of two; inbox_cap: rows one sender may send to one owner in a push, even
 *   shadow_base      byte offset inside every slab of a bf16 copy of the rows (fields in order, rows_per_shard * dim
 *                    bf16 each) that the apply pass keeps current and bf16 pulls read; 0: none. */
int tipsk_ps_configure(void* const* slabs, void* const* inboxes, void* const* accs, void* const* ulists,
                       void* const* ctls, void* const* item_slots, void* const* caches, int nranks, int nlocal,
                       const int32_t* servers, int nservers, const uint64_t* field_off, const uint64_t* state_off,
                       const int64_t* rows_per_shard, int nfields, int dim, uint64_t slots, uint64_t inbox_cap,
                       uint64_t item_cap, uint64_t shadow_base) {
  if (!servers) nservers = nranks;
  TIPSK_REQUIRE(nservers >= 1 && nservers <= nranks && nranks <= kMaxRanks, "ps: between one server and all ranks");
  for (int j = 0; servers && j < nservers; ++j)
    TIPSK_REQUIRE(servers[j] >= 0 && servers[j] < nranks && (j == 0 || servers[j] > servers[j - 1]),
                  "ps: server ranks must be ascending ranks of the job");
  TIPSK_REQUIRE(nfields >= 1 && nfields <= kMaxFields, "ps: 1..64 fields are supported");
  TIPSK_REQUIRE(dim >= 4 && dim % 4 == 0, "ps: the row dimension must be a multiple of 4");
  TIPSK_REQUIRE(slots >= 2 && (slots & (slots - 1)) == 0 && slots <= (1ull << 31), "ps: slots must be a power of two");
  TIPSK_REQUIRE(nranks >= 1 && nranks <= kMaxRanks, "ps: 1..8 ranks");
  TIPSK_REQUIRE(nlocal == 1 || nlocal == nranks, "ps: one local rank, or all of them (emulation)");
  TIPSK_REQUIRE(nranks == 1 || !accs || (inboxes && inbox_cap >= 2 && inbox_cap % 2 == 0),
                "ps: several ranks need inboxes with an even capacity");
  PsState& st = g_ps;
  memset(&st.meta, 0, sizeof(st.meta));
  for (int f = 0; f < nfields; ++f) {
    st.meta.field_off[f]      = field_off[f];
    st.meta.state_off[f]      = state_off ? state_off[f] : 0;
    st.meta.rows_per_shard[f] = rows_per_shard[f];
  }
  st.meta.nfields     = nfields;
  st.meta.dim         = dim;
  st.meta.shadow_base = shadow_base;
  st.nservers = nservers;
  for (int j = 0; j < kMaxRanks; ++j) st.server_rank[j] = j < nservers ? (servers ? servers[j] : j) : -1;
  for (int r = 0; r < kMaxRanks; ++r) {
    st.slab[r]      = r < nservers ? static_cast<char*>(slabs[r]) : nullptr;
    st.inbox[r]     = r < nservers && inboxes ? static_cast<char*>(inboxes[r]) : nullptr;
    st.acc[r]       = r < nlocal && accs ? static_cast<char*>(accs[r]) : nullptr;
    st.ulist[r]     = r < nlocal && ulists ? static_cast<uint32_t*>(ulists[r]) : nullptr;
    st.ctl[r]       = r < nlocal && ctls ? static_cast<PsCtl*>(ctls[r]) : nullptr;
    st.item_slot[r] = r < nlocal && item_slots ? static_cast<uint32_t*>(item_slots[r]) : nullptr;
    st.cache[r]     = r < nlocal && caches ? static_cast<char*>(caches[r]) : nullptr;
  }
  st.nlocal      = nlocal;
  st.slots       = slots;
  st.inbox_cap   = inbox_cap;
  st.item_cap    = item_cap;
  st.lead_fence  = true;
  st.index_items = -1;
  if (!st.error_dev) {
    TIPSK_CUDA(cudaMalloc(reinterpret_cast<void**>(&st.error_dev), sizeof(int32_t)));
    TIPSK_CUDA(cudaMemset(st.error_dev, 0, sizeof(int32_t)));
  }
  st.ready = true;
  return 0;
}

/* Reads and clears the PS error word (0 ok, 1 accumulation table full, 2 id out of range, 3 inbox full) and the
 * count of rows updated since the last call.  Synchronises the device. */
int tipsk_ps_status(int32_t* error, uint64_t* touched) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  TIPSK_CUDA(cudaMemcpy(error, st.error_dev, sizeof(int32_t), cudaMemcpyDeviceToHost));
  TIPSK_CUDA(cudaMemset(st.error_dev, 0, sizeof(int32_t)));
  uint64_t t = 0;
  for (int i = 0; i < st.nlocal; ++i) {
    if (!st.ctl[i]) continue;
    PsCtl c;
    TIPSK_CUDA(cudaMemcpy(&c, st.ctl[i], sizeof(c), cudaMemcpyDeviceToHost));
    t += c.applied;
    TIPSK_CUDA(cudaMemset(&st.ctl[i]->applied, 0, sizeof(unsigned long long)));
  }
  *touched = t;
  return 0;
}

/* Traffic counters since the last call: out[0] distinct rows of the pushed batches (after the local reduction of
 * duplicates; rows this rank owns itself included), out[1] those that crossed NVLink to their owner, out[2] rows
 * that indexed pulls read over NVLink.  Summed over the local ranks.  Synchronises the device. */
int tipsk_ps_traffic(uint64_t* out) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  out[0] = out[1] = out[2] = 0;
  for (int i = 0; i < st.nlocal; ++i) {
    if (!st.ctl[i]) continue;
    PsCtl c;
    TIPSK_CUDA(cudaMemcpy(&c, st.ctl[i], sizeof(c), cudaMemcpyDeviceToHost));
    out[0] += c.sent_total;
    out[1] += c.sent_remote;
    out[2] += c.fetched_remote;
    TIPSK_CUDA(cudaMemset(&st.ctl[i]->sent_total, 0, 2 * sizeof(unsigned long long)));
    TIPSK_CUDA(cudaMemset(&st.ctl[i]->fetched_remote, 0, sizeof(unsigned long long)));
  }
  return 0;
}

/* follow non-zero (the default): when the pushed gradients are bf16, each rank's per-row sum of its duplicates is
 * rounded to bf16 once and crosses NVLink in half the bytes; zero: rows always travel as fp32.  The same value on
 * every rank. */
int tipsk_ps_wire_follows_grads(int follow) {
  g_ps.wire_follows_grads = follow != 0;
  return 0;
}

/* Per-phase device timing of the next synchronous pushes (eager launches only, not under stream capture):
 * events are recorded around scatter / send / fence / reduce / apply.  tipsk_ps_phase_ms synchronises and
 * returns the five durations of the last push in milliseconds (0 for phases that did not run). */
int tipsk_ps_phase_timing(int enable) {
  PsState& st = g_ps;
  if (enable && !st.ev[0]) {
    for (auto& e : st.ev) TIPSK_CUDA(cudaEventCreate(&e));
    for (auto& e : st.pull_ev) TIPSK_CUDA(cudaEventCreate(&e));
  }
  st.timing       = enable != 0;
  st.ev_used      = 0;
  st.pull_ev_used = 0;
  return 0;
}
/* The durations of the last indexed pull: index, fence, fetch, expand (milliseconds). */
int tipsk_ps_pull_phase_ms(float* out4) {
  PsState& st = g_ps;
  for (int i = 0; i < 4; ++i) out4[i] = 0.f;
  if (!st.timing || st.pull_ev_used != 5) return 0;
  TIPSK_CUDA(cudaEventSynchronize(st.pull_ev[4]));
  for (int i = 0; i < 4; ++i) TIPSK_CUDA(cudaEventElapsedTime(&out4[i], st.pull_ev[i], st.pull_ev[i + 1]));
  return 0;
}
int tipsk_ps_phase_ms(float* out5) {
  PsState& st = g_ps;
  for (int i = 0; i < 5; ++i) out5[i] = 0.f;
  if (!st.timing || st.ev_used < 2) return 0;
  TIPSK_CUDA(cudaEventSynchronize(st.ev[st.ev_used - 1]));
  if (st.ev_used == 3) {  // one rank: scatter, apply
    TIPSK_CUDA(cudaEventElapsedTime(&out5[0], st.ev[0], st.ev[1]));
    TIPSK_CUDA(cudaEventElapsedTime(&out5[4], st.ev[1], st.ev[2]));
  } else if (st.ev_used == 6) {
    for (int i = 0; i < 5; ++i) TIPSK_CUDA(cudaEventElapsedTime(&out5[i], st.ev[i], st.ev[i + 1]));
  }
  return 0;
}

/* ids: [batch, nfields] int64 (one pointer per local rank); out: [batch, out_ld] of out_dtype (fp32/bf16),
 * field f lands at columns out_col0 + f*dim.  `fence` non-zero puts a cross-rank fence first, so that
 * rows updated by the previous push on any rank are visible.  `index` non-zero: the batch is first resolved into
 * its distinct rows, each of which is fetched once; the index stays in place for a following
 * tipsk_ps_push(..., reuse_index = 1) of the SAME ids (it is dropped by any other pull or push). */
int tipsk_ps_pull(const int64_t* const* ids, void* const* outs, int64_t batch, int64_t out_ld, int64_t out_col0,
                  int out_dtype, int fence, int index, void* stream) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  if (batch <= 0) return 0;
  TIPSK_REQUIRE(out_ld % 4 == 0 && out_col0 % 4 == 0, "ps pull: the output pitch and column offset must be multiples of 4");
  TIPSK_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "ps pull: output must be fp32 or bf16");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PsLaunch l;
  int local = MakePsLaunch(&l, ids, nullptr, outs);
  if (local < 0) return local;
  const int64_t items = batch * st.meta.nfields;
  const int lpi       = LanesPerItem(st.meta.dim);
  dim3 grid(PsGrid(items, lpi), local);
  if (index) {
    TIPSK_REQUIRE(st.acc[0] && st.ulist[0] && st.ctl[0] && st.item_slot[0] && st.cache[0],
                  "ps pull: the indexed pull needs the accumulation table, lists, item slots and row cache");
    TIPSK_REQUIRE(static_cast<uint64_t>(items) <= st.item_cap, "ps pull: the batch exceeds the configured item capacity");
    int rc = DropIndex(l, local, s);
    if (rc) return rc;
    st.pull_ev_used = 0;
    MarkPull(s);
    PsIndexKernel<<<dim3(PsGrid(items, 1), local), 256, 0, s>>>(l, st.meta, batch, st.slots);
    TIPSK_LAUNCH_CHECK();
    st.index_items = items;
    MarkPull(s);
  }
  if (fence) {
    int rc = tipsk_comm_fence(2, stream);
    if (rc) return rc;
    st.lead_fence = false;
  }
  if (!index) {
    if (out_dtype == kF32)
      PsPullKernel<float><<<grid, 256, 0, s>>>(l, st.meta, batch, out_ld, out_col0);
    else
      PsPullKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(l, st.meta, batch, out_ld, out_col0);
    TIPSK_LAUNCH_CHECK();
    return 0;
  }
  MarkPull(s);
  dim3 lgrid(ListGrid(items), local);
  if (out_dtype == kF32)
    PsFetchKernel<float><<<lgrid, 256, 0, s>>>(l, st.meta, st.slots);
  else
    PsFetchKernel<__nv_bfloat16><<<lgrid, 256, 0, s>>>(l, st.meta, st.slots);
  TIPSK_LAUNCH_CHECK();
  MarkPull(s);
  if (out_dtype == kF32)
    PsExpandKernel<float><<<grid, 256, 0, s>>>(l, st.meta, batch, out_ld, out_col0);
  else
    PsExpandKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(l, st.meta, batch, out_ld, out_col0);
  TIPSK_LAUNCH_CHECK();
  MarkPull(s);
  return 0;
}

/* grads: [batch, grad_ld] of grad_dtype, field f at columns grad_col0 + f*dim.  `reuse_index` non-zero: `ids` are
 * the ids of the last tipsk_ps_pull(..., index = 1), whose index gives every item's slot. */
int tipsk_ps_push(const int64_t* const* ids, const void* const* grads, int64_t batch, int64_t grad_ld,
                  int64_t grad_col0, int grad_dtype, float grad_scale, int rule, float lr, float eps, int reuse_index,
                  void* stream) {
  PsState& st = g_ps;
  TIPSK_REQUIRE(st.ready, "ps not configured");
  TIPSK_REQUIRE(st.acc[0] != nullptr && st.ulist[0] != nullptr && st.ctl[0] != nullptr,
                "ps push: no accumulation tables configured");
  TIPSK_REQUIRE(grad_dtype == kF32 || grad_dtype == kBF16, "ps push: gradients must be fp32 or bf16");
  if (batch <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PsLaunch l;
  int local = MakePsLaunch(&l, ids, grads, nullptr);
  if (local < 0) return local;
  const int nranks    = l.r[0].nranks;
  const int64_t items = batch * st.meta.nfields;
  TIPSK_REQUIRE(nranks == 1 || st.inbox[0] != nullptr, "ps push: no inboxes configured");
  TIPSK_REQUIRE(!reuse_index || st.index_items == items,
                "ps push: reuse_index needs the index of a pull of the same batch right before");
  if (!reuse_index) {
    int rc = DropIndex(l, local, s);
    if (rc) return rc;
  }
  if (nranks > 1 && st.lead_fence) {
    // every rank has finished reading its inbox and applying the previous push
    int rc = tipsk_comm_fence(2, stream);
    if (rc) return rc;
  }
  st.lead_fence  = true;
  st.index_items = -1;  // the push consumes the index: send and apply empty the table
  st.ev_used     = 0;
  const int lpi  = LanesPerItem(st.meta.dim);
  dim3 grid(PsGrid(items, lpi), local);
  bool vec = grad_ld % 4 == 0 && grad_col0 % 4 == 0;
  for (int i = 0; i < local; ++i) vec = vec && (reinterpret_cast<uintptr_t>(grads[i]) % 16 == 0);
  Mark(s);
  int rc = grad_dtype == kF32
               ? LaunchScatter<float>(l, grid, s, vec, reuse_index != 0, batch, grad_ld, grad_col0, grad_scale)
               : LaunchScatter<__nv_bfloat16>(l, grid, s, vec, reuse_index != 0, batch, grad_ld, grad_col0, grad_scale);
  if (rc) return rc;
  Mark(s);
  if (nranks > 1) {
    dim3 lgrid(ListGrid(items), local);
    const int wire_bf16 = st.wire_follows_grads && grad_dtype == kBF16 ? 1 : 0;
    PsSendKernel<<<lgrid, 256, 0, s>>>(l, st.meta, st.slots, st.inbox_cap, wire_bf16);
    TIPSK_LAUNCH_CHECK();
    Mark(s);
    rc = tipsk_comm_fence(2, stream);  // every rank's rows and counts have landed
    if (rc) return rc;
    Mark(s);
    PsOwnerReduceKernel<<<lgrid, 256, 0, s>>>(l, st.meta, st.slots, st.inbox_cap, wire_bf16);
    TIPSK_LAUNCH_CHECK();
    Mark(s);
  }
  PsPushApplyKernel<<<grid, 256, 0, s>>>(l, st.meta, st.slots, rule, lr, eps);
  TIPSK_LAUNCH_CHECK();
  Mark(s);
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

/* ---- tables keyed by arbitrary 64-bit ids (rows created on first pull) ----
 * keys / rows / states: one pointer per rank as mapped here ([cap] u64, [cap][dim] fp32, [cap][dim] fp32 or null);
 * all zero at creation.  ids / outs / grads: one pointer per LOCAL rank (nlocal = 1, or nranks when emulated).
 * error: device int32 (1 table full, 2 key 2^64-1), missing: device u64 counter of pushed rows never pulled. */
int tipsk_hash_pull(void* const* keys, void* const* rows, int nranks, uint64_t cap, int dim, const int64_t* const* ids,
                    void* const* outs, int nlocal, int64_t count, int64_t out_ld, int out_dtype, int32_t* error,
                    void* stream) {
  TIPSK_REQUIRE(nranks >= 1 && nranks <= kMaxRanks && (nlocal == 1 || nlocal == nranks), "hash pull: bad rank counts");
  TIPSK_REQUIRE(cap >= 2 && (cap & (cap - 1)) == 0 && cap <= (1ull << 31), "hash pull: cap must be a power of two");
  TIPSK_REQUIRE(dim >= 4 && dim % 4 == 0 && out_ld % 4 == 0, "hash pull: dim and the output pitch must be multiples of 4");
  TIPSK_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "hash pull: output must be fp32 or bf16");
  if (count <= 0) return 0;
  HashTables t;
  HashIO io;
  memset(&t, 0, sizeof(t));
  memset(&io, 0, sizeof(io));
  for (int r = 0; r < nranks; ++r) {
    t.keys[r] = static_cast<unsigned long long*>(keys[r]);
    t.rows[r] = static_cast<float*>(rows[r]);
  }
  t.cap = cap; t.dim = dim; t.nranks = nranks;
  for (int i = 0; i < nlocal; ++i) {
    io.ids[i] = ids[i];
    io.out[i] = outs[i];
  }
  io.error = error;
  dim3 grid(PsGrid(count, LanesPerItem(dim)), nlocal);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == kF32)
    HashPullKernel<float><<<grid, 256, 0, s>>>(t, io, count, out_ld);
  else
    HashPullKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(t, io, count, out_ld);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_hash_push(void* const* keys, void* const* rows, void* const* states, int nranks, uint64_t cap, int dim,
                    const int64_t* const* ids, const void* const* grads, int nlocal, int64_t count, int64_t grad_ld,
                    int grad_dtype, float grad_scale, int rule, float lr, float eps, int32_t* error,
                    unsigned long long* missing, void* stream) {
  TIPSK_REQUIRE(nranks >= 1 && nranks <= kMaxRanks && (nlocal == 1 || nlocal == nranks), "hash push: bad rank counts");
  TIPSK_REQUIRE(cap >= 2 && (cap & (cap - 1)) == 0 && cap <= (1ull << 31), "hash push: cap must be a power of two");
  TIPSK_REQUIRE(dim >= 4 && dim % 4 == 0, "hash push: dim must be a multiple of 4");
  TIPSK_REQUIRE(grad_dtype == kF32 || grad_dtype == kBF16, "hash push: gradients must be fp32 or bf16");
  TIPSK_REQUIRE(rule == 0 || (rule == 1 && states), "hash push: SGD, or Adagrad with accumulators");
  if (count <= 0) return 0;
  HashTables t;
  HashIO io;
  memset(&t, 0, sizeof(t));
  memset(&io, 0, sizeof(io));
  for (int r = 0; r < nranks; ++r) {
    t.keys[r]  = static_cast<unsigned long long*>(keys[r]);
    t.rows[r]  = static_cast<float*>(rows[r]);
    t.state[r] = states ? static_cast<float*>(states[r]) : nullptr;
  }
  t.cap = cap; t.dim = dim; t.nranks = nranks;
  for (int i = 0; i < nlocal; ++i) {
    io.ids[i]   = ids[i];
    io.grads[i] = grads[i];
  }
  io.error   = error;
  io.missing = missing;
  dim3 grid(PsGrid(count, LanesPerItem(dim)), nlocal);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (grad_dtype == kF32)
    HashPushKernel<float><<<grid, 256, 0, s>>>(t, io, count, grad_ld, grad_scale, rule, lr, eps);
  else
    HashPushKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(t, io, count, grad_ld, grad_scale, rule, lr, eps);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
