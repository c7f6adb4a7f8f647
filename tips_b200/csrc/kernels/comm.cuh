// Device-side building blocks of the NVLink collectives: the per-rank
// communication context, cross-rank block barriers on epoch flags with bounded
// waits, system-scope vector loads/stores on peer memory and NVLS multimem
// instructions.
//
// Memory model: data written before a barrier is published with
// __threadfence_system() + st.release.sys on the flag; the waiter polls the flag
// with ld.acquire.sys, so peer data read after the barrier is the data written
// before it.  Peer data is always accessed with .relaxed.sys loads/stores, never
// through a TMA or any cluster-multicast copy.
//
// Every wait is bounded: when the time budget runs out the waiting thread
// records {code, peer, phase, block, epoch} in a status block that the host can
// read, and the kernel carries on to its end without further waiting, so a lost
// peer costs one budget, not a hung GPU.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tipsk {

constexpr int kMaxRanks       = 8;
constexpr int kMaxCommBlocks  = 128;
constexpr int kNumChannels    = 4;  // 0 negotiated collectives, 1 frozen schedule, 2 parameter server, 3 spare
// Flag area at the start of every rank's window: [channel][block][src rank] u32.
constexpr size_t kFlagBytes   = sizeof(uint32_t) * kNumChannels * kMaxCommBlocks * kMaxRanks;
constexpr size_t kSignalBytes = 64 * 1024;  // flag area rounded up; the staging area starts here

enum CommStatusCode : int32_t { kCommOk = 0, kCommTimeout = 5 };

struct CommStatus {
  int32_t code;
  int32_t peer;
  int32_t phase;
  int32_t block;
  uint32_t epoch;
  int32_t channel;
  int32_t rank;
  int32_t pad;
};

struct CommCtx {
  char* peer[kMaxRanks];   // base of every rank's window as mapped in this process
  char* mc;                // multicast mapping of the window, or null
  uint32_t* epochs;        // local: [channel][block] last used epoch
  CommStatus* status;      // host-visible status block (mapped host memory: written on failure only)
  int32_t* failed;         // device-side copy of "a wait has timed out", polled by the barriers
  uint64_t budget_ns;
  int32_t rank;
  int32_t nranks;
  // Byte offset of this context's flag area inside every member's window: 0 = the area at the start of the
  // window (the collectives of all ranks); a sub-group of ranks has an area of its own further up, so that its
  // barriers and epochs are independent of everyone else's.
  uint64_t flag_off;
};

__device__ __forceinline__ uint64_t GlobalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void StReleaseSys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t LdAcquireSys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

struct alignas(16) U4 {
  uint32_t x, y, z, w;
};

__device__ __forceinline__ U4 LdSys(const void* addr) {
  U4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void StSys(void* addr, const U4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// NVLS: one load that returns the sum over every rank's copy / one store that
// lands in every rank's copy.  `addr` is an address inside the multicast mapping.
__device__ __forceinline__ U4 MultimemLdReduceF32(const void* addr) {
  U4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ U4 MultimemLdReduceBf16(const void* addr) {
  U4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ U4 MultimemLdReduceF16(const void* addr) {
  U4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void MultimemSt(void* addr, const U4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ uint32_t* FlagAddr(char* window, int channel, int block, int src_rank) {
  return reinterpret_cast<uint32_t*>(window) + (channel * kMaxCommBlocks + block) * kMaxRanks + src_rank;
}

__device__ __forceinline__ void ReportTimeout(const CommCtx& ctx, int peer, int phase, int block, uint32_t epoch,
                                              int channel) {
  if (atomicExch(ctx.failed, 1) == 0) {
    ctx.status->code    = kCommTimeout;
    ctx.status->peer    = peer;
    ctx.status->phase   = phase;
    ctx.status->block   = block;
    ctx.status->epoch   = epoch;
    ctx.status->channel = channel;
    ctx.status->rank    = ctx.rank;
    __threadfence_system();
  }
}

// Barrier between block `block` of this rank and the same block of every other
// rank.  All threads of the block call it.  Returns false if the wait ran out
// of budget (or an earlier wait of this kernel already had).
__device__ __forceinline__ bool BlockBarrier(const CommCtx& ctx, int channel, int block, uint32_t epoch, int phase) {
  __threadfence_system();
  __syncthreads();
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < ctx.nranks) {
    const int peer = threadIdx.x;
    StReleaseSys(FlagAddr(ctx.peer[peer] + ctx.flag_off, channel, block, ctx.rank), epoch);
    const uint32_t* mine = FlagAddr(ctx.peer[ctx.rank] + ctx.flag_off, channel, block, peer);
    // device memory, not the host-visible block: a PCIe read per barrier would serialise the blocks
    const bool already_failed = *reinterpret_cast<volatile int32_t*>(ctx.failed) != 0;
    if (already_failed) {
      s_ok = 0;
    } else {
      const uint64_t t0 = GlobalTimerNs();
      uint32_t spins    = 0;
      while (static_cast<int32_t>(LdAcquireSys(mine) - epoch) < 0) {
        if ((++spins & 0x3f) == 0) {
          if (GlobalTimerNs() - t0 > ctx.budget_ns) {
            ReportTimeout(ctx, peer, phase, block, epoch, channel);
            s_ok = 0;
            break;
          }
          __nanosleep(64);
        }
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

}  // namespace tipsk
