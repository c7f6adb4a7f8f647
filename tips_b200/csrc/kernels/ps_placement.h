// Placement of parameter-server rows on ranks: one rule, shared by the device
// kernels (pull, push, table initialisation) and mirrored by the host-side dump /
// load code, so that a row is found where it was stored.
//
// Row `id` of field `f` belongs to the group of n consecutive ids
// [lrow*n, lrow*n + n) with lrow = id div n; the group is dealt to the n ranks
// rotated by (f + hash(lrow)) mod n, and every rank stores its member of the
// group at local row `lrow`.  The rule is a bijection between ids and
// (owner, local row) pairs and needs no lookup table.  Without the rotation
// (owner = id mod n) the smallest ids of every field, which are the most
// frequent ones under a Zipf distribution, would all live on rank 0.
//
// The reference's two placement rules disagree with each other
// (tips/core/ps/route.h:104-134 against ps_server.h:202-210); this is the single
// rule used everywhere here.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define TIPS_HD __host__ __device__ __forceinline__
#else
#define TIPS_HD inline
#endif

namespace tipsk {

TIPS_HD uint32_t PsRotation(int field, int64_t lrow, int n) {
  const uint32_t h = static_cast<uint32_t>(static_cast<uint64_t>(lrow)) * 0x9E3779B1u;
  return ((h >> 16) + static_cast<uint32_t>(field)) % static_cast<uint32_t>(n);
}

// id -> (owner rank, local row)
TIPS_HD void PsPlace(int field, int64_t id, int n, int* owner, int64_t* lrow) {
  const int64_t l = id / n;
  const uint32_t j = static_cast<uint32_t>(id - l * n);
  *owner = static_cast<int>((j + PsRotation(field, l, n)) % static_cast<uint32_t>(n));
  *lrow  = l;
}

// (owner rank, local row) -> id
TIPS_HD int64_t PsGlobalId(int field, int64_t lrow, int owner, int n) {
  const uint32_t rot = PsRotation(field, lrow, n);
  const uint32_t j   = (static_cast<uint32_t>(owner) + static_cast<uint32_t>(n) - rot) % static_cast<uint32_t>(n);
  return lrow * n + j;
}

}  // namespace tipsk
