// CPU collectives over the runtime's TCP data mesh.
//
// Capability parity with the reference's MPI wrappers
// (tips/core/collective/utils.h:21-134, utils.cc:6-16): AllreduceCpu with
// SUM/MAX/MIN (plus PROD), AllgatherCpu (equal sizes), AllgathervCpu (per-rank
// first-dimension sizes, validated), BroadcastCpu (any root).  They serve CPU
// tensors and CPU-only jobs; device tensors use the CUDA kernels instead and
// never pass through here.
//
// Algorithms: allreduce = direct reduce-scatter (every rank owns 1/N of the
// elements, receives the N-1 foreign copies of its slice and reduces them)
// followed by a direct allgather; allgatherv = N-1 pairwise exchanges;
// broadcast = root sends to every rank.  Each step is a simultaneous
// send+receive driven by poll(), so no ordering of blocking calls can deadlock.
// 16-bit floats are reduced in fp32.
#pragma once

#include <cstdint>
#include <vector>

#include "core/common.h"
#include "core/datatype.h"

namespace tips {
namespace collective {

enum class ReduceOp : int32_t { kSum = 0, kMax = 1, kMin = 2, kProd = 3 };

// out may alias in. `count` elements of `dtype`.
Status AllreduceCpu(const void* in, void* out, int64_t count, Datatype dtype, ReduceOp op);

// Every rank contributes `count` elements; out holds size*count elements.
Status AllgatherCpu(const void* in, void* out, int64_t count, Datatype dtype);

// Rank r contributes first_dims[r] * trailing elements; out holds the
// concatenation in rank order.
Status AllgathervCpu(const void* in, void* out, const std::vector<int64_t>& first_dims, int64_t trailing,
                     Datatype dtype);

// In place on `data` (count elements); root's contents win.
Status BroadcastCpu(void* data, int64_t count, Datatype dtype, int root);

// Elementwise reduction of `src` into `dst` on the host; exposed for tests.
void ReduceInto(void* dst, const void* src, int64_t count, Datatype dtype, ReduceOp op);

}  // namespace collective
}  // namespace tips
