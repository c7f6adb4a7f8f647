#include "collective/cpu_collectives.h"

#include <algorithm>
#include <cstring>

#include "runtime/context.h"
#include "runtime/net.h"

namespace tips {
namespace collective {

namespace {

template <typename T>
void ReduceTyped(T* dst, const T* src, int64_t n, ReduceOp op) {
  switch (op) {
    case ReduceOp::kSum:
      for (int64_t i = 0; i < n; ++i) dst[i] += src[i];
      break;
    case ReduceOp::kMax:
      for (int64_t i = 0; i < n; ++i) dst[i] = std::max(dst[i], src[i]);
      break;
    case ReduceOp::kMin:
      for (int64_t i = 0; i < n; ++i) dst[i] = std::min(dst[i], src[i]);
      break;
    case ReduceOp::kProd:
      for (int64_t i = 0; i < n; ++i) dst[i] *= src[i];
      break;
  }
}

template <typename ToF, typename FromF>
void Reduce16(uint16_t* dst, const uint16_t* src, int64_t n, ReduceOp op, ToF to_f, FromF from_f) {
  for (int64_t i = 0; i < n; ++i) {
    float a = to_f(dst[i]), b = to_f(src[i]), r = 0.f;
    switch (op) {
      case ReduceOp::kSum: r = a + b; break;
      case ReduceOp::kMax: r = std::max(a, b); break;
      case ReduceOp::kMin: r = std::min(a, b); break;
      case ReduceOp::kProd: r = a * b; break;
    }
    dst[i] = from_f(r);
  }
}

bool Xchg(Context& ctx, int dst, const void* sbuf, size_t sn, int src, void* rbuf, size_t rn) {
  return net::Exchange(ctx.data_fd(dst), sbuf, sn, ctx.data_fd(src), rbuf, rn, ctx.data_timeout_ms());
}

Status TransportError(const char* what) {
  return Status(kUnavailable, std::string(what) + ": peer connection failed or timed out");
}

}  // namespace

void ReduceInto(void* dst, const void* src, int64_t n, Datatype dtype, ReduceOp op) {
  switch (dtype) {
    case Datatype::kFp32: ReduceTyped(static_cast<float*>(dst), static_cast<const float*>(src), n, op); break;
    case Datatype::kFp64: ReduceTyped(static_cast<double*>(dst), static_cast<const double*>(src), n, op); break;
    case Datatype::kInt32: ReduceTyped(static_cast<int32_t*>(dst), static_cast<const int32_t*>(src), n, op); break;
    case Datatype::kInt64: ReduceTyped(static_cast<int64_t*>(dst), static_cast<const int64_t*>(src), n, op); break;
    case Datatype::kInt8: ReduceTyped(static_cast<int8_t*>(dst), static_cast<const int8_t*>(src), n, op); break;
    case Datatype::kUInt8: ReduceTyped(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), n, op); break;
    case Datatype::kBf16:
      Reduce16(static_cast<uint16_t*>(dst), static_cast<const uint16_t*>(src), n, op, Bf16ToFloat, FloatToBf16);
      break;
    case Datatype::kFp16:
      Reduce16(static_cast<uint16_t*>(dst), static_cast<const uint16_t*>(src), n, op, Fp16ToFloat, FloatToFp16);
      break;
    default: TIPS_LOG(FATAL) << "ReduceInto: unsupported dtype";
  }
}

Status AllreduceCpu(const void* in, void* out, int64_t count, Datatype dtype, ReduceOp op) {
  Context& ctx   = Context::Global();
  const int n    = ctx.size();
  const int rank = ctx.rank();
  const size_t es = DatatypeNumBytes(dtype);
  if (out != in) memcpy(out, in, count * es);
  if (n == 1 || count == 0) return Status::OK();
  std::lock_guard<std::mutex> lock(ctx.data_mu());
  auto off = [&](int j) { return count * j / n; };
  char* o  = static_cast<char*>(out);
  const int64_t my_n = off(rank + 1) - off(rank);
  std::vector<char> tmp(std::max<int64_t>(my_n, 1) * es);
  // reduce-scatter: out[slice rank] accumulates every peer's copy of it.
  // Slices of other ranks in `out` still hold this rank's original values.
  for (int s = 1; s < n; ++s) {
    int dst = (rank + s) % n, src = (rank - s + n) % n;
    if (!Xchg(ctx, dst, o + off(dst) * es, (off(dst + 1) - off(dst)) * es, src, tmp.data(), my_n * es))
      return TransportError("allreduce");
    ReduceInto(o + off(rank) * es, tmp.data(), my_n, dtype, op);
  }
  // allgather of the reduced slices
  for (int s = 1; s < n; ++s) {
    int dst = (rank + s) % n, src = (rank - s + n) % n;
    if (!Xchg(ctx, dst, o + off(rank) * es, my_n * es, src, o + off(src) * es, (off(src + 1) - off(src)) * es))
      return TransportError("allreduce");
  }
  return Status::OK();
}

Status AllgathervCpu(const void* in, void* out, const std::vector<int64_t>& first_dims, int64_t trailing,
                     Datatype dtype) {
  Context& ctx   = Context::Global();
  const int n    = ctx.size();
  const int rank = ctx.rank();
  if (static_cast<int>(first_dims.size()) != n)
    return Status(kInvalidArgument, "allgatherv: need one first-dimension size per rank");
  if (trailing < 0) return Status(kInvalidArgument, "allgatherv: negative trailing size");
  const size_t es = DatatypeNumBytes(dtype);
  std::vector<int64_t> displ(n + 1, 0);
  for (int r = 0; r < n; ++r) {
    if (first_dims[r] < 0) return Status(kInvalidArgument, "allgatherv: negative first dimension");
    displ[r + 1] = displ[r] + first_dims[r] * trailing;
  }
  char* o = static_cast<char*>(out);
  memcpy(o + displ[rank] * es, in, (displ[rank + 1] - displ[rank]) * es);
  if (n == 1) return Status::OK();
  std::lock_guard<std::mutex> lock(ctx.data_mu());
  for (int s = 1; s < n; ++s) {
    int dst = (rank + s) % n, src = (rank - s + n) % n;
    if (!Xchg(ctx, dst, o + displ[rank] * es, (displ[rank + 1] - displ[rank]) * es, src, o + displ[src] * es,
              (displ[src + 1] - displ[src]) * es))
      return TransportError("allgatherv");
  }
  return Status::OK();
}

Status AllgatherCpu(const void* in, void* out, int64_t count, Datatype dtype) {
  std::vector<int64_t> dims(Context::Global().size(), count);
  return AllgathervCpu(in, out, dims, 1, dtype);
}

Status BroadcastCpu(void* data, int64_t count, Datatype dtype, int root) {
  Context& ctx = Context::Global();
  const int n  = ctx.size();
  if (root < 0 || root >= n) return Status(kInvalidArgument, "broadcast: bad root rank");
  if (n == 1 || count == 0) return Status::OK();
  const size_t bytes = count * DatatypeNumBytes(dtype);
  std::lock_guard<std::mutex> lock(ctx.data_mu());
  if (ctx.rank() == root) {
    for (int r = 0; r < n; ++r) {
      if (r == root) continue;
      if (!net::SendAll(ctx.data_fd(r), data, bytes)) return TransportError("broadcast");
    }
  } else {
    if (!net::Exchange(ctx.data_fd(root), nullptr, 0, ctx.data_fd(root), data, bytes, ctx.data_timeout_ms()))
      return TransportError("broadcast");
  }
  return Status::OK();
}

}  // namespace collective
}  // namespace tips
