// Device executor: the function the collective engine calls, on its background
// thread, to run one negotiated collective on the GPU.  It orders the collective
// after the producer (cudaStreamWaitEvent on the op's ready event), launches the
// fused kernel on the communication stream of the op's channel and records the
// done event that consumers wait on.  Tensors that already live inside the
// symmetric window are reduced in place; others go through the staging area.
#include <cstdio>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

#include "device_op.h"
#include "kernels/comm.cuh"
#include "kernels/common.cuh"
#include "kernels/tips_kernels.h"

namespace {
// NVTX range around the launch of one collective on the engine thread ("tips.allreduce 51380224 B ch1"); it costs
// a function-pointer check when no profiler is attached.
struct LaunchRange {
  LaunchRange(const tips_device_op* op, size_t es) {
    static const char* kNames[3] = {"tips.allreduce", "tips.allgather", "tips.broadcast"};
    char label[96];
    snprintf(label, sizeof(label), "%s %lld B ch%d", op->type >= 0 && op->type < 3 ? kNames[op->type] : "tips.op",
             static_cast<long long>(op->count) * static_cast<long long>(es), op->channel & 1);
    nvtxRangePushA(label);
  }
  ~LaunchRange() { nvtxRangePop(); }
};

int g_device = -1;
char* g_window = nullptr;
uint64_t g_window_bytes = 0;
}  // namespace

extern "C" {

int tipsk_executor_configure(int device, void* my_window, uint64_t window_bytes) {
  g_device       = device;
  g_window       = static_cast<char*>(my_window);
  g_window_bytes = window_bytes;
  return 0;
}

int tipsk_device_execute(const tips_device_op* op, char* err, int err_len) {
  auto fail = [&](int rc) {
    snprintf(err, err_len, "%s", tipsk_last_error());
    return rc ? rc : -7;
  };
  if (g_device >= 0 && cudaSetDevice(g_device) != cudaSuccess) {
    snprintf(err, err_len, "cudaSetDevice(%d) failed", g_device);
    return -7;
  }
  const int ch        = op->channel & 1;
  void* stream        = tipsk_comm_stream(ch);
  const size_t es     = tipsk::DTypeSize(op->dtype);
  if (es == 0) {
    snprintf(err, err_len, "unsupported dtype %d", op->dtype);
    return -2;
  }
  LaunchRange range(op, es);
  if (op->ready_event && tipsk_stream_wait_event(stream, op->ready_event) != 0) return fail(-7);
  int rc = 0;
  if (op->type == 0) {
    const uint64_t nbytes = static_cast<uint64_t>(op->count) * es;
    const char* in        = static_cast<const char*>(op->in);
    const bool in_window  = g_window && in >= g_window + tipsk::kSignalBytes && in + nbytes <= g_window + g_window_bytes &&
                           ((in - g_window) % 16) == 0;
    if (in_window && op->in == op->out && op->reduce_op == 0 && tipsk_comm_update_attached(in - g_window, nbytes)) {
      // this bucket carries an optimizer update: reduce, update the owned share, store the new parameters
      rc = tipsk_allreduce_update(in - g_window, static_cast<float>(op->prescale * op->postscale), ch, stream);
    } else if (in_window && op->in == op->out) {
      rc = tipsk_allreduce(nullptr, nullptr, in - g_window, nbytes, op->dtype, op->reduce_op,
                           static_cast<float>(op->prescale), static_cast<float>(op->postscale), ch, stream);
    } else if (in_window) {
      void* dst[1] = {op->out};
      rc = tipsk_allreduce(nullptr, dst, in - g_window, nbytes, op->dtype, op->reduce_op,
                           static_cast<float>(op->prescale), static_cast<float>(op->postscale), ch, stream);
    } else {
      const void* src[1] = {op->in};
      void* dst[1]       = {op->out};
      rc = tipsk_allreduce(src, dst, -1, nbytes, op->dtype, op->reduce_op, static_cast<float>(op->prescale),
                           static_cast<float>(op->postscale), ch, stream);
    }
  } else if (op->type == 1) {
    uint64_t bytes[tipsk::kMaxRanks] = {0};
    if (!op->counts || op->nranks > tipsk::kMaxRanks) {
      snprintf(err, err_len, "allgather without per-rank counts");
      return -2;
    }
    for (int r = 0; r < op->nranks; ++r) bytes[r] = static_cast<uint64_t>(op->counts[r]) * es;
    const void* src[1] = {op->in};
    void* dst[1]       = {op->out};
    rc = tipsk_allgatherv(src, dst, bytes, ch, stream);
  } else if (op->type == 2) {
    const void* src[1] = {op->in};
    void* dst[1]       = {op->out};
    rc = tipsk_broadcast(src, dst, static_cast<uint64_t>(op->count) * es, op->root_rank, ch, stream);
  } else {
    snprintf(err, err_len, "unknown collective type %d", op->type);
    return -2;
  }
  if (rc != 0) return fail(rc);
  if (op->done_event && tipsk_event_record(op->done_event, stream) != 0) return fail(-7);
  return 0;
}

void* tipsk_device_executor_ptr(void) { return reinterpret_cast<void*>(&tipsk_device_execute); }

}  // extern "C"
