// The collective engine: a background thread per rank plus a coordinator on
// rank 0 that decides one global execution order for all collectives.
//
// Capability parity with the reference (tips/core/collective/coordinator.h:33-139,
// coordinator.cc:15-589): EnqueueTensorCollective puts an op record in the
// tensor table and a request on the message queue; workers forward requests to
// rank 0; rank 0 counts requests per tensor name (IncreTensorCount), and when
// every rank has asked builds a response after cross-rank validation
// (ConstructResponseMessage: same dtype, same op, same shape; allgather: same
// rank and trailing dims, first dims collected), answers every worker and runs
// the op itself (PerformCollectiveOp).  All ranks therefore execute collectives
// in the order chosen by rank 0, whatever their local enqueue order.
//
// What this engine does differently, on purpose:
//  * Framework-neutral: an OpRecord carries raw pointers, dtype, shape, device
//    kind and stream/event handles, not a framework tensor (the reference stores
//    tensorflow::Tensor* and OpKernelContext*, coordinator.h:33-59).
//  * Errors reach the caller's handle on every rank instead of aborting the
//    process (reference: LOG(FATAL) on the worker, coordinator.cc:406-411); a
//    duplicate in-flight name is rejected (reference: silently dropped, :233-236).
//  * The broadcast root, the reduce operator and the scale factors are part of
//    the request and validated (reference: root fixed to 0, :280-291).
//  * Tensor fusion: allreduce responses that become ready in the same cycle and
//    agree on dtype/op/scales/device are merged into one response up to
//    fusion_threshold bytes; host tensors are packed into a fusion buffer and
//    reduced with ONE collective.
//  * Frozen schedule: once a step's bucket sequence has been negotiated it can
//    be frozen; from then on those names execute in the frozen order as soon as
//    they are locally ready, with zero control messages per step.
//  * Stall detector on rank 0, peer-failure propagation, a timeline tracer and
//    counters.
#pragma once

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "collective/cpu_collectives.h"
#include "collective/messages.h"
#include "core/channel.h"
#include "device_op.h"
#include "runtime/rpc.h"

namespace tips {
namespace collective {

// Allocates the output of an allgather once the per-rank first dimensions are
// known.  Returns the address of a buffer of `nbytes` bytes (host or device,
// matching the input), or nullptr on failure.
using AllocOutputFn = void* (*)(int64_t handle, int64_t nbytes, const int64_t* first_dims, int32_t n, void* user);

using DeviceOp = tips_device_op;
using DeviceExecutorFn = tips_device_executor_fn;

struct OpRecord {
  std::string name;
  RequestType type{RequestType::kAllreduce};
  Datatype dtype{Datatype::kFp32};
  std::vector<int64_t> shape;
  const void* in{nullptr};
  void* out{nullptr};  // allgather: filled by `alloc` when null
  int32_t device{0};
  int32_t root_rank{0};
  ReduceOp reduce_op{ReduceOp::kSum};
  double prescale{1.0};
  double postscale{1.0};
  void* stream{nullptr};
  void* ready_event{nullptr};
  void* done_event{nullptr};
  AllocOutputFn alloc{nullptr};
  void* alloc_user{nullptr};
  int64_t handle{0};
  int64_t enqueue_us{0};
};

// State of one asynchronous collective as seen by the caller.
struct HandleState {
  std::atomic<int> code{kInProgress};
  std::string error;
  std::vector<int64_t> sizes;  // allgather: per-rank first dims
  void* out{nullptr};
};

struct EngineOptions {
  int64_t fusion_threshold_bytes{64ll << 20};
  int cycle_time_ms{0};
  int stall_warn_ms{60000};
  int stall_abort_ms{0};  // 0 = never abort on a stall
};

struct EngineCounters {
  std::atomic<uint64_t> ops_enqueued{0};
  std::atomic<uint64_t> ops_completed{0};
  std::atomic<uint64_t> ops_failed{0};
  std::atomic<uint64_t> allreduce_bytes{0};
  std::atomic<uint64_t> allgather_bytes{0};
  std::atomic<uint64_t> broadcast_bytes{0};
  std::atomic<uint64_t> negotiation_requests{0};
  std::atomic<uint64_t> responses{0};
  std::atomic<uint64_t> fused_groups{0};
  std::atomic<uint64_t> fused_tensors{0};
  std::atomic<uint64_t> frozen_executions{0};
  std::atomic<uint64_t> stall_warnings{0};
};

struct TimelineEvent {
  std::string name;
  const char* phase;  // "NEGOTIATE", "EXECUTE"
  int64_t begin_us;
  int64_t end_us;
};

// Rank-0 bookkeeping: requests received so far for each tensor name.
struct PendingTensor {
  std::vector<RequestMessage> requests;     // indexed by arrival
  std::vector<RpcMsgHead> heads;            // where to answer (remote ranks only)
  std::vector<bool> seen;                   // by rank
  int64_t first_us{0};
  bool warned{false};
};
using MessageTable = std::unordered_map<std::string, PendingTensor>;

// Adds `msg` to the table; true when every rank has now asked for that name.
bool IncreTensorCount(MessageTable* table, const RequestMessage& msg, const RpcMsgHead* head, int world_size);

// Validates the requests collected for `name` and builds the response
// (type ERROR with a message when the ranks disagree).  Consumes the entry.
ResponseMessage ConstructResponseMessage(MessageTable* table, const std::string& name, int world_size);

class CollectiveEngine {
 public:
  static CollectiveEngine& Global();

  void Initialize(const EngineOptions& opts);
  bool initialized() const { return initialized_.load(); }
  // Fails everything still in flight with kAborted and joins the thread.
  void Finalize();

  // Returns a handle (> 0), or a negative StatusCode when the op is rejected
  // synchronously (engine down, duplicate in-flight name).
  int64_t Enqueue(OpRecord record, std::string* error = nullptr);

  // kInProgress until the op completed; then kOk or the error code.
  int Poll(int64_t handle);
  // Blocks up to timeout_ms (-1 = forever); returns the final code or kTimeout.
  int Wait(int64_t handle, int timeout_ms);
  std::shared_ptr<HandleState> Lookup(int64_t handle);
  void Release(int64_t handle);

  void SetDeviceExecutor(DeviceExecutorFn fn) { device_executor_ = fn; }

  // Frozen schedule.  `names` is the per-step sequence, identical on every
  // rank (take it from LastNegotiatedOrder()).
  Status FreezeSchedule(const std::vector<std::string>& names);
  void ThawSchedule();
  // Fails every collective in flight on this rank with `kAborted`, forgets partial negotiations and frozen
  // schedules, and returns once the engine thread has done so: the state a failed step leaves behind is gone and
  // the same tensor names can be submitted again.  Every rank calls it, then the ranks meet on a host barrier.
  Status Reset();
  bool schedule_frozen() const { return frozen_.load(); }
  // Names of the responses executed since the last call to this function.
  std::vector<std::string> TakeNegotiatedOrder();

  EngineCounters& counters() { return counters_; }
  const EngineOptions& options() const { return opts_; }

  void EnableTimeline(bool on) { timeline_on_ = on; }
  Status DumpTimeline(const std::string& path);

 private:
  CollectiveEngine() = default;

  struct Event {
    enum Kind { kLocalRequest, kRemoteRequest, kResponse, kFrozenReady, kPeerFailure, kReset, kShutdown, kStopMarker } kind;
    RequestMessage request;
    RpcMsgHead head;
    ResponseMessage response;
    int peer{-1};
  };

  void Loop();
  void HandleRequestOnCoordinator(const RequestMessage& req, const RpcMsgHead* head,
                                  std::vector<std::string>* ready);
  void FlushReady(std::vector<std::string>* ready);
  void Execute(const ResponseMessage& resp);
  Status ExecuteOne(OpRecord* rec, const ResponseMessage& resp, int channel);
  Status ExecuteFusedHost(std::vector<OpRecord*>& recs);
  void DrainFrozen();
  void Complete(const OpRecord& rec, const Status& st);
  void FailAll(const Status& st);
  void CheckStalls();
  void Trace(const std::string& name, const char* phase, int64_t b, int64_t e);

  std::atomic<bool> initialized_{false};
  std::atomic<bool> shut_down_{false};
  EngineOptions opts_;
  int rank_{0};
  int size_{1};
  std::thread thread_;
  Channel<Event> queue_;
  DeviceExecutorFn device_executor_{nullptr};

  std::mutex mu_;  // guards tensor_table_, handles_, frozen state, order log
  std::unordered_map<std::string, OpRecord> tensor_table_;
  std::unordered_map<int64_t, std::shared_ptr<HandleState>> handles_;
  std::condition_variable handle_cv_;
  uint64_t resets_requested_{0};  // guarded by mu_
  uint64_t resets_done_{0};
  std::condition_variable reset_cv_;
  int64_t next_handle_{1};

  MessageTable message_table_;  // rank 0, background thread only
  struct Signature {
    RequestType type;
    Datatype dtype;
    std::vector<int64_t> shape;
    int32_t device;
    int32_t reduce_op;
    int32_t root_rank;
  };
  std::unordered_map<std::string, Signature> negotiated_;  // name -> last validated signature
  std::vector<std::string> order_log_;

  // Frozen schedules: each FreezeSchedule call adds one cyclic sequence with its own cursor
  // (one per DistributedOptimizer).
  struct Schedule {
    std::vector<std::string> names;
    std::vector<Signature> sigs;
    std::vector<bool> ready;
    size_t cursor{0};
  };
  std::atomic<bool> frozen_{false};
  std::vector<Schedule> schedules_;
  std::unordered_map<std::string, std::pair<size_t, size_t>> schedule_index_;  // name -> (schedule, position)

  std::vector<uint8_t> fusion_buffer_;
  EngineCounters counters_;
  std::atomic<bool> timeline_on_{false};
  std::mutex timeline_mu_;
  std::deque<TimelineEvent> timeline_;
};

}  // namespace collective
}  // namespace tips
