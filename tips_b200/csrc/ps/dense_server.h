// Dense parameter-server tables over the runtime's RPC: a vector of `size`
// fp32 elements, range-partitioned over the servers' shards, pulled and pushed
// by index range, with the update rule applied on the owning shard's thread.
//
// Capability parity with the reference: DenseTable (range partition, Lookup,
// ForEach, Load/Save; tips/core/ps/dense_table.h:49-131) and the dense pull
// access method that copies a stored element into the worker's parameter
// (tips/core/ps/dense_access_method.h:10-25).  The reference stops there: its
// dense table is not compiled into the library and has no server, client or push
// rule.  Here the table is served like the sparse one: a pull returns the
// elements of [begin, end) gathered from every owning shard, a push sends a
// gradient for [begin, end) and each shard applies SGD (w -= lr*g), Adagrad, the
// reference's literal rule (w = lr*g) or a plain assignment to its part.
#pragma once

#include <atomic>
#include <memory>
#include <string>
#include <vector>

#include "ps/ps_server.h"
#include "ps/table.h"

namespace tips {
namespace ps {

enum class DenseRule : int32_t { kSgd = 0, kAdagrad = 1, kLiteralReference = 2 };
enum class DensePushOp : int32_t { kGradient = 0, kAssign = 1 };

// Element-wise update of a contiguous run of a shard.  State (Adagrad accumulators) is kept per local shard
// and only touched on that shard's thread.
class DensePushAccess {
 public:
  DensePushAccess(DenseRule rule, double lr, double eps) : rule_(rule), lr_(lr), eps_(eps) {}
  void Apply(float* w, float* state, const float* g, size_t n) const;
  bool needs_state() const { return rule_ == DenseRule::kAdagrad; }
  DenseRule rule() const { return rule_; }

 private:
  DenseRule rule_;
  double lr_, eps_;
};

// One range of a request, cut at shard boundaries by the client: [begin, end) lies inside global shard `shard`.
struct DenseRange {
  uint64_t begin{0}, end{0};
  int32_t shard{0};
};

struct DenseRequest {
  MessageMeta meta;
  int32_t op{0};                   // pull: unused; push: DensePushOp
  std::vector<DenseRange> ranges;
  std::vector<float> values;       // push: the ranges' gradients, concatenated
  void Serialize(NaiveBuffer* b) const;
  void Deserialize(NaiveBuffer* b);
};

class DensePsServer {
 public:
  DensePsServer(std::string name, DenseTable<float>* table, DenseRule rule, double lr, double eps);
  ~DensePsServer();
  void Start();
  void Stop();
  uint64_t elements_pulled() const { return pulled_.load(); }
  uint64_t elements_pushed() const { return pushed_.load(); }
  std::string pull_service_name() const { return "dense_pull_service." + name_; }
  std::string push_service_name() const { return "dense_push_service." + name_; }

 private:
  void PullTask(RpcMessage&& msg);
  void PushTask(RpcMessage&& msg);

  std::string name_;
  DenseTable<float>* table_;
  DensePushAccess access_;
  std::vector<std::vector<float>> state_;  // per local shard, sized on first use
  bool started_{false};
  std::atomic<uint64_t> pulled_{0}, pushed_{0};
};

class DensePsClient {
 public:
  DensePsClient(std::string name, DenseTable<float>* table, int client_id);
  // out receives end - begin elements.  The future completes once, after every contacted server answered.
  std::shared_ptr<PsFuture> Pull(uint64_t begin, uint64_t end, float* out);
  std::shared_ptr<PsFuture> Push(uint64_t begin, uint64_t end, const float* values, DensePushOp op);

 private:
  // Cuts [begin, end) at shard boundaries and groups the pieces by owning server.
  std::vector<std::vector<DenseRange>> Split(uint64_t begin, uint64_t end) const;

  std::string name_;
  DenseTable<float>* table_;
  int client_id_;
  std::atomic<uint64_t> next_message_id_{1};
};

}  // namespace ps
}  // namespace tips
