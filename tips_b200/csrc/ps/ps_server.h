// Parameter-server server and client over the runtime's RPC.
//
// Capability parity with the reference:
//   PsServer  tips/core/ps/ps_server.h:33-265  RPC services "pull_service" / "push_service";
//             a request's keys are bucketed by shard and one closure per shard runs on that
//             shard's thread; the last shard to finish builds the response (pull: values in
//             request order) and sends it
//   PsClient  tips/core/ps/ps_client.h:78-176  bucket records by owning server, one request
//             per server, asynchronous completion
// Beside the per-row messages of the reference there is a packed form for uniform rows (PullPacked / PushPacked),
// which the C API uses: no per-row allocation on either side, rows copied once between the message and the table.
// Differences: the completion fires ONCE per call, after every contacted server answered
// (the reference calls `done` once per server, ps_client.h:93-107,124-128); a push to a row
// that was never pulled is reported in the response instead of CHECK-failing the server
// (access_method.h:137-143); placement is the table's single rule for both directions.
#pragma once

#include <atomic>
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "ps/access_method.h"
#include "ps/ps_messages.h"
#include "ps/table.h"
#include "runtime/rpc.h"

namespace tips {
namespace ps {

class PsServer {
 public:
  // `name` distinguishes several tables served by one process; every rank registers
  // the services (only servers receive requests).
  PsServer(std::string name, SparseTable* table, std::shared_ptr<PullAccessMethod> pull,
           std::shared_ptr<PushAccessMethod> push);
  ~PsServer();
  void Start();  // registers the RPC services and starts the table's shard threads
  void Stop();
  uint64_t rows_pulled() const { return rows_pulled_.load(); }
  uint64_t rows_pushed() const { return rows_pushed_.load(); }
  std::string pull_service_name() const { return std::string(kPullServiceName) + "." + name_; }
  std::string push_service_name() const { return std::string(kPushServiceName) + "." + name_; }

 private:
  void PullTask(RpcMessage&& msg);
  void PushTask(RpcMessage&& msg);
  void PackedPullTask(RpcMessage&& msg);
  void PackedPushTask(RpcMessage&& msg);

  std::string name_;
  SparseTable* table_;
  PullAccessAgent pull_agent_;
  PushAccessAgent push_agent_;
  bool started_{false};
  std::atomic<uint64_t> rows_pulled_{0};
  std::atomic<uint64_t> rows_pushed_{0};
};

// Completion state of one client call.
struct PsFuture {
  std::mutex mu;
  std::condition_variable cv;
  int pending{0};
  Status status;
  // pull: value of every requested key, in request order
  std::vector<KeyItem> values;
  uint64_t missing_rows{0};  // push: rows that did not exist on the server
  uint64_t bad_rows{0};      // packed pull: rows that exist with another dtype or length
  bool cancelled{false};     // packed pull: the caller gave up; late responses must not touch its output buffer
  void Cancel();
  bool Wait(int timeout_ms);
};

class PsClient {
 public:
  PsClient(std::string name, SparseTable* table, int client_id);

  struct PullRecord {
    uint64_t key;
    Datatype dtype;
    uint32_t length;
  };
  // Asynchronous: the future completes once, when every server has answered.
  std::shared_ptr<PsFuture> Pull(const std::vector<PullRecord>& records, std::function<void()> done = nullptr);
  std::shared_ptr<PsFuture> Push(const std::vector<KeyItem>& records, std::function<void()> done = nullptr);
  // Uniform rows, packed on the wire (see ps_messages.h).  `out` / `values` hold n rows of `length` elements in key
  // order and must stay alive until the future completes; pulled rows are written straight into `out`.
  std::shared_ptr<PsFuture> PullPacked(const uint64_t* keys, size_t n, Datatype dtype, uint32_t length, void* out);
  std::shared_ptr<PsFuture> PushPacked(const uint64_t* keys, size_t n, Datatype dtype, uint32_t length,
                                       const void* values);

 private:
  std::string name_;
  SparseTable* table_;
  int client_id_;
  std::atomic<uint64_t> next_message_id_{1};
};

}  // namespace ps
}  // namespace tips
