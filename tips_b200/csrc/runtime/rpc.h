// Asynchronous request/response RPC between the ranks of a job.
//
// Capability parity with the reference's ZeroMQ RPC (tips/core/common/naive_rpc.h:38-178,
// naive_rpc.cc:25-290, zmq_message.h:12-67): named services registered on every
// rank, SendRequest with a completion callback that runs when the response
// arrives, SendResponse that echoes the request header, listener threads that
// run the callbacks, a self-loop so a rank can call itself, and a Finalize
// that drains and stops the listeners.
//
// Design differences: frames travel over a TCP mesh (no ZeroMQ on the target
// image); a service is addressed by a hash of its name and a request by an id
// in a local table, so no raw pointer ever crosses a process boundary
// (the reference ships `RpcRequest*` and per-rank service addresses,
// naive_rpc.cc:127-150,279-290); a peer that closes its socket unexpectedly
// fails every pending request to it and fires a failure hook, which is the
// host-side failure detector of the runtime.
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

#include "core/common.h"
#include "core/naive_buffer.h"

namespace tips {

enum RpcMsgType : int32_t { kRpcRequest = 0, kRpcResponse = 1 };

struct RpcMsgHead {
  int32_t type{kRpcRequest};
  int32_t src_rank{-1};
  int32_t dst_rank{-1};
  uint32_t service_hash{0};
  uint64_t request_id{0};
};

// One received or to-be-sent frame: [RpcMsgHead | payload]. Move-only owner of
// its bytes (the counterpart of the reference's ZmqMessage).
// Byte buffer whose resize() leaves new bytes uninitialised: frames of tens of MB are filled by recv() or memcpy
// right away, and zeroing them first costs as much as the copy.
template <typename T>
struct UninitAllocator : std::allocator<T> {
  template <typename U>
  struct rebind {
    using other = UninitAllocator<U>;
  };
  UninitAllocator() = default;
  template <typename U>
  UninitAllocator(const UninitAllocator<U>&) {}
  template <typename U>
  void construct(U* p) noexcept {
    ::new (static_cast<void*>(p)) U;  // default-initialisation: nothing for bytes
  }
  template <typename U, typename... A>
  void construct(U* p, A&&... a) {
    ::new (static_cast<void*>(p)) U(std::forward<A>(a)...);
  }
};
using FrameBytes = std::vector<uint8_t, UninitAllocator<uint8_t>>;

class RpcMessage {
 public:
  RpcMessage() = default;
  explicit RpcMessage(FrameBytes&& frame) : frame_(std::move(frame)) {}
  RpcMessage(RpcMessage&&) = default;
  RpcMessage& operator=(RpcMessage&&) = default;
  RpcMessage(const RpcMessage&) = delete;
  RpcMessage& operator=(const RpcMessage&) = delete;

  bool empty() const { return frame_.size() < sizeof(RpcMsgHead); }
  const RpcMsgHead& head() const { return *reinterpret_cast<const RpcMsgHead*>(frame_.data()); }
  const uint8_t* payload() const { return frame_.data() + sizeof(RpcMsgHead); }
  uint8_t* payload() { return frame_.data() + sizeof(RpcMsgHead); }
  size_t payload_size() const { return empty() ? 0 : frame_.size() - sizeof(RpcMsgHead); }
  size_t size() const { return frame_.size(); }

 private:
  FrameBytes frame_;
};

// Runs on a listener thread when a request for the service arrives. The
// handler answers with RpcServer::SendResponse(msg.head(), ...), possibly later
// and from another thread.
using RpcRequestHandler = std::function<void(RpcMessage&&)>;
// Runs on a listener thread when the response arrives; `status` is not OK when
// the peer died or the server shut down first (then `msg` is empty).
using RpcResponseCallback = std::function<void(const Status&, RpcMessage&&)>;

class RpcService {
 public:
  RpcService(std::string name, RpcRequestHandler handler);
  const std::string& name() const { return name_; }
  uint32_t hash() const { return hash_; }
  void Handle(RpcMessage&& msg) { handler_(std::move(msg)); }

 private:
  std::string name_;
  uint32_t hash_;
  RpcRequestHandler handler_;
};

class RpcServer {
 public:
  static RpcServer& Global();

  // `peer_fds[r]` is a connected stream socket to rank r; the entry of this
  // rank itself is ignored (a local socket pair is made for the self loop).
  // The server owns the fds from here on.
  void Initialize(int rank, int size, std::vector<int> peer_fds, int num_listen_threads = 1);
  bool initialized() const { return initialized_.load(); }

  // Registration is local; callers that need every rank to have the service
  // before the first request put a barrier after it.
  RpcService* AddService(const std::string& name, RpcRequestHandler handler);
  RpcService* LookupService(const std::string& name);

  Status SendRequest(int dst_rank, const RpcService* service, const void* payload, size_t size,
                     RpcResponseCallback on_response);
  Status SendRequest(int dst_rank, const std::string& service_name, const void* payload, size_t size,
                     RpcResponseCallback on_response);
  Status SendResponse(const RpcMsgHead& request_head, const void* payload, size_t size);

  // Called (on a listener thread) when a peer's connection drops while the
  // server is running.
  void SetPeerFailureHook(std::function<void(int)> hook);
  bool peer_alive(int r) const { return r >= 0 && r < size_ && !peer_dead_[r].load(); }

  // Test hook: drop the next `n` outgoing requests to `dst_rank` (-1 = any).
  void InjectDropRequests(int dst_rank, int n);

  int64_t pending_requests() const { return pending_count_.load(); }
  uint64_t messages_sent() const { return sent_count_.load(); }
  uint64_t messages_received() const { return recv_count_.load(); }

  // After this call a peer that closes its connection is an orderly shutdown,
  // not a failure.
  void SetQuiescing() { quiescing_ = true; }

  // Stops the listeners, fails whatever is still pending and closes the
  // sockets.  Callers synchronise the ranks before (a barrier) so that no
  // request is in flight.
  void Finalize();

 private:
  RpcServer() = default;
  void ListenLoop(int thread_index);
  void SenderLoop();
  bool ReadFrame(int fd, FrameBytes* frame);
  Status SendFrame(int dst_rank, const RpcMsgHead& head, const void* payload, size_t size);
  void Dispatch(RpcMessage&& msg);
  void OnPeerClosed(int peer);

  std::atomic<bool> initialized_{false};
  std::atomic<bool> stopping_{false};
  std::atomic<bool> quiescing_{false};
  int rank_{-1};
  int size_{0};
  int num_listen_threads_{1};
  std::vector<int> send_fds_;   // write side per destination
  std::vector<int> recv_fds_;   // read side per source
  std::vector<std::unique_ptr<std::mutex>> send_mus_;
  std::unique_ptr<std::atomic<bool>[]> peer_dead_;
  int wake_pipe_[2]{-1, -1};
  std::vector<std::thread> listeners_;
  // Frames produced on a listener thread (responses written by request handlers, requests sent from callbacks) are
  // handed to this thread: a listener that blocked in send() would stop draining its sockets, and two ranks whose
  // listeners send each other more than the socket buffers hold, or one rank answering itself, would never finish.
  std::thread sender_;
  std::mutex out_mu_;
  std::condition_variable out_cv_;
  std::deque<std::pair<int, FrameBytes>> out_queue_;
  bool sender_stop_{false};

  std::mutex services_mu_;
  std::unordered_map<uint32_t, std::unique_ptr<RpcService>> services_;

  struct Pending {
    int dst_rank;
    RpcResponseCallback cb;
  };
  std::mutex pending_mu_;
  std::unordered_map<uint64_t, Pending> pending_;
  std::atomic<uint64_t> next_request_id_{1};
  std::atomic<int64_t> pending_count_{0};
  std::atomic<uint64_t> sent_count_{0};
  std::atomic<uint64_t> recv_count_{0};

  std::mutex hook_mu_;
  std::function<void(int)> failure_hook_;
  std::atomic<int> drop_dst_{-2};
  std::atomic<int> drop_left_{0};
};

}  // namespace tips
