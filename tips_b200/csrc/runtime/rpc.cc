#include "runtime/rpc.h"

#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include "runtime/net.h"

namespace tips {

namespace {
uint32_t Fnv1a(const std::string& s) {
  uint32_t h = 2166136261u;
  for (unsigned char c : s) {
    h ^= c;
    h *= 16777619u;
  }
  return h ? h : 1u;
}
}  // namespace

RpcService::RpcService(std::string name, RpcRequestHandler handler)
    : name_(std::move(name)), hash_(Fnv1a(name_)), handler_(std::move(handler)) {}

namespace {
thread_local bool t_on_listener_thread = false;
}  // namespace

RpcServer& RpcServer::Global() {
  static RpcServer* server = new RpcServer;
  return *server;
}

void RpcServer::Initialize(int rank, int size, std::vector<int> peer_fds, int num_listen_threads) {
  TIPS_CHECK(!initialized_.load()) << "RpcServer initialised twice";
  TIPS_CHECK_EQ(static_cast<int>(peer_fds.size()), size);
  rank_ = rank;
  size_ = size;
  send_fds_.assign(size, -1);
  recv_fds_.assign(size, -1);
  send_mus_.clear();
  peer_dead_.reset(new std::atomic<bool>[size]);
  for (int r = 0; r < size; ++r) {
    send_mus_.emplace_back(new std::mutex);
    peer_dead_[r] = false;
    if (r == rank) {
      int sv[2];
      TIPS_ZCHECK(socketpair(AF_UNIX, SOCK_STREAM, 0, sv));
      send_fds_[r] = sv[0];
      recv_fds_[r] = sv[1];
    } else {
      send_fds_[r] = peer_fds[r];
      recv_fds_[r] = peer_fds[r];
    }
  }
  TIPS_ZCHECK(pipe(wake_pipe_));
  stopping_ = false;
  quiescing_ = false;
  {
    std::lock_guard<std::mutex> lock(pending_mu_);
    pending_.clear();
    pending_count_ = 0;
  }
  if (num_listen_threads < 1) num_listen_threads = 1;
  if (num_listen_threads > size) num_listen_threads = size;
  num_listen_threads_ = num_listen_threads;
  initialized_ = true;
  {
    std::lock_guard<std::mutex> lock(out_mu_);
    out_queue_.clear();
    sender_stop_ = false;
  }
  sender_ = std::thread([this] { SenderLoop(); });
  for (int t = 0; t < num_listen_threads; ++t) listeners_.emplace_back([this, t] { ListenLoop(t); });
}

RpcService* RpcServer::AddService(const std::string& name, RpcRequestHandler handler) {
  std::lock_guard<std::mutex> lock(services_mu_);
  auto svc      = std::make_unique<RpcService>(name, std::move(handler));
  uint32_t hash = svc->hash();
  auto it       = services_.find(hash);
  if (it != services_.end()) {
    TIPS_CHECK(it->second->name() == name) << "service name hash collision: " << name << " vs " << it->second->name();
    it->second = std::move(svc);  // re-registration replaces the handler
    return it->second.get();
  }
  RpcService* raw = svc.get();
  services_[hash] = std::move(svc);
  return raw;
}

RpcService* RpcServer::LookupService(const std::string& name) {
  std::lock_guard<std::mutex> lock(services_mu_);
  auto it = services_.find(Fnv1a(name));
  return it == services_.end() ? nullptr : it->second.get();
}

void RpcServer::SetPeerFailureHook(std::function<void(int)> hook) {
  std::lock_guard<std::mutex> lock(hook_mu_);
  failure_hook_ = std::move(hook);
}

void RpcServer::InjectDropRequests(int dst_rank, int n) {
  drop_dst_  = dst_rank;
  drop_left_ = n;
}

Status RpcServer::SendFrame(int dst_rank, const RpcMsgHead& head, const void* payload, size_t size) {
  if (!initialized_.load()) return Status(kUnavailable, "rpc server not initialised");
  if (dst_rank < 0 || dst_rank >= size_) return Status(kInvalidArgument, "bad destination rank");
  if (peer_dead_[dst_rank].load()) return Status(kUnavailable, "peer " + std::to_string(dst_rank) + " is gone");
  uint64_t len = sizeof(RpcMsgHead) + size;
  FrameBytes frame(sizeof(uint64_t) + len);
  memcpy(frame.data(), &len, sizeof(len));
  memcpy(frame.data() + sizeof(len), &head, sizeof(head));
  if (size) memcpy(frame.data() + sizeof(len) + sizeof(head), payload, size);
  if (t_on_listener_thread) {  // never block a listener in send(): the sender thread takes it from here
    {
      std::lock_guard<std::mutex> lock(out_mu_);
      out_queue_.emplace_back(dst_rank, std::move(frame));
    }
    out_cv_.notify_one();
    sent_count_++;
    return Status::OK();
  }
  std::lock_guard<std::mutex> lock(*send_mus_[dst_rank]);
  if (!net::SendAll(send_fds_[dst_rank], frame.data(), frame.size()))
    return Status(kUnavailable, "send to rank " + std::to_string(dst_rank) + " failed");
  sent_count_++;
  return Status::OK();
}

void RpcServer::SenderLoop() {
  for (;;) {
    std::pair<int, FrameBytes> item;
    {
      std::unique_lock<std::mutex> lock(out_mu_);
      out_cv_.wait(lock, [&] { return sender_stop_ || !out_queue_.empty(); });
      if (out_queue_.empty()) return;  // stop requested and everything handed over has been sent
      item = std::move(out_queue_.front());
      out_queue_.pop_front();
    }
    const int dst = item.first;
    if (peer_dead_[dst].load()) continue;
    std::lock_guard<std::mutex> lock(*send_mus_[dst]);
    if (!net::SendAll(send_fds_[dst], item.second.data(), item.second.size()) && !stopping_.load() && !quiescing_.load())
      TIPS_LOG(ERROR) << "send to rank " << dst << " failed";
  }
}

Status RpcServer::SendRequest(int dst_rank, const std::string& service_name, const void* payload, size_t size,
                              RpcResponseCallback on_response) {
  RpcService tmp(service_name, nullptr);
  return SendRequest(dst_rank, &tmp, payload, size, std::move(on_response));
}

Status RpcServer::SendRequest(int dst_rank, const RpcService* service, const void* payload, size_t size,
                              RpcResponseCallback on_response) {
  RpcMsgHead head;
  head.type         = kRpcRequest;
  head.src_rank     = rank_;
  head.dst_rank     = dst_rank;
  head.service_hash = service->hash();
  head.request_id   = next_request_id_++;
  {
    std::lock_guard<std::mutex> lock(pending_mu_);
    pending_[head.request_id] = Pending{dst_rank, std::move(on_response)};
    pending_count_++;
  }
  if (drop_left_.load() > 0 && (drop_dst_.load() == -1 || drop_dst_.load() == dst_rank)) {
    drop_left_--;
    return Status::OK();  // fault injection: the request silently vanishes
  }
  Status st = SendFrame(dst_rank, head, payload, size);
  if (!st.ok()) {
    std::lock_guard<std::mutex> lock(pending_mu_);
    if (pending_.erase(head.request_id)) pending_count_--;
  }
  return st;
}

Status RpcServer::SendResponse(const RpcMsgHead& request_head, const void* payload, size_t size) {
  RpcMsgHead head = request_head;
  head.type       = kRpcResponse;
  head.src_rank   = rank_;
  head.dst_rank   = request_head.src_rank;
  return SendFrame(head.dst_rank, head, payload, size);
}

bool RpcServer::ReadFrame(int fd, FrameBytes* frame) {
  uint64_t len = 0;
  if (!net::RecvAll(fd, &len, sizeof(len))) return false;
  if (len < sizeof(RpcMsgHead) || len > (1ull << 34)) return false;
  frame->resize(len);
  return net::RecvAll(fd, frame->data(), len);
}

void RpcServer::Dispatch(RpcMessage&& msg) {
  recv_count_++;
  const RpcMsgHead head = msg.head();
  if (head.type == kRpcRequest) {
    RpcService* svc = nullptr;
    {
      std::lock_guard<std::mutex> lock(services_mu_);
      auto it = services_.find(head.service_hash);
      if (it != services_.end()) svc = it->second.get();
    }
    if (!svc) {
      TIPS_LOG(ERROR) << "request for unknown service hash " << head.service_hash << " from rank " << head.src_rank;
      return;
    }
    try {
      svc->Handle(std::move(msg));
    } catch (const std::exception& e) {
      TIPS_LOG(ERROR) << "service " << svc->name() << " threw: " << e.what();
    }
  } else {
    RpcResponseCallback cb;
    {
      std::lock_guard<std::mutex> lock(pending_mu_);
      auto it = pending_.find(head.request_id);
      if (it == pending_.end()) return;  // already failed (peer death / timeout)
      cb = std::move(it->second.cb);
      pending_.erase(it);
      pending_count_--;
    }
    if (cb) {
      try {
        cb(Status::OK(), std::move(msg));
      } catch (const std::exception& e) {
        TIPS_LOG(ERROR) << "response callback threw: " << e.what();
      }
    }
  }
}

void RpcServer::OnPeerClosed(int peer) {
  if (stopping_.load() || quiescing_.load()) return;
  bool was = peer_dead_[peer].exchange(true);
  if (was) return;
  std::vector<RpcResponseCallback> failed;
  {
    std::lock_guard<std::mutex> lock(pending_mu_);
    for (auto it = pending_.begin(); it != pending_.end();) {
      if (it->second.dst_rank == peer) {
        failed.push_back(std::move(it->second.cb));
        it = pending_.erase(it);
        pending_count_--;
      } else {
        ++it;
      }
    }
  }
  Status st(kUnavailable, "rank " + std::to_string(peer) + " closed its connection");
  for (auto& cb : failed)
    if (cb) cb(st, RpcMessage());
  std::function<void(int)> hook;
  {
    std::lock_guard<std::mutex> lock(hook_mu_);
    hook = failure_hook_;
  }
  if (hook) hook(peer);
}

void RpcServer::ListenLoop(int thread_index) {
  t_on_listener_thread = true;
  std::vector<int> my_peers;
  const int total_threads = num_listen_threads_;
  for (int r = 0; r < size_; ++r)
    if (r % total_threads == thread_index) my_peers.push_back(r);

  std::vector<struct pollfd> pfds;
  while (!stopping_.load()) {
    pfds.clear();
    pfds.push_back({wake_pipe_[0], POLLIN, 0});
    for (int r : my_peers)
      if (!peer_dead_[r].load()) pfds.push_back({recv_fds_[r], POLLIN, 0});
    int n = ignore_signal_call(poll, pfds.data(), static_cast<nfds_t>(pfds.size()), 1000);
    if (n <= 0) continue;
    if (pfds[0].revents & POLLIN) break;
    size_t k = 1;
    for (int r : my_peers) {
      if (peer_dead_[r].load()) continue;
      if (k >= pfds.size()) break;
      short ev = pfds[k].revents;
      ++k;
      if (!(ev & (POLLIN | POLLHUP | POLLERR))) continue;
      FrameBytes frame;
      if (!ReadFrame(recv_fds_[r], &frame)) {
        OnPeerClosed(r);
        if (stopping_.load()) break;
        peer_dead_[r] = true;
        continue;
      }
      Dispatch(RpcMessage(std::move(frame)));
    }
  }
}

void RpcServer::Finalize() {
  if (!initialized_.load()) return;
  stopping_ = true;
  char b    = 1;
  if (write(wake_pipe_[1], &b, 1) < 0) {
  }
  for (auto& t : listeners_)
    if (t.joinable()) t.join();
  listeners_.clear();
  {
    std::lock_guard<std::mutex> lock(out_mu_);
    sender_stop_ = true;
  }
  out_cv_.notify_all();
  if (sender_.joinable()) sender_.join();  // sends what the listeners had handed over, then ends
  std::vector<RpcResponseCallback> failed;
  {
    std::lock_guard<std::mutex> lock(pending_mu_);
    for (auto& kv : pending_) failed.push_back(std::move(kv.second.cb));
    pending_.clear();
    pending_count_ = 0;
  }
  Status st(kAborted, "rpc server shut down");
  for (auto& cb : failed)
    if (cb) cb(st, RpcMessage());
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) {
      net::Close(send_fds_[r]);
      net::Close(recv_fds_[r]);
    } else {
      net::Close(send_fds_[r]);
    }
  }
  net::Close(wake_pipe_[0]);
  net::Close(wake_pipe_[1]);
  wake_pipe_[0] = wake_pipe_[1] = -1;
  send_fds_.clear();
  recv_fds_.clear();
  {
    std::lock_guard<std::mutex> lock(services_mu_);
    services_.clear();
  }
  {
    std::lock_guard<std::mutex> lock(hook_mu_);
    failure_hook_ = nullptr;
  }
  initialized_ = false;
}

}  // namespace tips
