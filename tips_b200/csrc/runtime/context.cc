#include "runtime/context.h"

#include <algorithm>
#include <cstdlib>

#include "runtime/net.h"

namespace tips {

namespace {

const char kGatherService[] = "tips_host_gather";

bool IsLoopback(const std::string& host) {
  return host == "127.0.0.1" || host == "localhost" || host.rfind("127.", 0) == 0;
}

int EnvInt(const char* name, int dflt) {
  const char* v = getenv(name);
  if (!v || !*v) return dflt;
  return atoi(v);
}

bool SendString(int fd, const std::string& s) {
  uint32_t n = static_cast<uint32_t>(s.size());
  return net::SendAll(fd, &n, sizeof(n)) && net::SendAll(fd, s.data(), n);
}
bool RecvString(int fd, std::string* s) {
  uint32_t n = 0;
  if (!net::RecvAll(fd, &n, sizeof(n))) return false;
  if (n > (1u << 20)) return false;
  s->resize(n);
  return net::RecvAll(fd, &(*s)[0], n);
}

struct GatherWait {
  std::mutex mu;
  std::condition_variable cv;
  bool done{false};
  Status status;
  std::vector<std::string> result;
};

}  // namespace

// ---------------------------------------------------------------- Group ----

Group::Group(uint64_t id, std::vector<int> world_ranks, int my_world_rank) : id_(id) {
  std::sort(world_ranks.begin(), world_ranks.end());
  world_ranks.erase(std::unique(world_ranks.begin(), world_ranks.end()), world_ranks.end());
  ranks_ = std::move(world_ranks);
  my_group_rank_ = ToGroupRank(my_world_rank);
}

int Group::ToGroupRank(int world_rank) const {
  auto it = std::lower_bound(ranks_.begin(), ranks_.end(), world_rank);
  if (it == ranks_.end() || *it != world_rank) return -1;
  return static_cast<int>(it - ranks_.begin());
}

Status Group::Barrier(int timeout_ms) {
  std::vector<std::string> all;
  return AllgatherBytes(std::string(), &all, timeout_ms);
}

Status Group::AllgatherBytes(const std::string& mine, std::vector<std::string>* all, int timeout_ms) {
  return Context::Global().GroupGather(this, mine, all, timeout_ms);
}

// -------------------------------------------------------------- Context ----

Context& Context::Global() {
  static Context* ctx = new Context;
  return *ctx;
}

InitOptions Context::OptionsFromEnv() {
  InitOptions o;
  o.rank = EnvInt("TIPS_RANK", EnvInt("RANK", EnvInt("OMPI_COMM_WORLD_RANK", 0)));
  o.size = EnvInt("TIPS_SIZE", EnvInt("WORLD_SIZE", EnvInt("OMPI_COMM_WORLD_SIZE", 1)));
  if (const char* a = getenv("MASTER_ADDR")) o.master_addr = a;
  int torch_port     = EnvInt("MASTER_PORT", 29400);
  o.master_port      = EnvInt("TIPS_MASTER_PORT", torch_port + 1000 > 65000 ? torch_port - 1000 : torch_port + 1000);
  o.connect_timeout_ms = EnvInt("TIPS_CONNECT_TIMEOUT_MS", 120000);
  o.rpc_listen_threads = EnvInt("TIPS_RPC_LISTEN_THREADS", 1);
  return o;
}

Status Context::Initialize(const InitOptions& opts) {
  if (initialized_) return Status(kPrecondition, "tips runtime already initialised");
  if (opts.size < 1 || opts.rank < 0 || opts.rank >= opts.size)
    return Status(kInvalidArgument, StringFormat("bad rank/size %d/%d", opts.rank, opts.size));
  rank_ = opts.rank;
  size_ = opts.size;
  LogConfig::SetRank(rank_, size_);
  host_timeout_ms_ = EnvInt("TIPS_HOST_TIMEOUT_MS", 300000);
  data_timeout_ms_ = EnvInt("TIPS_DATA_TIMEOUT_MS", host_timeout_ms_);

  const std::string my_ip = getenv("TIPS_LOCAL_IP") ? std::string(getenv("TIPS_LOCAL_IP"))
                            : IsLoopback(opts.master_addr) ? std::string("127.0.0.1")
                                                           : GetLocalIp();
  ips_.assign(size_, my_ip);
  std::vector<int> ports(size_, 0);
  std::vector<int> rpc_fds(size_, -1);
  data_fds_.assign(size_, -1);

  int listen_fd = -1;
  if (size_ > 1) {
    int my_port = 0;
    listen_fd   = net::Listen(0, &my_port);

    // ---- rendezvous at the master ----
    int master_fd = -1;
    if (rank_ == 0) {
      int bound = 0;
      master_fd = net::Listen(opts.master_port, &bound);
    }
    int c = net::Connect(opts.master_addr, opts.master_port, opts.connect_timeout_ms);
    if (c < 0) {
      net::Close(listen_fd);
      net::Close(master_fd);
      return Status(kUnavailable, StringFormat("rank %d cannot reach the rendezvous at %s:%d", rank_,
                                               opts.master_addr.c_str(), opts.master_port));
    }
    int32_t reg[2] = {rank_, my_port};
    bool ok        = net::SendAll(c, reg, sizeof(reg)) && SendString(c, my_ip);
    if (rank_ == 0) {
      std::vector<int> conns(size_, -1);
      for (int i = 0; i < size_ && ok; ++i) {
        int fd = net::Accept(master_fd, opts.connect_timeout_ms);
        if (fd < 0) {
          ok = false;
          break;
        }
        int32_t r[2];
        std::string ip;
        if (!net::RecvAll(fd, r, sizeof(r)) || !RecvString(fd, &ip) || r[0] < 0 || r[0] >= size_ ||
            conns[r[0]] != -1) {
          net::Close(fd);
          ok = false;
          break;
        }
        conns[r[0]] = fd;
        ports[r[0]] = r[1];
        ips_[r[0]]  = ip;
      }
      for (int i = 0; i < size_; ++i) {
        if (conns[i] < 0) continue;
        if (ok) {
          ok = net::SendAll(conns[i], ports.data(), sizeof(int) * size_);
          for (int j = 0; j < size_ && ok; ++j) ok = SendString(conns[i], ips_[j]);
        }
        net::Close(conns[i]);
      }
      net::Close(master_fd);
    }
    if (ok) {
      ok = net::RecvAll(c, ports.data(), sizeof(int) * size_);
      for (int j = 0; j < size_ && ok; ++j) ok = RecvString(c, &ips_[j]);
    }
    net::Close(c);
    if (!ok) {
      net::Close(listen_fd);
      return Status(kUnavailable, "rendezvous failed");
    }

    // ---- two full meshes: kind 0 = rpc, kind 1 = data ----
    for (int kind = 0; kind < 2 && ok; ++kind) {
      for (int j = 0; j < rank_ && ok; ++j) {
        int fd = net::Connect(ips_[j], ports[j], opts.connect_timeout_ms);
        if (fd < 0) {
          ok = false;
          break;
        }
        int32_t hello[2] = {kind, rank_};
        ok               = net::SendAll(fd, hello, sizeof(hello));
        (kind == 0 ? rpc_fds : data_fds_)[j] = fd;
      }
    }
    int to_accept = 2 * (size_ - 1 - rank_);
    for (int i = 0; i < to_accept && ok; ++i) {
      int fd = net::Accept(listen_fd, opts.connect_timeout_ms);
      if (fd < 0) {
        ok = false;
        break;
      }
      int32_t hello[2];
      if (!net::RecvAll(fd, hello, sizeof(hello)) || hello[0] < 0 || hello[0] > 1 || hello[1] <= rank_ ||
          hello[1] >= size_) {
        net::Close(fd);
        ok = false;
        break;
      }
      (hello[0] == 0 ? rpc_fds : data_fds_)[hello[1]] = fd;
    }
    net::Close(listen_fd);
    if (!ok) {
      for (int fd : rpc_fds) net::Close(fd);
      for (int fd : data_fds_) net::Close(fd);
      return Status(kUnavailable, "building the TCP mesh failed");
    }
  }

  // local rank = position among the ranks that share this host
  local_rank_ = 0;
  local_size_ = 0;
  for (int r = 0; r < size_; ++r) {
    if (ips_[r] == ips_[rank_]) {
      if (r < rank_) ++local_rank_;
      ++local_size_;
    }
  }
  local_rank_ = EnvInt("LOCAL_RANK", local_rank_);
  local_size_ = EnvInt("LOCAL_WORLD_SIZE", local_size_);

  std::vector<int> all(size_);
  for (int i = 0; i < size_; ++i) all[i] = i;
  world_.reset(new Group(0, all, rank_));
  next_group_id_ = 1;

  // The gather service is registered before the listeners start, so a request
  // from a faster rank can never find the service table empty.
  RpcServer::Global().AddService(kGatherService, [this](RpcMessage&& m) { HandleGatherRequest(std::move(m)); });
  RpcServer::Global().Initialize(rank_, size_, rpc_fds, opts.rpc_listen_threads);
  initialized_ = true;
  Status st = Barrier(opts.connect_timeout_ms);
  if (!st.ok()) {
    initialized_ = false;
    return st;
  }
  TIPS_VLOG(1) << "runtime up: local_rank " << local_rank_ << "/" << local_size_ << " ip " << ips_[rank_];
  return Status::OK();
}

void Context::Finalize() {
  if (!initialized_) return;
  Barrier(30000);
  RpcServer::Global().SetQuiescing();
  Barrier(30000);
  RpcServer::Global().Finalize();
  for (int& fd : data_fds_) {
    net::Close(fd);
    fd = -1;
  }
  data_fds_.clear();
  groups_.clear();
  world_.reset();
  {
    std::lock_guard<std::mutex> lock(gather_mu_);
    gather_slots_.clear();
  }
  initialized_ = false;
  LogConfig::SetRank(-1, 0);
}

Group* Context::NewGroup(const std::vector<int>& world_ranks) {
  TIPS_CHECK(initialized_);
  for (int r : world_ranks) TIPS_CHECK(r >= 0 && r < size_) << "group rank out of range: " << r;
  std::lock_guard<std::mutex> lock(groups_mu_);
  groups_.emplace_back(new Group(next_group_id_++, world_ranks, rank_));
  return groups_.back().get();
}

Group* Context::FindGroup(uint64_t id) {
  if (id == 0) return world_.get();
  std::lock_guard<std::mutex> lock(groups_mu_);
  for (auto& g : groups_)
    if (g->id() == id) return g.get();
  return nullptr;
}

Status Context::BroadcastBytes(std::string* inout, int root, int timeout_ms) {
  std::vector<std::string> all;
  Status st = AllgatherBytes(rank_ == root ? *inout : std::string(), &all, timeout_ms);
  if (!st.ok()) return st;
  *inout = all.at(root);
  return Status::OK();
}

Status Context::GroupGather(Group* g, const std::string& mine, std::vector<std::string>* all, int timeout_ms) {
  if (!initialized_) return Status(kPrecondition, "tips runtime not initialised");
  if (!g->valid()) return Status(kInvalidArgument, "this rank is not a member of the group");
  if (timeout_ms < 0) timeout_ms = host_timeout_ms_;
  uint64_t seq;
  {
    std::lock_guard<std::mutex> lock(g->seq_mu_);
    seq = g->seq_++;
  }
  if (g->size() == 1) {
    all->assign(1, mine);
    return Status::OK();
  }
  NaiveBuffer buf;
  buf << g->id() << seq << static_cast<int32_t>(g->size()) << static_cast<int32_t>(g->rank()) << mine;
  auto wait = std::make_shared<GatherWait>();
  Status st = RpcServer::Global().SendRequest(
      g->leader(), kGatherService, buf.data(), buf.size(), [wait](const Status& s, RpcMessage&& m) {
        std::lock_guard<std::mutex> lock(wait->mu);
        wait->status = s;
        if (s.ok()) {
          NaiveBuffer rb(m.payload(), m.payload_size());
          uint64_t n = 0;
          rb >> n;
          wait->result.resize(n);
          for (uint64_t i = 0; i < n; ++i) rb >> wait->result[i];
        }
        wait->done = true;
        wait->cv.notify_all();
      });
  if (!st.ok()) return st;
  std::unique_lock<std::mutex> lock(wait->mu);
  if (!wait->cv.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return wait->done; }))
    return Status(kTimeout, StringFormat("host collective #%llu of group %llu timed out after %d ms",
                                         (unsigned long long)seq, (unsigned long long)g->id(), timeout_ms));
  if (!wait->status.ok()) return wait->status;
  *all = std::move(wait->result);
  return Status::OK();
}

void Context::HandleGatherRequest(RpcMessage&& msg) {
  NaiveBuffer rb(msg.payload(), msg.payload_size());
  uint64_t gid = 0, seq = 0;
  int32_t gsize = 0, grank = 0;
  std::string data;
  rb >> gid >> seq >> gsize >> grank >> data;
  std::vector<std::pair<RpcMsgHead, std::string>> ready;
  {
    std::lock_guard<std::mutex> lock(gather_mu_);
    GatherSlot& slot = gather_slots_[{gid, seq}];
    if (slot.expected == 0) {
      slot.expected = gsize;
      slot.arrivals.resize(gsize);
      slot.present.assign(gsize, false);
    }
    if (grank < 0 || grank >= slot.expected || slot.present[grank]) {
      TIPS_LOG(ERROR) << "bad gather request: group " << gid << " seq " << seq << " rank " << grank;
      return;
    }
    slot.arrivals[grank] = {msg.head(), std::move(data)};
    slot.present[grank]  = true;
    if (++slot.count == slot.expected) {
      ready = std::move(slot.arrivals);
      gather_slots_.erase({gid, seq});
    }
  }
  if (ready.empty()) return;
  NaiveBuffer out;
  out << static_cast<uint64_t>(ready.size());
  for (auto& a : ready) out << a.second;
  for (auto& a : ready) {
    Status st = RpcServer::Global().SendResponse(a.first, out.data(), out.size());
    if (!st.ok()) TIPS_LOG(WARNING) << "gather response to rank " << a.first.src_rank << ": " << st.ToString();
  }
}

}  // namespace tips
