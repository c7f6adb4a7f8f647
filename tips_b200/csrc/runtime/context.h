// Process runtime: bootstrap, rank table, rank groups and host-side collectives.
//
// Capability parity with the reference's MPI layer:
//   MpiContext  tips/core/mpi/tips_mpi.h:57-181, tips_mpi.cc:9-82  (singleton, rank/size,
//               IP table of every rank, barrier that does not busy-wait, scalar allreduce,
//               serialised broadcast of arbitrary values)
//   MpiGroup    tips/core/mpi/mpi_group.h:15-96, mpi_group.cc:5-52 (sorted subset of world
//               ranks, group rank <-> world rank, Barrier, AllReduce)
//
// Design: there is no MPI on the target image, and device tensors never cross
// the host, so the job is bootstrapped from the environment that a one
// process-per-GPU launcher provides (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT):
// rank 0 runs a short-lived rendezvous socket where every rank registers
// (ip, port); the table is sent back and the ranks build two TCP meshes, one
// handed to the RpcServer, one kept as the synchronous CPU data plane.  All
// host collectives (barrier, allgather of byte strings, broadcast, scalar
// allreduce) are one RPC service on the group leader; waiters block on a
// condition variable, never spin.
#pragma once

#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "core/common.h"
#include "runtime/rpc.h"

namespace tips {

struct InitOptions {
  int rank{0};
  int size{1};
  std::string master_addr{"127.0.0.1"};
  int master_port{29400};
  int connect_timeout_ms{120000};
  int rpc_listen_threads{1};
};

class Context;

// A subset of world ranks with its own numbering.
class Group {
 public:
  Group() = default;
  // `world_ranks` may be unsorted and contain duplicates; they are normalised.
  Group(uint64_t id, std::vector<int> world_ranks, int my_world_rank);

  uint64_t id() const { return id_; }
  int size() const { return static_cast<int>(ranks_.size()); }
  // Rank of this process inside the group, -1 if it is not a member.
  int rank() const { return my_group_rank_; }
  bool valid() const { return my_group_rank_ >= 0; }
  int ToWorldRank(int group_rank) const { return ranks_.at(group_rank); }
  int ToWorldRank() const { return ranks_.at(my_group_rank_); }
  int ToGroupRank(int world_rank) const;
  bool Contains(int world_rank) const { return ToGroupRank(world_rank) >= 0; }
  int leader() const { return ranks_.front(); }
  const std::vector<int>& ranks() const { return ranks_; }

  // Host collectives restricted to the group (members only).
  Status Barrier(int timeout_ms = -1);
  Status AllgatherBytes(const std::string& mine, std::vector<std::string>* all, int timeout_ms = -1);
  template <typename T>
  Status AllReduceSum(T* value, int timeout_ms = -1);

 private:
  friend class Context;
  uint64_t id_{0};
  std::vector<int> ranks_;
  int my_group_rank_{-1};
  uint64_t seq_{0};
  std::mutex seq_mu_;
};

class Context {
 public:
  static Context& Global();

  // Reads RANK / WORLD_SIZE / MASTER_ADDR / TIPS_MASTER_PORT (default
  // MASTER_PORT + 1000) from the environment.
  static InitOptions OptionsFromEnv();

  Status Initialize(const InitOptions& opts);
  // Orderly shutdown: barrier, mark the RPC server quiescing, barrier, close.
  void Finalize();
  bool initialized() const { return initialized_; }

  int rank() const { return rank_; }
  int size() const { return size_; }
  int local_rank() const { return local_rank_; }
  int local_size() const { return local_size_; }
  const std::string& ip(int r) const { return ips_.at(r); }
  const std::vector<std::string>& ip_table() const { return ips_; }

  Group* world() { return world_.get(); }
  // Collective over the world: every rank calls it with the same list, in
  // the same order relative to other NewGroup calls.
  Group* NewGroup(const std::vector<int>& world_ranks);
  // The group created with that id by NewGroup (0 = the world), or null.
  Group* FindGroup(uint64_t id);

  // Host collectives over the world group.
  Status Barrier(int timeout_ms = -1) { return world_->Barrier(timeout_ms); }
  Status AllgatherBytes(const std::string& mine, std::vector<std::string>* all, int timeout_ms = -1) {
    return world_->AllgatherBytes(mine, all, timeout_ms);
  }
  Status BroadcastBytes(std::string* inout, int root, int timeout_ms = -1);

  // CPU data plane: connected socket to `peer` and the mutex that serialises
  // its users (one collective at a time).
  int data_fd(int peer) const { return data_fds_.at(peer); }
  std::mutex& data_mu() { return data_mu_; }
  int data_timeout_ms() const { return data_timeout_ms_; }

  int default_timeout_ms() const { return host_timeout_ms_; }

 private:
  friend class Group;
  Context() = default;
  Status GroupGather(Group* g, const std::string& mine, std::vector<std::string>* all, int timeout_ms);
  void HandleGatherRequest(RpcMessage&& msg);

  bool initialized_{false};
  int rank_{0};
  int size_{1};
  int local_rank_{0};
  int local_size_{1};
  std::vector<std::string> ips_;
  std::vector<int> data_fds_;
  std::mutex data_mu_;
  int data_timeout_ms_{300000};
  int host_timeout_ms_{300000};
  std::unique_ptr<Group> world_;
  std::vector<std::unique_ptr<Group>> groups_;
  std::mutex groups_mu_;  // guards groups_ and next_group_id_
  uint64_t next_group_id_{1};

  // Leader-side state of the gather service: (group id, seq) -> arrivals.
  struct GatherSlot {
    int expected{0};
    std::vector<std::pair<RpcMsgHead, std::string>> arrivals;  // indexed by group rank
    std::vector<bool> present;
    int count{0};
  };
  std::mutex gather_mu_;
  std::map<std::pair<uint64_t, uint64_t>, GatherSlot> gather_slots_;
};

template <typename T>
Status Group::AllReduceSum(T* value, int timeout_ms) {
  std::string mine(reinterpret_cast<const char*>(value), sizeof(T));
  std::vector<std::string> all;
  Status st = AllgatherBytes(mine, &all, timeout_ms);
  if (!st.ok()) return st;
  T acc = T();
  for (auto& s : all) {
    T v;
    memcpy(&v, s.data(), sizeof(T));
    acc += v;
  }
  *value = acc;
  return Status::OK();
}

}  // namespace tips
