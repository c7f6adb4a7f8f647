// Host parameter-server tables: node roles, the sharded table base with one
// executor thread per local shard, the sparse (hash-map) table and the dense
// (range-partitioned) table.
//
// Capability parity with the reference:
//   Route            tips/core/ps/route.h:22-134   (PS_WORKER / PS_SERVER rank sets -> groups)
//   Table            tips/core/ps/table.h:10-36, table.cc:6-73 (shard maps, one Channel<function>
//                    and one thread per local shard, so updates to a shard are serialised)
//   SparseTableShard tips/core/ps/sparse_table.h:38-104 (hash map + RW lock, Find/Assign, text dump)
//   SparseTable      tips/core/ps/sparse_table.h:112-185
//   DenseTable       tips/core/ps/dense_table.h:49-131 (declared in the reference, disabled in its build)
//
// Placement (one rule for pull and push, valid for any number of servers; the
// reference indexes local arrays with global shard ids and only works with one
// server, sparse_table.h:139-142,164-165):
//   server      = hash(key) mod n_servers
//   local shard = (hash(key) div n_servers) mod local_shards
#pragma once

#include <condition_variable>
#include <functional>
#include <mutex>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/channel.h"
#include "core/common.h"
#include "core/datatype.h"
#include "core/threads.h"
#include "runtime/context.h"

namespace tips {
namespace ps {

enum class NodeKind : int { kWorker = 0, kServer = 1 };

class Route {
 public:
  static Route& Global();
  void RegisterNode(NodeKind kind, int world_rank);
  // Builds the groups; every rank calls it after the same RegisterNode calls.
  void Initialize();
  void Finalize();
  bool initialized() const { return initialized_; }
  Group* GetGroup(NodeKind kind) { return groups_[static_cast<int>(kind)]; }
  bool IsInGroup(NodeKind kind, int world_rank) const;
  const std::vector<int>& ranks(NodeKind kind) const { return ranks_[static_cast<int>(kind)]; }

 private:
  std::vector<int> ranks_[2];
  Group* groups_[2]{nullptr, nullptr};
  bool initialized_{false};
};

class Table {
 public:
  // `servers` = sorted world ranks that hold shards; `local_shards` per server.
  Table(std::vector<int> servers, int my_world_rank, int local_shards = 1);
  virtual ~Table();

  int num_servers() const { return static_cast<int>(servers_.size()); }
  int local_shard_num() const { return local_shards_; }
  int shard_num() const { return num_servers() * local_shards_; }
  bool is_server() const { return my_server_index_ >= 0; }
  int server_index() const { return my_server_index_; }
  int ServerWorldRank(int server_index) const { return servers_.at(server_index); }

  int ToServerId(uint64_t key) const { return static_cast<int>(HashKey(key) % static_cast<uint64_t>(num_servers())); }
  int ToLocalShard(uint64_t key) const {
    return static_cast<int>((HashKey(key) / static_cast<uint64_t>(num_servers())) % static_cast<uint64_t>(local_shards_));
  }
  // global shard id <-> (server, local shard)
  int ToGlobalShard(int server, int local) const { return local * num_servers() + server; }

  // Starts / stops the per-shard executor threads (servers only).
  void StartService();
  void StopService();
  bool running() const { return running_; }
  // Runs `task` on the thread that owns local shard `local`. False once stopped.
  bool Submit(int local, std::function<void()> task);

 private:
  std::vector<int> servers_;
  int my_server_index_{-1};
  int local_shards_{1};
  bool running_{false};
  std::vector<std::unique_ptr<Channel<std::function<void()>>>> channels_;
  std::vector<std::thread> threads_;
};

class SparseTableShard {
 public:
  // Pointer to the stored row or nullptr. The pointer stays valid until the row is erased.
  AnyVec* Find(uint64_t key);
  bool Find(uint64_t key, AnyVec* shadow);   // shadow copy of the row
  void Assign(uint64_t key, const AnyVec& value);  // deep copy
  // The stored row, made empty first if the key is new (`created`); the caller fills a new row in place.
  AnyVec* FindOrCreate(uint64_t key, bool* created);
  size_t size() const;
  void Dump(std::ostream& os) const;          // "<key>\t<Vec text>\n" per row
  template <typename F>
  void ForEach(F&& f) const {
    RWLockReadGuard guard(lock_);
    for (auto& kv : rows_) f(kv.first, kv.second);
  }
  void Clear();

 private:
  mutable RWLock lock_;
  std::unordered_map<uint64_t, AnyVec> rows_;
};

class SparseTable : public Table {
 public:
  SparseTable(std::vector<int> servers, int my_world_rank, int local_shards = 1);

  SparseTableShard& local_shard(int local) { return *shards_.at(local); }
  // Local lookups (the key must belong to this server).
  AnyVec* Find(uint64_t key);
  void Assign(uint64_t key, const AnyVec& value);
  AnyVec* FindOrCreate(uint64_t key, bool* created);
  size_t size() const;

  // Text dump of the local shards, one "<key>\tVec:\t<e> <e> ... \n" line per row
  // (the reference's WriteToFile format), and its loader.
  Status WriteToFile(const std::string& path) const;
  Status LoadFromFile(const std::string& path, Datatype dtype, bool only_owned = true);
  // Binary dump: u64 n_rows, then per row u64 key, i32 dtype, u64 len, raw values.
  Status SaveBinary(const std::string& path) const;
  Status LoadBinary(const std::string& path, bool only_owned = true);
  std::string ToString() const;

 private:
  std::vector<std::unique_ptr<SparseTableShard>> shards_;
};

// Dense vector of `size` elements split into contiguous ranges, one per global shard.
template <typename T>
class DenseTable : public Table {
 public:
  DenseTable(std::vector<int> servers, int my_world_rank, int local_shards = 1)
      : Table(std::move(servers), my_world_rank, local_shards) {}

  void Resize(size_t size) {
    size_ = size;
    const int n = shard_num();
    boundaries_.resize(n + 1);
    for (int i = 0; i <= n; ++i) boundaries_[i] = size * i / n;
    data_.assign(local_shard_num(), {});
    if (is_server())
      for (int l = 0; l < local_shard_num(); ++l) {
        int g = ToGlobalShard(server_index(), l);
        data_[l].assign(boundaries_[g + 1] - boundaries_[g], T());
      }
  }
  size_t size() const { return size_; }
  // Global shard that owns element `index`.
  int ShardOf(size_t index) const {
    int lo = 0, hi = shard_num();
    while (hi - lo > 1) {
      int mid = (lo + hi) / 2;
      (boundaries_[mid] <= index ? lo : hi) = mid;
    }
    return lo;
  }
  size_t shard_begin(int global_shard) const { return boundaries_[global_shard]; }
  size_t shard_end(int global_shard) const { return boundaries_[global_shard + 1]; }
  // Pointer to a locally stored element or nullptr.
  T* Lookup(size_t index) {
    int g = ShardOf(index);
    if (!is_server() || g % num_servers() != server_index()) return nullptr;
    return &data_[g / num_servers()][index - boundaries_[g]];
  }
  // Applies f(index, value&) to every local element.  While the table's service runs, every local shard is
  // visited on its own shard thread (in parallel with the others, serialised with the pushes to that shard) and
  // the call returns when all are done; otherwise the shards are visited one after the other on the caller.
  void ForEach(const std::function<void(size_t, T&)>& f) {
    auto visit = [this, &f](int l) {
      int g = ToGlobalShard(server_index(), l);
      for (size_t i = 0; i < data_[l].size(); ++i) f(boundaries_[g] + i, data_[l][i]);
    };
    if (!is_server()) return;
    if (!running()) {
      for (int l = 0; l < local_shard_num(); ++l) visit(l);
      return;
    }
    std::mutex mu;
    std::condition_variable cv;
    int pending = local_shard_num();
    for (int l = 0; l < local_shard_num(); ++l) {
      bool ok = Submit(l, [&, l] {
        visit(l);
        std::lock_guard<std::mutex> lock(mu);
        if (--pending == 0) cv.notify_all();
      });
      if (!ok) {
        visit(l);
        std::lock_guard<std::mutex> lock(mu);
        --pending;
      }
    }
    std::unique_lock<std::mutex> lock(mu);
    cv.wait(lock, [&] { return pending == 0; });
  }
  Status Save(const std::string& path) const;
  Status Load(const std::string& path);

 private:
  size_t size_{0};
  std::vector<size_t> boundaries_;
  std::vector<std::vector<T>> data_;
};

}  // namespace ps
}  // namespace tips
