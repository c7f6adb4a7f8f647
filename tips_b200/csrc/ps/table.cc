#include "ps/table.h"

#include <algorithm>
#include <fstream>
#include <sstream>

#include "core/naive_buffer.h"

namespace tips {
namespace ps {

// ---------------------------------------------------------------- Route ----

Route& Route::Global() {
  static Route* r = new Route;
  return *r;
}

void Route::RegisterNode(NodeKind kind, int world_rank) {
  TIPS_CHECK(!initialized_) << "Route::RegisterNode after Initialize";
  auto& v = ranks_[static_cast<int>(kind)];
  if (std::find(v.begin(), v.end(), world_rank) == v.end()) v.push_back(world_rank);
}

void Route::Initialize() {
  TIPS_CHECK(!initialized_);
  for (int k = 0; k < 2; ++k) {
    std::sort(ranks_[k].begin(), ranks_[k].end());
    groups_[k] = ranks_[k].empty() ? nullptr : Context::Global().NewGroup(ranks_[k]);
  }
  initialized_ = true;
}

void Route::Finalize() {
  for (int k = 0; k < 2; ++k) {
    ranks_[k].clear();
    groups_[k] = nullptr;
  }
  initialized_ = false;
}

bool Route::IsInGroup(NodeKind kind, int world_rank) const {
  const auto& v = ranks_[static_cast<int>(kind)];
  return std::find(v.begin(), v.end(), world_rank) != v.end();
}

// ---------------------------------------------------------------- Table ----

Table::Table(std::vector<int> servers, int my_world_rank, int local_shards)
    : servers_(std::move(servers)), local_shards_(local_shards) {
  TIPS_CHECK(!servers_.empty()) << "a table needs at least one server";
  TIPS_CHECK_GE(local_shards_, 1);
  std::sort(servers_.begin(), servers_.end());
  servers_.erase(std::unique(servers_.begin(), servers_.end()), servers_.end());
  auto it = std::find(servers_.begin(), servers_.end(), my_world_rank);
  my_server_index_ = it == servers_.end() ? -1 : static_cast<int>(it - servers_.begin());
}

Table::~Table() { StopService(); }

void Table::StartService() {
  if (running_ || !is_server()) return;
  channels_.clear();
  for (int l = 0; l < local_shards_; ++l) channels_.emplace_back(new Channel<std::function<void()>>());
  for (int l = 0; l < local_shards_; ++l) {
    Channel<std::function<void()>>* ch = channels_[l].get();
    threads_.emplace_back([ch] {
      std::function<void()> task;
      while (ch->Read(&task)) {
        try {
          task();
        } catch (const std::exception& e) {
          TIPS_LOG(ERROR) << "table shard task threw: " << e.what();
        }
      }
    });
  }
  running_ = true;
}

void Table::StopService() {
  if (!running_) return;
  for (auto& ch : channels_) ch->Close();
  for (auto& t : threads_)
    if (t.joinable()) t.join();
  threads_.clear();
  channels_.clear();
  running_ = false;
}

bool Table::Submit(int local, std::function<void()> task) {
  if (!running_ || local < 0 || local >= local_shards_) return false;
  return channels_[local]->WriteMove(std::move(task));
}

// ----------------------------------------------------- SparseTableShard ----

AnyVec* SparseTableShard::Find(uint64_t key) {
  RWLockReadGuard guard(lock_);
  auto it = rows_.find(key);
  return it == rows_.end() ? nullptr : &it->second;
}

bool SparseTableShard::Find(uint64_t key, AnyVec* shadow) {
  RWLockReadGuard guard(lock_);
  auto it = rows_.find(key);
  if (it == rows_.end()) return false;
  shadow->ShadowCopyFrom(it->second);
  return true;
}

void SparseTableShard::Assign(uint64_t key, const AnyVec& value) {
  RWLockWriteGuard guard(lock_);
  rows_[key].CopyFrom(value);
}

AnyVec* SparseTableShard::FindOrCreate(uint64_t key, bool* created) {
  {
    RWLockReadGuard guard(lock_);
    auto it = rows_.find(key);
    if (it != rows_.end()) {
      *created = false;
      return &it->second;
    }
  }
  RWLockWriteGuard guard(lock_);
  auto ins = rows_.emplace(key, AnyVec());
  *created = ins.second;
  return &ins.first->second;
}

size_t SparseTableShard::size() const {
  RWLockReadGuard guard(lock_);
  return rows_.size();
}

void SparseTableShard::Dump(std::ostream& os) const {
  RWLockReadGuard guard(lock_);
  for (auto& kv : rows_) os << kv.first << "\t" << kv.second << std::endl;
}

void SparseTableShard::Clear() {
  RWLockWriteGuard guard(lock_);
  rows_.clear();
}

// ---------------------------------------------------------- SparseTable ----

SparseTable::SparseTable(std::vector<int> servers, int my_world_rank, int local_shards)
    : Table(std::move(servers), my_world_rank, local_shards) {
  for (int l = 0; l < local_shard_num(); ++l) shards_.emplace_back(new SparseTableShard);
}

AnyVec* SparseTable::Find(uint64_t key) { return local_shard(ToLocalShard(key)).Find(key); }

void SparseTable::Assign(uint64_t key, const AnyVec& value) { local_shard(ToLocalShard(key)).Assign(key, value); }

AnyVec* SparseTable::FindOrCreate(uint64_t key, bool* created) {
  return local_shard(ToLocalShard(key)).FindOrCreate(key, created);
}

size_t SparseTable::size() const {
  size_t n = 0;
  for (auto& s : shards_) n += s->size();
  return n;
}

Status SparseTable::WriteToFile(const std::string& path) const {
  std::ofstream file(path.c_str(), std::ios::out);
  if (!file) return Status(kInvalidArgument, "cannot open " + path);
  file.precision(9);
  for (auto& s : shards_) s->Dump(file);
  return Status::OK();
}

Status SparseTable::LoadFromFile(const std::string& path, Datatype dtype, bool only_owned) {
  std::ifstream file(path.c_str());
  if (!file) return Status(kInvalidArgument, "cannot open " + path);
  std::string line;
  while (std::getline(file, line)) {
    if (line.empty()) continue;
    std::istringstream ss(line);
    uint64_t key;
    std::string tag;
    ss >> key >> tag;
    if (tag != "Vec:") return Status(kInvalidArgument, "bad line in " + path + ": " + line);
    std::vector<double> vals;
    double v;
    while (ss >> v) vals.push_back(v);
    if (only_owned && (!is_server() || ToServerId(key) != server_index())) continue;
    AnyVec row(dtype, vals.size());
    for (size_t i = 0; i < vals.size(); ++i) row.SetFromDouble(i, vals[i]);
    Assign(key, row);
  }
  return Status::OK();
}

Status SparseTable::SaveBinary(const std::string& path) const {
  NaiveBuffer buf;
  buf << static_cast<uint64_t>(size());
  for (auto& s : shards_) {
    s->ForEach([&](uint64_t key, const AnyVec& row) {
      buf << key << static_cast<int32_t>(row.dtype()) << static_cast<uint64_t>(row.size());
      buf.WriteRaw(row.buffer(), row.num_bytes());
    });
  }
  try {
    buf.SaveToFile(path);
  } catch (const std::exception& e) {
    return Status(kInvalidArgument, e.what());
  }
  return Status::OK();
}

Status SparseTable::LoadBinary(const std::string& path, bool only_owned) {
  try {
    NaiveBuffer buf;
    buf.LoadFromFile(path);
    uint64_t n = 0;
    buf >> n;
    for (uint64_t i = 0; i < n; ++i) {
      uint64_t key = 0, len = 0;
      int32_t dt   = 0;
      buf >> key >> dt >> len;
      AnyVec row(static_cast<Datatype>(dt), len);
      buf.ReadRaw(row.buffer(), row.num_bytes());
      if (only_owned && (!is_server() || ToServerId(key) != server_index())) continue;
      Assign(key, row);
    }
  } catch (const std::exception& e) {
    return Status(kInvalidArgument, e.what());
  }
  return Status::OK();
}

std::string SparseTable::ToString() const {
  std::ostringstream ss;
  ss << "SparseTable(servers=" << num_servers() << ", local_shards=" << local_shard_num() << ", rows=" << size() << ")";
  return ss.str();
}

// ----------------------------------------------------------- DenseTable ----

template <typename T>
Status DenseTable<T>::Save(const std::string& path) const {
  NaiveBuffer buf;
  buf << static_cast<uint64_t>(size_) << static_cast<int32_t>(DatatypeOf<T>::value);
  buf << static_cast<uint64_t>(data_.size());
  for (int l = 0; l < static_cast<int>(data_.size()); ++l) {
    int g = ToGlobalShard(server_index(), l);
    buf << static_cast<uint64_t>(boundaries_[g]) << data_[l];
  }
  try {
    buf.SaveToFile(path);
  } catch (const std::exception& e) {
    return Status(kInvalidArgument, e.what());
  }
  return Status::OK();
}

template <typename T>
Status DenseTable<T>::Load(const std::string& path) {
  try {
    NaiveBuffer buf;
    buf.LoadFromFile(path);
    uint64_t total = 0, nshards = 0;
    int32_t dt = 0;
    buf >> total >> dt >> nshards;
    if (static_cast<Datatype>(dt) != DatatypeOf<T>::value) return Status(kInvalidArgument, "dtype mismatch in " + path);
    if (total != size_) Resize(total);
    for (uint64_t s = 0; s < nshards; ++s) {
      uint64_t begin = 0;
      std::vector<T> vals;
      buf >> begin >> vals;
      for (size_t i = 0; i < vals.size(); ++i) {
        T* slot = Lookup(begin + i);
        if (slot) *slot = vals[i];
      }
    }
  } catch (const std::exception& e) {
    return Status(kInvalidArgument, e.what());
  }
  return Status::OK();
}

template class DenseTable<float>;
template class DenseTable<double>;
template class DenseTable<int32_t>;
template class DenseTable<int64_t>;

}  // namespace ps
}  // namespace tips
