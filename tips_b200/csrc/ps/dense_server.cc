#include "ps/dense_server.h"

#include <cmath>
#include <cstring>

namespace tips {
namespace ps {

void DensePushAccess::Apply(float* w, float* state, const float* g, size_t n) const {
  switch (rule_) {
    case DenseRule::kSgd:
      for (size_t i = 0; i < n; ++i) w[i] -= static_cast<float>(lr_) * g[i];
      break;
    case DenseRule::kAdagrad:
      for (size_t i = 0; i < n; ++i) {
        state[i] += g[i] * g[i];
        w[i] -= static_cast<float>(lr_ * g[i] / (std::sqrt(static_cast<double>(state[i])) + eps_));
      }
      break;
    case DenseRule::kLiteralReference:
      for (size_t i = 0; i < n; ++i) w[i] = static_cast<float>(lr_) * g[i];
      break;
  }
}

void DenseRequest::Serialize(NaiveBuffer* b) const {
  *b << meta.client_id << meta.message_id << op << static_cast<uint64_t>(ranges.size());
  for (const DenseRange& r : ranges) *b << r.begin << r.end << r.shard;
  *b << values;
}

void DenseRequest::Deserialize(NaiveBuffer* b) {
  uint64_t n = 0;
  *b >> meta.client_id >> meta.message_id >> op >> n;
  ranges.resize(n);
  for (DenseRange& r : ranges) *b >> r.begin >> r.end >> r.shard;
  *b >> values;
}

DensePsServer::DensePsServer(std::string name, DenseTable<float>* table, DenseRule rule, double lr, double eps)
    : name_(std::move(name)), table_(table), access_(rule, lr, eps) {}

DensePsServer::~DensePsServer() { Stop(); }

void DensePsServer::Start() {
  if (started_) return;
  state_.assign(table_->local_shard_num(), {});
  RpcServer::Global().AddService(pull_service_name(), [this](RpcMessage&& m) { PullTask(std::move(m)); });
  RpcServer::Global().AddService(push_service_name(), [this](RpcMessage&& m) { PushTask(std::move(m)); });
  table_->StartService();
  started_ = true;
}

void DensePsServer::Stop() {
  if (!started_) return;
  table_->StopService();
  started_ = false;
}

namespace {

struct DenseJob {
  RpcMsgHead head;
  DenseRequest request;
  std::vector<float> out;          // pull: the ranges' values, concatenated in request order
  std::vector<size_t> offsets;     // start of every range inside `out` / `request.values`
  std::atomic<int> remaining{0};
  std::atomic<uint64_t> rejected{0};
};

// Offsets of the ranges in the concatenated value vector, and the ranges grouped by local shard.
std::vector<std::vector<size_t>> Bucket(const DenseTable<float>& table, DenseJob* job) {
  std::vector<std::vector<size_t>> buckets(table.local_shard_num());
  size_t off = 0;
  job->offsets.resize(job->request.ranges.size());
  for (size_t i = 0; i < job->request.ranges.size(); ++i) {
    const DenseRange& r = job->request.ranges[i];
    job->offsets[i] = off;
    off += r.end - r.begin;
    const bool mine = table.is_server() && r.shard >= 0 && r.shard < table.shard_num() &&
                      r.shard % table.num_servers() == table.server_index() && r.begin >= table.shard_begin(r.shard) &&
                      r.end <= table.shard_end(r.shard) && r.begin <= r.end;
    if (!mine) {
      job->rejected++;
      continue;
    }
    buckets[r.shard / table.num_servers()].push_back(i);
  }
  return buckets;
}

}  // namespace

void DensePsServer::PullTask(RpcMessage&& msg) {
  auto job  = std::make_shared<DenseJob>();
  job->head = msg.head();
  {
    NaiveBuffer rb(msg.payload(), msg.payload_size());
    job->request.Deserialize(&rb);
  }
  auto buckets = Bucket(*table_, job.get());
  size_t total = 0;
  for (const DenseRange& r : job->request.ranges) total += r.end - r.begin;
  job->out.assign(total, 0.f);
  auto finish = [job] {
    NaiveBuffer out;
    out << job->request.meta.client_id << job->request.meta.message_id << job->rejected.load() << job->out;
    Status st = RpcServer::Global().SendResponse(job->head, out.data(), out.size());
    if (!st.ok()) TIPS_LOG(WARNING) << "dense pull response failed: " << st.ToString();
  };
  int used = 0;
  for (auto& b : buckets) used += b.empty() ? 0 : 1;
  if (used == 0) {
    finish();
    return;
  }
  job->remaining = used;
  for (int l = 0; l < table_->local_shard_num(); ++l) {
    if (buckets[l].empty()) continue;
    auto idx = std::make_shared<std::vector<size_t>>(std::move(buckets[l]));
    bool ok  = table_->Submit(l, [this, job, idx, finish] {
      for (size_t i : *idx) {
        const DenseRange& r = job->request.ranges[i];
        if (r.end == r.begin) continue;
        const float* src = table_->Lookup(r.begin);
        memcpy(job->out.data() + job->offsets[i], src, (r.end - r.begin) * sizeof(float));
        pulled_ += r.end - r.begin;
      }
      if (job->remaining.fetch_sub(1) == 1) finish();
    });
    if (!ok && job->remaining.fetch_sub(1) == 1) finish();
  }
}

void DensePsServer::PushTask(RpcMessage&& msg) {
  auto job  = std::make_shared<DenseJob>();
  job->head = msg.head();
  {
    NaiveBuffer rb(msg.payload(), msg.payload_size());
    job->request.Deserialize(&rb);
  }
  auto buckets = Bucket(*table_, job.get());
  size_t total = 0;
  for (const DenseRange& r : job->request.ranges) total += r.end - r.begin;
  if (total != job->request.values.size()) {
    job->rejected += job->request.ranges.size();
    for (auto& b : buckets) b.clear();
  }
  auto finish = [job] {
    NaiveBuffer out;
    out << job->request.meta.client_id << job->request.meta.message_id << job->rejected.load();
    Status st = RpcServer::Global().SendResponse(job->head, out.data(), out.size());
    if (!st.ok()) TIPS_LOG(WARNING) << "dense push response failed: " << st.ToString();
  };
  int used = 0;
  for (auto& b : buckets) used += b.empty() ? 0 : 1;
  if (used == 0) {
    finish();
    return;
  }
  job->remaining = used;
  for (int l = 0; l < table_->local_shard_num(); ++l) {
    if (buckets[l].empty()) continue;
    auto idx = std::make_shared<std::vector<size_t>>(std::move(buckets[l]));
    bool ok  = table_->Submit(l, [this, job, idx, finish, l] {
      const int g          = table_->ToGlobalShard(table_->server_index(), l);
      const size_t sbegin  = table_->shard_begin(g);
      std::vector<float>& st = state_[l];
      if (access_.needs_state() && st.size() != table_->shard_end(g) - sbegin) st.assign(table_->shard_end(g) - sbegin, 0.f);
      for (size_t i : *idx) {
        const DenseRange& r = job->request.ranges[i];
        if (r.end == r.begin) continue;
        float* w       = table_->Lookup(r.begin);
        const float* v = job->request.values.data() + job->offsets[i];
        const size_t n = r.end - r.begin;
        if (job->request.op == static_cast<int32_t>(DensePushOp::kAssign))
          memcpy(w, v, n * sizeof(float));
        else
          access_.Apply(w, access_.needs_state() ? st.data() + (r.begin - sbegin) : nullptr, v, n);
        pushed_ += n;
      }
      if (job->remaining.fetch_sub(1) == 1) finish();
    });
    if (!ok && job->remaining.fetch_sub(1) == 1) finish();
  }
}

// --------------------------------------------------------------- client ----

DensePsClient::DensePsClient(std::string name, DenseTable<float>* table, int client_id)
    : name_(std::move(name)), table_(table), client_id_(client_id) {}

std::vector<std::vector<DenseRange>> DensePsClient::Split(uint64_t begin, uint64_t end) const {
  std::vector<std::vector<DenseRange>> per_server(table_->num_servers());
  uint64_t at = begin;
  while (at < end) {
    const int g        = table_->ShardOf(at);
    const uint64_t hi  = std::min<uint64_t>(end, table_->shard_end(g));
    DenseRange r;
    r.begin = at;
    r.end   = hi;
    r.shard = g;
    per_server[g % table_->num_servers()].push_back(r);
    at = hi;
  }
  return per_server;
}

std::shared_ptr<PsFuture> DensePsClient::Pull(uint64_t begin, uint64_t end, float* out) {
  auto fut = std::make_shared<PsFuture>();
  if (end > table_->size() || begin > end) {
    fut->status = Status(kInvalidArgument, "dense pull: range outside the table");
    return fut;
  }
  auto per_server = Split(begin, end);
  int contacted   = 0;
  for (auto& v : per_server) contacted += v.empty() ? 0 : 1;
  fut->pending = contacted;
  for (int s = 0; s < table_->num_servers(); ++s) {
    if (per_server[s].empty()) continue;
    DenseRequest req;
    req.meta.client_id  = client_id_;
    req.meta.message_id = next_message_id_++;
    req.ranges          = per_server[s];
    NaiveBuffer buf;
    req.Serialize(&buf);
    auto ranges = std::make_shared<std::vector<DenseRange>>(std::move(per_server[s]));
    auto cb     = [fut, ranges, out, begin](const Status& st, RpcMessage&& m) {
      bool last;
      {
        std::lock_guard<std::mutex> lock(fut->mu);
        if (!st.ok()) {
          fut->status = st;
        } else {
          NaiveBuffer rb(m.payload(), m.payload_size());
          int32_t cid = 0;
          uint64_t mid = 0, rejected = 0;
          std::vector<float> vals;
          rb >> cid >> mid >> rejected >> vals;
          size_t off = 0;
          for (const DenseRange& r : *ranges) {
            const size_t n = r.end - r.begin;
            if (off + n <= vals.size()) memcpy(out + (r.begin - begin), vals.data() + off, n * sizeof(float));
            off += n;
          }
          if (rejected || off != vals.size())
            fut->status = Status(kPrecondition, "dense pull: the server does not own a requested range");
        }
        last = --fut->pending == 0;
      }
      if (last) fut->cv.notify_all();
    };
    Status st = RpcServer::Global().SendRequest(table_->ServerWorldRank(s), "dense_pull_service." + name_, buf.data(),
                                                buf.size(), cb);
    if (!st.ok()) cb(st, RpcMessage());
  }
  return fut;
}

std::shared_ptr<PsFuture> DensePsClient::Push(uint64_t begin, uint64_t end, const float* values, DensePushOp op) {
  auto fut = std::make_shared<PsFuture>();
  if (end > table_->size() || begin > end) {
    fut->status = Status(kInvalidArgument, "dense push: range outside the table");
    return fut;
  }
  auto per_server = Split(begin, end);
  int contacted   = 0;
  for (auto& v : per_server) contacted += v.empty() ? 0 : 1;
  fut->pending = contacted;
  for (int s = 0; s < table_->num_servers(); ++s) {
    if (per_server[s].empty()) continue;
    DenseRequest req;
    req.meta.client_id  = client_id_;
    req.meta.message_id = next_message_id_++;
    req.op              = static_cast<int32_t>(op);
    req.ranges          = std::move(per_server[s]);
    for (const DenseRange& r : req.ranges)
      req.values.insert(req.values.end(), values + (r.begin - begin), values + (r.end - begin));
    NaiveBuffer buf;
    req.Serialize(&buf);
    auto cb = [fut](const Status& st, RpcMessage&& m) {
      bool last;
      {
        std::lock_guard<std::mutex> lock(fut->mu);
        if (!st.ok()) {
          fut->status = st;
        } else {
          NaiveBuffer rb(m.payload(), m.payload_size());
          int32_t cid = 0;
          uint64_t mid = 0, rejected = 0;
          rb >> cid >> mid >> rejected;
          fut->missing_rows += rejected;
        }
        last = --fut->pending == 0;
      }
      if (last) fut->cv.notify_all();
    };
    Status st = RpcServer::Global().SendRequest(table_->ServerWorldRank(s), "dense_push_service." + name_, buf.data(),
                                                buf.size(), cb);
    if (!st.ok()) cb(st, RpcMessage());
  }
  return fut;
}

}  // namespace ps
}  // namespace tips
