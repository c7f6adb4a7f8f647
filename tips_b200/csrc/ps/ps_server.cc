#include "ps/ps_server.h"

namespace tips {
namespace ps {

PsServer::PsServer(std::string name, SparseTable* table, std::shared_ptr<PullAccessMethod> pull,
                   std::shared_ptr<PushAccessMethod> push)
    : name_(std::move(name)), table_(table), pull_agent_(table, std::move(pull)), push_agent_(table, std::move(push)) {}

PsServer::~PsServer() { Stop(); }

void PsServer::Start() {
  if (started_) return;
  RpcServer::Global().AddService(pull_service_name(), [this](RpcMessage&& m) { PullTask(std::move(m)); });
  RpcServer::Global().AddService(push_service_name(), [this](RpcMessage&& m) { PushTask(std::move(m)); });
  table_->StartService();
  started_ = true;
}

void PsServer::Stop() {
  if (!started_) return;
  table_->StopService();
  started_ = false;
}

namespace {
// Shared between the shard closures of one request.
struct PullJob {
  RpcMsgHead head;
  PullResponse response;
  std::atomic<int> remaining{0};
};
struct PushJob {
  RpcMsgHead head;
  PushRequest request;
  MessageMeta meta;
  std::atomic<int> remaining{0};
  std::atomic<uint64_t> missing{0};
};
}  // namespace

void PsServer::PullTask(RpcMessage&& msg) {
  auto job  = std::make_shared<PullJob>();
  job->head = msg.head();
  PullRequest req;
  {
    NaiveBuffer rb(msg.payload(), msg.payload_size());
    req.Deserialize(&rb);
  }
  const size_t n = req.keys.size();
  job->response.meta = req.meta;
  job->response.data.resize(n);
  // bucket by local shard, remembering each key's position in the request
  std::vector<std::vector<size_t>> buckets(table_->local_shard_num());
  for (size_t i = 0; i < n; ++i) buckets[table_->ToLocalShard(req.keys[i])].push_back(i);
  int used = 0;
  for (auto& b : buckets) used += b.empty() ? 0 : 1;
  auto finish = [this, job] {
    NaiveBuffer out;
    job->response.Serialize(&out);
    Status st = RpcServer::Global().SendResponse(job->head, out.data(), out.size());
    if (!st.ok()) TIPS_LOG(WARNING) << "pull response failed: " << st.ToString();
  };
  if (used == 0) {
    finish();
    return;
  }
  job->remaining = used;
  auto shared_req = std::make_shared<PullRequest>(std::move(req));
  for (int l = 0; l < table_->local_shard_num(); ++l) {
    if (buckets[l].empty()) continue;
    auto idx = std::make_shared<std::vector<size_t>>(std::move(buckets[l]));
    bool ok  = table_->Submit(l, [this, job, shared_req, idx, finish] {
      for (size_t i : *idx) {
        AnyVec value;
        pull_agent_.GetPullValue(shared_req->keys[i], ToDatatype(shared_req->dtypes[i]), shared_req->lengths[i], &value);
        KeyItem& item = job->response.data[i];  // distinct slots per key: no lock needed
        item.key      = shared_req->keys[i];
        item.dtype    = value.dtype();
        item.value.assign(value.buffer(), value.buffer() + value.num_bytes());
      }
      rows_pulled_ += idx->size();
      if (job->remaining.fetch_sub(1) == 1) finish();
    });
    if (!ok && job->remaining.fetch_sub(1) == 1) finish();
  }
}

void PsServer::PushTask(RpcMessage&& msg) {
  auto job  = std::make_shared<PushJob>();
  job->head = msg.head();
  {
    NaiveBuffer rb(msg.payload(), msg.payload_size());
    job->request.Deserialize(&rb);
  }
  job->meta = job->request.meta;
  std::vector<std::vector<size_t>> buckets(table_->local_shard_num());
  for (size_t i = 0; i < job->request.data.size(); ++i)
    buckets[table_->ToLocalShard(job->request.data[i].key)].push_back(i);
  int used = 0;
  for (auto& b : buckets) used += b.empty() ? 0 : 1;
  auto finish = [job] {
    NaiveBuffer out;
    PushResponse resp;
    resp.meta = job->meta;
    resp.Serialize(&out);
    out << job->missing.load();
    Status st = RpcServer::Global().SendResponse(job->head, out.data(), out.size());
    if (!st.ok()) TIPS_LOG(WARNING) << "push response failed: " << st.ToString();
  };
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
        KeyItem& item = job->request.data[i];
        const size_t es = DatatypeNumBytes(item.dtype);
        AnyVec view(item.dtype, es ? item.value.size() / es : 0, item.value.data());  // borrows the message bytes
        if (!push_agent_.ApplyPushValue(item.key, view)) job->missing++;
      }
      rows_pushed_ += idx->size();
      if (job->remaining.fetch_sub(1) == 1) finish();
    });
    if (!ok && job->remaining.fetch_sub(1) == 1) finish();
  }
}

// --------------------------------------------------------------- client ----

bool PsFuture::Wait(int timeout_ms) {
  std::unique_lock<std::mutex> lock(mu);
  if (timeout_ms < 0) {
    cv.wait(lock, [&] { return pending == 0; });
    return true;
  }
  return cv.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return pending == 0; });
}

PsClient::PsClient(std::string name, SparseTable* table, int client_id)
    : name_(std::move(name)), table_(table), client_id_(client_id) {}

std::shared_ptr<PsFuture> PsClient::Pull(const std::vector<PullRecord>& records, std::function<void()> done) {
  auto fut = std::make_shared<PsFuture>();
  fut->values.resize(records.size());
  const int ns = table_->num_servers();
  std::vector<PullRequest> reqs(ns);
  std::vector<std::vector<size_t>> positions(ns);
  for (size_t i = 0; i < records.size(); ++i) {
    int s = table_->ToServerId(records[i].key);
    reqs[s].keys.push_back(records[i].key);
    reqs[s].dtypes.push_back(ToMessageDataType(records[i].dtype));
    reqs[s].lengths.push_back(records[i].length);
    positions[s].push_back(i);
  }
  int contacted = 0;
  for (int s = 0; s < ns; ++s) contacted += reqs[s].keys.empty() ? 0 : 1;
  fut->pending = contacted;
  if (contacted == 0) {
    if (done) done();
    return fut;
  }
  const std::string service = std::string(kPullServiceName) + "." + name_;
  for (int s = 0; s < ns; ++s) {
    if (reqs[s].keys.empty()) continue;
    reqs[s].meta.client_id  = client_id_;
    reqs[s].meta.message_id = next_message_id_++;
    NaiveBuffer buf;
    reqs[s].Serialize(&buf);
    auto pos = std::make_shared<std::vector<size_t>>(std::move(positions[s]));
    auto cb  = [fut, pos, done](const Status& st, RpcMessage&& m) {
      bool last;
      {
        std::lock_guard<std::mutex> lock(fut->mu);
        if (!st.ok()) {
          fut->status = st;
        } else {
          PullResponse resp;
          NaiveBuffer rb(m.payload(), m.payload_size());
          resp.Deserialize(&rb);
          for (size_t k = 0; k < resp.data.size() && k < pos->size(); ++k) fut->values[(*pos)[k]] = std::move(resp.data[k]);
        }
        last = --fut->pending == 0;
      }
      if (last) {
        fut->cv.notify_all();
        if (done) done();
      }
    };
    Status st = RpcServer::Global().SendRequest(table_->ServerWorldRank(s), service, buf.data(), buf.size(), cb);
    if (!st.ok()) cb(st, RpcMessage());
  }
  return fut;
}

std::shared_ptr<PsFuture> PsClient::Push(const std::vector<KeyItem>& records, std::function<void()> done) {
  auto fut = std::make_shared<PsFuture>();
  const int ns = table_->num_servers();
  std::vector<PushRequest> reqs(ns);
  for (const KeyItem& it : records) reqs[table_->ToServerId(it.key)].data.push_back(it);
  int contacted = 0;
  for (int s = 0; s < ns; ++s) contacted += reqs[s].data.empty() ? 0 : 1;
  fut->pending = contacted;
  if (contacted == 0) {
    if (done) done();
    return fut;
  }
  const std::string service = std::string(kPushServiceName) + "." + name_;
  for (int s = 0; s < ns; ++s) {
    if (reqs[s].data.empty()) continue;
    reqs[s].meta.client_id  = client_id_;
    reqs[s].meta.message_id = next_message_id_++;
    NaiveBuffer buf;
    reqs[s].Serialize(&buf);
    auto cb = [fut, done](const Status& st, RpcMessage&& m) {
      bool last;
      {
        std::lock_guard<std::mutex> lock(fut->mu);
        if (!st.ok()) {
          fut->status = st;
        } else {
          PushResponse resp;
          NaiveBuffer rb(m.payload(), m.payload_size());
          resp.Deserialize(&rb);
          uint64_t missing = 0;
          rb >> missing;
          fut->missing_rows += missing;
        }
        last = --fut->pending == 0;
      }
      if (last) {
        fut->cv.notify_all();
        if (done) done();
      }
    };
    Status st = RpcServer::Global().SendRequest(table_->ServerWorldRank(s), service, buf.data(), buf.size(), cb);
    if (!st.ok()) cb(st, RpcMessage());
  }
  return fut;
}

}  // namespace ps
}  // namespace tips
