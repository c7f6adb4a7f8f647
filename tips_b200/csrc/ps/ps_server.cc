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
  RpcServer::Global().AddService(std::string(kPackedPullServiceName) + "." + name_,
                                 [this](RpcMessage&& m) { PackedPullTask(std::move(m)); });
  RpcServer::Global().AddService(std::string(kPackedPushServiceName) + "." + name_,
                                 [this](RpcMessage&& m) { PackedPushTask(std::move(m)); });
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

namespace {
struct PackedPullJob {
  RpcMsgHead head;
  PackedHeader req;
  NaiveBuffer out;          // the whole response; rows are written in place
  char* rows{nullptr};      // start of the row block inside `out`
  uint64_t* bad_slot{nullptr};
  std::atomic<int> remaining{0};
  std::atomic<uint64_t> bad{0};
};
struct PackedPushJob {
  RpcMsgHead head;
  RpcMessage msg;           // keeps the payload alive: gradients are applied from it
  PackedHeader req;
  const char* rows{nullptr};
  std::atomic<int> remaining{0};
  std::atomic<uint64_t> missing{0};
};
}  // namespace

void PsServer::PackedPullTask(RpcMessage&& msg) {
  auto job  = std::make_shared<PackedPullJob>();
  job->head = msg.head();
  {
    NaiveBuffer rb(msg.payload(), msg.payload_size());
    job->req.Deserialize(&rb);
  }
  const size_t n = job->req.keys.size(), row_bytes = job->req.row_bytes();
  job->out << job->req.meta.client_id << job->req.meta.message_id << static_cast<uint64_t>(n);
  const size_t bad_at = job->out.cursor_pos();
  job->out << static_cast<uint64_t>(0);
  const size_t rows_at = job->out.cursor_pos();
  job->out.Require(n * row_bytes);
  job->out.Consume(n * row_bytes);
  job->rows     = static_cast<char*>(job->out.data()) + rows_at;
  job->bad_slot = reinterpret_cast<uint64_t*>(static_cast<char*>(job->out.data()) + bad_at);
  auto finish = [job] {
    const uint64_t bad = job->bad.load();
    memcpy(job->bad_slot, &bad, sizeof(bad));
    Status st = RpcServer::Global().SendResponse(job->head, job->out.data(), job->out.size());
    if (!st.ok()) TIPS_LOG(WARNING) << "pull response failed: " << st.ToString();
  };
  std::vector<std::vector<size_t>> buckets(table_->local_shard_num());
  for (size_t i = 0; i < n; ++i) buckets[table_->ToLocalShard(job->req.keys[i])].push_back(i);
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
    bool ok  = table_->Submit(l, [this, job, idx, finish, row_bytes] {
      const Datatype dtype = job->req.dtype;
      const size_t length  = job->req.length;
      for (size_t i : *idx) {
        AnyVec value;  // borrows the stored row
        pull_agent_.GetPullValue(job->req.keys[i], dtype, length, &value);
        char* slot = job->rows + i * row_bytes;
        if (value.dtype() == dtype && value.size() == length) {
          memcpy(slot, value.buffer(), row_bytes);
        } else {
          memset(slot, 0, row_bytes);
          job->bad++;
        }
      }
      rows_pulled_ += idx->size();
      if (job->remaining.fetch_sub(1) == 1) finish();
    });
    if (!ok && job->remaining.fetch_sub(1) == 1) finish();
  }
}

void PsServer::PackedPushTask(RpcMessage&& msg) {
  auto job  = std::make_shared<PackedPushJob>();
  job->head = msg.head();
  job->msg  = std::move(msg);
  const size_t rows_at = PackedHeader::EncodedSize(job->msg.payload(), job->msg.payload_size());
  if (rows_at == 0) {
    TIPS_LOG(ERROR) << "malformed packed push request";
    return;
  }
  {
    NaiveBuffer rb(job->msg.payload(), rows_at);  // the header alone: the rows stay in the message
    job->req.Deserialize(&rb);
  }
  const size_t n = job->req.keys.size(), row_bytes = job->req.row_bytes();
  auto finish = [job] {
    NaiveBuffer out;
    PushResponse resp;
    resp.meta = job->req.meta;
    resp.Serialize(&out);
    out << job->missing.load();
    Status st = RpcServer::Global().SendResponse(job->head, out.data(), out.size());
    if (!st.ok()) TIPS_LOG(WARNING) << "push response failed: " << st.ToString();
  };
  if (rows_at + n * row_bytes > job->msg.payload_size()) {  // truncated message: nothing is applied
    TIPS_LOG(ERROR) << "packed push of " << n << " rows is shorter than its header says";
    job->missing = n;
    finish();
    return;
  }
  job->rows = reinterpret_cast<const char*>(job->msg.payload()) + rows_at;
  std::vector<std::vector<size_t>> buckets(table_->local_shard_num());
  for (size_t i = 0; i < n; ++i) buckets[table_->ToLocalShard(job->req.keys[i])].push_back(i);
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
    bool ok  = table_->Submit(l, [this, job, idx, finish, row_bytes] {
      for (size_t i : *idx) {
        // borrows the message bytes; the methods only read the pushed value
        AnyVec view(job->req.dtype, job->req.length, const_cast<char*>(job->rows + i * row_bytes));
        if (!push_agent_.ApplyPushValue(job->req.keys[i], view)) job->missing++;
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

void PsFuture::Cancel() {
  std::lock_guard<std::mutex> lock(mu);
  cancelled = true;
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

std::shared_ptr<PsFuture> PsClient::PullPacked(const uint64_t* keys, size_t n, Datatype dtype, uint32_t length,
                                               void* out) {
  auto fut = std::make_shared<PsFuture>();
  const int ns = table_->num_servers();
  std::vector<PackedHeader> reqs(ns);
  std::vector<std::vector<size_t>> positions(ns);
  for (size_t i = 0; i < n; ++i) {
    const int s = table_->ToServerId(keys[i]);
    reqs[s].keys.push_back(keys[i]);
    positions[s].push_back(i);
  }
  int contacted = 0;
  for (int s = 0; s < ns; ++s) contacted += reqs[s].keys.empty() ? 0 : 1;
  fut->pending = contacted;
  if (contacted == 0) return fut;
  const size_t row_bytes    = DatatypeNumBytes(dtype) * length;
  const std::string service = std::string(kPackedPullServiceName) + "." + name_;
  for (int s = 0; s < ns; ++s) {
    if (reqs[s].keys.empty()) continue;
    reqs[s].meta.client_id  = client_id_;
    reqs[s].meta.message_id = next_message_id_++;
    reqs[s].dtype           = dtype;
    reqs[s].length          = length;
    NaiveBuffer buf;
    reqs[s].Serialize(&buf);
    auto pos = std::make_shared<std::vector<size_t>>(std::move(positions[s]));
    auto cb  = [fut, pos, out, row_bytes](const Status& st, RpcMessage&& m) {
      Status result = st;
      uint64_t bad  = 0;
      if (st.ok()) {
        constexpr size_t at = sizeof(int32_t) + 3 * sizeof(uint64_t);  // client, message, count, bad
        int32_t client = 0;
        uint64_t message = 0, count = 0;
        if (m.payload_size() >= at) {
          NaiveBuffer rb(m.payload(), at);
          rb >> client >> message >> count >> bad;
        }
        if (m.payload_size() < at || count != pos->size() || at + count * row_bytes > m.payload_size())
          result = Status(kInternal, "packed pull response does not match the request");
      }
      bool last;
      {
        // the rows are copied under the future's lock: a caller that gives up (Cancel) takes the same lock, so its
        // output buffer is never written after it has been told that the call is over
        std::lock_guard<std::mutex> lock(fut->mu);
        if (result.ok() && !fut->cancelled) {
          const char* rows = reinterpret_cast<const char*>(m.payload()) + sizeof(int32_t) + 3 * sizeof(uint64_t);
          for (size_t k = 0; k < pos->size(); ++k)
            memcpy(static_cast<char*>(out) + (*pos)[k] * row_bytes, rows + k * row_bytes, row_bytes);
        }
        if (!result.ok()) fut->status = result;
        fut->bad_rows += bad;
        last = --fut->pending == 0;
      }
      if (last) fut->cv.notify_all();
    };
    Status st = RpcServer::Global().SendRequest(table_->ServerWorldRank(s), service, buf.data(), buf.size(), cb);
    if (!st.ok()) cb(st, RpcMessage());
  }
  return fut;
}

std::shared_ptr<PsFuture> PsClient::PushPacked(const uint64_t* keys, size_t n, Datatype dtype, uint32_t length,
                                               const void* values) {
  auto fut = std::make_shared<PsFuture>();
  const int ns = table_->num_servers();
  std::vector<PackedHeader> reqs(ns);
  std::vector<std::vector<size_t>> positions(ns);
  for (size_t i = 0; i < n; ++i) {
    const int s = table_->ToServerId(keys[i]);
    reqs[s].keys.push_back(keys[i]);
    positions[s].push_back(i);
  }
  int contacted = 0;
  for (int s = 0; s < ns; ++s) contacted += reqs[s].keys.empty() ? 0 : 1;
  fut->pending = contacted;
  if (contacted == 0) return fut;
  const size_t row_bytes    = DatatypeNumBytes(dtype) * length;
  const std::string service = std::string(kPackedPushServiceName) + "." + name_;
  for (int s = 0; s < ns; ++s) {
    if (reqs[s].keys.empty()) continue;
    reqs[s].meta.client_id  = client_id_;
    reqs[s].meta.message_id = next_message_id_++;
    reqs[s].dtype           = dtype;
    reqs[s].length          = length;
    NaiveBuffer buf;
    reqs[s].Serialize(&buf);
    const size_t at = buf.cursor_pos();
    buf.Require(positions[s].size() * row_bytes);
    char* rows = static_cast<char*>(buf.data()) + at;
    for (size_t k = 0; k < positions[s].size(); ++k)
      memcpy(rows + k * row_bytes, static_cast<const char*>(values) + positions[s][k] * row_bytes, row_bytes);
    buf.Consume(positions[s].size() * row_bytes);
    auto cb = [fut](const Status& st, RpcMessage&& m) {
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
      if (last) fut->cv.notify_all();
    };
    Status st = RpcServer::Global().SendRequest(table_->ServerWorldRank(s), service, buf.data(), buf.size(), cb);
    if (!st.ok()) cb(st, RpcMessage());
  }
  return fut;
}

}  // namespace ps
}  // namespace tips
