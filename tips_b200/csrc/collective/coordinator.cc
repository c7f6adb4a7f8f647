#include "collective/coordinator.h"

#include <algorithm>
#include <cstdio>
#include <cstring>

#include "runtime/context.h"

namespace tips {
namespace collective {

namespace {

const char kCoordinatorService[] = "collective_coordinator";
const char kEngineStopService[]  = "collective_stop";

int64_t NumElements(const std::vector<int64_t>& shape) {
  int64_t n = 1;
  for (int64_t d : shape) n *= d;
  return n;
}

void ScaleHost(void* data, int64_t n, Datatype dtype, double f) {
  if (f == 1.0) return;
  switch (dtype) {
    case Datatype::kFp32: {
      float* p = static_cast<float*>(data);
      float s  = static_cast<float>(f);
      for (int64_t i = 0; i < n; ++i) p[i] *= s;
    } break;
    case Datatype::kFp64: {
      double* p = static_cast<double*>(data);
      for (int64_t i = 0; i < n; ++i) p[i] *= f;
    } break;
    default: {
      AnyVec v(dtype, static_cast<size_t>(n), data);
      for (int64_t i = 0; i < n; ++i) v.SetFromDouble(i, v.GetAsDouble(i) * f);
    }
  }
}

RequestMessage RequestOf(const OpRecord& rec, int rank) {
  RequestMessage req;
  req.request_rank = rank;
  req.request_type = rec.type;
  req.tensor_type  = rec.dtype;
  req.tensor_name  = rec.name;
  req.tensor_shape = rec.shape.empty() ? std::vector<int64_t>{1} : rec.shape;  // a scalar travels as [1]
  req.root_rank    = rec.root_rank;
  req.reduce_op    = static_cast<int32_t>(rec.reduce_op);
  req.device       = rec.device;
  req.prescale     = rec.prescale;
  req.postscale    = rec.postscale;
  return req;
}

}  // namespace

// ------------------------------------------------ rank-0 negotiation table --

bool IncreTensorCount(MessageTable* table, const RequestMessage& msg, const RpcMsgHead* head, int world_size) {
  PendingTensor& p = (*table)[msg.tensor_name];
  if (p.seen.empty()) {
    p.seen.assign(world_size, false);
    p.first_us = NowMicros();
  }
  int r = msg.request_rank;
  if (r < 0 || r >= world_size || p.seen[r]) {
    TIPS_LOG(ERROR) << "unexpected request for '" << msg.tensor_name << "' from rank " << r;
    return false;
  }
  p.seen[r] = true;
  p.requests.push_back(msg);
  if (head) p.heads.push_back(*head);
  return static_cast<int>(p.requests.size()) == world_size;
}

ResponseMessage ConstructResponseMessage(MessageTable* table, const std::string& name, int world_size) {
  ResponseMessage resp;
  resp.tensor_names = {name};
  auto it = table->find(name);
  if (it == table->end() || static_cast<int>(it->second.requests.size()) != world_size) {
    resp.response_type = ResponseType::kError;
    resp.error_message = "internal: response requested before every rank asked for '" + name + "'";
    return resp;
  }
  std::vector<RequestMessage> reqs = std::move(it->second.requests);
  std::sort(reqs.begin(), reqs.end(),
            [](const RequestMessage& a, const RequestMessage& b) { return a.request_rank < b.request_rank; });
  const RequestMessage& first = reqs[0];
  std::string err;
  for (int r = 1; r < world_size && err.empty(); ++r) {
    const RequestMessage& q = reqs[r];
    if (q.request_type != first.request_type) {
      err = StringFormat("mismatched collective operations for '%s': rank 0 did %s, rank %d did %s", name.c_str(),
                         RequestTypeName(first.request_type), r, RequestTypeName(q.request_type));
    } else if (q.tensor_type != first.tensor_type) {
      err = StringFormat("mismatched data types for '%s': rank 0 has %s, rank %d has %s", name.c_str(),
                         DatatypeName(first.tensor_type), r, DatatypeName(q.tensor_type));
    } else if (q.device != first.device) {
      err = StringFormat("mismatched devices for '%s': rank 0 uses %s memory, rank %d uses %s memory", name.c_str(),
                         first.device ? "device" : "host", r, q.device ? "device" : "host");
    }
  }
  if (err.empty()) {
    switch (first.request_type) {
      case RequestType::kAllreduce:
      case RequestType::kBroadcast:
        for (int r = 1; r < world_size && err.empty(); ++r) {
          const RequestMessage& q = reqs[r];
          if (q.tensor_shape != first.tensor_shape)
            err = StringFormat("mismatched %s tensor shapes for '%s': rank 0 has %s, rank %d has %s",
                               RequestTypeName(first.request_type), name.c_str(),
                               ToString(first.tensor_shape).c_str(), r, ToString(q.tensor_shape).c_str());
          else if (q.root_rank != first.root_rank && first.request_type == RequestType::kBroadcast)
            err = StringFormat("mismatched broadcast roots for '%s': rank 0 says %d, rank %d says %d", name.c_str(),
                               first.root_rank, r, q.root_rank);
          else if (first.request_type == RequestType::kAllreduce &&
                   (q.reduce_op != first.reduce_op || q.prescale != first.prescale || q.postscale != first.postscale))
            err = StringFormat("mismatched reduce operator or scale factors for '%s' on rank %d", name.c_str(), r);
        }
        if (err.empty() && first.request_type == RequestType::kBroadcast &&
            (first.root_rank < 0 || first.root_rank >= world_size))
          err = StringFormat("broadcast root %d out of range for '%s'", first.root_rank, name.c_str());
        break;
      case RequestType::kAllgather:
        if (first.tensor_shape.empty()) err = "allgather of a rank-0 tensor '" + name + "'";
        for (int r = 0; r < world_size && err.empty(); ++r) {
          const RequestMessage& q = reqs[r];
          if (q.tensor_shape.size() != first.tensor_shape.size()) {
            err = StringFormat("mismatched allgather tensor ranks for '%s': rank 0 has %zu dims, rank %d has %zu",
                               name.c_str(), first.tensor_shape.size(), r, q.tensor_shape.size());
            break;
          }
          for (size_t d = 1; d < q.tensor_shape.size(); ++d)
            if (q.tensor_shape[d] != first.tensor_shape[d]) {
              err = StringFormat("mismatched allgather trailing dimension %zu for '%s': rank 0 has %lld, rank %d has %lld",
                                 d, name.c_str(), (long long)first.tensor_shape[d], r, (long long)q.tensor_shape[d]);
              break;
            }
          resp.tensor_sizes.push_back(q.tensor_shape[0]);
        }
        break;
    }
  }
  table->erase(it);
  if (!err.empty()) {
    resp.response_type = ResponseType::kError;
    resp.error_message = err;
    resp.tensor_sizes.clear();
    return resp;
  }
  resp.response_type = static_cast<ResponseType>(static_cast<int16_t>(first.request_type));
  resp.root_rank     = first.root_rank;
  return resp;
}

// ----------------------------------------------------------- the engine ----

CollectiveEngine& CollectiveEngine::Global() {
  static CollectiveEngine* e = new CollectiveEngine;
  return *e;
}

void CollectiveEngine::Initialize(const EngineOptions& opts) {
  TIPS_CHECK(!initialized_.load()) << "collective engine initialised twice";
  Context& ctx = Context::Global();
  TIPS_CHECK(ctx.initialized());
  opts_  = opts;
  rank_  = ctx.rank();
  size_  = ctx.size();
  shut_down_ = false;
  frozen_    = false;
  queue_.Open();
  message_table_.clear();
  negotiated_.clear();
  order_log_.clear();
  RpcServer::Global().AddService(kCoordinatorService, [this](RpcMessage&& m) {
    Event ev;
    ev.kind = Event::kRemoteRequest;
    ev.head = m.head();
    NaiveBuffer rb(m.payload(), m.payload_size());
    ev.request.Deserialize(&rb);
    queue_.WriteMove(std::move(ev));
  });
  // Rank 0 ends a job's negotiation with this message, sent after its last response on the same connection
  // (see Loop): a rank stops executing responses exactly where rank 0 stopped sending them.
  RpcServer::Global().AddService(kEngineStopService, [this](RpcMessage&&) {
    Event ev;
    ev.kind = Event::kStopMarker;
    queue_.WriteMove(std::move(ev));
  });
  RpcServer::Global().SetPeerFailureHook([this](int peer) {
    Event ev;
    ev.kind = Event::kPeerFailure;
    ev.peer = peer;
    queue_.WriteMove(std::move(ev));
  });
  thread_      = std::thread([this] { Loop(); });
  initialized_ = true;
  ctx.Barrier();
}

void CollectiveEngine::Finalize() {
  if (!initialized_.load()) return;
  shut_down_ = true;
  Event ev;
  ev.kind = Event::kShutdown;
  queue_.WriteMove(std::move(ev));
  if (thread_.joinable()) thread_.join();
  queue_.Close();
  Event drop;
  while (queue_.TryRead(&drop)) {
  }
  {
    std::lock_guard<std::mutex> lock(mu_);
    tensor_table_.clear();
    schedules_.clear();
    schedule_index_.clear();
  }
  frozen_      = false;
  initialized_ = false;
}

int64_t CollectiveEngine::Enqueue(OpRecord record, std::string* error) {
  auto fail = [&](StatusCode c, const std::string& m) {
    if (error) *error = m;
    return -static_cast<int64_t>(c);
  };
  if (!initialized_.load() || shut_down_.load()) return fail(kAborted, "collective engine is not running");
  if (record.name.empty()) return fail(kInvalidArgument, "a collective needs a tensor name");
  if (record.device == 1 && !device_executor_) return fail(kPrecondition, "no device executor registered");
  record.enqueue_us = NowMicros();
  bool frozen_hit   = false;
  std::string frozen_err;
  int64_t handle;
  {
    std::lock_guard<std::mutex> lock(mu_);
    if (tensor_table_.count(record.name))
      return fail(kDuplicateName, "a collective named '" + record.name + "' is already in flight");
    handle        = next_handle_++;
    record.handle = handle;
    handles_[handle] = std::make_shared<HandleState>();
    if (frozen_.load()) {
      auto it = schedule_index_.find(record.name);
      if (it != schedule_index_.end()) {
        Schedule& sched    = schedules_[it->second.first];
        const Signature& s = sched.sigs[it->second.second];
        std::vector<int64_t> shape = record.shape.empty() ? std::vector<int64_t>{1} : record.shape;
        if (s.type != record.type || s.dtype != record.dtype || s.shape != shape || s.device != record.device ||
            s.reduce_op != static_cast<int32_t>(record.reduce_op) || s.root_rank != record.root_rank) {
          frozen_err = "'" + record.name + "' no longer matches the frozen schedule; thaw it first";
        } else {
          frozen_hit = true;
          tensor_table_[record.name]    = record;
          sched.ready[it->second.second] = true;
        }
      }
    }
    if (!frozen_hit && frozen_err.empty()) tensor_table_[record.name] = record;
  }
  counters_.ops_enqueued++;
  if (!frozen_err.empty()) {
    Complete(record, Status(kPrecondition, frozen_err));
    return handle;
  }
  Event ev;
  if (frozen_hit) {
    ev.kind = Event::kFrozenReady;
  } else {
    ev.kind    = Event::kLocalRequest;
    ev.request = RequestOf(record, rank_);
  }
  if (!queue_.WriteMove(std::move(ev))) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      tensor_table_.erase(record.name);
    }
    Complete(record, Status(kAborted, "collective engine shut down"));
  }
  return handle;
}

int CollectiveEngine::Poll(int64_t handle) {
  auto h = Lookup(handle);
  if (!h) return kInvalidArgument;
  return h->code.load();
}

int CollectiveEngine::Wait(int64_t handle, int timeout_ms) {
  auto h = Lookup(handle);
  if (!h) return kInvalidArgument;
  std::unique_lock<std::mutex> lock(mu_);
  auto done = [&] { return h->code.load() != kInProgress; };
  if (timeout_ms < 0) {
    handle_cv_.wait(lock, done);
  } else if (!handle_cv_.wait_for(lock, std::chrono::milliseconds(timeout_ms), done)) {
    return kTimeout;
  }
  return h->code.load();
}

std::shared_ptr<HandleState> CollectiveEngine::Lookup(int64_t handle) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = handles_.find(handle);
  return it == handles_.end() ? nullptr : it->second;
}

void CollectiveEngine::Release(int64_t handle) {
  std::lock_guard<std::mutex> lock(mu_);
  handles_.erase(handle);
}

void CollectiveEngine::Complete(const OpRecord& rec, const Status& st) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = handles_.find(rec.handle);
    if (it != handles_.end()) {
      it->second->error = st.message();
      it->second->code  = st.ok() ? kOk : static_cast<int>(st.code());
    }
  }
  handle_cv_.notify_all();
  if (st.ok())
    counters_.ops_completed++;
  else
    counters_.ops_failed++;
}

void CollectiveEngine::FailAll(const Status& st) {
  std::vector<OpRecord> recs;
  {
    std::lock_guard<std::mutex> lock(mu_);
    for (auto& kv : tensor_table_) recs.push_back(kv.second);
    tensor_table_.clear();
    for (Schedule& sched : schedules_) std::fill(sched.ready.begin(), sched.ready.end(), false);
  }
  for (auto& r : recs) Complete(r, st);
}

void CollectiveEngine::Trace(const std::string& name, const char* phase, int64_t b, int64_t e) {
  if (!timeline_on_.load()) return;
  std::lock_guard<std::mutex> lock(timeline_mu_);
  if (timeline_.size() >= (1u << 20)) timeline_.pop_front();
  timeline_.push_back(TimelineEvent{name, phase, b, e});
}

Status CollectiveEngine::DumpTimeline(const std::string& path) {
  FILE* f = fopen(path.c_str(), "w");
  if (!f) return Status(kInvalidArgument, "cannot open " + path);
  std::lock_guard<std::mutex> lock(timeline_mu_);
  fprintf(f, "[\n");
  bool first = true;
  for (auto& ev : timeline_) {
    std::string safe;
    for (char c : ev.name) safe += (c == '"' || c == '\\') ? '_' : c;
    fprintf(f, "%s{\"name\": \"%s\", \"cat\": \"%s\", \"ph\": \"X\", \"ts\": %lld, \"dur\": %lld, \"pid\": %d, \"tid\": \"%s\"}",
            first ? "" : ",\n", safe.c_str(), ev.phase, (long long)ev.begin_us, (long long)(ev.end_us - ev.begin_us),
            rank_, ev.phase);
    first = false;
  }
  fprintf(f, "\n]\n");
  fclose(f);
  return Status::OK();
}

}  // namespace collective
}  // namespace tips
