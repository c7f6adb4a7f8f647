// Background-thread half of the collective engine: the event loop, rank-0
// response construction with tensor fusion, op execution (host and device),
// the frozen schedule, the stall detector and peer-failure handling.
// Reference counterpart: BackgroundThreadLoop / PerformCollectiveOp
// (tips/core/collective/coordinator.cc:243-513).
#include <algorithm>
#include <cstring>
#include <thread>

#include "collective/coordinator.h"
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
  if (dtype == Datatype::kFp32) {
    float* p = static_cast<float*>(data);
    float s  = static_cast<float>(f);
    for (int64_t i = 0; i < n; ++i) p[i] *= s;
    return;
  }
  if (dtype == Datatype::kFp64) {
    double* p = static_cast<double*>(data);
    for (int64_t i = 0; i < n; ++i) p[i] *= f;
    return;
  }
  AnyVec v(dtype, static_cast<size_t>(n), data);
  for (int64_t i = 0; i < n; ++i) v.SetFromDouble(i, v.GetAsDouble(i) * f);
}

}  // namespace

void CollectiveEngine::Loop() {
  // Shutdown with collectives in flight: every rank has to execute the same responses, or a rank that stopped
  // early leaves the others inside a collective it never joins.  So rank 0 decides where the job ends: on its own
  // shutdown it stops answering and tells every rank so, after its last response on the same connection; the other
  // ranks keep executing what arrives until that message (or a lost peer, or `kStopWaitMs`).
  constexpr int64_t kStopWaitMs = 10000;
  bool stopping         = false;
  int64_t stop_deadline = 0;
  std::vector<std::string> ready;
  while (true) {
    Event first;
    int got = queue_.ReadFor(&first, stopping ? 50 : 500);
    if (got < 0) break;
    if (stopping && NowMicros() > stop_deadline) break;
    if (got == 0) {
      if (rank_ == 0) CheckStalls();
      continue;
    }
    std::vector<Event> batch;
    batch.emplace_back(std::move(first));
    if (opts_.cycle_time_ms > 0 && batch[0].kind != Event::kShutdown)
      std::this_thread::sleep_for(std::chrono::milliseconds(opts_.cycle_time_ms));
    Event more;
    while (queue_.TryRead(&more)) batch.emplace_back(std::move(more));

    bool stop = false;
    for (Event& ev : batch) {
      switch (ev.kind) {
        case Event::kShutdown:
          if (rank_ == 0 || size_ == 1) {
            for (int r = 1; r < size_; ++r)
              RpcServer::Global().SendRequest(r, kEngineStopService, nullptr, 0, [](const Status&, RpcMessage&&) {});
            stop = true;
          } else if (!stopping) {
            stopping      = true;
            stop_deadline = NowMicros() + kStopWaitMs * 1000;
          }
          break;
        case Event::kStopMarker:
          // rank 0 has sent its last response: nothing that arrives later is executed anywhere
          stop = true;
          break;
        case Event::kLocalRequest:
          counters_.negotiation_requests++;
          if (rank_ == 0) {
            HandleRequestOnCoordinator(ev.request, nullptr, &ready);
          } else {
            NaiveBuffer buf;
            ev.request.Serialize(&buf);
            std::string name = ev.request.tensor_name;
            Status st        = RpcServer::Global().SendRequest(
                0, kCoordinatorService, buf.data(), buf.size(), [this, name](const Status& s, RpcMessage&& m) {
                  Event rev;
                  rev.kind = Event::kResponse;
                  if (s.ok()) {
                    NaiveBuffer rb(m.payload(), m.payload_size());
                    rev.response.Deserialize(&rb);
                  } else {
                    rev.response.response_type = ResponseType::kError;
                    rev.response.tensor_names  = {name};
                    rev.response.error_message = "negotiation failed: " + s.message();
                  }
                  queue_.WriteMove(std::move(rev));
                });
            if (!st.ok()) {
              ResponseMessage err;
              err.response_type = ResponseType::kError;
              err.tensor_names  = {name};
              err.error_message = "cannot reach the coordinator: " + st.message();
              Execute(err);
            }
          }
          break;
        case Event::kRemoteRequest: HandleRequestOnCoordinator(ev.request, &ev.head, &ready); break;
        case Event::kResponse: Execute(ev.response); break;
        case Event::kFrozenReady: DrainFrozen(); break;
        case Event::kPeerFailure:
          TIPS_LOG(ERROR) << "rank " << ev.peer << " left the job; failing the collectives in flight";
          message_table_.clear();
          FailAll(Status(kUnavailable, "rank " + std::to_string(ev.peer) + " left the job"));
          if (stopping) stop = true;
          break;
        case Event::kReset:
          message_table_.clear();
          ready.clear();
          FailAll(Status(kAborted, "the collective engine was reset"));
          ThawSchedule();
          {
            std::lock_guard<std::mutex> lock(mu_);
            negotiated_.clear();
            order_log_.clear();
            ++resets_done_;
          }
          reset_cv_.notify_all();
          break;
      }
      if (stop) break;
    }
    if (stop) break;
    if (rank_ == 0) {
      FlushReady(&ready);
      CheckStalls();
    }
  }
  FailAll(Status(kAborted, "tips shut down while the collective was in flight"));
}

void CollectiveEngine::HandleRequestOnCoordinator(const RequestMessage& req, const RpcMsgHead* head,
                                                  std::vector<std::string>* ready) {
  if (IncreTensorCount(&message_table_, req, head, size_)) ready->push_back(req.tensor_name);
}

void CollectiveEngine::FlushReady(std::vector<std::string>* ready) {
  if (ready->empty()) return;
  struct Item {
    ResponseMessage resp;
    RequestMessage exemplar;
    std::vector<RpcMsgHead> heads;
    int64_t bytes;
  };
  std::vector<Item> items;
  for (const std::string& name : *ready) {
    Item it;
    auto p = message_table_.find(name);
    if (p == message_table_.end()) continue;
    it.exemplar = p->second.requests.front();
    it.heads    = p->second.heads;
    it.bytes    = it.exemplar.NumElements() * static_cast<int64_t>(DatatypeNumBytes(it.exemplar.tensor_type));
    it.resp     = ConstructResponseMessage(&message_table_, name, size_);
    items.emplace_back(std::move(it));
  }
  ready->clear();

  auto fusable = [&](const Item& a, const Item& b) {
    return a.resp.response_type == ResponseType::kAllreduce && b.resp.response_type == ResponseType::kAllreduce &&
           a.exemplar.device == 0 && b.exemplar.device == 0 && a.exemplar.tensor_type == b.exemplar.tensor_type &&
           a.exemplar.reduce_op == b.exemplar.reduce_op && a.exemplar.prescale == b.exemplar.prescale &&
           a.exemplar.postscale == b.exemplar.postscale;
  };
  size_t i = 0;
  while (i < items.size()) {
    size_t j      = i + 1;
    int64_t total = items[i].bytes;
    while (j < items.size() && opts_.fusion_threshold_bytes > 0 && fusable(items[i], items[j]) &&
           total + items[j].bytes <= opts_.fusion_threshold_bytes) {
      total += items[j].bytes;
      ++j;
    }
    ResponseMessage resp = items[i].resp;
    for (size_t k = i + 1; k < j; ++k) resp.tensor_names.push_back(items[k].resp.tensor_names[0]);
    if (j - i > 1) {
      counters_.fused_groups++;
      counters_.fused_tensors += j - i;
    }
    NaiveBuffer full;
    resp.Serialize(&full);
    ResponseMessage covered;  // "this name is part of another response"
    covered.response_type = resp.response_type;
    NaiveBuffer cov;
    covered.Serialize(&cov);
    for (size_t k = i; k < j; ++k) {
      const NaiveBuffer& payload = (k == i) ? full : cov;
      for (const RpcMsgHead& h : items[k].heads) {
        Status st = RpcServer::Global().SendResponse(h, payload.data(), payload.size());
        if (!st.ok()) TIPS_LOG(WARNING) << "response to rank " << h.src_rank << " failed: " << st.ToString();
      }
    }
    counters_.responses++;
    Execute(resp);
    i = j;
  }
}

void CollectiveEngine::Execute(const ResponseMessage& resp) {
  if (resp.tensor_names.empty()) return;  // covered by a fused response
  std::vector<OpRecord> recs;
  {
    std::lock_guard<std::mutex> lock(mu_);
    for (const std::string& name : resp.tensor_names) {
      auto it = tensor_table_.find(name);
      if (it == tensor_table_.end()) continue;  // already failed (peer loss, shutdown)
      recs.push_back(it->second);
    }
  }
  if (recs.empty()) return;
  Status st;
  const int64_t t0 = NowMicros();
  for (auto& r : recs) Trace(r.name, "NEGOTIATE", r.enqueue_us, t0);
  if (resp.response_type == ResponseType::kError) {
    // a tensor that the stall detector gave up on is a timeout (a retry may succeed), anything else a mismatch
    st = Status(resp.error_message.rfind("stalled:", 0) == 0 ? kTimeout : kPrecondition, resp.error_message);
  } else if (resp.response_type == ResponseType::kShutdown) {
    st = Status(kAborted, "coordinator shut down");
  } else if (recs.size() == 1) {
    st = ExecuteOne(&recs[0], resp, 0);
  } else {
    std::vector<OpRecord*> ptrs;
    for (auto& r : recs) ptrs.push_back(&r);
    st = ExecuteFusedHost(ptrs);
  }
  const int64_t t1 = NowMicros();
  {
    std::lock_guard<std::mutex> lock(mu_);
    for (auto& r : recs) {
      tensor_table_.erase(r.name);
      if (st.ok()) {
        Signature s{r.type, r.dtype, r.shape.empty() ? std::vector<int64_t>{1} : r.shape,
                    r.device, static_cast<int32_t>(r.reduce_op), r.root_rank};
        negotiated_[r.name] = std::move(s);
        order_log_.push_back(r.name);
      }
    }
  }
  for (auto& r : recs) {
    Trace(r.name, "EXECUTE", t0, t1);
    Complete(r, st);
  }
}

Status CollectiveEngine::ExecuteOne(OpRecord* rec, const ResponseMessage& resp, int channel) {
  const int64_t count = NumElements(rec->shape);
  const size_t es     = DatatypeNumBytes(rec->dtype);
  std::vector<int64_t> counts;
  int64_t trailing = 1;
  if (rec->type == RequestType::kAllgather) {
    if (static_cast<int>(resp.tensor_sizes.size()) != size_)
      return Status(kInternal, "allgather response without per-rank sizes");
    for (size_t d = 1; d < rec->shape.size(); ++d) trailing *= rec->shape[d];
    int64_t total_first = 0;
    for (int64_t s : resp.tensor_sizes) {
      counts.push_back(s * trailing);
      total_first += s;
    }
    {
      std::lock_guard<std::mutex> lock(mu_);
      auto it = handles_.find(rec->handle);
      if (it != handles_.end()) it->second->sizes = resp.tensor_sizes;
    }
    if (!rec->out) {
      if (!rec->alloc) return Status(kInvalidArgument, "allgather without an output buffer or allocator");
      rec->out = rec->alloc(rec->handle, total_first * trailing * static_cast<int64_t>(es), resp.tensor_sizes.data(),
                            size_, rec->alloc_user);
      if (!rec->out && total_first * trailing > 0) return Status(kInternal, "allgather output allocation failed");
    }
    {
      std::lock_guard<std::mutex> lock(mu_);
      auto it = handles_.find(rec->handle);
      if (it != handles_.end()) it->second->out = rec->out;
    }
  }

  if (rec->device == 1) {
    if (!device_executor_) return Status(kPrecondition, "no device executor registered");
    DeviceOp op;
    memset(&op, 0, sizeof(op));
    op.type        = static_cast<int32_t>(rec->type);
    op.dtype       = static_cast<int32_t>(rec->dtype);
    op.reduce_op   = static_cast<int32_t>(rec->reduce_op);
    op.root_rank   = rec->type == RequestType::kBroadcast ? resp.root_rank : rec->root_rank;
    op.in          = rec->in;
    op.out         = rec->out;
    op.count       = count;
    op.counts      = counts.empty() ? nullptr : counts.data();
    op.nranks      = size_;
    op.channel     = channel;
    op.prescale    = rec->prescale;
    op.postscale   = rec->postscale;
    op.stream      = rec->stream;
    op.ready_event = rec->ready_event;
    op.done_event  = rec->done_event;
    char err[512]  = {0};
    int rc         = device_executor_(&op, err, sizeof(err));
    if (rc != 0) return Status(rc == kTimeout ? kTimeout : kInternal, std::string("device collective failed: ") + err);
  } else {
    switch (rec->type) {
      case RequestType::kAllreduce: {
        if (rec->out != rec->in) memcpy(rec->out, rec->in, count * es);
        ScaleHost(rec->out, count, rec->dtype, rec->prescale);
        Status st = AllreduceCpu(rec->out, rec->out, count, rec->dtype, rec->reduce_op);
        if (!st.ok()) return st;
        ScaleHost(rec->out, count, rec->dtype, rec->postscale);
      } break;
      case RequestType::kBroadcast: {
        if (rank_ == resp.root_rank && rec->out != rec->in) memcpy(rec->out, rec->in, count * es);
        Status st = BroadcastCpu(rec->out, count, rec->dtype, resp.root_rank);
        if (!st.ok()) return st;
      } break;
      case RequestType::kAllgather: {
        Status st = AllgathervCpu(rec->in, rec->out, resp.tensor_sizes, trailing, rec->dtype);
        if (!st.ok()) return st;
      } break;
    }
  }
  const uint64_t bytes = static_cast<uint64_t>(count) * es;
  if (rec->type == RequestType::kAllreduce) counters_.allreduce_bytes += bytes;
  if (rec->type == RequestType::kBroadcast) counters_.broadcast_bytes += bytes;
  if (rec->type == RequestType::kAllgather) {
    uint64_t total = 0;
    for (int64_t c : counts) total += static_cast<uint64_t>(c) * es;
    counters_.allgather_bytes += total;
  }
  return Status::OK();
}

Status CollectiveEngine::ExecuteFusedHost(std::vector<OpRecord*>& recs) {
  // Pack -> one allreduce -> unpack. All records agree on dtype/op/scales.
  const Datatype dtype = recs[0]->dtype;
  const size_t es      = DatatypeNumBytes(dtype);
  int64_t total        = 0;
  for (OpRecord* r : recs) total += NumElements(r->shape);
  if (fusion_buffer_.size() < static_cast<size_t>(total) * es) fusion_buffer_.resize(static_cast<size_t>(total) * es);
  int64_t off = 0;
  for (OpRecord* r : recs) {
    int64_t n = NumElements(r->shape);
    memcpy(fusion_buffer_.data() + off * es, r->in, n * es);
    off += n;
  }
  ScaleHost(fusion_buffer_.data(), total, dtype, recs[0]->prescale);
  Status st = AllreduceCpu(fusion_buffer_.data(), fusion_buffer_.data(), total, dtype, recs[0]->reduce_op);
  if (!st.ok()) return st;
  ScaleHost(fusion_buffer_.data(), total, dtype, recs[0]->postscale);
  off = 0;
  for (OpRecord* r : recs) {
    int64_t n = NumElements(r->shape);
    memcpy(r->out, fusion_buffer_.data() + off * es, n * es);
    off += n;
  }
  counters_.allreduce_bytes += static_cast<uint64_t>(total) * es;
  return Status::OK();
}

// ------------------------------------------------------ frozen schedule ----

Status CollectiveEngine::FreezeSchedule(const std::vector<std::string>& names) {
  std::lock_guard<std::mutex> lock(mu_);
  if (names.empty()) return Status(kInvalidArgument, "empty schedule");
  Schedule sched;
  std::unordered_map<std::string, size_t> seen;
  for (size_t i = 0; i < names.size(); ++i) {
    auto it = negotiated_.find(names[i]);
    if (it == negotiated_.end())
      return Status(kPrecondition, "'" + names[i] + "' has not been negotiated yet; run one step first");
    if (it->second.type == RequestType::kAllgather)
      return Status(kInvalidArgument, "allgather '" + names[i] + "' cannot be frozen: its sizes may change");
    if (seen.count(names[i])) return Status(kInvalidArgument, "'" + names[i] + "' appears twice in the schedule");
    if (schedule_index_.count(names[i]))
      return Status(kInvalidArgument, "'" + names[i] + "' already belongs to a frozen schedule");
    if (tensor_table_.count(names[i])) return Status(kPrecondition, "'" + names[i] + "' is still in flight");
    seen[names[i]] = i;
    sched.sigs.push_back(it->second);
  }
  sched.names = names;
  sched.ready.assign(names.size(), false);
  const size_t sid = schedules_.size();
  for (size_t i = 0; i < names.size(); ++i) schedule_index_[names[i]] = {sid, i};
  schedules_.push_back(std::move(sched));
  frozen_ = true;
  return Status::OK();
}

Status CollectiveEngine::Reset() {
  if (!initialized_.load() || shut_down_.load()) return Status(kPrecondition, "the engine is not running");
  uint64_t ticket;
  {
    std::lock_guard<std::mutex> lock(mu_);
    ticket = ++resets_requested_;
  }
  Event ev;
  ev.kind = Event::kReset;
  queue_.WriteMove(std::move(ev));
  std::unique_lock<std::mutex> lock(mu_);
  if (!reset_cv_.wait_for(lock, std::chrono::seconds(30), [&] { return resets_done_ >= ticket; }))
    return Status(kTimeout, "the engine thread did not answer the reset");
  return Status::OK();
}

void CollectiveEngine::ThawSchedule() {
  std::lock_guard<std::mutex> lock(mu_);
  frozen_ = false;
  schedules_.clear();
  schedule_index_.clear();
}

std::vector<std::string> CollectiveEngine::TakeNegotiatedOrder() {
  std::lock_guard<std::mutex> lock(mu_);
  std::vector<std::string> out;
  out.swap(order_log_);
  return out;
}

void CollectiveEngine::DrainFrozen() {
  // Execute, for every schedule, the entries at its cursor for as long as they are ready.
  bool progress = true;
  while (progress) {
    progress = false;
    size_t nsched;
    {
      std::lock_guard<std::mutex> lock(mu_);
      nsched = schedules_.size();
    }
    for (size_t sid = 0; sid < nsched; ++sid) {
      OpRecord rec;
      {
        std::lock_guard<std::mutex> lock(mu_);
        if (!frozen_.load() || sid >= schedules_.size()) return;
        Schedule& sched = schedules_[sid];
        if (sched.names.empty() || !sched.ready[sched.cursor]) continue;
        auto it = tensor_table_.find(sched.names[sched.cursor]);
        if (it == tensor_table_.end()) {
          sched.ready[sched.cursor] = false;
          continue;
        }
        rec = it->second;
      }
      ResponseMessage resp;
      resp.response_type = static_cast<ResponseType>(static_cast<int16_t>(rec.type));
      resp.tensor_names  = {rec.name};
      resp.root_rank     = rec.root_rank;
      const int64_t t0   = NowMicros();
      Status st          = ExecuteOne(&rec, resp, 1);
      Trace(rec.name, "EXECUTE", t0, NowMicros());
      {
        std::lock_guard<std::mutex> lock(mu_);
        tensor_table_.erase(rec.name);
        if (sid < schedules_.size()) {
          Schedule& sched = schedules_[sid];
          sched.ready[sched.cursor] = false;
          sched.cursor              = (sched.cursor + 1) % sched.names.size();
        }
      }
      counters_.frozen_executions++;
      Complete(rec, st);
      progress = true;
    }
  }
}

// -------------------------------------------------------- stall detector ---

void CollectiveEngine::CheckStalls() {
  if (message_table_.empty()) return;
  const int64_t now = NowMicros();
  std::vector<std::string> to_abort;
  for (auto& kv : message_table_) {
    PendingTensor& p = kv.second;
    const int64_t waited_ms = (now - p.first_us) / 1000;
    if (opts_.stall_warn_ms > 0 && waited_ms > opts_.stall_warn_ms && !p.warned) {
      std::string missing;
      for (int r = 0; r < size_; ++r)
        if (!p.seen[r]) missing += (missing.empty() ? "" : ", ") + std::to_string(r);
      TIPS_LOG(WARNING) << "collective '" << kv.first << "' has waited " << waited_ms
                        << " ms for ranks [" << missing << "]: one or more ranks may have stopped submitting it";
      p.warned = true;
      counters_.stall_warnings++;
    }
    if (opts_.stall_abort_ms > 0 && waited_ms > opts_.stall_abort_ms) to_abort.push_back(kv.first);
  }
  for (const std::string& name : to_abort) {
    PendingTensor p = std::move(message_table_[name]);
    message_table_.erase(name);
    std::string missing;
    for (int r = 0; r < size_; ++r)
      if (!p.seen[r]) missing += (missing.empty() ? "" : ", ") + std::to_string(r);
    ResponseMessage resp;
    resp.response_type = ResponseType::kError;
    resp.tensor_names  = {name};
    resp.error_message = StringFormat("stalled: '%s' was never submitted by ranks [%s] within %d ms", name.c_str(),
                                      missing.c_str(), opts_.stall_abort_ms);
    NaiveBuffer buf;
    resp.Serialize(&buf);
    for (const RpcMsgHead& h : p.heads) RpcServer::Global().SendResponse(h, buf.data(), buf.size());
    Execute(resp);
  }
}

}  // namespace collective
}  // namespace tips
