// extern "C" surface of the native runtime; see tips_c_api.h.
// Lifecycle order follows the reference's tips_init / tips_shutdown
// (tips/core/operations.cc:12-44): context (bootstrap + RPC) first, then the
// collective engine; shutdown drains the engine, then the context with
// barriers around the RPC teardown.
#include "tips_c_api.h"

#include <cstring>
#include <chrono>
#include <sstream>

#include "collective/coordinator.h"
#include "runtime/context.h"

using namespace tips;
using namespace tips::collective;

namespace {

thread_local std::string tl_error;
EngineOptions g_engine_opts;

int Fail(const Status& st) {
  tl_error = st.message();
  return -static_cast<int>(st.code());
}
int Fail(StatusCode c, const std::string& m) {
  tl_error = m;
  return -static_cast<int>(c);
}

template <typename F>
int Guard(F&& f) {
  try {
    return f();
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

int EnvInt(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

int InitWith(const InitOptions& opts) {
  return Guard([&] {
    if (Context::Global().initialized()) return 0;
    LogConfig::Reload();
    Status st = Context::Global().Initialize(opts);
    if (!st.ok()) return Fail(st);
    if (const char* v = getenv("TIPS_FUSION_THRESHOLD")) g_engine_opts.fusion_threshold_bytes = atoll(v);
    g_engine_opts.cycle_time_ms  = EnvInt("TIPS_CYCLE_TIME_MS", g_engine_opts.cycle_time_ms);
    g_engine_opts.stall_warn_ms  = EnvInt("TIPS_STALL_WARN_MS", g_engine_opts.stall_warn_ms);
    g_engine_opts.stall_abort_ms = EnvInt("TIPS_STALL_ABORT_MS", g_engine_opts.stall_abort_ms);
    CollectiveEngine::Global().Initialize(g_engine_opts);
    return 0;
  });
}

}  // namespace

extern "C" {

int tips_init(void) { return InitWith(Context::OptionsFromEnv()); }

int tips_init_ex(int rank, int size, const char* master_addr, int master_port) {
  InitOptions o = Context::OptionsFromEnv();
  o.rank        = rank;
  o.size        = size;
  if (master_addr && *master_addr) o.master_addr = master_addr;
  if (master_port > 0) o.master_port = master_port;
  return InitWith(o);
}

int tips_shutdown(void) {
  return Guard([] {
    if (!Context::Global().initialized()) return 0;
    Context::Global().Barrier(30000);
    CollectiveEngine::Global().Finalize();
    Context::Global().Finalize();
    return 0;
  });
}

int tips_is_initialized(void) {
  return Context::Global().initialized() && RpcServer::Global().initialized() &&
                 CollectiveEngine::Global().initialized()
             ? 1
             : 0;
}
int tips_is_initialize(void) { return tips_is_initialized(); }
int tips_size(void) { return Context::Global().initialized() ? Context::Global().size() : -1; }
int tips_rank(void) { return Context::Global().initialized() ? Context::Global().rank() : -1; }
int tips_local_rank(void) { return Context::Global().initialized() ? Context::Global().local_rank() : -1; }
int tips_local_size(void) { return Context::Global().initialized() ? Context::Global().local_size() : -1; }
const char* tips_last_error(void) { return tl_error.c_str(); }

int tips_rank_ip(int rank, char* out, int out_len) {
  return Guard([&] {
    if (!Context::Global().initialized()) return Fail(kPrecondition, "not initialised");
    if (rank < 0 || rank >= Context::Global().size()) return Fail(kInvalidArgument, "bad rank");
    const std::string& ip = Context::Global().ip(rank);
    int n = static_cast<int>(ip.size()) < out_len - 1 ? static_cast<int>(ip.size()) : out_len - 1;
    memcpy(out, ip.data(), n);
    out[n] = 0;
    return n;
  });
}

int tips_barrier(void) {
  return Guard([] {
    Status st = Context::Global().initialized() ? Context::Global().Barrier()
                                                : Status(kPrecondition, "tips is not initialised");
    return st.ok() ? 0 : Fail(st);
  });
}

int tips_host_allgather(const void* in, int64_t n, void* out, int64_t max_n, int64_t* out_sizes) {
  return Guard([&] {
    if (!Context::Global().initialized()) return Fail(kPrecondition, "tips is not initialised");
    std::vector<std::string> all;
    Status st = Context::Global().AllgatherBytes(std::string(static_cast<const char*>(in), n), &all);
    if (!st.ok()) return Fail(st);
    for (size_t r = 0; r < all.size(); ++r) {
      if (static_cast<int64_t>(all[r].size()) > max_n) return Fail(kInvalidArgument, "allgather output too small");
      memcpy(static_cast<char*>(out) + r * max_n, all[r].data(), all[r].size());
      out_sizes[r] = static_cast<int64_t>(all[r].size());
    }
    return 0;
  });
}

// ---- sub-groups of ranks (the reference's MpiGroup, tips/core/mpi_group.h:15-96) ----
int64_t tips_group_new(const int32_t* world_ranks, int n) {
  int64_t id = -1;
  int rc = Guard([&] {
    if (!Context::Global().initialized()) return Fail(kPrecondition, "tips is not initialised");
    if (n < 1 || !world_ranks) return Fail(kInvalidArgument, "a group needs at least one rank");
    std::vector<int> ranks(world_ranks, world_ranks + n);
    for (int r : ranks)
      if (r < 0 || r >= Context::Global().size()) return Fail(kInvalidArgument, "group rank out of range");
    id = static_cast<int64_t>(Context::Global().NewGroup(ranks)->id());
    return 0;
  });
  return rc == 0 ? id : rc;
}

static Group* GroupOf(int64_t id) {
  if (!Context::Global().initialized() || id < 0) return nullptr;
  return Context::Global().FindGroup(static_cast<uint64_t>(id));
}

int tips_group_size(int64_t id) {
  Group* g = GroupOf(id);
  return g ? g->size() : -1;
}
int tips_group_rank(int64_t id) {  // -1 when this process is not a member
  Group* g = GroupOf(id);
  return g ? g->rank() : -1;
}
int tips_group_to_world(int64_t id, int group_rank) {
  Group* g = GroupOf(id);
  return (g && group_rank >= 0 && group_rank < g->size()) ? g->ToWorldRank(group_rank) : -1;
}
int tips_group_barrier(int64_t id, int timeout_ms) {
  return Guard([&] {
    Group* g = GroupOf(id);
    if (!g) return Fail(kInvalidArgument, "unknown group");
    Status st = g->Barrier(timeout_ms);
    return st.ok() ? 0 : Fail(st);
  });
}
int tips_group_allgather(int64_t id, const void* in, int64_t n, void* out, int64_t max_n, int64_t* out_sizes,
                         int timeout_ms) {
  return Guard([&] {
    Group* g = GroupOf(id);
    if (!g) return Fail(kInvalidArgument, "unknown group");
    std::vector<std::string> all;
    Status st = g->AllgatherBytes(std::string(static_cast<const char*>(in), n), &all, timeout_ms);
    if (!st.ok()) return Fail(st);
    for (size_t r = 0; r < all.size(); ++r) {
      if (static_cast<int64_t>(all[r].size()) > max_n) return Fail(kInvalidArgument, "allgather output too small");
      memcpy(static_cast<char*>(out) + r * max_n, all[r].data(), all[r].size());
      out_sizes[r] = static_cast<int64_t>(all[r].size());
    }
    return 0;
  });
}

int tips_host_broadcast(void* data, int64_t n, int root) {
  return Guard([&] {
    if (!Context::Global().initialized()) return Fail(kPrecondition, "tips is not initialised");
    std::string s(static_cast<const char*>(data), n);
    Status st = Context::Global().BroadcastBytes(&s, root);
    if (!st.ok()) return Fail(st);
    if (static_cast<int64_t>(s.size()) != n) return Fail(kPrecondition, "broadcast size differs from the root's");
    memcpy(data, s.data(), n);
    return 0;
  });
}

int tips_set_fusion_threshold(int64_t bytes) {
  g_engine_opts.fusion_threshold_bytes = bytes;
  if (CollectiveEngine::Global().initialized())
    const_cast<EngineOptions&>(CollectiveEngine::Global().options()).fusion_threshold_bytes = bytes;
  return 0;
}
int tips_set_cycle_time_ms(int ms) {
  g_engine_opts.cycle_time_ms = ms;
  if (CollectiveEngine::Global().initialized())
    const_cast<EngineOptions&>(CollectiveEngine::Global().options()).cycle_time_ms = ms;
  return 0;
}
int tips_set_stall_check(int warn_ms, int abort_ms) {
  g_engine_opts.stall_warn_ms  = warn_ms;
  g_engine_opts.stall_abort_ms = abort_ms;
  if (CollectiveEngine::Global().initialized()) {
    auto& o          = const_cast<EngineOptions&>(CollectiveEngine::Global().options());
    o.stall_warn_ms  = warn_ms;
    o.stall_abort_ms = abort_ms;
  }
  return 0;
}

int64_t tips_enqueue(const tips_op_t* op) {
  try {
    if (!op || !op->name) return Fail(kInvalidArgument, "null op");
    OpRecord rec;
    rec.name = op->name;
    rec.type = static_cast<RequestType>(op->type);
    if (op->type < 0 || op->type > 2) return Fail(kInvalidArgument, "bad collective type");
    rec.dtype = static_cast<Datatype>(op->dtype);
    if (op->dtype < 0 || op->dtype > 7) return Fail(kInvalidArgument, "unsupported dtype");
    rec.shape.assign(op->shape, op->shape + op->ndim);
    rec.in          = op->in;
    rec.out         = op->out;
    rec.device      = op->device;
    rec.root_rank   = op->root_rank;
    rec.reduce_op   = static_cast<ReduceOp>(op->reduce_op);
    rec.prescale    = op->prescale;
    rec.postscale   = op->postscale;
    rec.stream      = op->stream;
    rec.ready_event = op->ready_event;
    rec.done_event  = op->done_event;
    rec.alloc       = op->alloc;
    rec.alloc_user  = op->alloc_user;
    std::string err;
    int64_t h = CollectiveEngine::Global().Enqueue(std::move(rec), &err);
    if (h < 0) tl_error = err;
    return h;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

int tips_poll(int64_t handle) { return CollectiveEngine::Global().Poll(handle); }
int tips_wait(int64_t handle, int timeout_ms) { return CollectiveEngine::Global().Wait(handle, timeout_ms); }

int tips_handle_error(int64_t handle, char* out, int out_len) {
  auto h = CollectiveEngine::Global().Lookup(handle);
  if (!h || out_len <= 0) return -kInvalidArgument;
  int n = static_cast<int>(h->error.size()) < out_len - 1 ? static_cast<int>(h->error.size()) : out_len - 1;
  memcpy(out, h->error.data(), n);
  out[n] = 0;
  return n;
}

int tips_handle_sizes(int64_t handle, int64_t* out, int n) {
  auto h = CollectiveEngine::Global().Lookup(handle);
  if (!h) return -kInvalidArgument;
  int m = static_cast<int>(h->sizes.size()) < n ? static_cast<int>(h->sizes.size()) : n;
  for (int i = 0; i < m; ++i) out[i] = h->sizes[i];
  return m;
}

void* tips_handle_output(int64_t handle) {
  auto h = CollectiveEngine::Global().Lookup(handle);
  return h ? h->out : nullptr;
}

int tips_release(int64_t handle) {
  CollectiveEngine::Global().Release(handle);
  return 0;
}

int tips_set_device_executor(void* fn) {
  CollectiveEngine::Global().SetDeviceExecutor(reinterpret_cast<DeviceExecutorFn>(fn));
  return 0;
}

int tips_take_negotiated_order(char* out, int out_len) {
  std::vector<std::string> names = CollectiveEngine::Global().TakeNegotiatedOrder();
  std::string joined;
  for (size_t i = 0; i < names.size(); ++i) joined += (i ? "\n" : "") + names[i];
  if (static_cast<int>(joined.size()) >= out_len) return Fail(kInvalidArgument, "buffer too small");
  memcpy(out, joined.data(), joined.size());
  out[joined.size()] = 0;
  return static_cast<int>(names.size());
}

int tips_freeze_schedule(const char* names) {
  return Guard([&] {
    std::vector<std::string> v;
    std::istringstream ss(names ? names : "");
    std::string line;
    while (std::getline(ss, line))
      if (!line.empty()) v.push_back(line);
    Status st = CollectiveEngine::Global().FreezeSchedule(v);
    return st.ok() ? 0 : Fail(st);
  });
}

int tips_thaw_schedule(void) {
  CollectiveEngine::Global().ThawSchedule();
  return 0;
}

int tips_reset_collectives(void) {
  return Guard([&] {
    Status st = CollectiveEngine::Global().Reset();
    return st.ok() ? 0 : Fail(st);
  });
}

int tips_timeline_enable(int on) {
  CollectiveEngine::Global().EnableTimeline(on != 0);
  return 0;
}

int tips_timeline_dump(const char* path) {
  return Guard([&] {
    Status st = CollectiveEngine::Global().DumpTimeline(path);
    return st.ok() ? 0 : Fail(st);
  });
}

const char* tips_counter_names(void) {
  return "ops_enqueued,ops_completed,ops_failed,allreduce_bytes,allgather_bytes,broadcast_bytes,"
         "negotiation_requests,responses,fused_groups,fused_tensors,frozen_executions,stall_warnings,"
         "rpc_messages_sent,rpc_messages_received";
}

int tips_counters(uint64_t* out, int n) {
  EngineCounters& c = CollectiveEngine::Global().counters();
  uint64_t v[] = {c.ops_enqueued.load(),     c.ops_completed.load(),        c.ops_failed.load(),
                  c.allreduce_bytes.load(),  c.allgather_bytes.load(),      c.broadcast_bytes.load(),
                  c.negotiation_requests.load(), c.responses.load(),        c.fused_groups.load(),
                  c.fused_tensors.load(),    c.frozen_executions.load(),    c.stall_warnings.load(),
                  RpcServer::Global().messages_sent(), RpcServer::Global().messages_received()};
  int m = static_cast<int>(sizeof(v) / sizeof(v[0]));
  if (n < m) m = n;
  for (int i = 0; i < m; ++i) out[i] = v[i];
  return m;
}

int tips_set_log_level(int min_level, int verbose) {
  LogConfig::MinLevel()     = min_level;
  LogConfig::VerboseLevel() = verbose;
  return 0;
}

/* Cost of the control-plane messages, the counterpart of the reference's serializer timing test
 * (tips/core/message/flatbuffers_test.cc:12-66, 1000 x build / read of a message): `iters` round trips of a
 * request (name of 24 characters, 4 dimensions) and of a response (8 fused tensor names) through the wire format.
 * out = {request encode, request decode, response encode, response decode} in nanoseconds per message. */
int tips_bench_messages(int iters, double* out4) {
  using namespace tips::collective;
  if (iters < 1) iters = 1;
  RequestMessage req;
  req.request_rank = 3;
  req.tensor_name  = "tips.opt0.bucket.17.grad";
  req.tensor_shape = {256, 3, 224, 224};
  ResponseMessage resp;
  resp.response_type = ResponseType::kAllreduce;
  for (int i = 0; i < 8; ++i) resp.tensor_names.push_back("tips.opt0.bucket." + std::to_string(i));
  resp.tensor_sizes = {1, 2, 3, 4, 5, 6, 7, 8};
  auto now = [] { return std::chrono::steady_clock::now(); };
  auto ns  = [&](std::chrono::steady_clock::time_point a) {
    return std::chrono::duration<double, std::nano>(now() - a).count() / iters;
  };
  volatile int64_t sink = 0;
  NaiveBuffer rbuf, pbuf;
  auto t = now();
  for (int i = 0; i < iters; ++i) {
    NaiveBuffer b;
    req.request_rank = i;
    req.Serialize(&b);
    sink += static_cast<int64_t>(b.size());
    if (i == 0) rbuf = b;
  }
  out4[0] = ns(t);
  t       = now();
  for (int i = 0; i < iters; ++i) {
    NaiveBuffer b(rbuf.data(), rbuf.size());
    RequestMessage m;
    m.Deserialize(&b);
    sink += m.NumElements();
  }
  out4[1] = ns(t);
  t       = now();
  for (int i = 0; i < iters; ++i) {
    NaiveBuffer b;
    resp.root_rank = i;
    resp.Serialize(&b);
    sink += static_cast<int64_t>(b.size());
    if (i == 0) pbuf = b;
  }
  out4[2] = ns(t);
  t       = now();
  for (int i = 0; i < iters; ++i) {
    NaiveBuffer b(pbuf.data(), pbuf.size());
    ResponseMessage m;
    m.Deserialize(&b);
    sink += static_cast<int64_t>(m.tensor_names.size());
  }
  out4[3] = ns(t);
  (void)sink;
  return 0;
}

int tips_inject_drop_requests(int dst_rank, int n) {
  RpcServer::Global().InjectDropRequests(dst_rank, n);
  return 0;
}

}  // extern "C"
