// extern "C" surface of the host parameter server (the reference has no binding for
// its parameter server at all: it is reachable only from C++ tests,
// tips/core/ps/ps_server_test.cc, ps_client_test.cc).
//
// A "ps table" handle bundles a SparseTable, the PsServer that serves its local shards and a
// PsClient.  Creation is collective in the sense that every rank must create the same tables
// with the same names and server lists, then synchronise (tips_barrier) before the first
// pull, so that the RPC services exist everywhere.
#include <cstring>
#include <map>
#include <memory>
#include <mutex>

#include "ps/dense_server.h"
#include "ps/ps_server.h"
#include "runtime/context.h"

using namespace tips;
using namespace tips::ps;

namespace {

struct PsBundle {
  std::unique_ptr<SparseTable> table;
  std::unique_ptr<PsServer> server;
  std::unique_ptr<PsClient> client;
};

struct DenseBundle {
  std::unique_ptr<DenseTable<float>> table;
  std::unique_ptr<DensePsServer> server;
  std::unique_ptr<DensePsClient> client;
};

std::mutex g_mu;
// Calls in flight that were started with the *_async entry points, by handle.
struct AsyncCall {
  std::shared_ptr<PsFuture> future;
  bool is_pull{false};
};
std::map<int64_t, AsyncCall> g_calls;
int64_t g_next_call = 1;
std::map<int64_t, std::unique_ptr<PsBundle>> g_tables;
std::map<int64_t, std::unique_ptr<DenseBundle>> g_dense;
int64_t g_next = 1;
thread_local std::string tl_ps_error;

int Fail(int code, const std::string& m) {
  tl_ps_error = m;
  return -code;
}

PsBundle* Get(int64_t id) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_tables.find(id);
  return it == g_tables.end() ? nullptr : it->second.get();
}

DenseBundle* GetDense(int64_t id) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_dense.find(id);
  return it == g_dense.end() ? nullptr : it->second.get();
}

}  // namespace

extern "C" {

const char* tips_ps_last_error(void) { return tl_ps_error.c_str(); }

/* rule: 0 SGD (w -= lr*g), 1 Adagrad, 2 the reference's literal rule (w = lr*g). */
int64_t tips_ps_table_create(const char* name, const int* servers, int nservers, int local_shards, int rule, double lr,
                             double eps) {
  try {
    Context& ctx = Context::Global();
    if (!ctx.initialized()) return Fail(kPrecondition, "tips is not initialised");
    std::vector<int> sv(servers, servers + nservers);
    for (int s : sv)
      if (s < 0 || s >= ctx.size()) return Fail(kInvalidArgument, "server rank out of range");
    auto b   = std::make_unique<PsBundle>();
    b->table = std::make_unique<SparseTable>(sv, ctx.rank(), local_shards);
    std::shared_ptr<PushAccessMethod> push;
    if (rule == 0)
      push = std::make_shared<SparseTableSgdPushAccess>(lr);
    else if (rule == 1)
      push = std::make_shared<AdagradPushAccess>(lr, eps);
    else if (rule == 2)
      push = std::make_shared<LiteralReferencePushAccess>(lr);
    else
      return Fail(kInvalidArgument, "unknown update rule");
    b->server = std::make_unique<PsServer>(name, b->table.get(), std::make_shared<SparseTablePullAccess>(), push);
    b->server->Start();
    b->client = std::make_unique<PsClient>(name, b->table.get(), ctx.rank());
    std::lock_guard<std::mutex> lock(g_mu);
    int64_t id   = g_next++;
    g_tables[id] = std::move(b);
    return id;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

int tips_ps_table_destroy(int64_t id) {
  std::unique_ptr<PsBundle> b;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_tables.find(id);
    if (it == g_tables.end()) return 0;
    b = std::move(it->second);
    g_tables.erase(it);
  }
  b->server->Stop();
  return 0;
}

/* Pulls n rows of `length` elements of `dtype`; out receives n*length elements in key order. */
int tips_ps_pull(int64_t id, const uint64_t* keys, int64_t n, int dtype, int length, void* out, int timeout_ms) {
  try {
    PsBundle* b = Get(id);
    if (!b) return Fail(kInvalidArgument, "unknown ps table");
    auto fut = b->client->PullPacked(keys, static_cast<size_t>(n), static_cast<Datatype>(dtype),
                                     static_cast<uint32_t>(length), out);
    if (!fut->Wait(timeout_ms)) {
      fut->Cancel();  // a late answer must not write into `out` any more
      return Fail(kTimeout, "ps pull timed out");
    }
    if (!fut->status.ok()) return Fail(fut->status.code(), fut->status.message());
    if (fut->bad_rows)
      return Fail(kPrecondition, std::to_string(fut->bad_rows) + " row(s) have a different length or dtype on the server");
    return 0;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

/* Pushes n gradient rows; returns the number of rows that did not exist on their server (>= 0). */
int64_t tips_ps_push(int64_t id, const uint64_t* keys, int64_t n, int dtype, int length, const void* values,
                     int timeout_ms) {
  try {
    PsBundle* b = Get(id);
    if (!b) return Fail(kInvalidArgument, "unknown ps table");
    auto fut = b->client->PushPacked(keys, static_cast<size_t>(n), static_cast<Datatype>(dtype),
                                     static_cast<uint32_t>(length), values);
    if (!fut->Wait(timeout_ms)) return Fail(kTimeout, "ps push timed out");
    if (!fut->status.ok()) return Fail(fut->status.code(), fut->status.message());
    return static_cast<int64_t>(fut->missing_rows);
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

/* Asynchronous forms: the call returns a handle (> 0) at once; tips_ps_wait collects the result.  A pull writes into
 * `out` when the servers answer, so `out` must stay valid until tips_ps_wait returned; `keys` and the pushed `values`
 * are copied into the requests before the call returns. */
int64_t tips_ps_pull_async(int64_t id, const uint64_t* keys, int64_t n, int dtype, int length, void* out) {
  try {
    PsBundle* b = Get(id);
    if (!b) return Fail(kInvalidArgument, "unknown ps table");
    AsyncCall call;
    call.is_pull = true;
    call.future  = b->client->PullPacked(keys, static_cast<size_t>(n), static_cast<Datatype>(dtype),
                                         static_cast<uint32_t>(length), out);
    std::lock_guard<std::mutex> lock(g_mu);
    const int64_t h = g_next_call++;
    g_calls[h]      = std::move(call);
    return h;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

int64_t tips_ps_push_async(int64_t id, const uint64_t* keys, int64_t n, int dtype, int length, const void* values) {
  try {
    PsBundle* b = Get(id);
    if (!b) return Fail(kInvalidArgument, "unknown ps table");
    AsyncCall call;
    call.future = b->client->PushPacked(keys, static_cast<size_t>(n), static_cast<Datatype>(dtype),
                                        static_cast<uint32_t>(length), values);
    std::lock_guard<std::mutex> lock(g_mu);
    const int64_t h = g_next_call++;
    g_calls[h]      = std::move(call);
    return h;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

/* Waits for an asynchronous call.  Returns -kTimeout while it is still running after `timeout_ms` (the handle stays
 * valid; timeout_ms = 0 polls); otherwise the handle is released and the result is 0 for a pull, the number of rows
 * that did not exist for a push, or a negative status. */
int64_t tips_ps_wait(int64_t handle, int timeout_ms) {
  try {
    AsyncCall call;
    {
      std::lock_guard<std::mutex> lock(g_mu);
      auto it = g_calls.find(handle);
      if (it == g_calls.end()) return Fail(kInvalidArgument, "unknown ps call handle");
      call = it->second;
    }
    if (!call.future->Wait(timeout_ms)) return Fail(kTimeout, "ps call still running");
    {
      std::lock_guard<std::mutex> lock(g_mu);
      g_calls.erase(handle);
    }
    if (!call.future->status.ok()) return Fail(call.future->status.code(), call.future->status.message());
    if (call.is_pull) {
      if (call.future->bad_rows)
        return Fail(kPrecondition,
                    std::to_string(call.future->bad_rows) + " row(s) have a different length or dtype on the server");
      return 0;
    }
    return static_cast<int64_t>(call.future->missing_rows);
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

/* Gives up on an asynchronous call: its output buffer is not written after this returns. */
int tips_ps_cancel(int64_t handle) {
  AsyncCall call;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_calls.find(handle);
    if (it == g_calls.end()) return 0;
    call = it->second;
    g_calls.erase(it);
  }
  call.future->Cancel();
  return 0;
}

int64_t tips_ps_table_size(int64_t id) {
  PsBundle* b = Get(id);
  return b ? static_cast<int64_t>(b->table->size()) : -1;
}

int tips_ps_table_server_of(int64_t id, uint64_t key) {
  PsBundle* b = Get(id);
  return b ? b->table->ServerWorldRank(b->table->ToServerId(key)) : -1;
}

int tips_ps_table_save(int64_t id, const char* path, int binary) {
  PsBundle* b = Get(id);
  if (!b) return Fail(kInvalidArgument, "unknown ps table");
  Status st = binary ? b->table->SaveBinary(path) : b->table->WriteToFile(path);
  return st.ok() ? 0 : Fail(st.code(), st.message());
}

int tips_ps_table_load(int64_t id, const char* path, int binary, int dtype) {
  PsBundle* b = Get(id);
  if (!b) return Fail(kInvalidArgument, "unknown ps table");
  Status st = binary ? b->table->LoadBinary(path) : b->table->LoadFromFile(path, static_cast<Datatype>(dtype));
  return st.ok() ? 0 : Fail(st.code(), st.message());
}

int tips_ps_server_counters(int64_t id, uint64_t* rows_pulled, uint64_t* rows_pushed) {
  PsBundle* b = Get(id);
  if (!b) return Fail(kInvalidArgument, "unknown ps table");
  *rows_pulled = b->server->rows_pulled();
  *rows_pushed = b->server->rows_pushed();
  return 0;
}

/* ---- dense tables: `size` fp32 elements range-partitioned over the servers' shards ----
 * rule: 0 SGD (w -= lr*g), 1 Adagrad, 2 the reference's literal rule (w = lr*g).  Creation is collective like the
 * sparse tables': every rank creates the same table, then the ranks synchronise before the first pull. */
int64_t tips_ps_dense_create(const char* name, const int* servers, int nservers, int local_shards, int64_t size,
                             int rule, double lr, double eps) {
  try {
    Context& ctx = Context::Global();
    if (!ctx.initialized()) return Fail(kPrecondition, "tips is not initialised");
    if (size < 0 || rule < 0 || rule > 2) return Fail(kInvalidArgument, "bad size or update rule");
    std::vector<int> sv(servers, servers + nservers);
    for (int s : sv)
      if (s < 0 || s >= ctx.size()) return Fail(kInvalidArgument, "server rank out of range");
    auto b   = std::make_unique<DenseBundle>();
    b->table = std::make_unique<DenseTable<float>>(sv, ctx.rank(), local_shards);
    b->table->Resize(static_cast<size_t>(size));
    b->server = std::make_unique<DensePsServer>(name, b->table.get(), static_cast<DenseRule>(rule), lr, eps);
    b->server->Start();
    b->client = std::make_unique<DensePsClient>(name, b->table.get(), ctx.rank());
    std::lock_guard<std::mutex> lock(g_mu);
    int64_t id  = g_next++;
    g_dense[id] = std::move(b);
    return id;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

int tips_ps_dense_destroy(int64_t id) {
  std::unique_ptr<DenseBundle> b;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_dense.find(id);
    if (it == g_dense.end()) return 0;
    b = std::move(it->second);
    g_dense.erase(it);
  }
  b->server->Stop();
  return 0;
}

/* out receives the elements [begin, end). */
int tips_ps_dense_pull(int64_t id, int64_t begin, int64_t end, float* out, int timeout_ms) {
  try {
    DenseBundle* b = GetDense(id);
    if (!b) return Fail(kInvalidArgument, "unknown dense ps table");
    auto fut = b->client->Pull(static_cast<uint64_t>(begin), static_cast<uint64_t>(end), out);
    if (!fut->Wait(timeout_ms)) return Fail(kTimeout, "dense pull timed out");
    if (!fut->status.ok()) return Fail(fut->status.code(), fut->status.message());
    return 0;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

/* op 0: `values` is the gradient of [begin, end), the owning shards apply the table's rule; op 1: assignment. */
int tips_ps_dense_push(int64_t id, int64_t begin, int64_t end, const float* values, int op, int timeout_ms) {
  try {
    DenseBundle* b = GetDense(id);
    if (!b) return Fail(kInvalidArgument, "unknown dense ps table");
    auto fut = b->client->Push(static_cast<uint64_t>(begin), static_cast<uint64_t>(end), values,
                               static_cast<DensePushOp>(op));
    if (!fut->Wait(timeout_ms)) return Fail(kTimeout, "dense push timed out");
    if (!fut->status.ok()) return Fail(fut->status.code(), fut->status.message());
    if (fut->missing_rows) return Fail(kPrecondition, "dense push: a server rejected a range");
    return 0;
  } catch (const std::exception& e) {
    return Fail(kInternal, e.what());
  }
}

/* Elements stored on this rank, and the sum of them (computed on the shard threads in parallel). */
int tips_ps_dense_local(int64_t id, int64_t* count, double* sum) {
  DenseBundle* b = GetDense(id);
  if (!b) return Fail(kInvalidArgument, "unknown dense ps table");
  std::mutex mu;
  int64_t n = 0;
  double s  = 0;
  b->table->ForEach([&](size_t, float& v) {
    std::lock_guard<std::mutex> lock(mu);
    ++n;
    s += v;
  });
  *count = n;
  *sum   = s;
  return 0;
}

int tips_ps_dense_save(int64_t id, const char* path) {
  DenseBundle* b = GetDense(id);
  if (!b) return Fail(kInvalidArgument, "unknown dense ps table");
  Status st = b->table->Save(path);
  return st.ok() ? 0 : Fail(st.code(), st.message());
}

int tips_ps_dense_load(int64_t id, const char* path) {
  DenseBundle* b = GetDense(id);
  if (!b) return Fail(kInvalidArgument, "unknown dense ps table");
  Status st = b->table->Load(path);
  return st.ok() ? 0 : Fail(st.code(), st.message());
}

int tips_ps_dense_counters(int64_t id, uint64_t* pulled, uint64_t* pushed) {
  DenseBundle* b = GetDense(id);
  if (!b) return Fail(kInvalidArgument, "unknown dense ps table");
  *pulled = b->server->elements_pulled();
  *pushed = b->server->elements_pushed();
  return 0;
}

}  // extern "C"
