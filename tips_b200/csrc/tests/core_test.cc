// Unit tests of the native L0 utilities; the cases mirror the reference's gtest files
// (tips/core/common/channel_test.cc, naive_buffer_test.cc, thread_group_test.cc, any_vec_test.cc)
// with value assertions throughout.  Plain executable: exit code 0 = all passed.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <thread>

#include "collective/coordinator.h"
#include "core/channel.h"
#include "core/common.h"
#include "core/datatype.h"
#include "core/naive_buffer.h"
#include "core/threads.h"
#include "ps/access_method.h"
#include "ps/ps_messages.h"

using namespace tips;

static int g_failed = 0;
#define EXPECT(cond)                                                    \
  do {                                                                  \
    if (!(cond)) {                                                      \
      fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++g_failed;                                                       \
    }                                                                   \
  } while (0)

static void TestChannel() {
  Channel<int> ch;
  std::thread w([&] {
    for (int i = 0; i < 100; ++i) EXPECT(ch.Write(i));
    ch.Close();
  });
  int v, n = 0, sum = 0;
  while (ch.Read(&v)) {
    sum += v;
    ++n;
  }
  w.join();
  EXPECT(n == 100 && sum == 4950);
  EXPECT(!ch.Write(1));
  // 5 writers, 3 readers, bounded capacity
  Channel<int> bounded(4);
  std::atomic<int> total{0}, count{0};
  std::vector<std::thread> ts;
  for (int i = 0; i < 5; ++i) ts.emplace_back([&] { for (int k = 1; k <= 50; ++k) bounded.Write(k); });
  std::vector<std::thread> rs;
  for (int i = 0; i < 3; ++i)
    rs.emplace_back([&] {
      int x;
      while (bounded.Read(&x)) {
        total += x;
        count++;
      }
    });
  for (auto& t : ts) t.join();
  bounded.Close();
  for (auto& t : rs) t.join();
  EXPECT(count == 250 && total == 5 * 1275);
  Channel<int> timed;
  EXPECT(timed.ReadFor(&v, 20) == 0);
  timed.Close();
  EXPECT(timed.ReadFor(&v, 20) == -1);
}

static void TestNaiveBuffer() {
  NaiveBuffer buf;
  std::string s = "hello world!";
  std::vector<int64_t> shape{3, 4, 5};
  buf << 1.23 << 123 << true << s << shape << static_cast<uint8_t>(7);
  NaiveBuffer rd(buf.data(), buf.size());
  double d; int i; bool b; std::string s2; std::vector<int64_t> sh2; uint8_t u;
  rd >> d >> i >> b >> s2 >> sh2 >> u;
  EXPECT(d == 1.23 && i == 123 && b && s2 == s && sh2 == shape && u == 7);
  EXPECT(rd.free_size() == 0);
  bool threw = false;
  try { rd >> i; } catch (const FatalError&) { threw = true; }
  EXPECT(threw);
  // wire format: string = u64 length + bytes
  NaiveBuffer w;
  w << std::string("ab");
  EXPECT(w.size() == 10 && w.bytes()[0] == 2 && w.bytes()[8] == 97);
  // builders
  NaiveBuffer tb;
  StructBuilder st(&tb);
  st.NewField<Int32Builder>("rank")->set(3);
  st.NewField<StringBuilder>("name")->set("grad/w");
  st.NewField<PrimaryListBuilder<int64_t>>("shape")->set(shape);
  st.Flush();
  NaiveBuffer tr(tb.data(), tb.size());
  StructBuilder st2(&tr);
  auto* r = st2.NewField<Int32Builder>("rank");
  auto* n = st2.NewField<StringBuilder>("name");
  auto* sh = st2.NewField<PrimaryListBuilder<int64_t>>("shape");
  st2.Load();
  EXPECT(r->data() == 3 && n->data() == "grad/w" && sh->data() == shape);
  // files
  const char* path = "/tmp/tips_naive_buffer_test.bin";
  buf.SaveToFile(path);
  buf.AppendToFile(path);
  NaiveBuffer f;
  f.LoadFromFile(path, buf.size(), buf.size());
  EXPECT(f.size() == buf.size() && memcmp(f.data(), buf.data(), buf.size()) == 0);
  remove(path);
}

static void TestThreads() {
  ThreadGroup group(4);
  std::atomic<int> hits{0};
  std::vector<int> ids(4, -1);
  group.Run([&](int tid) {
    ids[tid] = ThreadGroup::thread_id();
    hits++;
    group.BarrierWait();
  });
  EXPECT(hits == 4);
  for (int i = 0; i < 4; ++i) EXPECT(ids[i] == i);
  group.SetThreadNum(3);
  std::vector<int> data(1000, 1);
  std::atomic<long> sum{0};
  ParallelRunRange(group, data.size(), [&](int, size_t b, size_t e) {
    long s = 0;
    for (size_t i = b; i < e; ++i) s += data[i];
    sum += s;
  });
  EXPECT(sum == 1000);
  ManagedThread mt;
  int x = 0;
  mt.Start([&] { x = 42; });
  mt.Join();
  EXPECT(x == 42);
  mt.Start([&] { x = 43; });
  mt.Join();
  EXPECT(x == 43);
  ThreadPool pool(3);
  EXPECT(pool.parallel_num() == 3);
  auto f1 = pool.Submit([] { return 7; });
  auto f2 = pool.Submit([] { return std::string("ok"); });
  EXPECT(f1.get() == 7 && f2.get() == "ok");
  Semaphore sem(0);
  std::thread poster([&] { sem.Post(); });
  sem.Wait();
  poster.join();
  EXPECT(!sem.TryWait());
  RWLock lock;
  { RWLockReadGuard a(lock); RWLockReadGuard b(lock); }
  { RWLockWriteGuard w(lock); }
}

template <typename T>
static void TestAnyVecTyped(Datatype dt) {
  AnyVec a(dt, 5), b(dt, 5), c(dt, 5);
  auto va = a.ToVec<T>(), vb = b.ToVec<T>();
  for (int i = 0; i < 5; ++i) {
    va[i] = static_cast<T>(i + 1);
    vb[i] = static_cast<T>(2 * i);
  }
  AnyVec::Add(a, b, &c);
  for (int i = 0; i < 5; ++i) EXPECT(c.ToVec<T>()[i] == static_cast<T>(3 * i + 1));
  AnyVec::Mul(a, b, &c);
  for (int i = 0; i < 5; ++i) EXPECT(c.ToVec<T>()[i] == static_cast<T>((i + 1) * 2 * i));
  AnyVec::Mul(a, 3.0, &c);
  for (int i = 0; i < 5; ++i) EXPECT(c.ToVec<T>()[i] == static_cast<T>(3 * (i + 1)));
  AnyVec shadow = a.ShadowCopy();
  EXPECT(!shadow.own_data() && shadow.buffer() == a.buffer());
  AnyVec deep = a.Copy();
  EXPECT(deep.own_data() && deep.buffer() != a.buffer() && deep.ToVec<T>()[4] == static_cast<T>(5));
  EXPECT(va.dot(vb) == static_cast<T>(0 + 4 + 12 + 24 + 40));
}

static void TestDatatypes() {
  TestAnyVecTyped<float>(Datatype::kFp32);
  TestAnyVecTyped<double>(Datatype::kFp64);
  TestAnyVecTyped<int32_t>(Datatype::kInt32);
  TestAnyVecTyped<int64_t>(Datatype::kInt64);
  EXPECT(DatatypeNumBytes(Datatype::kInt8) == 1 && DatatypeNumBytes(Datatype::kBf16) == 2);
  EXPECT(std::string(DatatypeName(Datatype::kFp16)) == "fp16" && DatatypeFromName("int64") == Datatype::kInt64);
  for (float f : {0.f, 1.f, -2.5f, 3.14159f, 65504.f, 1e-5f}) {
    EXPECT(std::fabs(Bf16ToFloat(FloatToBf16(f)) - f) <= std::fabs(f) * 0.008f + 1e-30f);
    EXPECT(std::fabs(Fp16ToFloat(FloatToFp16(f)) - f) <= std::fabs(f) * 0.001f + 1e-7f);
  }
  float data[3] = {1.5f, 2.f, -3.f};
  Vec<float> v(data, 3);
  EXPECT(v.ToStr() == "Vec:\t1.5 2 -3 ");
  v *= 2.f;
  EXPECT(data[0] == 3.f && v.sum() == 1.f);
  OrderedMap<std::string, int> om;
  om.Set("b", 1);
  om.Set("a", 2);
  om.Set("b", 3);
  EXPECT(om.size() == 2 && om.items()[0].first == "b" && om.Get("b") == 3 && om.Has("a") && !om.Has("c"));
  EXPECT(StringFormat("%d-%s", 7, "x") == "7-x");
  EXPECT(ToString(std::vector<int>{1, 2, 3}) == "[1, 2, 3]");
  EXPECT(!GetLocalIp().empty());
  int calls = 0;
  EXPECT(ignore_signal_call([&](int) { ++calls; errno = EINTR; return calls < 3 ? -1 : 5; }, 0) == 5 && calls == 3);
}

static void TestNegotiationTable() {
  using namespace collective;
  MessageTable table;
  auto mk = [](int rank, std::vector<int64_t> shape, Datatype dt = Datatype::kFp32, RequestType t = RequestType::kAllreduce) {
    RequestMessage m;
    m.request_rank = rank;
    m.tensor_name  = "t";
    m.tensor_shape = std::move(shape);
    m.tensor_type  = dt;
    m.request_type = t;
    return m;
  };
  EXPECT(!IncreTensorCount(&table, mk(1, {4, 2}), nullptr, 3));
  EXPECT(!IncreTensorCount(&table, mk(0, {4, 2}), nullptr, 3));
  EXPECT(IncreTensorCount(&table, mk(2, {4, 2}), nullptr, 3));
  ResponseMessage ok = ConstructResponseMessage(&table, "t", 3);
  EXPECT(ok.response_type == ResponseType::kAllreduce && table.empty());
  IncreTensorCount(&table, mk(0, {4, 2}), nullptr, 2);
  IncreTensorCount(&table, mk(1, {4, 3}), nullptr, 2);
  ResponseMessage bad = ConstructResponseMessage(&table, "t", 2);
  EXPECT(bad.response_type == ResponseType::kError && bad.error_message.find("shapes") != std::string::npos);
  IncreTensorCount(&table, mk(0, {4}, Datatype::kFp32), nullptr, 2);
  IncreTensorCount(&table, mk(1, {4}, Datatype::kInt32), nullptr, 2);
  EXPECT(ConstructResponseMessage(&table, "t", 2).error_message.find("data types") != std::string::npos);
  IncreTensorCount(&table, mk(0, {1, 5}, Datatype::kFp32, RequestType::kAllgather), nullptr, 2);
  IncreTensorCount(&table, mk(1, {3, 5}, Datatype::kFp32, RequestType::kAllgather), nullptr, 2);
  ResponseMessage g = ConstructResponseMessage(&table, "t", 2);
  EXPECT(g.response_type == ResponseType::kAllgather && g.tensor_sizes == (std::vector<int64_t>{1, 3}));
  NaiveBuffer b;
  g.Serialize(&b);
  NaiveBuffer r(b.data(), b.size());
  ResponseMessage g2;
  g2.Deserialize(&r);
  EXPECT(g2.tensor_sizes == g.tensor_sizes && g2.tensor_names == g.tensor_names);
}

static void TestPsPieces() {
  using namespace ps;
  SparseTable table({0}, 0, 4);
  PullAccessAgent pull(&table, std::make_shared<SparseTablePullAccess>());
  PushAccessAgent sgd(&table, std::make_shared<SparseTableSgdPushAccess>(0.01));
  AnyVec got;
  pull.GetPullValue(42, Datatype::kFp32, 4, &got);
  EXPECT(got.size() == 4 && got.ToVec<float>()[0] == 0.f && table.size() == 1);
  AnyVec grad(Datatype::kFp32, 4);
  grad.ToVec<float>().Fill(1.f);
  EXPECT(sgd.ApplyPushValue(42, grad));
  EXPECT(!sgd.ApplyPushValue(43, grad));
  EXPECT(std::fabs(table.Find(42)->ToVec<float>()[0] + 0.01f) < 1e-7f);
  PushAccessAgent literal(&table, std::make_shared<LiteralReferencePushAccess>(0.01));
  literal.ApplyPushValue(42, grad);
  EXPECT(std::fabs(table.Find(42)->ToVec<float>()[0] - 0.01f) < 1e-7f);
  PushAccessAgent ada(&table, std::make_shared<AdagradPushAccess>(0.1, 0.0));
  table.Find(42)->ToVec<float>().Fill(1.f);
  ada.ApplyPushValue(42, grad);  // G = 1 -> w = 1 - 0.1
  EXPECT(std::fabs(table.Find(42)->ToVec<float>()[0] - 0.9f) < 1e-6f);
  // placement: one rule, every shard index in range, servers balanced-ish
  SparseTable multi({0, 1, 2, 3}, 2, 2);
  int per_server[4] = {0, 0, 0, 0};
  for (uint64_t k = 0; k < 4000; ++k) {
    int s = multi.ToServerId(k), l = multi.ToLocalShard(k);
    EXPECT(s >= 0 && s < 4 && l >= 0 && l < 2);
    per_server[s]++;
  }
  for (int s = 0; s < 4; ++s) EXPECT(per_server[s] > 800 && per_server[s] < 1200);
  EXPECT(multi.server_index() == 2 && multi.shard_num() == 8);
  DenseTable<float> dense({0}, 0, 3);
  dense.Resize(10);
  *dense.Lookup(9) = 2.5f;
  EXPECT(dense.ShardOf(0) == 0 && dense.ShardOf(9) == 2 && *dense.Lookup(9) == 2.5f);
  EXPECT(dense.Save("/tmp/tips_dense_test.bin").ok());
  DenseTable<float> dense2({0}, 0, 2);
  dense2.Resize(10);
  EXPECT(dense2.Load("/tmp/tips_dense_test.bin").ok() && *dense2.Lookup(9) == 2.5f);
  // text dump round trip
  EXPECT(table.WriteToFile("/tmp/tips_sparse_test.txt").ok());
  SparseTable again({0}, 0, 2);
  EXPECT(again.LoadFromFile("/tmp/tips_sparse_test.txt", Datatype::kFp32).ok());
  EXPECT(again.size() == 1 && std::fabs(again.Find(42)->ToVec<float>()[0] - 0.9f) < 1e-5f);
  EXPECT(table.SaveBinary("/tmp/tips_sparse_test.bin").ok());
  SparseTable bin({0}, 0, 1);
  EXPECT(bin.LoadBinary("/tmp/tips_sparse_test.bin").ok() && bin.Find(42)->ToVec<float>()[3] == table.Find(42)->ToVec<float>()[3]);
  PullRequest req;
  req.meta = {3, 9};
  req.keys = {1, 2};
  req.dtypes = {0, 0};
  req.lengths = {4, 8};
  NaiveBuffer b;
  req.Serialize(&b);
  NaiveBuffer r(b.data(), b.size());
  PullRequest req2;
  req2.Deserialize(&r);
  EXPECT(req2.meta.message_id == 9 && req2.lengths == req.lengths);
  // packed form of a uniform request: the header can be measured and parsed without touching the row block
  PackedHeader ph;
  ph.meta   = {5, 77};
  ph.dtype  = Datatype::kFp32;
  ph.length = 4;
  ph.keys   = {10, 11, 12};
  NaiveBuffer pb;
  ph.Serialize(&pb);
  const size_t header_bytes = pb.size();
  const float block[12]     = {1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12};
  pb.WriteRaw(block, sizeof(block));
  EXPECT(PackedHeader::EncodedSize(pb.data(), pb.size()) == header_bytes);
  EXPECT(PackedHeader::EncodedSize(pb.data(), 10) == 0);                 // shorter than the fixed fields
  EXPECT(PackedHeader::EncodedSize(pb.data(), header_bytes - 1) == 0);  // key array cut short
  NaiveBuffer hb(pb.data(), header_bytes);
  PackedHeader ph2;
  ph2.Deserialize(&hb);
  EXPECT(ph2.meta.client_id == 5 && ph2.meta.message_id == 77 && ph2.keys == ph.keys && ph2.row_bytes() == 16);
  EXPECT(memcmp(pb.data() + header_bytes + 2 * ph2.row_bytes(), block + 8, 16) == 0);
  // find-or-create leaves an empty row for the caller to fill; Adagrad's typed path equals the generic one
  bool created = false;
  AnyVec* fresh = table.FindOrCreate(4242, &created);
  EXPECT(created && fresh != nullptr && fresh->size() == 0);
  EXPECT(table.FindOrCreate(4242, &created) == fresh && !created);
  {
    SparseTable t32({0}, 0, 1), t64({0}, 0, 1);
    PullAccessAgent p32(&t32, std::make_shared<SparseTablePullAccess>()), p64(&t64, std::make_shared<SparseTablePullAccess>());
    PushAccessAgent a32(&t32, std::make_shared<AdagradPushAccess>(0.05, 1e-8)), a64(&t64, std::make_shared<AdagradPushAccess>(0.05, 1e-8));
    AnyVec tmp;
    p32.GetPullValue(1, Datatype::kFp32, 3, &tmp);
    p64.GetPullValue(1, Datatype::kFp64, 3, &tmp);
    for (int step = 0; step < 3; ++step) {
      AnyVec g32(Datatype::kFp32, 3), g64(Datatype::kFp64, 3);
      for (int i = 0; i < 3; ++i) {
        g32.ToVec<float>()[i]  = 0.25f * (i + 1) * (step + 1);
        g64.ToVec<double>()[i] = 0.25 * (i + 1) * (step + 1);
      }
      EXPECT(a32.ApplyPushValue(1, g32) && a64.ApplyPushValue(1, g64));
    }
    for (int i = 0; i < 3; ++i)
      EXPECT(std::fabs(t32.Find(1)->ToVec<float>()[i] - t64.Find(1)->ToVec<double>()[i]) < 1e-6);
  }
  WorkerParamCache cache;
  cache.SetParam(1, grad);
  cache.AccumulateGrad(1, grad);
  cache.AccumulateGrad(1, grad);
  auto grads = cache.TakeGrads();
  EXPECT(grads.size() == 1 && grads[1].ToVec<float>()[0] == 2.f && cache.num_params() == 1);
}

int main() {
  TestChannel();
  TestNaiveBuffer();
  TestThreads();
  TestDatatypes();
  TestNegotiationTable();
  TestPsPieces();
  if (g_failed) {
    fprintf(stderr, "%d checks failed\n", g_failed);
    return 1;
  }
  printf("all native core tests passed\n");
  return 0;
}
