// Multi-rank test of the host runtime through its C API, as one executable: the parent forks one child per rank
// (before any thread exists), every child initialises the runtime over TCP on 127.0.0.1, runs negotiated
// allreduce / allgather / broadcast on host buffers (several tensors in flight, so the coordinator fuses them),
// a host barrier and the sparse and dense parameter-server tables, checks every value and shuts down.
// Exit code 0 = every rank passed.  The same source is linked against the ThreadSanitizer and AddressSanitizer
// builds of the library; the reference's multi-process tests run under mpirun instead
// (tips/core/collective/coordinator_test.cc, tips/core/ps/ps_server_test.cc:55-131).
//
//   ranks_test [ranks=3] [port=0 -> derived from the pid]
#include <sys/wait.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "tips_c_api.h"

extern "C" {
int64_t tips_ps_table_create(const char* name, const int* servers, int nservers, int local_shards, int rule, double lr,
                             double eps);
int tips_ps_table_destroy(int64_t id);
int tips_ps_pull(int64_t id, const uint64_t* keys, int64_t n, int dtype, int length, void* out, int timeout_ms);
int64_t tips_ps_push(int64_t id, const uint64_t* keys, int64_t n, int dtype, int length, const void* values,
                     int timeout_ms);
int64_t tips_ps_dense_create(const char* name, const int* servers, int nservers, int local_shards, int64_t size,
                             int rule, double lr, double eps);
int tips_ps_dense_destroy(int64_t id);
int tips_ps_dense_pull(int64_t id, int64_t begin, int64_t end, float* out, int timeout_ms);
int tips_ps_dense_push(int64_t id, int64_t begin, int64_t end, const float* values, int op, int timeout_ms);
}

static int g_failed = 0;
#define EXPECT(cond)                                                               \
  do {                                                                             \
    if (!(cond)) {                                                                 \
      fprintf(stderr, "rank %d FAILED %s:%d: %s\n", g_rank, __FILE__, __LINE__, #cond); \
      ++g_failed;                                                                  \
    }                                                                              \
  } while (0)
static int g_rank = -1;

static int64_t Enqueue(const char* name, int type, const float* in, float* out, int64_t n, int root) {
  tips_op_t op;
  memset(&op, 0, sizeof(op));
  op.name      = name;
  op.type      = type;
  op.dtype     = 0;  // fp32
  op.ndim      = 1;
  op.shape     = &n;
  op.in        = in;
  op.out       = out;
  op.root_rank = root;
  op.prescale  = 1.0;
  op.postscale = 1.0;
  return tips_enqueue(&op);
}

static int RunRank(int rank, int size, int port) {
  g_rank = rank;
  if (tips_init_ex(rank, size, "127.0.0.1", port) != 0) {
    fprintf(stderr, "rank %d: init failed: %s\n", rank, tips_last_error());
    return 1;
  }
  EXPECT(tips_rank() == rank && tips_size() == size);
  for (int step = 0; step < 3; ++step) {
    // eight allreduces in flight at once (fused by the coordinator), sizes 1..4097
    const int64_t sizes[8] = {1, 7, 64, 255, 1024, 1025, 4096, 4097};
    std::vector<std::vector<float>> in(8), out(8);
    std::vector<int64_t> h(8);
    std::vector<std::string> names(8);
    for (int t = 0; t < 8; ++t) {
      in[t].resize(sizes[t]);
      out[t].assign(sizes[t], -1.f);
      for (int64_t i = 0; i < sizes[t]; ++i) in[t][i] = static_cast<float>((rank + 1) * (i % 13 + 1) + step);
      names[t] = "ar." + std::to_string(t);
      h[t]     = Enqueue(names[t].c_str(), 0, in[t].data(), out[t].data(), sizes[t], 0);
      EXPECT(h[t] > 0);
    }
    for (int t = 0; t < 8; ++t) {
      EXPECT(tips_wait(h[t], 60000) == 0);
      tips_release(h[t]);
      for (int64_t i = 0; i < sizes[t]; ++i) {
        const float want = static_cast<float>(size * (size + 1) / 2 * (i % 13 + 1) + size * step);
        if (out[t][i] != want) {
          EXPECT(out[t][i] == want);
          break;
        }
      }
    }
    // broadcast from the last rank
    std::vector<float> b(300, static_cast<float>(rank * 10 + step));
    int64_t hb = Enqueue("bc", 2, b.data(), b.data(), 300, size - 1);
    EXPECT(hb > 0 && tips_wait(hb, 60000) == 0);
    tips_release(hb);
    EXPECT(b[0] == static_cast<float>((size - 1) * 10 + step) && b[299] == b[0]);
    // allgather of equal parts
    std::vector<float> g(5, static_cast<float>(rank)), go(5 * size, -1.f);
    int64_t hg = Enqueue("ag", 1, g.data(), go.data(), 5, 0);
    EXPECT(hg > 0 && tips_wait(hg, 60000) == 0);
    tips_release(hg);
    for (int r = 0; r < size; ++r) EXPECT(go[5 * r] == static_cast<float>(r) && go[5 * r + 4] == static_cast<float>(r));
    EXPECT(tips_barrier() == 0);
  }
  // sparse table on ranks {0, 1}: every rank pushes a gradient of ones for three keys
  {
    int servers[2] = {0, size > 1 ? 1 : 0};
    int64_t id = tips_ps_table_create("rt", servers, size > 1 ? 2 : 1, 2, 0, 0.5, 1e-8);
    EXPECT(id > 0);
    EXPECT(tips_barrier() == 0);
    uint64_t keys[3] = {3, 200, 0x123456789abull};
    float rows[12];
    EXPECT(tips_ps_pull(id, keys, 3, 0, 4, rows, 60000) == 0);
    EXPECT(tips_barrier() == 0);
    float ones[12];
    for (float& v : ones) v = 1.f;
    EXPECT(tips_ps_push(id, keys, 3, 0, 4, ones, 60000) == 0);
    EXPECT(tips_barrier() == 0);
    EXPECT(tips_ps_pull(id, keys, 3, 0, 4, rows, 60000) == 0);
    for (float v : rows) EXPECT(std::fabs(v + 0.5f * size) < 1e-6f);
    EXPECT(tips_barrier() == 0);
    tips_ps_table_destroy(id);
  }
  // dense table over every rank
  {
    std::vector<int> servers(size);
    for (int r = 0; r < size; ++r) servers[r] = r;
    int64_t id = tips_ps_dense_create("rd", servers.data(), size, 2, 1000, 0, 0.1, 1e-8);
    EXPECT(id > 0);
    EXPECT(tips_barrier() == 0);
    std::vector<float> g(1000, 1.f), w(1000, 7.f);
    EXPECT(tips_ps_dense_push(id, 0, 1000, g.data(), 0, 60000) == 0);
    EXPECT(tips_barrier() == 0);
    EXPECT(tips_ps_dense_pull(id, 0, 1000, w.data(), 60000) == 0);
    for (float v : w) {
      if (std::fabs(v + 0.1f * size) > 1e-6f) {
        EXPECT(std::fabs(v + 0.1f * size) <= 1e-6f);
        break;
      }
    }
    EXPECT(tips_barrier() == 0);
    tips_ps_dense_destroy(id);
  }
  EXPECT(tips_shutdown() == 0);
  if (getenv("TIPS_TEST_VERBOSE")) fprintf(stderr, "rank %d of %d: %d failed expectations\n", rank, size, g_failed);
  return g_failed ? 1 : 0;
}

int main(int argc, char** argv) {
  const int size = argc > 1 ? atoi(argv[1]) : 3;
  int port       = argc > 2 ? atoi(argv[2]) : 0;
  if (port == 0) port = 20000 + static_cast<int>(getpid() % 20000);
  std::vector<pid_t> kids;
  for (int r = 0; r < size; ++r) {
    pid_t pid = fork();
    if (pid == 0) _exit(RunRank(r, size, port));
    kids.push_back(pid);
  }
  int bad = 0;
  for (pid_t pid : kids) {
    int status = 0;
    waitpid(pid, &status, 0);
    if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) ++bad;
  }
  if (bad) fprintf(stderr, "%d of %d ranks failed\n", bad, size);
  return bad ? 1 : 0;
}
