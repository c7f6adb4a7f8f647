/* C API of the native runtime (libtips_core.so).
 *
 * Lifecycle parity with the reference's exported functions
 * (tips/core/operations.h:7-21): tips_init, tips_shutdown, tips_is_initialize,
 * tips_size, tips_rank.  tips_is_initialized is the spelling the reference's
 * Python loader expects (tips/tensorflow/basics.py:25); both are exported.
 * Everything below the lifecycle block has no C counterpart in the reference,
 * which reaches its engine only through TensorFlow ops (tips/tensorflow/ops.cc).
 *
 * All functions return 0 / a non-negative value on success and a negative
 * tips status code on failure unless stated otherwise; tips_last_error() gives
 * the message of the calling thread's last failure.
 */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- lifecycle -------------------------------------------------------- */
/* Rank, size and rendezvous address come from the environment (RANK,
 * WORLD_SIZE, MASTER_ADDR, TIPS_MASTER_PORT or MASTER_PORT+1000). */
int tips_init(void);
int tips_init_ex(int rank, int size, const char* master_addr, int master_port);
int tips_shutdown(void);
int tips_is_initialized(void);
int tips_is_initialize(void);
int tips_size(void);
int tips_rank(void);
int tips_local_rank(void);
int tips_local_size(void);
const char* tips_last_error(void);
/* IP of `rank` as registered at bootstrap; returns bytes written. */
int tips_rank_ip(int rank, char* out, int out_len);

/* ---- host collectives (control plane) --------------------------------- */
int tips_barrier(void);
/* Gathers `n` bytes from every rank; `out` holds size*max_n bytes, `out_sizes` size entries. */
int tips_host_allgather(const void* in, int64_t n, void* out, int64_t max_n, int64_t* out_sizes);
int tips_host_broadcast(void* data, int64_t n, int root);

/* ---- sub-groups of ranks ------------------------------------------------ */
/* Collective over the world: every rank calls it with the same list, in the same order relative to other
 * tips_group_new calls.  Returns the group id (> 0), or a negative error.  Id 0 is the world. */
int64_t tips_group_new(const int32_t* world_ranks, int n);
int tips_group_size(int64_t id);
int tips_group_rank(int64_t id);                     /* -1: this process is not a member */
int tips_group_to_world(int64_t id, int group_rank);
/* Members only: */
int tips_group_barrier(int64_t id, int timeout_ms);
int tips_group_allgather(int64_t id, const void* in, int64_t n, void* out, int64_t max_n, int64_t* out_sizes,
                         int timeout_ms);

/* ---- engine options ---------------------------------------------------- */
int tips_set_fusion_threshold(int64_t bytes);
int tips_set_cycle_time_ms(int ms);
int tips_set_stall_check(int warn_ms, int abort_ms);

/* ---- asynchronous tensor collectives ---------------------------------- */
typedef void* (*tips_alloc_fn)(int64_t handle, int64_t nbytes, const int64_t* first_dims, int32_t n, void* user);

typedef struct {
  const char* name;
  int32_t type;      /* 0 allreduce, 1 allgather, 2 broadcast */
  int32_t dtype;     /* tips Datatype value */
  int32_t ndim;
  const int64_t* shape;
  const void* in;
  void* out;         /* allgather: may be NULL when alloc is given */
  int32_t device;    /* 0 host, 1 CUDA */
  int32_t root_rank;
  int32_t reduce_op; /* 0 sum, 1 max, 2 min, 3 prod */
  double prescale;
  double postscale;
  void* stream;
  void* ready_event;
  void* done_event;
  tips_alloc_fn alloc;
  void* alloc_user;
} tips_op_t;

/* Returns a handle > 0, or a negative status code. */
int64_t tips_enqueue(const tips_op_t* op);
/* 1 = still running, 0 = done OK, other positive = failed with that status code. */
int tips_poll(int64_t handle);
int tips_wait(int64_t handle, int timeout_ms);
int tips_handle_error(int64_t handle, char* out, int out_len);
/* Allgather: per-rank first dimensions and the output address. */
int tips_handle_sizes(int64_t handle, int64_t* out, int n);
void* tips_handle_output(int64_t handle);
int tips_release(int64_t handle);

/* Device executor hook: int fn(const DeviceOp*, char* err, int err_len). */
int tips_set_device_executor(void* fn);

/* ---- frozen schedule --------------------------------------------------- */
/* Names executed through negotiation since the last call, '\n'-separated. */
int tips_take_negotiated_order(char* out, int out_len);
int tips_freeze_schedule(const char* names_newline_separated);
int tips_thaw_schedule(void);
/* Fails every collective in flight on this rank (status 4), forgets partial negotiations and frozen schedules;
 * every rank calls it after a failed step, then the ranks meet on tips_barrier() before the next collective. */
int tips_reset_collectives(void);

/* ---- observability ----------------------------------------------------- */
int tips_timeline_enable(int on);
int tips_timeline_dump(const char* path);
/* Fills up to n counters in a fixed order (see CounterNames in c_api.cc); returns the count. */
int tips_counters(uint64_t* out, int n);
const char* tips_counter_names(void);
int tips_set_log_level(int min_level, int verbose);

/* Nanoseconds per message for request encode / decode and response encode / decode (see c_api.cc). */
int tips_bench_messages(int iters, double* out4);

/* ---- fault injection (tests) ------------------------------------------- */
int tips_inject_drop_requests(int dst_rank, int n);

#ifdef __cplusplus
}
#endif
