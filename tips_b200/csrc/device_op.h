/* Description of one device-side collective, handed by the collective engine
 * (libtips_core.so) to the device executor (libtips_kernels.so).  Plain C
 * layout because it crosses a shared-library boundary. */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tips_device_op {
  int32_t type;          /* 0 allreduce, 1 allgather, 2 broadcast */
  int32_t dtype;         /* tips Datatype code */
  int32_t reduce_op;     /* 0 sum, 1 max, 2 min, 3 prod */
  int32_t root_rank;
  const void* in;
  void* out;
  int64_t count;         /* elements (allreduce / broadcast) */
  const int64_t* counts; /* allgather: elements contributed by every rank */
  int32_t nranks;
  int32_t channel;       /* 0 = negotiated order, 1 = frozen schedule */
  double prescale;
  double postscale;
  void* stream;          /* producer stream (informational) */
  void* ready_event;     /* recorded by the producer once the input is written; may be null */
  void* done_event;      /* recorded by the executor after the collective; may be null */
} tips_device_op;

/* Returns 0 on success; on failure writes a message into err. */
typedef int (*tips_device_executor_fn)(const tips_device_op* op, char* err, int err_len);

#ifdef __cplusplus
}
#endif
