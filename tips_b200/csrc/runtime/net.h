// Blocking TCP helpers for the host control plane and the CPU data plane.
//
// The reference moves control messages over ZeroMQ PUSH/PULL sockets and CPU
// tensors through OpenMPI (tips/core/common/naive_rpc.cc:201-246,
// tips/core/collective/utils.h:52-134).  Neither library exists on the target
// image, and GPU tensors never touch the host here, so the host transport is a
// plain full mesh of TCP sockets: one mesh for length-prefixed RPC frames, one
// for synchronous CPU collectives.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

#include "core/common.h"

namespace tips {
namespace net {

// Creates a listening socket bound to `port` (0 = ephemeral) on all
// interfaces; returns the fd and stores the bound port.
int Listen(int port, int* bound_port, int backlog = 3000);

// Connects to host:port, retrying until `timeout_ms` elapses. Returns fd or -1.
int Connect(const std::string& host, int port, int timeout_ms);

// Accepts one connection, waiting at most timeout_ms (-1 = forever). -1 on timeout/error.
int Accept(int listen_fd, int timeout_ms);

void SetNoDelay(int fd);
void SetNonBlocking(int fd, bool on);
void Close(int fd);

// Full-length blocking send/recv. False on error or EOF.
bool SendAll(int fd, const void* data, size_t n);
bool RecvAll(int fd, void* data, size_t n);

// Sends `sn` bytes to `send_fd` while receiving `rn` bytes from `recv_fd`
// (the two may be the same socket); progress on both directions is driven by
// poll() so two peers that exchange large buffers cannot deadlock on full
// socket buffers.  timeout_ms bounds the time without progress.
bool Exchange(int send_fd, const void* sbuf, size_t sn, int recv_fd, void* rbuf, size_t rn, int timeout_ms);

}  // namespace net
}  // namespace tips
