#include "runtime/net.h"

#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <thread>

namespace tips {
namespace net {

int Listen(int port, int* bound_port, int backlog) {
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  TIPS_CHECK_GE(fd, 0) << "socket() failed";
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in addr;
  memset(&addr, 0, sizeof(addr));
  addr.sin_family      = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port        = htons(static_cast<uint16_t>(port));
  if (bind(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) != 0) {
    int e = errno;
    close(fd);
    TIPS_LOG(FATAL) << "bind to port " << port << " failed: " << strerror(e);
  }
  TIPS_ZCHECK(listen(fd, backlog));
  socklen_t len = sizeof(addr);
  TIPS_ZCHECK(getsockname(fd, reinterpret_cast<struct sockaddr*>(&addr), &len));
  if (bound_port) *bound_port = ntohs(addr.sin_port);
  return fd;
}

int Connect(const std::string& host, int port, int timeout_ms) {
  struct addrinfo hints;
  memset(&hints, 0, sizeof(hints));
  hints.ai_family   = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  const std::string port_str = std::to_string(port);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  int backoff_ms = 1;
  while (true) {
    struct addrinfo* res = nullptr;
    if (getaddrinfo(host.c_str(), port_str.c_str(), &hints, &res) == 0 && res) {
      int fd = socket(res->ai_family, res->ai_socktype, res->ai_protocol);
      if (fd >= 0) {
        if (ignore_signal_call(connect, fd, res->ai_addr, res->ai_addrlen) == 0) {
          freeaddrinfo(res);
          SetNoDelay(fd);
          return fd;
        }
        close(fd);
      }
      freeaddrinfo(res);
    }
    if (std::chrono::steady_clock::now() >= deadline) return -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(backoff_ms));
    if (backoff_ms < 64) backoff_ms *= 2;
  }
}

int Accept(int listen_fd, int timeout_ms) {
  struct pollfd p;
  p.fd     = listen_fd;
  p.events = POLLIN;
  int r    = ignore_signal_call(poll, &p, 1, timeout_ms);
  if (r <= 0) return -1;
  int fd = ignore_signal_call(accept, listen_fd, nullptr, nullptr);
  if (fd >= 0) SetNoDelay(fd);
  return fd;
}

void SetNoDelay(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

void SetNonBlocking(int fd, bool on) {
  int flags = fcntl(fd, F_GETFL, 0);
  if (flags < 0) return;
  fcntl(fd, F_SETFL, on ? (flags | O_NONBLOCK) : (flags & ~O_NONBLOCK));
}

void Close(int fd) {
  if (fd >= 0) close(fd);
}

bool SendAll(int fd, const void* data, size_t n) {
  const char* p = static_cast<const char*>(data);
  while (n > 0) {
    ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) {
        struct pollfd pf = {fd, POLLOUT, 0};
        poll(&pf, 1, 1000);
        continue;
      }
      return false;
    }
    p += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}

bool RecvAll(int fd, void* data, size_t n) {
  char* p = static_cast<char*>(data);
  while (n > 0) {
    ssize_t r = recv(fd, p, n, 0);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) {
        struct pollfd pf = {fd, POLLIN, 0};
        poll(&pf, 1, 1000);
        continue;
      }
      return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

bool Exchange(int send_fd, const void* sbuf, size_t sn, int recv_fd, void* rbuf, size_t rn, int timeout_ms) {
  const char* sp = static_cast<const char*>(sbuf);
  char* rp       = static_cast<char*>(rbuf);
  while (sn > 0 || rn > 0) {
    struct pollfd pf[2];
    int n = 0, si = -1, ri = -1;
    if (sn > 0 && rn > 0 && send_fd == recv_fd) {
      pf[0] = {send_fd, static_cast<short>(POLLIN | POLLOUT), 0};
      si = ri = 0;
      n       = 1;
    } else {
      if (sn > 0) {
        si    = n;
        pf[n] = {send_fd, POLLOUT, 0};
        ++n;
      }
      if (rn > 0) {
        ri    = n;
        pf[n] = {recv_fd, POLLIN, 0};
        ++n;
      }
    }
    int r = ignore_signal_call(poll, pf, static_cast<nfds_t>(n), timeout_ms);
    if (r <= 0) return false;
    if (si >= 0 && (pf[si].revents & (POLLOUT | POLLERR | POLLHUP))) {
      ssize_t w = send(send_fd, sp, sn, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (w < 0) {
        if (errno != EINTR && errno != EAGAIN && errno != EWOULDBLOCK) return false;
      } else {
        sp += w;
        sn -= static_cast<size_t>(w);
      }
    }
    if (ri >= 0 && (pf[ri].revents & (POLLIN | POLLERR | POLLHUP))) {
      ssize_t g = recv(recv_fd, rp, rn, MSG_DONTWAIT);
      if (g == 0) return false;
      if (g < 0) {
        if (errno != EINTR && errno != EAGAIN && errno != EWOULDBLOCK) return false;
      } else {
        rp += g;
        rn -= static_cast<size_t>(g);
      }
    }
  }
  return true;
}

}  // namespace net
}  // namespace tips
