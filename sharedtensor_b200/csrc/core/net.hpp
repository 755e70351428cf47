// Socket helpers: exact-length reads and writes that can be interrupted by a stop flag and that
// report end-of-stream and errors to the caller.
//
// The reference's helpers (src/sharedtensor.c:53-104) retry on EINTR, spin forever on a closed
// peer (read()==0 is not handled, lines 56-67) and call exit(-1) on every other error.  Here a
// closed peer and an error are ordinary return values, and blocking calls wake up every
// `kPollMs` to look at a stop flag, which replaces the SIGALRM wake-up trick (lines 47-50, 404-411).
#pragma once
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/types.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <string>

namespace st {

enum class IoStatus { Ok = 0, Eof = 1, Error = 2, Stopped = 3, Timeout = 4 };

constexpr int kPollMs = 100;

inline const char* io_status_name(IoStatus s) {
  switch (s) {
    case IoStatus::Ok: return "ok";
    case IoStatus::Eof: return "eof";
    case IoStatus::Error: return "error";
    case IoStatus::Stopped: return "stopped";
    case IoStatus::Timeout: return "timeout";
  }
  return "?";
}

// Reads exactly `count` bytes.  `deadline_ms` < 0 means no deadline.
inline IoStatus read_full(int fd, void* buf, size_t count, const std::atomic<bool>* stop,
                          int deadline_ms = -1) {
  uint8_t* p = static_cast<uint8_t*>(buf);
  int waited = 0;
  while (count) {
    if (stop && stop->load(std::memory_order_acquire)) return IoStatus::Stopped;
    struct pollfd pfd = {fd, POLLIN, 0};
    int pr = ::poll(&pfd, 1, kPollMs);
    if (pr < 0) {
      if (errno == EINTR) continue;
      return IoStatus::Error;
    }
    if (pr == 0) {
      waited += kPollMs;
      if (deadline_ms >= 0 && waited >= deadline_ms) return IoStatus::Timeout;
      continue;
    }
    ssize_t r = ::recv(fd, p, count, 0);
    if (r == 0) return IoStatus::Eof;
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
      return IoStatus::Error;
    }
    p += r;
    count -= size_t(r);
  }
  return IoStatus::Ok;
}

// Writes exactly `count` bytes; never raises SIGPIPE.
inline IoStatus write_full(int fd, const void* buf, size_t count, const std::atomic<bool>* stop) {
  const uint8_t* p = static_cast<const uint8_t*>(buf);
  while (count) {
    if (stop && stop->load(std::memory_order_acquire)) return IoStatus::Stopped;
    struct pollfd pfd = {fd, POLLOUT, 0};
    int pr = ::poll(&pfd, 1, kPollMs);
    if (pr < 0) {
      if (errno == EINTR) continue;
      return IoStatus::Error;
    }
    if (pr == 0) continue;
    if (pfd.revents & (POLLERR | POLLHUP | POLLNVAL)) {
      // fall through to send() to get the precise errno
    }
    ssize_t r = ::send(fd, p, count, MSG_NOSIGNAL | MSG_DONTWAIT);
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
      if (errno == EPIPE || errno == ECONNRESET) return IoStatus::Eof;
      return IoStatus::Error;
    }
    p += r;
    count -= size_t(r);
  }
  return IoStatus::Ok;
}

inline std::string addr_to_string(const sockaddr_in& a) {
  char buf[64];
  inet_ntop(AF_INET, &a.sin_addr, buf, sizeof(buf));
  return std::string(buf) + ":" + std::to_string(ntohs(a.sin_port));
}

inline void close_fd(int& fd) {
  if (fd >= 0) {
    ::shutdown(fd, SHUT_RDWR);
    ::close(fd);
    fd = -1;
  }
}

}  // namespace st
