#include "tree.hpp"

#include <netdb.h>

namespace st {

bool resolve_ipv4(const std::string& host, int port, sockaddr_in* out, std::string* err) {
  std::memset(out, 0, sizeof(*out));
  out->sin_family = AF_INET;
  out->sin_port = htons(uint16_t(port));
  if (inet_pton(AF_INET, host.c_str(), &out->sin_addr) == 1) return true;
  struct addrinfo hints;
  std::memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  struct addrinfo* res = nullptr;
  int rc = getaddrinfo(host.c_str(), nullptr, &hints, &res);
  if (rc != 0 || !res) {
    if (err) *err = std::string("cannot resolve host '") + host + "': " + gai_strerror(rc);
    return false;
  }
  out->sin_addr = reinterpret_cast<sockaddr_in*>(res->ai_addr)->sin_addr;
  freeaddrinfo(res);
  return true;
}

static int make_tcp_socket(std::string* err) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) {
    if (err) *err = std::string("socket: ") + std::strerror(errno);
    return -1;
  }
  int yes = 1;
  if (setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &yes, sizeof(yes)) < 0) {
    if (err) *err = std::string("setsockopt(SO_REUSEADDR): ") + std::strerror(errno);
    ::close(fd);
    return -1;
  }
  return fd;
}

JoinResult join_tree(const std::string& host, int port, const std::atomic<bool>* stop, int max_hops,
                     int reply_timeout_ms, const std::vector<sockaddr_in>* self) {
  JoinResult r;
  sockaddr_in root;
  if (!resolve_ipv4(host, port, &root, &r.error)) return r;
  sockaddr_in target = root;
  int restarts = 0;
  for (int hop = 0; hop <= max_hops; hop++) {
    if (stop && stop->load()) {
      r.error = "stopped";
      return r;
    }
    bool to_self = false;
    if (self)
      for (const sockaddr_in& a : *self)
        to_self |= a.sin_port == target.sin_port && a.sin_addr.s_addr == target.sin_addr.s_addr;
    if (to_self) {  // redirected to this very node: its old parent still lists it; start over
      if (++restarts > 8) {
        r.error = "redirected to this node itself";
        return r;
      }
      target = root;
      ::usleep(50 * 1000);
      continue;
    }
    int fd = make_tcp_socket(&r.error);
    if (fd < 0) return r;
    if (::connect(fd, reinterpret_cast<sockaddr*>(&target), sizeof(target)) < 0) {
      ::close(fd);
      bool at_root = std::memcmp(&target, &root, sizeof(root)) == 0;
      if (at_root) {  // nobody serves host:port: this node is the master
        r.ok = true;
        r.master = true;
        r.listen_addr = root;
        r.hops = hop;
        return r;
      }
      // a redirect pointed at a node that is gone: start over from the root a few times
      if (++restarts > 8) {
        r.error = "redirect target " + addr_to_string(target) + " unreachable";
        return r;
      }
      target = root;
      ::usleep(50 * 1000);
      continue;
    }
    uint8_t reply = 0;
    IoStatus st = read_full(fd, &reply, 1, stop, reply_timeout_ms);
    if (st != IoStatus::Ok) {
      ::close(fd);
      if (st == IoStatus::Stopped) {
        r.error = "stopped";
        return r;
      }
      if (++restarts > 8) {
        r.error = std::string("no join reply from ") + addr_to_string(target) + ": " + io_status_name(st);
        return r;
      }
      target = root;
      ::usleep(50 * 1000);
      continue;
    }
    if (reply == 'Y') {
      socklen_t len = sizeof(r.listen_addr);
      if (getsockname(fd, reinterpret_cast<sockaddr*>(&r.listen_addr), &len) < 0) {
        r.error = std::string("getsockname: ") + std::strerror(errno);
        ::close(fd);
        return r;
      }
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      r.ok = true;
      r.fd = fd;
      r.parent_addr = target;
      r.hops = hop;
      return r;
    }
    // 'N' (or anything else, like the reference): the next 16 bytes are a raw sockaddr_in
    sockaddr_in next;
    st = read_full(fd, &next, sizeof(next), stop, reply_timeout_ms);
    ::close(fd);
    if (st != IoStatus::Ok) {
      r.error = std::string("truncated redirect from ") + addr_to_string(target);
      return r;
    }
    next.sin_family = AF_INET;
    target = next;
  }
  r.error = "too many redirects";
  return r;
}

int open_listener(const sockaddr_in& addr, int backlog, std::string* err) {
  int fd = make_tcp_socket(err);
  if (fd < 0) return -1;
  if (::bind(fd, reinterpret_cast<const sockaddr*>(&addr), sizeof(addr)) < 0) {
    if (err) *err = "bind " + addr_to_string(addr) + ": " + std::strerror(errno);
    ::close(fd);
    return -1;
  }
  if (::listen(fd, backlog) < 0) {
    if (err) *err = std::string("listen: ") + std::strerror(errno);
    ::close(fd);
    return -1;
  }
  return fd;
}

TreeListener::TreeListener(PickSlot pick, Adopt adopt, ChildAddr child_addr)
    : pick_(std::move(pick)), adopt_(std::move(adopt)), child_addr_(std::move(child_addr)) {}

TreeListener::~TreeListener() { stop(); }

void TreeListener::add_listen_fd(int fd) {
  std::lock_guard<std::mutex> g(mu_);
  fds_.push_back(fd);
}

void TreeListener::start() { th_ = std::thread([this] { run(); }); }

void TreeListener::stop() {
  stop_.store(true);
  if (th_.joinable()) th_.join();
  std::lock_guard<std::mutex> g(mu_);
  for (int& fd : fds_) {
    if (fd >= 0) ::close(fd);
    fd = -1;
  }
  fds_.clear();
}

void TreeListener::run() {
  while (!stop_.load()) {
    std::vector<pollfd> pfds;
    {
      std::lock_guard<std::mutex> g(mu_);
      for (int fd : fds_) pfds.push_back({fd, POLLIN, 0});
    }
    if (pfds.empty()) {
      ::usleep(kPollMs * 1000);
      continue;
    }
    int pr = ::poll(pfds.data(), pfds.size(), kPollMs);
    if (pr <= 0) continue;
    for (auto& p : pfds) {
      if (!(p.revents & POLLIN)) continue;
      sockaddr_in peer;
      socklen_t len = sizeof(peer);
      int fd = ::accept(p.fd, reinterpret_cast<sockaddr*>(&peer), &len);
      if (fd < 0) continue;
      int slot = pick_();
      if (slot >= 0) {
        if (write_full(fd, "Y", 1, &stop_) != IoStatus::Ok) {
          ::close(fd);
          continue;
        }
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        adopt_(slot, fd, peer);
        continue;
      }
      // Full: hand out a child's address, right first, then left, alternating.
      sockaddr_in give;
      int first = (lr_counter_++ & 1) ? kSlotLeft : kSlotRight;
      int second = first == kSlotLeft ? kSlotRight : kSlotLeft;
      bool have = child_addr_(first, &give) || child_addr_(second, &give);
      if (have) {
        uint8_t msg[1 + sizeof(sockaddr_in)];
        msg[0] = 'N';
        std::memcpy(msg + 1, &give, sizeof(give));
        write_full(fd, msg, sizeof(msg), &stop_);
        redirects_.fetch_add(1);
      }
      ::shutdown(fd, SHUT_WR);
      ::close(fd);
    }
  }
}

}  // namespace st
