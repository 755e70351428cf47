// Tree membership over TCP: the join walk of a new node and the accept/redirect server every node runs.
//
// Wire behaviour is the reference's (src/sharedtensor.c:192-242 server, 244-332 client):
//   * the server answers every inbound connection with one byte, 'Y' (adopted as left/right child)
//     or 'N' followed by the raw 16-byte sockaddr_in of one of its children; redirect targets
//     alternate right, left, right, ... per server;
//   * a child's address is the peer address accept() reported for it, because every joiner binds its
//     own listening socket to the local ip:port of its up connection (SO_REUSEADDR on both);
//   * the joiner sends nothing; if the very first connect fails the caller is the master and binds
//     the requested host:port itself.
// Differences: a freed child slot is re-used before redirecting, a failed redirect target restarts
// the walk from the root instead of silently turning the joiner into a second master, and all
// blocking calls can be interrupted by a stop flag.
#pragma once
#include <atomic>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "net.hpp"

namespace st {

constexpr int kSlotUp = 0, kSlotLeft = 1, kSlotRight = 2, kNumSlots = 3;

struct JoinResult {
  bool ok = false;
  bool master = false;      // nobody answered at host:port
  int fd = -1;              // connected up socket (when !master)
  sockaddr_in listen_addr;  // where this node must listen (host:port for the master, else own up-socket address)
  sockaddr_in parent_addr;  // address of the node that adopted us
  int hops = 0;             // number of redirects followed
  std::string error;
};

bool resolve_ipv4(const std::string& host, int port, sockaddr_in* out, std::string* err);

// Walks the tree from host:port until some node answers 'Y'.  `self`: addresses this node itself listens on; a
// redirect to one of them (a parent that has not noticed yet that this node's old connection is gone hands out the
// node's own address) is treated like an unreachable target, so that a re-joining node cannot adopt itself.
JoinResult join_tree(const std::string& host, int port, const std::atomic<bool>* stop,
                     int max_hops = 64, int reply_timeout_ms = 10000, const std::vector<sockaddr_in>* self = nullptr);

// socket + SO_REUSEADDR + bind + listen(backlog).  Returns -1 and fills err on failure.
int open_listener(const sockaddr_in& addr, int backlog, std::string* err);

// Accept loop.  `pick_slot` returns kSlotLeft/kSlotRight if a child slot is free, else -1.
// `adopt` takes ownership of an accepted fd that has already been told 'Y'.
// `child_addr(slot, &addr)` returns false if that child is not connected any more.
class TreeListener {
 public:
  using PickSlot = std::function<int()>;
  using Adopt = std::function<void(int slot, int fd, const sockaddr_in& peer)>;
  using ChildAddr = std::function<bool(int slot, sockaddr_in* out)>;

  TreeListener(PickSlot pick, Adopt adopt, ChildAddr child_addr);
  ~TreeListener();
  void add_listen_fd(int fd);  // takes ownership; may be called while running
  void start();
  void stop();
  uint64_t redirects() const { return redirects_.load(); }

 private:
  void run();
  PickSlot pick_;
  Adopt adopt_;
  ChildAddr child_addr_;
  std::vector<int> fds_;
  std::mutex mu_;
  std::thread th_;
  std::atomic<bool> stop_{false};
  std::atomic<uint64_t> redirects_{0};
  unsigned lr_counter_ = 0;
};

}  // namespace st
