// GPU node = tree membership + GPU replica.
//
// Membership is the reference's TCP protocol, byte for byte (see ../core/tree.hpp): a joiner connects to
// host:port, is adopted ('Y') or redirected ('N' + sockaddr_in), and listens on the local address of its
// up connection.  What is new is what happens after 'Y' when both ends are GPU nodes on the same host:
// every node also listens on an abstract AF_UNIX socket named after its TCP listen address.  The child
// connects to its parent's, the two exchange a hello (element count, block size, ring geometry) and the
// file descriptors of their edge blocks, map each other's block, and from then on the edge is a pair of
// rings in peer memory; the TCP connection carries no data and serves as the liveness signal (EOF = the
// neighbour is gone).  The parent then copies its replica into the child's with one kernel and sets its
// mirror for the edge to the same snapshot, which replaces the reference's implicit state transfer
// (streaming the whole history through the 1-bit codec, src/sharedtensor.c:379-387) by one bulk copy.
// If the parent has no such socket (a CPU node, the reference, another host) the edge stays on TCP; that
// case is handled by the TCP edge classes, not here.
//
// The class is defined in this header (its methods are short and are used by one translation unit each: the
// Python bindings in gpu_node.cpp and C++ tests that drive a node directly).
#pragma once
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime_api.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cmath>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../core/tree.hpp"
#include "engine.hpp"
#include "vmm.hpp"

namespace st {

namespace gpu_node_detail {

constexpr uint32_t kHelloMagic = 0x32425453;  // "STB2"
constexpr uint32_t kHelloVersion = 2;

struct Hello {
  uint32_t magic = kHelloMagic;
  uint32_t version = kHelloVersion;
  int64_t n = 0;
  int32_t block = 0;
  int32_t ring_slots = 0;
  int32_t bits = 0;            // bits per element of a frame
  int32_t reserved = 0;
  uint64_t edge_bytes = 0;     // mapped size of the sender's edge block
  uint64_t values_bytes = 0;   // mapped size of the sender's values block
  sockaddr_in listen_addr{};   // the sender's TCP listen address (identifies the child to its parent)
  int32_t device = 0;
  int32_t status = 0;          // reply only: 0 ok, else refusal code
  char message[64] = {0};
};

inline uint64_t now_ms() {
  using namespace std::chrono;
  return uint64_t(duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count());
}

inline std::string unix_name(const sockaddr_in& a) { return "sharedtensor_b200/" + addr_to_string(a); }
}  // namespace gpu_node_detail
using namespace gpu_node_detail;

struct GpuNodeOptions {
  bool rejoin = true;
  int rejoin_backoff_ms = 200;
  int upgrade_timeout_ms = 5000;
  int listen_backlog = 5;
  bool start_engine = true;
};

class GpuNode {
 public:
  GpuNode(int device, int64_t n, const GpuConfig& gcfg, const GpuNodeOptions& opt)
      : rep_(new GpuReplica(device, n, gcfg)), gcfg_(gcfg), opt_(opt), device_(device), n_(n) {
    for (int s = 0; s < kNumSlots; s++) edges_[s].slot = s;
    rep_->set_doorbell([this] { ring_neighbours(-1); });
  }
  ~GpuNode() { close(); }

  GpuReplica& replica() { return *rep_; }

  void start(const std::string& host, int port, const float* init_dev, void* stream) {
    if (started_.exchange(true)) throw std::runtime_error("node already started");
    host_ = host;
    port_ = port;
    listener_.reset(new TreeListener(
        [this]() -> int {
          std::lock_guard<std::mutex> g(mu_);
          if (closed_.load()) return -1;
          if (edges_[kSlotLeft].state == 0) return kSlotLeft;
          if (edges_[kSlotRight].state == 0) return kSlotRight;
          return -1;
        },
        [this](int slot, int fd, const sockaddr_in& peer) {
          // adopted over TCP; the edge becomes usable once the child has come in over the unix socket
          std::lock_guard<std::mutex> g(mu_);
          Edge& e = edges_[slot];
          e.state = 1;
          e.tcp_fd = fd;
          e.peer = peer;
          e.adopted_ms = now_ms();
          cv_.notify_all();
        },
        [this](int slot, sockaddr_in* out) -> bool {
          std::lock_guard<std::mutex> g(mu_);
          if (edges_[slot].state == 0) return false;
          *out = edges_[slot].peer;
          return true;
        }));
    // a first join can fail for a passing reason (the ephemeral port this node has to listen on was just taken by
    // another process's listener): a new connection gets a new port
    bool joined = false;
    for (int attempt = 0; attempt < 4 && !joined && !stop_.load(); attempt++) {
      if (attempt) ::usleep(50 * 1000);
      joined = join(true, init_dev, stream);
    }
    if (!joined) {
      started_.store(false);
      listener_.reset();
      throw std::runtime_error("shared tensor could not join or found a tree at " + host + ":" + std::to_string(port));
    }
    listener_->start();
    upgrade_thread_ = std::thread([this] { upgrade_loop(); });
    watch_thread_ = std::thread([this] { watch_loop(); });
    if (opt_.start_engine) rep_->start_engine();
  }

  bool wait_ready(int timeout_ms) {
    std::unique_lock<std::mutex> lk(mu_);
    return cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return ready_ || closed_.load(); }) && ready_;
  }
  bool is_master() const { return master_.load(); }

  void close() {
    if (closed_.exchange(true)) return;
    stop_.store(true);
    cv_.notify_all();
    if (rep_) rep_->set_doorbell(nullptr);
    if (rep_) rep_->stop_engine();
    if (listener_) listener_->stop();
    if (unix_fd_ >= 0) ::shutdown(unix_fd_, SHUT_RDWR);
    {
      std::lock_guard<std::mutex> g(mu_);
      for (int fd : extra_unix_fds_) ::shutdown(fd, SHUT_RDWR);
    }
    if (upgrade_thread_.joinable()) upgrade_thread_.join();
    if (watch_thread_.joinable()) watch_thread_.join();
    if (unix_fd_ >= 0) {
      ::close(unix_fd_);
      unix_fd_ = -1;
    }
    for (int fd : extra_unix_fds_) ::close(fd);
    extra_unix_fds_.clear();
    for (int s = 0; s < kNumSlots; s++) drop_edge(s, false);
    rep_.reset();
  }

  pybind11::dict stats() {
    namespace py = pybind11;
    py::dict d;
    std::vector<uint64_t> st;
    {
      py::gil_scoped_release rel;
      st = rep_->status();
    }
    std::lock_guard<std::mutex> g(mu_);
    d["master"] = master_.load();
    d["ready"] = ready_;
    d["closed"] = closed_.load();
    d["n"] = n_;
    d["listen_addr"] = addr_to_string(listen_addr_);
    d["rejoins"] = rejoins_;
    d["edge_failures"] = edge_failures_;
    d["redirects"] = listener_ ? listener_->redirects() : 0;
    d["launches"] = rep_->launches();
    static const char* names[] = {"up", "left", "right"};
    static const char* states[] = {"free", "adopted", "connected"};
    py::dict edges;
    for (int s = 0; s < kNumSlots; s++) {
      py::dict e;
      e["state"] = states[edges_[s].state];
      e["peer"] = edges_[s].state ? addr_to_string(edges_[s].peer) : std::string();
      e["transport"] = edges_[s].state == 2 ? (edges_[s].tcp ? "tcp" : "p2p") : "";
      if (edges_[s].tcp && tcp_[s]) {
        e["frames_sent"] = tcp_[s]->frames_sent.load();
        e["frames_recv"] = tcp_[s]->frames_recv.load();
      }
      e["link"] = edges_[s].link;
      edges[names[s]] = e;
    }
    d["edges"] = edges;
    py::dict dev;
    static const char* snames[] = {"rounds", "tiles_processed", "frames_sent", "frames_recv", "blocked_no_credit", "errors",
                                   "last_work_count", "residual_max0", "residual_max1", "residual_max2", "pending_tiles",
                                   "wait_timeouts"};
    for (int i = 0; i < 12; i++) {
      if (i >= 7 && i <= 9) {
        uint32_t bits = uint32_t(st[i]);
        float v;
        std::memcpy(&v, &bits, 4);
        dev[snames[i]] = v;
      } else {
        dev[snames[i]] = st[i];
      }
    }
    d["device"] = dev;
    return d;
  }

  // host-side fault injection for tests: cut the liveness connection of an edge
  void inject_sever(int slot) {
    std::lock_guard<std::mutex> g(mu_);
    if (edges_[slot].tcp_fd >= 0) ::shutdown(edges_[slot].tcp_fd, SHUT_RDWR);
  }

 private:
  struct Edge {
    int slot = 0;
    int state = 0;        // 0 free, 1 adopted over TCP (waiting for the peer-memory upgrade), 2 connected
    int tcp_fd = -1;
    sockaddr_in peer{};
    uint64_t adopted_ms = 0;
    bool upgrading = false;  // the parent side of the upgrade is at work on this edge
    bool tcp = false;        // frames travel over the TCP connection (see TcpEdge)
    int link = -1, peer_id = -1, block = -1;
    VmmBlock remote;      // neighbour's edge block mapped here
  };

  // An edge whose other end does not speak the peer-memory upgrade (a CPU node, the reference, another host):
  // tensor-scale frames over the TCP connection, encoded and decoded on the device, bytes moved by two threads
  // (the counterpart of the reference's synca / sync_in pair, src/sharedtensor.c:113-189).
  struct TcpEdge {
    int slot = 0, fd = -1, link = -1;
    std::thread tx, rx;
    std::atomic<bool> stop{false}, failed{false};
    std::atomic<uint64_t> frames_sent{0}, frames_recv{0};
  };

  void start_tcp_edge(int slot, int fd, const sockaddr_in& peer) {
    int link = rep_->add_link();
    if (link < 0) {
      ::close(fd);
      return;
    }
    std::unique_ptr<TcpEdge> te(new TcpEdge());
    te->slot = slot;
    te->fd = fd;
    te->link = link;
    TcpEdge* raw = te.get();
    {
      std::lock_guard<std::mutex> g(mu_);
      Edge& e = edges_[slot];
      e.state = 2;
      e.tcp = true;
      e.tcp_fd = fd;
      e.peer = peer;
      e.link = link;
      tcp_[slot] = std::move(te);
    }
    raw->tx = std::thread([this, raw] { tcp_tx_loop(raw); });
    raw->rx = std::thread([this, raw] { tcp_rx_loop(raw); });
    std::fprintf(stderr, "[sharedtensor] edge %d to %s runs over TCP (reference wire format)\n", slot, addr_to_string(peer).c_str());
  }

  void tcp_tx_loop(TcpEdge* e) {
    cudaSetDevice(device_);
    const size_t n_words = size_t((n_ + 31) / 32), n_bytes = size_t((n_ + 7) / 8);
    std::vector<uint32_t> words(n_words);
    std::vector<uint8_t> frame(4 + n_bytes);
    bool sent_first = false, idle_announced = false;
    uint64_t seen = 0;
    while (!e->stop.load()) {
      const uint64_t ep = rep_->change_epoch();
      if (sent_first && idle_announced && ep == seen) {
        ::usleep(500);
        continue;
      }
      seen = ep;
      float scale = 0.f;
      try {
        scale = rep_->tcp_encode(e->link, words.data(), 0.f, 2.3841858e-07f);
      } catch (const std::exception&) {
        e->failed.store(true);
        break;
      }
      const bool noop = scale == 0.f;
      if (noop && sent_first && idle_announced) continue;  // nothing new; one no-op frame already ended the burst
      std::memcpy(frame.data(), &scale, 4);
      std::memcpy(frame.data() + 4, words.data(), n_bytes);
      IoStatus st = write_full(e->fd, frame.data(), frame.size(), &e->stop);
      if (st != IoStatus::Ok) {
        // not written: the frame counts as never made, its content goes out over the next connection
        try {
          rep_->tcp_unsend(e->link, words.data(), scale);
        } catch (const std::exception&) {
        }
        if (st != IoStatus::Stopped) e->failed.store(true);
        break;
      }
      sent_first = true;
      idle_announced = noop;
      if (!noop) seen = 0;  // keep draining until a pass has nothing to say
      e->frames_sent++;
    }
  }

  void tcp_rx_loop(TcpEdge* e) {
    cudaSetDevice(device_);
    const size_t n_words = size_t((n_ + 31) / 32), n_bytes = size_t((n_ + 7) / 8);
    std::vector<uint32_t> words(n_words, 0u);
    std::vector<uint8_t> frame(4 + n_bytes);
    float first_scale = 0.f;
    const uint64_t t0 = now_ms();
    while (!e->stop.load()) {
      IoStatus st = read_full(e->fd, frame.data(), frame.size(), &e->stop);
      if (st != IoStatus::Ok) {
        if (st != IoStatus::Stopped) e->failed.store(true);
        break;
      }
      float scale;
      std::memcpy(&scale, frame.data(), 4);
      if (!(scale >= 0.f) || scale > 3.0e38f) {  // NaN, negative or infinite: the peer's state is broken
        e->failed.store(true);
        break;
      }
      std::memcpy(words.data(), frame.data() + 4, n_bytes);
      try {
        rep_->tcp_decode(e->link, words.data(), scale);
      } catch (const std::exception&) {
        e->failed.store(true);
        break;
      }
      e->frames_recv++;
      if (e->slot == kSlotUp) {
        std::lock_guard<std::mutex> g(mu_);
        if (!ready_) {
          if (first_scale == 0.f && scale > 0.f) first_scale = scale;
          if (scale == 0.f || scale <= std::ldexp(first_scale, -12) || now_ms() - t0 > 30000) {
            ready_ = true;
            cv_.notify_all();
          }
        }
      }
    }
  }

  Hello my_hello() const { return my_hello(listen_addr_); }
  // `seen_as`: the source address of the TCP connection this hello belongs to (what the parent matches it by)
  Hello my_hello(const sockaddr_in& seen_as) const {
    Hello h;
    h.n = n_;
    h.block = gcfg_.block;
    h.ring_slots = gcfg_.ring_slots;
    h.bits = gcfg_.bits;
    h.edge_bytes = 0;
    h.values_bytes = rep_->values_block().bytes;
    h.listen_addr = seen_as;
    h.device = device_;
    return h;
  }

  bool join(bool first, const float* init_dev, void* stream) {
    JoinResult jr = join_tree(host_, port_, &stop_, 64, 10000, &my_addrs_);
    if (!jr.ok) {
      std::fprintf(stderr, "[sharedtensor] join failed: %s\n", jr.error.c_str());
      return false;
    }
    std::string err;
    if (jr.master) {
      int lfd = open_listener(jr.listen_addr, opt_.listen_backlog, &err);
      if (lfd < 0) {
        std::fprintf(stderr, "[sharedtensor] cannot serve %s:%d as master: %s\n", host_.c_str(), port_, err.c_str());
        return false;
      }
      my_addrs_.push_back(jr.listen_addr);
      if (first) {
        listen_addr_ = jr.listen_addr;
        if (!open_unix(&err)) {
          ::close(lfd);
          std::fprintf(stderr, "[sharedtensor] %s\n", err.c_str());
          return false;
        }
        if (init_dev) rep_->load_values(init_dev, stream);
      } else {
        // took over the tensor's address: joiners will look for the peer-memory endpoint under that address
        int ufd = unix_listen_abstract(unix_name(jr.listen_addr), &err);
        if (ufd >= 0) {
          std::lock_guard<std::mutex> g(mu_);
          extra_unix_fds_.push_back(ufd);
        }
      }
      listener_->add_listen_fd(lfd);
      drop_orphan_link();  // became the root: the values are intact, nothing to add back
      {
        std::lock_guard<std::mutex> g(mu_);
        master_.store(true);
        ready_ = true;
      }
      cv_.notify_all();
      std::fprintf(stderr, "[sharedtensor] master of %s:%d (%lld elements, GPU %d)\n", host_.c_str(), port_, (long long)n_, device_);
      return true;
    }
    if (first) {
      int lfd = open_listener(jr.listen_addr, opt_.listen_backlog, &err);
      if (lfd < 0) {
        std::fprintf(stderr, "[sharedtensor] cannot listen on %s: %s\n", addr_to_string(jr.listen_addr).c_str(), err.c_str());
        ::close(jr.fd);
        return false;
      }
      listen_addr_ = jr.listen_addr;
      my_addrs_.push_back(jr.listen_addr);
      listener_->add_listen_fd(lfd);
      if (!open_unix(&err)) {
        ::close(jr.fd);
        std::fprintf(stderr, "[sharedtensor] %s\n", err.c_str());
        return false;
      }
    } else {
      // The new parent knows this node by the source address of the new connection and will hand that address to
      // later joiners: accept TCP joins and peer-memory hellos there too (the first address stays open for the
      // redirects already handed out).  Best effort: without it this node is simply never a redirect target.
      int lfd = open_listener(jr.listen_addr, opt_.listen_backlog, &err);
      if (lfd >= 0) {
        listener_->add_listen_fd(lfd);
        my_addrs_.push_back(jr.listen_addr);
      }
      int ufd = unix_listen_abstract(unix_name(jr.listen_addr), &err);
      if (ufd >= 0) {
        std::lock_guard<std::mutex> g(mu_);
        extra_unix_fds_.push_back(ufd);
      }
    }
    master_.store(false);
    bool no_endpoint = false;
    if (!upgrade_as_child(jr, first, &err, &no_endpoint)) {
      if (no_endpoint) {
        // the parent is a CPU node, the reference, or on another host: speak TCP frames with it.  A node that
        // re-joins keeps only what its lost parent had not been told (like the CPU node).
        if (!first && orphan_link_ >= 0) {
          rep_->gate_lock();
          float* carry = make_carry();
          if (carry) {
            cudaSetDevice(device_);
            cudaMemcpy(rep_->values(), carry, size_t(n_) * 4, cudaMemcpyDeviceToDevice);
            cudaDeviceSynchronize();
            cudaFree(carry);
          }
          drop_orphan_link();
          rep_->gate_unlock();
        }
        start_tcp_edge(kSlotUp, jr.fd, jr.parent_addr);
        std::fprintf(stderr, "[sharedtensor] joined %s:%d below %s after %d redirect(s), GPU %d, TCP edge\n", host_.c_str(), port_,
                     addr_to_string(jr.parent_addr).c_str(), jr.hops, device_);
        return true;
      }
      std::fprintf(stderr, "[sharedtensor] peer-memory upgrade with %s failed: %s\n", addr_to_string(jr.parent_addr).c_str(),
                   err.c_str());
      ::close(jr.fd);
      return false;
    }
    std::fprintf(stderr, "[sharedtensor] joined %s:%d below %s after %d redirect(s), GPU %d, peer-memory edge\n", host_.c_str(), port_,
                 addr_to_string(jr.parent_addr).c_str(), jr.hops, device_);
    return true;
  }

  bool open_unix(std::string* err) {
    unix_fd_ = unix_listen_abstract(unix_name(listen_addr_), err);
    return unix_fd_ >= 0;
  }

  // ---- child side of the upgrade ----
  bool upgrade_as_child(const JoinResult& jr, bool first, std::string* err, bool* no_endpoint) {
    int us = unix_connect_abstract(unix_name(jr.parent_addr), 300);
    if (us < 0) {
      *err = "parent has no peer-memory endpoint on this host (TCP-only parent)";
      *no_endpoint = true;
      return false;
    }
    // A re-joining node takes its old up link along: its mirror says what the lost parent had been told.
    const bool reuse = !first && orphan_link_ >= 0;
    bool ok = false, gate_held = false;
    int block = -1, link = -1;
    float* carry = nullptr;
    VmmBlock remote;
    do {
      // the hello goes out first, so that the parent knows at once that this child will not speak TCP frames
      Hello h = my_hello(jr.listen_addr);
      if (!unix_send_fd(us, -1, &h, sizeof(h))) {
        *err = "hello send failed";
        break;
      }
      block = rep_->alloc_edge_block();
      link = reuse ? orphan_link_ : rep_->add_link();
      if (block < 0 || link < 0) {
        *err = "out of links or edge blocks";
        break;
      }
      Hello reply;
      if (!unix_recv_fd(us, nullptr, &reply, sizeof(reply), opt_.upgrade_timeout_ms) || reply.magic != kHelloMagic) {
        *err = "no hello reply";
        break;
      }
      if (reply.status != 0) {
        *err = std::string("parent refused: ") + reply.message;
        break;
      }
      // our fds: edge block, values
      std::string e2;
      int fd_edge = vmm_export_fd(rep_->edge_block(block), &e2);
      int fd_vals = vmm_export_fd(rep_->values_block(), &e2);
      if (fd_edge < 0 || fd_vals < 0) {
        *err = "cannot export device memory: " + e2;
        if (fd_edge >= 0) ::close(fd_edge);
        if (fd_vals >= 0) ::close(fd_vals);
        break;
      }
      if (reuse) {
        // From here until the snapshot has arrived and the carry is back on top of it, nobody else may change the
        // values: what the lost parent had not been told, u = values - mirror, is set aside now, updates made
        // while the edge was down included.
        rep_->gate_lock();
        gate_held = true;
        carry = make_carry();
        if (!carry) {
          *err = "no memory for the carry";
          ::close(fd_edge);
          ::close(fd_vals);
          break;
        }
      }
      const uint64_t sz_edge = rep_->edge_block(block).bytes, sz_vals = rep_->values_block().bytes;
      bool sent = unix_send_fd(us, fd_edge, &sz_edge, 8) && unix_send_fd(us, fd_vals, &sz_vals, 8);
      ::close(fd_edge);
      ::close(fd_vals);
      if (!sent) {
        *err = "fd send failed";
        break;
      }
      int fd_remote = -1;
      uint64_t sz_remote = 0;
      if (!unix_recv_fd(us, &fd_remote, &sz_remote, 8, opt_.upgrade_timeout_ms) || fd_remote < 0) {
        *err = "parent's edge block did not arrive";
        break;
      }
      remote = vmm_import_fd(fd_remote, size_t(sz_remote), device_, &e2);
      ::close(fd_remote);
      if (!remote.ptr) {
        *err = "cannot map parent's edge block: " + e2;
        break;
      }
      // wait for the snapshot
      char rdy = 0;
      if (!unix_recv_fd(us, nullptr, &rdy, 1, 60000) || rdy != 'R') {
        *err = "snapshot did not arrive";
        break;
      }
      rep_->copy_mirror_from_values(link);  // the parent knows exactly what it just gave us
      if (carry) {
        rep_->add_gate_held(carry);
        rep_->sync();
      }
      int pid = rep_->attach_peer(link, block, remote.ptr);
      {
        std::lock_guard<std::mutex> g(mu_);
        Edge& e = edges_[kSlotUp];
        e.state = 2;
        e.tcp_fd = jr.fd;
        e.peer = jr.parent_addr;
        e.link = link;
        e.block = block;
        e.peer_id = pid;
        e.remote = remote;
        ready_ = true;
      }
      if (reuse) orphan_link_ = -1;  // it is the up link again
      cv_.notify_all();
      ok = true;
    } while (false);
    if (carry) {
      cudaSetDevice(device_);
      cudaFree(carry);
    }
    if (gate_held) rep_->gate_unlock();
    ::close(us);
    if (!ok) {
      if (remote.ptr) vmm_free(&remote);
      if (link >= 0 && !reuse) rep_->remove_link(link);
      if (block >= 0) rep_->free_edge_block(block);
    }
    return ok;
  }

  // u = values - mirror of the lost parent's link, in a scratch buffer (the caller holds the update gate and frees it)
  float* make_carry() {
    if (orphan_link_ < 0) return nullptr;
    cudaSetDevice(device_);
    float* carry = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&carry), size_t(n_) * 4) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cudaStream_t cs = static_cast<cudaStream_t>(rep_->comm_stream());
    cudaMemsetAsync(carry, 0, size_t(n_) * 4, cs);
    launch_sub_add(carry, rep_->values(), rep_->mirror(orphan_link_), n_, 0, rep_->comm_stream());
    rep_->sync();
    return carry;
  }

  void drop_orphan_link() {
    if (orphan_link_ < 0) return;
    rep_->remove_link(orphan_link_);
    orphan_link_ = -1;
  }

  // ---- parent side of the upgrade ----
  void upgrade_loop() {
    while (!stop_.load()) {
      std::vector<pollfd> pfds;
      pfds.push_back({unix_fd_, POLLIN, 0});
      {
        std::lock_guard<std::mutex> g(mu_);
        for (int fd : extra_unix_fds_) pfds.push_back({fd, POLLIN, 0});
      }
      int pr = ::poll(pfds.data(), pfds.size(), kPollMs);
      if (pr <= 0) continue;
      for (auto& pfd : pfds) {
        if (!(pfd.revents & POLLIN)) continue;
        int us = ::accept(pfd.fd, nullptr, nullptr);
        if (us < 0) continue;
        serve_upgrade(us);
        ::close(us);
      }
    }
  }

  void refuse(int us, const char* why) {
    Hello r = my_hello();
    r.status = 1;
    std::snprintf(r.message, sizeof(r.message), "%s", why);
    unix_send_fd(us, -1, &r, sizeof(r));
  }

  void serve_upgrade(int us) {
    Hello h;
    if (!unix_recv_fd(us, nullptr, &h, sizeof(h), opt_.upgrade_timeout_ms) || h.magic != kHelloMagic) return;
    if (h.version != kHelloVersion) return refuse(us, "protocol version mismatch");
    if (h.n != n_) return refuse(us, "Not the right size!");
    if (h.block != gcfg_.block || h.ring_slots != gcfg_.ring_slots || h.bits != gcfg_.bits)
      return refuse(us, "scale block / frame bits / ring geometry mismatch");
    // find the TCP adoption this child belongs to (the two connections race)
    int slot = -1;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait_for(lk, std::chrono::milliseconds(opt_.upgrade_timeout_ms), [&] {
        for (int s = kSlotLeft; s <= kSlotRight; s++) {
          if (edges_[s].state == 1 && edges_[s].peer.sin_port == h.listen_addr.sin_port &&
              edges_[s].peer.sin_addr.s_addr == h.listen_addr.sin_addr.s_addr) {
            slot = s;
            edges_[s].upgrading = true;
            return true;
          }
        }
        return stop_.load();
      });
    }
    if (slot < 0) return refuse(us, "no matching TCP adoption");
    int block = rep_->alloc_edge_block();
    int link = rep_->add_link();
    VmmBlock remote, child_values;
    bool ok = false;
    std::string err;
    do {
      if (block < 0 || link < 0) {
        refuse(us, "parent is out of links");
        break;
      }
      Hello r = my_hello();
      if (!unix_send_fd(us, -1, &r, sizeof(r))) break;
      int fd_edge = -1, fd_vals = -1;
      uint64_t sz_edge = 0, sz_vals = 0;
      if (!unix_recv_fd(us, &fd_edge, &sz_edge, 8, opt_.upgrade_timeout_ms * 4) || fd_edge < 0) break;
      if (!unix_recv_fd(us, &fd_vals, &sz_vals, 8, opt_.upgrade_timeout_ms) || fd_vals < 0) {
        ::close(fd_edge);
        break;
      }
      remote = vmm_import_fd(fd_edge, size_t(sz_edge), device_, &err);
      child_values = vmm_import_fd(fd_vals, size_t(sz_vals), device_, &err);
      ::close(fd_edge);
      ::close(fd_vals);
      if (!remote.ptr || !child_values.ptr) {
        std::fprintf(stderr, "[sharedtensor] cannot map child's memory: %s\n", err.c_str());
        break;
      }
      int my_fd = vmm_export_fd(rep_->edge_block(block), &err);
      if (my_fd < 0) break;
      const uint64_t my_sz = rep_->edge_block(block).bytes;
      bool sent = unix_send_fd(us, my_fd, &my_sz, 8);
      ::close(my_fd);
      if (!sent) break;
      // state transfer: one pass over the replica, in stream order with the rounds
      rep_->push_snapshot(link, reinterpret_cast<float*>(static_cast<uint8_t*>(child_values.ptr) + kGuardBytes));
      int pid = rep_->attach_peer(link, block, remote.ptr);
      {
        std::lock_guard<std::mutex> g(mu_);
        Edge& e = edges_[slot];
        e.state = 2;
        e.upgrading = false;
        e.link = link;
        e.block = block;
        e.peer_id = pid;
        e.remote = remote;
      }
      unix_send_fd(us, -1, "R", 1);
      ok = true;
    } while (false);
    if (child_values.ptr) vmm_free(&child_values);
    if (!ok) {
      if (remote.ptr) vmm_free(&remote);
      if (link >= 0) rep_->remove_link(link);
      if (block >= 0) rep_->free_edge_block(block);
      drop_edge(slot, true);
    }
  }

  // One byte on the otherwise silent TCP connection of every peer-memory edge except `except_slot`.  A GPU cannot
  // interrupt a host thread, so an engine that pauses between rounds would find the first frames of a burst only
  // at its next poll; the doorbell travels ahead of the frames and ends the pause.
  void ring_neighbours(int except_slot) {
    std::lock_guard<std::mutex> g(mu_);
    for (int s = 0; s < kNumSlots; s++) {
      const Edge& e = edges_[s];
      if (s == except_slot || e.state != 2 || e.tcp || e.tcp_fd < 0 || e.peer_id < 0) continue;
      (void)!::send(e.tcp_fd, "W", 1, MSG_DONTWAIT | MSG_NOSIGNAL);
    }
  }

  // ---- liveness ----
  void watch_loop() {
    while (!stop_.load()) {
      std::vector<pollfd> pfds;
      std::vector<int> slots;
      {
        std::lock_guard<std::mutex> g(mu_);
        for (int s = 0; s < kNumSlots; s++) {
          if (edges_[s].state && edges_[s].tcp_fd >= 0 && !edges_[s].tcp) {
            pfds.push_back({edges_[s].tcp_fd, POLLIN, 0});
            slots.push_back(s);
          }
          if (edges_[s].tcp && tcp_[s] && tcp_[s]->failed.load()) {
            pfds.push_back({-1, 0, 0});
            slots.push_back(100 + s);
          }
          // a child that was adopted over TCP but never came in over the unix socket is a TCP-only
          // peer (CPU node, reference, other host): not served by this class
          if (edges_[s].state == 1 && !edges_[s].upgrading && now_ms() - edges_[s].adopted_ms > 600) {
            pfds.push_back({-1, 0, 0});
            slots.push_back(-(s + 1));
          }
        }
      }
      if (pfds.empty()) {
        ::usleep(kPollMs * 1000);
        continue;
      }
      int pr = ::poll(pfds.data(), pfds.size(), kPollMs);
      for (size_t i = 0; i < pfds.size(); i++) {
        if (slots[i] < 0) {
          // adopted over TCP and no peer-memory hello followed: a TCP-only child (CPU node, reference, other host)
          int s = -slots[i] - 1;
          int fd;
          sockaddr_in peer;
          {
            std::lock_guard<std::mutex> g(mu_);
            if (edges_[s].state != 1 || edges_[s].upgrading) continue;
            fd = edges_[s].tcp_fd;
            peer = edges_[s].peer;
            edges_[s].upgrading = true;  // claimed
          }
          start_tcp_edge(s, fd, peer);
          continue;
        }
        int s = slots[i];
        if (s < 100) {
          if (pr <= 0 || !(pfds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
          char buf[256];
          ssize_t r = ::recv(pfds[i].fd, buf, sizeof(buf), MSG_DONTWAIT);
          if (r > 0) {
            // a doorbell: the neighbour is about to send frames.  Poll at full rate, and pass the doorbell on if
            // this engine had been pausing (the rest of the tree then is, too).
            if (rep_->wake(true)) ring_neighbours(s);
            continue;
          }
          if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) continue;
        } else {
          s -= 100;  // a TCP edge whose thread reported a failure
        }
        if (stop_.load()) break;
        std::fprintf(stderr, "[sharedtensor] edge %d lost (neighbour closed its connection)\n", s);
        bool was_up = s == kSlotUp;
        // the up link of a node that will re-join stays (without its rings): its mirror is what the lost parent knew
        drop_edge(s, true, was_up && opt_.rejoin);
        if (was_up) {
          if (!opt_.rejoin) {
            master_.store(true);
            continue;
          }
          {
            std::lock_guard<std::mutex> g(mu_);
            ready_ = false;
          }
          // the new parent writes its snapshot into this replica's values: no round may run meanwhile
          rep_->stop_engine();
          int backoff = opt_.rejoin_backoff_ms;
          while (!stop_.load()) {
            if (join(false, nullptr, nullptr)) {
              std::lock_guard<std::mutex> g(mu_);
              rejoins_++;
              break;
            }
            ::usleep(useconds_t(backoff) * 1000);
            if (backoff < 5000) backoff *= 2;
          }
          if (opt_.start_engine && !stop_.load()) rep_->start_engine();
        }
      }
    }
  }

  void drop_edge(int slot, bool count, bool keep_link = false) {
    Edge old;
    std::unique_ptr<TcpEdge> te;
    {
      std::lock_guard<std::mutex> g(mu_);
      te = std::move(tcp_[slot]);
    }
    if (te) {
      te->stop.store(true);
      if (te->fd >= 0) ::shutdown(te->fd, SHUT_RDWR);
      if (te->tx.joinable()) te->tx.join();
      if (te->rx.joinable()) te->rx.join();
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      old = edges_[slot];
      edges_[slot] = Edge();
      edges_[slot].slot = slot;
      if (count && old.state) edge_failures_++;
    }
    if (!old.state) return;
    if (rep_) {
      if (old.peer_id >= 0 && keep_link && orphan_link_ < 0 && old.remote.ptr) {
        // the lost parent never acknowledged these frames: what they said counts as not yet told
        try {
          const uint64_t back = rep_->unsend_unacknowledged(old.peer_id);
          if (back) std::fprintf(stderr, "[sharedtensor] took %llu unacknowledged tile-frames back from the lost edge\n", (unsigned long long)back);
        } catch (const std::exception&) {
        }
      }
      if (old.peer_id >= 0) rep_->detach_peer(old.peer_id);
      if (old.link >= 0) {
        if (keep_link && orphan_link_ < 0) orphan_link_ = old.link;
        else rep_->remove_link(old.link);
      }
      if (old.block >= 0) rep_->free_edge_block(old.block);
    }
    if (old.remote.ptr) vmm_free(&old.remote);
    if (old.tcp_fd >= 0) {
      ::shutdown(old.tcp_fd, SHUT_RDWR);
      ::close(old.tcp_fd);
    }
  }

  std::unique_ptr<GpuReplica> rep_;
  GpuConfig gcfg_;
  GpuNodeOptions opt_;
  int device_;
  int64_t n_;
  std::string host_;
  int port_ = 0;
  sockaddr_in listen_addr_{};
  std::unique_ptr<TreeListener> listener_;
  int unix_fd_ = -1;
  Edge edges_[kNumSlots];
  std::unique_ptr<TcpEdge> tcp_[kNumSlots];
  std::mutex mu_;
  std::condition_variable cv_;
  bool ready_ = false;
  std::atomic<bool> master_{false}, closed_{false}, started_{false}, stop_{false};
  std::thread upgrade_thread_, watch_thread_;
  uint64_t rejoins_ = 0, edge_failures_ = 0;
  std::vector<sockaddr_in> my_addrs_;  // every address this node listens on (start / watch thread only)
  int orphan_link_ = -1;  // the lost parent's link, kept (with its mirror) until a new parent has been found
  std::vector<int> extra_unix_fds_;  // peer-memory endpoints under the addresses of later up connections
};

}  // namespace st
