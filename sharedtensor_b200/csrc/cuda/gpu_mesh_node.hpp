// Mesh group of GPU replicas (see the banner below); defined in a header for the same reason as GpuNode.
#pragma once
#include "gpu_node.hpp"

namespace st {

// =================================================================================================
// Mesh group: a fixed set of GPU replicas on one NVSwitch box, fully connected.
//
// Every member has ONE link (one mirror) with a ring pair to every other member: its frames are pushed to all
// peers, frames from a peer are applied and not forwarded (the peer's own push already reaches everybody).
// An update therefore crosses exactly one hop and is quantised once, instead of being re-quantised along a
// tree path; NVSwitch gives every pair full bandwidth, so the tree's purpose (bounded fan-out per node on a
// network of point-to-point links) does not apply inside the box.  Membership is fixed at creation: member r
// listens on an abstract unix socket derived from the group's host:port and its rank, the higher rank of each
// pair connects to the lower.  Member 0 holds the initial values and copies them into every other member
// before anybody's createOrFetch returns.  A member whose connection closes is dropped from the group.
// =================================================================================================
struct MeshHello {
  uint32_t magic = 0x4d425453;  // "STBM"
  int32_t rank = 0, world = 0;
  int64_t n = 0;
  int32_t block = 0, ring_slots = 0;
  int32_t bits = 0, reserved = 0;
  uint64_t edge_bytes = 0, values_bytes = 0;
};

class GpuMeshNode {
 public:
  GpuMeshNode(int device, int64_t n, const GpuConfig& gcfg, int rank, int world, bool start_engine)
      : rep_(new GpuReplica(device, n, gcfg)), gcfg_(gcfg), device_(device), n_(n), rank_(rank), world_(world),
        start_engine_(start_engine) {
    if (world < 1 || world > kMaxRings + 1 || rank < 0 || rank >= world)
      throw std::invalid_argument("mesh group needs 1..9 members and a rank inside it");
    peers_.resize(size_t(world));
    rep_->set_doorbell([this] { ring_members(); });
  }
  ~GpuMeshNode() { close(); }
  GpuReplica& replica() { return *rep_; }

  void start(const std::string& host, int port, const float* init_dev, void* stream, int timeout_ms) {
    std::string err;
    const std::string base = "sharedtensor_b200/mesh/" + host + ":" + std::to_string(port) + "/";
    listen_fd_ = unix_listen_abstract(base + std::to_string(rank_), &err);
    if (listen_fd_ < 0) throw std::runtime_error("mesh: " + err);
    link_ = rep_->add_link();
    if (rank_ == 0 && init_dev) rep_->load_values(init_dev, stream);
    rep_->sync();
    // lower ranks are connected to, higher ranks are accepted from
    for (int j = 0; j < rank_; j++) {
      int fd = unix_connect_abstract(base + std::to_string(j), timeout_ms);
      if (fd < 0) throw std::runtime_error("mesh: member " + std::to_string(j) + " is not there");
      handshake(fd, j);
    }
    for (int k = rank_ + 1; k < world_; k++) {
      struct pollfd pfd = {listen_fd_, POLLIN, 0};
      if (::poll(&pfd, 1, timeout_ms) <= 0) throw std::runtime_error("mesh: timed out waiting for the other members");
      int fd = ::accept(listen_fd_, nullptr, nullptr);
      if (fd < 0) throw std::runtime_error("mesh: accept failed");
      handshake(fd, -1);
    }
    // common initial state, then the go signal
    if (rank_ == 0) {
      for (int j = 1; j < world_; j++) {
        rep_->push_snapshot(link_, reinterpret_cast<float*>(static_cast<uint8_t*>(peers_[size_t(j)].values.ptr) + kGuardBytes));
        vmm_free(&peers_[size_t(j)].values);
      }
      if (world_ == 1) rep_->copy_mirror_from_values(link_);
      for (int j = 1; j < world_; j++) unix_send_fd(peers_[size_t(j)].fd, -1, "R", 1);
    } else {
      char c = 0;
      if (!unix_recv_fd(peers_[0].fd, nullptr, &c, 1, timeout_ms) || c != 'R') throw std::runtime_error("mesh: initial state did not arrive");
      rep_->copy_mirror_from_values(link_);
    }
    rep_->sync();
    watch_ = std::thread([this] { watch_loop(); });
    if (start_engine_) rep_->start_engine();
  }

  int members_alive() {
    std::lock_guard<std::mutex> g(mu_);
    int c = 1;
    for (auto& p : peers_) c += p.fd >= 0;
    return c;
  }
  int dropped() {
    std::lock_guard<std::mutex> g(mu_);
    return dropped_;
  }

  void close() {
    if (closed_.exchange(true)) return;
    stop_.store(true);
    if (rep_) rep_->set_doorbell(nullptr);
    if (rep_) rep_->stop_engine();
    if (watch_.joinable()) watch_.join();
    for (int j = 0; j < world_; j++) drop_peer(j);
    if (listen_fd_ >= 0) ::close(listen_fd_);
    listen_fd_ = -1;
    rep_.reset();
  }

 private:
  struct Peer {
    int fd = -1;
    int block = -1, peer_id = -1;
    VmmBlock remote, values;
  };

  void handshake(int fd, int expect_rank) {
    std::string err;
    int block = rep_->alloc_edge_block();
    if (block < 0) throw std::runtime_error("mesh: out of edge blocks");
    MeshHello h;
    h.rank = rank_;
    h.world = world_;
    h.n = n_;
    h.block = gcfg_.block;
    h.ring_slots = gcfg_.ring_slots;
    h.bits = gcfg_.bits;
    h.edge_bytes = rep_->edge_block(block).bytes;
    h.values_bytes = rep_->values_block().bytes;
    MeshHello o;
    if (!unix_send_fd(fd, -1, &h, sizeof(h)) || !unix_recv_fd(fd, nullptr, &o, sizeof(o), 10000) || o.magic != h.magic)
      throw std::runtime_error("mesh: hello failed");
    if (o.n != n_ || o.block != h.block || o.ring_slots != h.ring_slots || o.bits != h.bits || o.world != world_ || o.rank == rank_ ||
        (expect_rank >= 0 && o.rank != expect_rank))
      throw std::runtime_error("mesh: members disagree on size, block, ring geometry or group");
    int my_fd = vmm_export_fd(rep_->edge_block(block), &err);
    if (my_fd < 0) throw std::runtime_error("mesh: " + err);
    bool ok = unix_send_fd(fd, my_fd, "E", 1);
    ::close(my_fd);
    int their_fd = -1;
    char tag = 0;
    ok = ok && unix_recv_fd(fd, &their_fd, &tag, 1, 10000) && their_fd >= 0;
    if (!ok) throw std::runtime_error("mesh: edge block exchange failed");
    Peer& p = peers_[size_t(o.rank)];
    p.remote = vmm_import_fd(their_fd, size_t(o.edge_bytes), device_, &err);
    ::close(their_fd);
    if (!p.remote.ptr) throw std::runtime_error("mesh: cannot map peer memory: " + err);
    // member 0 gets everybody's values to write the initial state into
    if (o.rank == 0) {
      int vfd = vmm_export_fd(rep_->values_block(), &err);
      if (vfd < 0) throw std::runtime_error("mesh: " + err);
      ok = unix_send_fd(fd, vfd, "V", 1);
      ::close(vfd);
      if (!ok) throw std::runtime_error("mesh: values exchange failed");
    } else if (rank_ == 0) {
      int vfd = -1;
      if (!unix_recv_fd(fd, &vfd, &tag, 1, 10000) || vfd < 0) throw std::runtime_error("mesh: values exchange failed");
      p.values = vmm_import_fd(vfd, size_t(o.values_bytes), device_, &err);
      ::close(vfd);
      if (!p.values.ptr) throw std::runtime_error("mesh: cannot map peer values: " + err);
    }
    p.fd = fd;
    p.block = block;
    p.peer_id = rep_->attach_peer(link_, block, p.remote.ptr);
  }

  void watch_loop() {
    while (!stop_.load()) {
      std::vector<pollfd> pfds;
      std::vector<int> who;
      {
        std::lock_guard<std::mutex> g(mu_);
        for (int j = 0; j < world_; j++)
          if (peers_[size_t(j)].fd >= 0) {
            pfds.push_back({peers_[size_t(j)].fd, POLLIN, 0});
            who.push_back(j);
          }
      }
      if (pfds.empty()) {
        ::usleep(kPollMs * 1000);
        continue;
      }
      if (::poll(pfds.data(), pfds.size(), kPollMs) <= 0) continue;
      for (size_t i = 0; i < pfds.size(); i++) {
        if (!(pfds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
        char buf[64];
        ssize_t r = ::recv(pfds[i].fd, buf, sizeof(buf), MSG_DONTWAIT);
        if (r > 0) {
          rep_->wake(true);  // a doorbell: that member is about to send frames (one hop: nothing to pass on)
          continue;
        }
        if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) continue;
        if (stop_.load()) break;
        std::fprintf(stderr, "[sharedtensor] mesh member %d is gone, dropping its rings\n", who[i]);
        drop_peer(who[i]);
        std::lock_guard<std::mutex> g(mu_);
        dropped_++;
      }
    }
  }

  void ring_members() {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& p : peers_)
      if (p.fd >= 0 && p.peer_id >= 0) (void)!::send(p.fd, "W", 1, MSG_DONTWAIT | MSG_NOSIGNAL);
  }

  void drop_peer(int j) {
    Peer old;
    {
      std::lock_guard<std::mutex> g(mu_);
      old = peers_[size_t(j)];
      peers_[size_t(j)] = Peer();
    }
    if (old.fd < 0 && !old.remote.ptr) return;
    if (rep_) {
      if (old.peer_id >= 0) rep_->detach_peer(old.peer_id);
      if (old.block >= 0) rep_->free_edge_block(old.block);
    }
    if (old.remote.ptr) vmm_free(&old.remote);
    if (old.values.ptr) vmm_free(&old.values);
    if (old.fd >= 0) ::close(old.fd);
  }

  std::unique_ptr<GpuReplica> rep_;
  GpuConfig gcfg_;
  int device_;
  int64_t n_;
  int rank_, world_;
  bool start_engine_;
  int listen_fd_ = -1, link_ = -1;
  std::vector<Peer> peers_;
  std::mutex mu_;
  std::thread watch_;
  std::atomic<bool> stop_{false}, closed_{false};
  int dropped_ = 0;
};

}  // namespace st
