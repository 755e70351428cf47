#include "node.hpp"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <stdexcept>

namespace st {

uint64_t now_ms() {
  using namespace std::chrono;
  return uint64_t(duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count());
}

CpuNode::CpuNode(int64_t n, const NodeConfig& cfg) : n_(n), cfg_(cfg) {
  if (n <= 0) throw std::invalid_argument("shared tensor needs at least one element");
  if (cfg_.tcp_block != 0) {
    int b = cfg_.tcp_block;
    if (b < 32 || b > 4096 || (b & (b - 1))) throw std::invalid_argument("tcp_block must be 0 or a power of two in 32..4096");
  }
  if (cfg_.tcp_bits != 1 && cfg_.tcp_bits != 8) throw std::invalid_argument("tcp_bits must be 1 or 8");
  if (cfg_.tcp_bits == 8 && cfg_.tcp_block == 0) throw std::invalid_argument("8-bit frames need a block scale mode (tcp_block)");
  values_.assign(size_t(n), 0.0f);
  for (int s = 0; s < kNumSlots; s++) edges_[s].slot = s;
}

CpuNode::~CpuNode() { close(); }

size_t CpuNode::frame_bytes() const {
  if (cfg_.tcp_block == 0) return 4 + sign_bytes(size_t(n_));
  if (cfg_.tcp_bits == 8) return block_scales(size_t(n_), cfg_.tcp_block) + size_t(n_);  // scale bytes, one code byte per element
  return block_scales(size_t(n_), cfg_.tcp_block) + 4 * block_words(size_t(n_));
}

void CpuNode::start(const std::string& host, int port, const float* init) {
  if (started_.exchange(true)) throw std::runtime_error("node already started");
  host_ = host;
  port_ = port;
  listener_.reset(new TreeListener(
      [this]() -> int {
        std::lock_guard<std::mutex> g(mu_);
        if (closed_.load()) return -1;
        if (edges_[kSlotLeft].state.load() == 0) return kSlotLeft;
        if (edges_[kSlotRight].state.load() == 0) return kSlotRight;
        return -1;
      },
      [this](int slot, int fd, const sockaddr_in& peer) { attach_edge(slot, fd, peer); },
      [this](int slot, sockaddr_in* out) -> bool {
        std::lock_guard<std::mutex> g(mu_);
        if (edges_[slot].state.load() != 1) return false;
        *out = edges_[slot].peer;
        return true;
      }));
  // A first join can fail for a passing reason: the node listens on the source address of its up connection, and on
  // a busy host that ephemeral port may just have been taken by another process's listener.  A new connection gets a
  // new port, so a few attempts are made before giving up.
  bool joined = false;
  for (int attempt = 0; attempt < 4 && !joined && !stop_.load(); attempt++) {
    if (attempt) ::usleep(50 * 1000);
    joined = do_join(true, init);
  }
  if (!joined) {
    started_.store(false);
    listener_.reset();
    throw std::runtime_error("shared tensor could not join or found a tree at " + host + ":" + std::to_string(port));
  }
  listener_->start();
  supervisor_ = std::thread([this] { supervisor_loop(); });
}

bool CpuNode::do_join(bool first, const float* init) {
  JoinResult jr = join_tree(host_, port_, &stop_, 64, 10000, &my_addrs_);
  if (!jr.ok) {
    std::fprintf(stderr, "[sharedtensor] join failed: %s\n", jr.error.c_str());
    return false;
  }
  std::string err;
  if (jr.master) {
    int lfd = open_listener(jr.listen_addr, cfg_.listen_backlog, &err);
    if (lfd < 0) {
      // Either host:port is not an address of this machine, or another orphan won the race to
      // become the new master.  The caller retries.
      std::fprintf(stderr, "[sharedtensor] cannot serve %s:%d as master: %s\n", host_.c_str(), port_, err.c_str());
      return false;
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      if (first && init)
        for (int64_t i = 0; i < n_; i++) values_[size_t(i)] += init[i];
      if (first) listen_addr_ = jr.listen_addr;
      my_addrs_.push_back(jr.listen_addr);
      master_.store(true);
      ready_.store(true);
      for (int s = kSlotLeft; s <= kSlotRight; s++) edges_[s].paused.store(false);
    }
    listener_->add_listen_fd(lfd);
    ready_cv_.notify_all();
    std::fprintf(stderr, "[sharedtensor] master of %s:%d (%lld elements)\n", host_.c_str(), port_, (long long)n_);
    log_event(first ? "master" : "took_over", host_ + ":" + std::to_string(port_));
    return true;
  }
  if (first) {
    int lfd = open_listener(jr.listen_addr, cfg_.listen_backlog, &err);
    if (lfd < 0) {
      std::fprintf(stderr, "[sharedtensor] cannot listen on %s: %s\n", addr_to_string(jr.listen_addr).c_str(), err.c_str());
      ::close(jr.fd);
      return false;
    }
    listen_addr_ = jr.listen_addr;
    my_addrs_.push_back(jr.listen_addr);
    listener_->add_listen_fd(lfd);
  } else {
    // The new parent knows this node by the source address of the new connection and hands that address to later
    // joiners: accept joins there too (best effort; the first address stays open for redirects already handed out).
    int lfd = open_listener(jr.listen_addr, cfg_.listen_backlog, &err);
    if (lfd >= 0) {
      listener_->add_listen_fd(lfd);
      my_addrs_.push_back(jr.listen_addr);
    }
    // Re-join keeping the part of the state the lost parent had not been told yet:
    // values <- values - mirror_up, so that it is sent up the new edge (whose mirror starts at 0)
    // while the new parent streams its whole state down.  Child edges pause meanwhile.
    std::lock_guard<std::mutex> g(mu_);
    Edge& up = edges_[kSlotUp];
    if (up.mirror.size() == size_t(n_))
      for (int64_t i = 0; i < n_; i++) values_[size_t(i)] -= up.mirror[size_t(i)];
    for (int s = kSlotLeft; s <= kSlotRight; s++) edges_[s].paused.store(true);
    ready_.store(false);
  }
  master_.store(false);
  attach_edge(kSlotUp, jr.fd, jr.parent_addr);
  log_event(first ? "joined" : "rejoined", "below " + addr_to_string(jr.parent_addr) + " after " + std::to_string(jr.hops) + " redirect(s)");
  std::fprintf(stderr, "[sharedtensor] joined %s:%d below %s after %d redirect(s)\n", host_.c_str(), port_,
               addr_to_string(jr.parent_addr).c_str(), jr.hops);
  return true;
}

void CpuNode::log_event(const char* kind, const std::string& detail) {
  NodeEvent ev;
  ev.ms = uint64_t(std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
  ev.kind = kind;
  ev.detail = detail;
  std::lock_guard<std::mutex> g(ev_mu_);
  events_.push_back(std::move(ev));
  if (events_.size() > 64) events_.pop_front();
}

void CpuNode::attach_edge(int slot, int fd, const sockaddr_in& peer) {
  Edge& e = edges_[slot];
  std::lock_guard<std::mutex> g(mu_);
  if (closed_.load() || e.state.load() != 0) {
    ::close(fd);
    return;
  }
  e.fd = fd;
  e.peer = peer;
  e.mirror.assign(size_t(n_), 0.0f);
  e.stop.store(false);
  e.drop_frames.store(0);
  e.sent_first = false;
  e.idle_announced = false;
  e.idle = false;
  e.first_scale_recv = 0;
  e.last_recv_ms = now_ms();
  e.st = EdgeStats();
  e.st.peer = addr_to_string(peer);
  e.state.store(1);
  if (slot != kSlotUp) log_event("adopted", std::string(slot == kSlotLeft ? "left " : "right ") + addr_to_string(peer));
  e.tx = std::thread([this, &e] { tx_loop(&e); });
  e.rx = std::thread([this, &e] { rx_loop(&e); });
}

void CpuNode::edge_failed(Edge* e, const char* why, IoStatus st) {
  int expect = 1;
  if (!e->state.compare_exchange_strong(expect, 2)) return;
  e->stop.store(true);
  if (!stop_.load()) log_event("edge_lost", std::string(e->slot == kSlotUp ? "up " : (e->slot == kSlotLeft ? "left " : "right ")) + e->st.peer + ": " + why);
  if (!stop_.load())
    std::fprintf(stderr, "[sharedtensor] edge %d (%s) lost: %s (%s)\n", e->slot, e->st.peer.c_str(), why,
                 io_status_name(st));
  if (e->fd >= 0) ::shutdown(e->fd, SHUT_RDWR);
  work_cv_.notify_all();
  {
    std::lock_guard<std::mutex> g(sup_mu_);
    dead_slots_.push_back(e->slot);
  }
  sup_cv_.notify_all();
}

void CpuNode::tx_loop(Edge* e) {
  std::vector<uint8_t> frame(frame_bytes());
  const size_t n = size_t(n_);
  const int B = cfg_.tcp_block;
  uint64_t last_sent = 0;
  uint64_t my_version = 0;
  while (!e->stop.load()) {
    bool noop;
    {
      std::unique_lock<std::mutex> lk(mu_);
      if (e->paused.load() || (e->idle && e->sent_first && my_version == e->dirty)) {
        int wait_ms = cfg_.idle_keepalive_ms > 0 ? cfg_.idle_keepalive_ms : 200;
        work_cv_.wait_for(lk, std::chrono::milliseconds(wait_ms));
        if (e->stop.load()) break;
        if (e->paused.load()) continue;
        bool keepalive = cfg_.idle_keepalive_ms > 0 && now_ms() - last_sent >= uint64_t(cfg_.idle_keepalive_ms);
        if (my_version == e->dirty && !keepalive) continue;
      }
      my_version = e->dirty;
      double resid = 0.0;
      if (B == 0) {
        // smallest step worth sending, relative to the replica's largest element: a step of at least
        // 2^-22 of it is a whole number of ulps of every element, so it can never round away
        float scale;
        if (cfg_.tcp_rule == 1) {
          scale = encode_tensor_fast(values_.data(), e->mirror.data(), n, frame.data() + 4, cfg_.min_scale_abs, cfg_.min_scale_rel);
        } else {
          float min_scale = cfg_.min_scale_abs;
          if (cfg_.min_scale_rel > 0.0f) {
            float vmax = 0.0f;
            for (size_t i = 0; i < n; i++) {
              float a = std::fabs(values_[i]);
              if (a > vmax) vmax = a;
            }
            float rel = vmax * cfg_.min_scale_rel;
            if (rel > min_scale) min_scale = rel;
          }
          scale = encode_tensor(values_.data(), e->mirror.data(), n, frame.data() + 4, min_scale, cfg_.tcp_rule);
        }
        std::memcpy(frame.data(), &scale, 4);
        noop = scale == 0.0f;
        e->st.last_scale_sent = scale;
        resid = double(scale);
      } else {
        size_t ns = block_scales(n, B);
        uint8_t* scales = frame.data();
        double ss;
        if (cfg_.tcp_bits == 8) {
          ss = encode_block_int8_fast(values_.data(), e->mirror.data(), n, B, cfg_.gate, frame.data() + ns, scales);
        } else {
          uint32_t* words = reinterpret_cast<uint32_t*>(frame.data() + ns);
          // words need 4-byte alignment: ns may be odd, so encode into an aligned scratch
          static thread_local std::vector<uint32_t> wtmp;
          wtmp.assign(block_words(n), 0u);
          ss = encode_block_fast(values_.data(), e->mirror.data(), n, B, cfg_.gate, wtmp.data(), scales);
          std::memcpy(words, wtmp.data(), 4 * wtmp.size());
        }
        noop = true;
        int maxc = 0;
        for (size_t i = 0; i < ns; i++) {
          if (scales[i]) noop = false;
          if (scales[i] > maxc) maxc = scales[i];
        }
        e->st.last_scale_sent = maxc ? exp2i(maxc - 127) : 0.0f;
        resid = ss;  // largest outstanding |residual|
      }
      e->st.residual_rms = resid;
      e->idle = noop;
    }
    // A no-op frame is sent once when a burst ends: it tells the peer (a joiner waiting for its
    // state in particular) that this side has nothing more to say for now.
    bool must_send = !noop || !e->sent_first || !e->idle_announced ||
                     (cfg_.idle_keepalive_ms > 0 && now_ms() - last_sent >= uint64_t(cfg_.idle_keepalive_ms));
    if (!must_send) continue;
    if (cfg_.max_frames_per_s > 0.0) {
      uint64_t gap = uint64_t(1000.0 / cfg_.max_frames_per_s);
      uint64_t now = now_ms();
      if (last_sent && now - last_sent < gap) ::usleep(useconds_t((gap - (now - last_sent)) * 1000));
    }
    IoStatus st = write_full(e->fd, frame.data(), frame.size(), &e->stop);
    if (st != IoStatus::Ok) {
      // Not written: the mirror's step is taken back, so that the frame's content is still in values - mirror when
      // the node re-joins.  (A frame the kernel accepted but the peer never read is lost for good: no resend.)
      if (!noop) {
        std::lock_guard<std::mutex> g(mu_);
        if (e->mirror.size() == n) {
          if (B == 0) {
            float scale;
            std::memcpy(&scale, frame.data(), 4);
            decode_tensor_add_fast(frame.data() + 4, -scale, n, e->mirror.data(), nullptr);
          } else if (cfg_.tcp_bits == 8) {
            size_t ns = block_scales(n, B);
            decode_block_int8_add_fast(frame.data() + ns, frame.data(), n, B, -1.0f, e->mirror.data(), nullptr);
          } else {
            size_t ns = block_scales(n, B);
            std::vector<uint32_t> flipped(block_words(n));
            std::memcpy(flipped.data(), frame.data() + ns, 4 * flipped.size());
            for (auto& w : flipped) w = ~w;
            decode_block_add_fast(flipped.data(), frame.data(), n, B, e->mirror.data(), nullptr);
          }
        }
      }
      if (st != IoStatus::Stopped) edge_failed(e, "send", st);
      break;
    }
    last_sent = now_ms();
    {
      std::lock_guard<std::mutex> g(mu_);
      e->sent_first = true;
      e->idle_announced = noop;
      e->st.frames_sent++;
      e->st.bytes_sent += frame.size();
      if (noop) e->st.noop_sent++;
    }
  }
}

void CpuNode::rx_loop(Edge* e) {
  std::vector<uint8_t> frame(frame_bytes());
  std::vector<uint32_t> wtmp;
  const size_t n = size_t(n_);
  const int B = cfg_.tcp_block;
  const uint64_t t_attach = now_ms();
  while (!e->stop.load()) {
    IoStatus st = read_full(e->fd, frame.data(), frame.size(), &e->stop);
    if (st != IoStatus::Ok) {
      if (st != IoStatus::Stopped) edge_failed(e, "receive", st);
      break;
    }
    std::unique_lock<std::mutex> lk(mu_);
    e->st.frames_recv++;
    e->st.bytes_recv += frame.size();
    e->last_recv_ms = now_ms();
    if (e->drop_frames.load() > 0) {
      e->drop_frames.fetch_sub(1);
      e->st.dropped_by_injection++;
      continue;
    }
    float level;  // magnitude indicator of this frame, 0 for a no-op
    if (B == 0) {
      float scale;
      std::memcpy(&scale, frame.data(), 4);
      if (!std::isfinite(scale) || scale < 0.0f) {
        lk.unlock();
        edge_failed(e, "malformed frame (scale)", IoStatus::Error);
        break;
      }
      decode_tensor_add_fast(frame.data() + 4, scale, n, values_.data(), e->mirror.data());
      level = scale;
    } else {
      size_t ns = block_scales(n, B);
      int maxc = 0;
      for (size_t i = 0; i < ns; i++)
        if (frame[i] > maxc) maxc = frame[i];
      if (maxc == 255) {  // no encoder emits this code (it would decode to infinity): the peer's stream is broken
        lk.unlock();
        edge_failed(e, "malformed frame (scale code)", IoStatus::Error);
        break;
      }
      if (cfg_.tcp_bits == 8) {
        decode_block_int8_add_fast(frame.data() + ns, frame.data(), n, B, 1.0f, values_.data(), e->mirror.data());
      } else {
        wtmp.resize(block_words(n));
        std::memcpy(wtmp.data(), frame.data() + ns, 4 * wtmp.size());
        decode_block_add_fast(wtmp.data(), frame.data(), n, B, values_.data(), e->mirror.data());
      }
      level = maxc ? exp2i(maxc - 127) : 0.0f;
    }
    e->st.last_scale_recv = level;
    if (level == 0.0f) {
      e->st.noop_recv++;
    } else {
      for (int s = 0; s < kNumSlots; s++)  // the other edges now have something to forward
        if (s != e->slot) edges_[s].dirty++;
    }
    if (e->slot == kSlotUp && !ready_.load()) {
      if (e->first_scale_recv == 0.0f && level > 0.0f) e->first_scale_recv = level;
      bool rdy = level == 0.0f || cfg_.ready_mode == 0 ||
                 level <= std::ldexp(e->first_scale_recv, -cfg_.ready_bits) ||
                 now_ms() - t_attach > uint64_t(cfg_.ready_timeout_ms);
      if (rdy) {
        ready_.store(true);
        for (int s = kSlotLeft; s <= kSlotRight; s++) edges_[s].paused.store(false);
        ready_cv_.notify_all();
      }
    }
    lk.unlock();
    if (level != 0.0f) work_cv_.notify_all();
  }
}

void CpuNode::reap_edge(Edge* e) {
  if (e->tx.joinable()) e->tx.join();
  if (e->rx.joinable()) e->rx.join();
  std::lock_guard<std::mutex> g(mu_);
  if (e->fd >= 0) {
    ::close(e->fd);
    e->fd = -1;
  }
  edge_failures_++;
  if (e->slot != kSlotUp) {
    std::vector<float>().swap(e->mirror);  // a new child in this slot starts from scratch
    e->state.store(0);
  }
  // the up mirror is kept until the re-join has used it
}

void CpuNode::supervisor_loop() {
  while (true) {
    int slot = -1;
    {
      std::unique_lock<std::mutex> lk(sup_mu_);
      sup_cv_.wait(lk, [&] { return stop_.load() || !dead_slots_.empty(); });
      if (stop_.load()) return;
      slot = dead_slots_.front();
      dead_slots_.pop_front();
    }
    Edge* e = &edges_[slot];
    reap_edge(e);
    if (slot != kSlotUp) continue;
    if (!cfg_.rejoin) {
      std::lock_guard<std::mutex> g(mu_);
      std::vector<float>().swap(e->mirror);
      e->state.store(0);
      master_.store(true);  // detached root of its own subtree
      continue;
    }
    // re-join: keep trying until it works or the node is closed
    int backoff = cfg_.rejoin_backoff_ms;
    while (!stop_.load()) {
      {
        std::lock_guard<std::mutex> g(mu_);
        e->state.store(0);
      }
      if (do_join(false, nullptr)) {
        std::lock_guard<std::mutex> g(mu_);
        rejoins_++;
        if (master_.load()) std::vector<float>().swap(e->mirror);
        break;
      }
      {
        std::lock_guard<std::mutex> g(mu_);
        e->state.store(2);
      }
      ::usleep(useconds_t(backoff) * 1000);
      if (backoff < 5000) backoff *= 2;
    }
  }
}

bool CpuNode::wait_ready(int timeout_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  return ready_cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return ready_.load() || closed_.load(); }) &&
         ready_.load();
}

void CpuNode::add(const float* delta, int64_t n) {
  if (n != n_) throw std::invalid_argument("Not the right size!");
  if (closed_.load()) throw std::runtime_error("shared tensor is closed");
  {
    std::lock_guard<std::mutex> g(mu_);
    add_fast(values_.data(), delta, size_t(n_));
    for (int s = 0; s < kNumSlots; s++) edges_[s].dirty++;
    adds_++;
  }
  work_cv_.notify_all();
}

void CpuNode::sub_add(const float* neu, const float* old, int64_t n) {
  if (n != n_) throw std::invalid_argument("Not the right size!");
  if (closed_.load()) throw std::runtime_error("shared tensor is closed");
  {
    std::lock_guard<std::mutex> g(mu_);
    sub_add_fast(values_.data(), neu, old, size_t(n_));
    for (int s = 0; s < kNumSlots; s++) edges_[s].dirty++;
    adds_++;
  }
  work_cv_.notify_all();
}

void CpuNode::copy_to(float* out, int64_t n) {
  if (n != n_) throw std::invalid_argument("Not the right size!");
  std::lock_guard<std::mutex> g(mu_);
  copy_fast(out, values_.data(), size_t(n_));
  copies_++;
}

void CpuNode::export_state(std::vector<float>* values, std::vector<float> mirrors[kNumSlots]) {
  std::lock_guard<std::mutex> g(mu_);
  *values = values_;
  for (int s = 0; s < kNumSlots; s++)
    if (edges_[s].state.load() == 1) mirrors[s] = edges_[s].mirror;
}

void CpuNode::import_values(const float* v, int64_t n) {
  if (n != n_) throw std::invalid_argument("Not the right size!");
  {
    std::lock_guard<std::mutex> g(mu_);
    std::memcpy(values_.data(), v, size_t(n_) * sizeof(float));
    for (int s = 0; s < kNumSlots; s++) edges_[s].dirty++;
  }
  work_cv_.notify_all();
}

bool CpuNode::flush(int timeout_ms, int quiet_ms) {
  uint64_t t0 = now_ms();
  while (now_ms() - t0 < uint64_t(timeout_ms)) {
    {
      std::lock_guard<std::mutex> g(mu_);
      bool quiet = true;
      uint64_t now = now_ms();
      for (int s = 0; s < kNumSlots; s++) {
        Edge& e = edges_[s];
        if (e.state.load() != 1) continue;
        if (!(e.idle && e.sent_first) || now - e.last_recv_ms < uint64_t(quiet_ms)) quiet = false;
      }
      if (quiet) return true;
    }
    ::usleep(2000);
  }
  return false;
}

void CpuNode::inject_drop_frames(int slot, int k) { edges_[slot].drop_frames.store(k); }

void CpuNode::inject_sever(int slot) {
  std::lock_guard<std::mutex> g(mu_);
  if (edges_[slot].fd >= 0) ::shutdown(edges_[slot].fd, SHUT_RDWR);
}

NodeStats CpuNode::stats() {
  NodeStats s;
  std::lock_guard<std::mutex> g(mu_);
  s.master = master_.load();
  s.ready = ready_.load();
  s.closed = closed_.load();
  s.n = n_;
  s.listen_addr = started_.load() ? addr_to_string(listen_addr_) : "";
  for (int i = 0; i < kNumSlots; i++) {
    s.edge[i] = edges_[i].st;
    s.edge[i].state = edges_[i].state.load();
  }
  s.adds = adds_;
  s.copies = copies_;
  s.redirects = listener_ ? listener_->redirects() : 0;
  s.rejoins = rejoins_;
  {
    std::lock_guard<std::mutex> g2(ev_mu_);
    s.events.assign(events_.begin(), events_.end());
  }
  s.edge_failures = edge_failures_;
  return s;
}

void CpuNode::close() {
  if (closed_.exchange(true)) return;
  {
    // under the supervisor's mutex: set between its check of the flag and its wait, the notification would find
    // nobody waiting and the supervisor would sleep for good
    std::lock_guard<std::mutex> g(sup_mu_);
    stop_.store(true);
  }
  sup_cv_.notify_all();
  if (supervisor_.joinable()) supervisor_.join();
  if (listener_) listener_->stop();
  for (int s = 0; s < kNumSlots; s++) {
    Edge& e = edges_[s];
    e.stop.store(true);
    {
      std::lock_guard<std::mutex> g(mu_);
      if (e.fd >= 0) ::shutdown(e.fd, SHUT_RDWR);
    }
  }
  work_cv_.notify_all();
  ready_cv_.notify_all();
  for (int s = 0; s < kNumSlots; s++) {
    Edge& e = edges_[s];
    if (e.tx.joinable()) e.tx.join();
    if (e.rx.joinable()) e.rx.join();
    if (e.fd >= 0) {
      ::close(e.fd);
      e.fd = -1;
    }
    e.state.store(0);
  }
}

}  // namespace st
