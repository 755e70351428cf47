// CPU replica node: the full shared-tensor behaviour with host memory and TCP edges.
//
// One node = one replica `values` plus up to three tree edges (up, left, right), like the
// reference's SharedTensor struct (src/sharedtensor.c:24-44).  Per connected edge there is a mirror
// array (see codec.hpp), one sender thread and one receiver thread (reference: synca 133-189 and
// sync_in 113-131).  Unlike the reference every access to values/mirrors happens under one node
// mutex, buffers are zero-initialised, sizes are 64-bit, a closed or failing peer only kills its
// edge, and close() tears everything down without ending the process (reference: __gc calls
// exit(-1) once any edge was ever connected, 421-430).
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "codec.hpp"
#include "tree.hpp"

namespace st {

struct NodeConfig {
  // wire format on TCP edges: 0 = tensor scale (what the reference speaks), else block size (32..4096)
  int tcp_block = 0;
  // block mode: bits per element of a frame, 1 (sign frames) or 8 (integer frames: one frame brings a fresh update
  // to under one percent; between nodes of this framework, where the link has eight times the bytes to spare)
  int tcp_bits = 1;
  int tcp_rule = 1;               // tensor mode scale: 0 = the reference's RMS rule, 1 = bisection (see codec.hpp)
  BlockGate gate;                 // block mode cut-offs
  float min_scale_abs = 0.0f;     // tensor mode: frames with a smaller scale become no-ops
  float min_scale_rel = 2.3841858e-07f;  // ... or smaller than this times max|values|   (2^-22)
  double max_frames_per_s = 0.0;  // per-edge rate cap, 0 = as fast as TCP takes them
  int idle_keepalive_ms = 0;      // send a scale-0 frame this often while idle (0 = never)
  int listen_backlog = 5;
  int ready_mode = 1;             // 0 = first frame (reference behaviour), 1 = scale fell by 2^-ready_bits or idle frame
  int ready_bits = 12;
  int ready_timeout_ms = 30000;
  bool rejoin = true;             // re-run the join walk when the up edge dies
  int rejoin_backoff_ms = 200;
};

struct EdgeStats {
  int state = 0;  // 0 free, 1 connected, 2 dead
  std::string peer;
  uint64_t frames_sent = 0, frames_recv = 0, noop_sent = 0, noop_recv = 0;
  uint64_t bytes_sent = 0, bytes_recv = 0;
  float last_scale_sent = 0, last_scale_recv = 0;
  double residual_rms = 0;
  uint64_t dropped_by_injection = 0;
};

// One membership event (joined, master, edge_lost, rejoined, adopted, ...), kept in a small ring for stats().
struct NodeEvent {
  uint64_t ms = 0;  // wall clock, milliseconds since the epoch
  std::string kind, detail;
};

struct NodeStats {
  std::vector<NodeEvent> events;  // oldest first, at most 64
  bool master = false, ready = false, closed = false;
  int64_t n = 0;
  std::string listen_addr;
  EdgeStats edge[kNumSlots];
  uint64_t adds = 0, copies = 0, redirects = 0, rejoins = 0, edge_failures = 0;
};

class CpuNode {
 public:
  CpuNode(int64_t n, const NodeConfig& cfg);
  ~CpuNode();
  CpuNode(const CpuNode&) = delete;

  // Joins (or founds) the tree at host:port.  `init` (n floats) seeds the replica if this node turns
  // out to be the master and is ignored otherwise (reference: src/sharedtensor.c:379-387).
  void start(const std::string& host, int port, const float* init);
  bool wait_ready(int timeout_ms);
  void add(const float* delta, int64_t n);          // values += delta             (334-344)
  void sub_add(const float* neu, const float* old, int64_t n);  // values += neu - old
  void copy_to(float* out, int64_t n);              // out = values                (435-446)
  void close();
  NodeStats stats();
  int64_t size() const { return n_; }
  bool is_master() const { return master_.load(); }

  // checkpoint support: values and the three mirrors (absent mirrors come back empty)
  void export_state(std::vector<float>* values, std::vector<float> mirrors[kNumSlots]);
  void import_values(const float* v, int64_t n);

  // Blocks until every connected edge has nothing left to send (its last frame was a no-op) and
  // nothing was received for `quiet_ms`; false on timeout.
  bool flush(int timeout_ms, int quiet_ms = 50);

  // Host-side fault injection for tests: drop the next `k` received frames on an edge after
  // reading them (the stream stays framed), or cut an edge's socket.
  void inject_drop_frames(int slot, int k);
  void inject_sever(int slot);

 private:
  struct Edge {
    int slot = 0;
    std::atomic<int> state{0};
    int fd = -1;
    sockaddr_in peer{};
    std::vector<float> mirror;
    std::thread tx, rx;
    std::atomic<bool> stop{false};
    std::atomic<int> drop_frames{0};
    std::atomic<bool> paused{false};  // no sending while the node re-fetches state through `up`
    bool sent_first = false;
    bool idle_announced = false;      // the no-op frame that ends a burst has gone out
    bool idle = false;                // last encode produced a no-op
    uint64_t dirty = 1;               // bumped whenever values change in a way this edge must forward
    EdgeStats st;
    float first_scale_recv = 0;
    uint64_t last_recv_ms = 0;
  };

  void attach_edge(int slot, int fd, const sockaddr_in& peer);
  void tx_loop(Edge* e);
  void rx_loop(Edge* e);
  void edge_failed(Edge* e, const char* why, IoStatus st);
  void supervisor_loop();
  void reap_edge(Edge* e);
  bool do_join(bool first, const float* init);
  size_t frame_bytes() const;

  const int64_t n_;
  NodeConfig cfg_;
  std::string host_;
  int port_ = 0;
  std::vector<float> values_;
  Edge edges_[kNumSlots];
  std::mutex mu_;                  // guards values_, mirrors, edge stats
  std::condition_variable work_cv_;  // new data to send
  std::unique_ptr<TreeListener> listener_;
  sockaddr_in listen_addr_{};
  std::mutex ev_mu_;
  std::deque<NodeEvent> events_;
  void log_event(const char* kind, const std::string& detail);
  std::vector<sockaddr_in> my_addrs_;  // every address this node listens on (supervisor/start thread only)
  std::atomic<bool> master_{false}, ready_{false}, closed_{false}, started_{false};
  std::condition_variable ready_cv_;
  // supervisor
  std::thread supervisor_;
  std::mutex sup_mu_;
  std::condition_variable sup_cv_;
  std::deque<int> dead_slots_;
  std::atomic<bool> stop_{false};
  uint64_t adds_ = 0, copies_ = 0, rejoins_ = 0, edge_failures_ = 0;
};

uint64_t now_ms();

}  // namespace st
