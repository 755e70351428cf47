// GPU replica: device-resident values and mirrors, ring bookkeeping, and the stream/thread that runs
// sync rounds.  This is the device-side counterpart of CpuNode (../core/node.hpp); it knows nothing
// about sockets or membership, which live in gpu_node.hpp.
//
// Stream discipline: mirrors are written by the round kernel only, on the replica's own comm stream.
// `values` has many writers (the round kernel adds what it received, addFromTensor adds from the caller's
// stream, TCP frames are added by their receiver threads) and every one of them adds with a reduction at
// the L2, so they commute and none waits for another: an update never queues behind a round in flight.
// (The reference adds from the user thread while its sender and receiver threads run, without any
// synchronisation, src/sharedtensor.c:334-344.)  Whoever changes the values marks the tiles as changed
// AFTER the change, on the same stream; the round kernel clears a tile's mark BEFORE it reads the tile,
// so a change it does not see is looked at in the next sweep.  copyToTensor reads `values` from the
// caller's stream and may overlap a round (per-element tearing is impossible, per-tensor tearing is
// allowed, as in the reference, src/sharedtensor.c:442-444).
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "round.h"
#include "vmm.hpp"

namespace st {

struct GpuConfig {
  int block = 32;            // scale block, power of two 32..4096
  int ring_slots = 4;
  int min_exp = -60;
  int rel_bits = 22;
  int comm_ctas = 0;         // 0 = one CTA per SM
  bool shareable = true;     // allocate edge blocks and values with the VMM API (needed across processes)
  int rounds_in_flight = 2;
  int idle_sleep_us = 1000;  // longest pause of the engine thread between rounds while nothing moves
  int round_interval_us = 0; // pause after every busy round (0 = run rounds back to back)
  int bits = 8;              // bits per element of a frame: 1 (sign frames), 2, 4 or 8 (integer frames)
  int sweeps = 0;            // passes over the tensor per launch of the engine thread (0 = one)
  int poll_deadline_us = 1000;  // upper bound of every wait inside the round kernel
  int shape = 1;             // make-up of the round kernel's CTAs, see launch_round
  bool yield_to_updates = true;  // a running round kernel gives up its SMs when addFromTensor has an update ready
  bool comm_high_priority = false;  // comm stream at the highest stream priority (switches yield_to_updates off)
  int chunk_tiles = 0;       // > 0: short-lived CTAs, a group takes this many consecutive tiles (0: one CTA per SM per launch)
  int window_tiles = 0;      // tiles a launch covers (0: 6144 for tensors above 8192 tiles, else the whole tensor)
};

constexpr size_t kGuardBytes = 256;  // canary before and after every mirror, edge block and the values

struct EdgeBlockLayout {
  size_t off_payload = 0, off_flags = 0, off_credit = 0, bytes = 0;
};

class GpuReplica {
 public:
  GpuReplica(int device, int64_t n, const GpuConfig& cfg);
  ~GpuReplica();
  GpuReplica(const GpuReplica&) = delete;

  int device() const { return device_; }
  int64_t size() const { return n_; }
  int64_t padded() const { return n_padded_; }
  int tiles() const { return n_tiles_; }
  float* values() const { return reinterpret_cast<float*>(static_cast<uint8_t*>(values_.ptr) + kGuardBytes); }
  const VmmBlock& values_block() const { return values_; }
  float* mirror(int link) const { return reinterpret_cast<float*>(static_cast<uint8_t*>(links_[link].mirror.ptr) + kGuardBytes); }
  EdgeBlockLayout edge_layout() const { return layout_; }
  void* comm_stream() const { return comm_; }

  // ---- topology ----
  int add_link();                      // new mirror (zero); returns link id, -1 if none is free
  void remove_link(int link);          // detaches the link's peers and frees the mirror
  int alloc_edge_block();              // zeroed local block a neighbour will store into
  void free_edge_block(int id);
  const VmmBlock& edge_block(int id) const { return blocks_[id].mem; }
  // Frames from the neighbour arrive in local block `local_block`; frames to it go to its block, mapped
  // at `remote_base` in this process (same layout).  Returns a peer id.
  int attach_peer(int link, int local_block, void* remote_base);
  void detach_peer(int peer);
  // The neighbour behind `peer` is gone: the frames it never acknowledged (they are still in its ring, which stays
  // mapped) are taken off the link's mirror again.  Returns how many tile-frames that were.  Call before detach_peer.
  uint64_t unsend_unacknowledged(int peer);
  int n_links() const;
  int n_peers() const;

  // ---- data path ----
  void load_values(const float* src, void* user_stream);
  // Updates run on the caller's stream, concurrently with rounds (every add is a reduction at the L2).
  void add(const float* delta, void* user_stream);
  void sub_add(const float* neu, const float* old, void* user_stream);
  void add_scaled_bf16(const void* g_bf16, float alpha, void* user_stream);  // values += alpha * g
  // While the gate is held every update of the values from outside the rounds (add, sub_add, add_scaled_bf16,
  // load_values, tcp_decode) waits.  A node that re-joins holds it from the moment it works out what its lost parent
  // had not been told until that has been added back on top of the new parent's snapshot, so that an update made in
  // between is neither overwritten by the snapshot nor counted twice.
  void gate_lock();   // also waits until the updates issued so far have run on the device
  void gate_unlock() { gate_mu_.unlock(); }
  void add_gate_held(const float* delta);   // values += delta on the comm stream; the caller holds the gate
  void snapshot(float* out, void* user_stream);
  void snapshot_bf16(void* out, void* user_stream);
  void copy_mirror_from_values(int link);                 // mirror <- values (neighbour is given a snapshot)
  void push_snapshot(int link, float* remote_values);     // neighbour's values <- values, mirror <- values
  void round(bool do_rx = true, bool do_tx = true, int sweeps = 1);
  // Test hook: while set (>= 0), the round kernel's copy barrier of this tile expects more bytes than are copied,
  // so the bounded wait of the group that owns the tile runs out.
  void set_test_stall_tile(int tile);
  // Compares the canaries around the values, every mirror and every edge block; returns the number of damaged ones.
  int check_guards();
  // TCP links: a link with a mirror and no ring peers; its tensor-scale frames (the reference's wire format) are
  // made and applied on the device, host threads only move bytes.  `words` is host memory of ceil(n/32) words.
  float tcp_encode(int link, uint32_t* words, float min_scale_abs, float min_scale_rel);  // returns the frame's scale
  void tcp_decode(int link, const uint32_t* words, float scale);
  // A frame made by tcp_encode that could not be written to the socket: the mirror's step is taken back, so that
  // the frame's content stays in the residual and goes out over the next connection.
  void tcp_unsend(int link, const uint32_t* words, float scale);
  void sync();

  // ---- engine thread: free-running rounds ----
  void start_engine();
  void stop_engine();
  bool engine_running() const { return engine_on_.load(); }
  // Ends the engine thread's idle pause at once.  `from_neighbour` marks a doorbell that came over a socket; the
  // return value says whether the engine had been idle (the caller then passes the doorbell on).
  bool wake(bool from_neighbour = false);
  // Called (from the thread that made the update) when a local update finds the engine idle: the node rings its
  // neighbours so that their engines are polling by the time the first frames arrive.
  void set_doorbell(std::function<void()> fn);

  // ---- observation ----
  std::vector<uint64_t> status();      // StatusWord order, then the trace ring; synchronises the comm stream
  int bits() const { return cfg_.bits; }
  std::vector<uint32_t> debug_crumbs() const;   // debug builds of the round kernel: its progress marks, 8 words per CTA
  uint64_t launches() const { return launches_.load(); }
  uint64_t change_epoch() const { return epoch_.load(); }  // bumped whenever values may have changed
  std::string last_error() const;

 private:
  struct Link {
    bool used = false;
    VmmBlock mirror;
  };
  struct Block {
    bool used = false;
    VmmBlock mem;
  };
  struct Peer {
    bool used = false;
    int link = -1;
    int local_block = -1;
    uint8_t* remote = nullptr;
    uint32_t* rx_seq = nullptr;
    uint32_t* tx_seq = nullptr;
  };
  void rebuild_params();               // under mu_
  void publish_pending();              // under mu_
  void launch(bool do_rx, bool do_tx, int sweeps);  // under mu_
  int auto_sweeps() const;
  void grid_for_launch(int tiles, int* grid, int* chunk, int* tiles_per_group) const;
  int window_tiles() const;
  int n_windows() const;
  void fill_guards(const VmmBlock& b, size_t used_bytes);
  void ask_for_sms(void* user_stream, bool on);
  void check(int cuda_err, const char* what);
  void engine_loop();
  void order_after_user(void* user_stream);
  void order_user_after(void* user_stream);

  int device_;
  int64_t n_, n_padded_;
  int n_tiles_;
  GpuConfig cfg_;
  EdgeBlockLayout layout_;
  VmmBlock values_;
  std::vector<Link> links_;
  std::vector<Block> blocks_;
  std::vector<Peer> peers_;
  uint32_t* tile_state_ = nullptr;     // change mark per tile
  uint64_t* status_ = nullptr;         // DevStatus layout
  uint32_t* yield_flag_ = nullptr;     // non-zero while an update wants the SMs the round kernel holds
  uint32_t* dbg_host_ = nullptr;       // mapped host memory for the debug build's progress marks
  uint64_t* status_host_ = nullptr;    // pinned
  uint32_t* tcp_words_dev_ = nullptr;  // ceil(n/32) words, staging of TCP frames
  uint32_t* tcp_stat_dev_ = nullptr;   // 2 words
  uint32_t* tcp_pinned_ = nullptr;     // pinned host staging: 2 stat words + ceil(n/32) frame words
  RoundParams params_{};
  int map_link_[kMaxLinks] = {0, 0, 0};  // dense link index of each link id
  int round_no_ = 0;
  int last_parity_ = 0;                // which half of the per-cycle status words the last launch used
  int next_window_ = 0;                // the window of the tensor the next launch covers
  int cycle_no_ = 0;                   // passes over the whole tensor started so far
  int ctas_ = 148;
  int sms_ = 148;
  void* comm_ = nullptr;               // cudaStream_t
  void* ev_user_ = nullptr;            // cudaEvent_t: user stream -> comm
  void* ev_comm_ = nullptr;            // cudaEvent_t: comm -> user stream
  std::vector<void*> ev_round_;       // per launch in flight: its work count has been read back
  std::vector<void*> ev_kernel_;      // per launch in flight: the kernel has finished (comm stream)
  void* stat_ = nullptr;               // cudaStream_t: reads work counts back beside the comm stream, so that launches follow each other without a copy in between
  mutable std::mutex mu_;
  std::mutex gate_mu_;                 // taken before mu_ by every update from outside the rounds
  std::mutex engine_mu_;               // serialises start_engine / stop_engine
  std::thread engine_;
  std::atomic<bool> engine_on_{false}, engine_stop_{false};
  std::atomic<uint64_t> last_wake_ns_{0};  // when wake() was last called (steady clock)
  std::atomic<bool> idle_{false};      // the engine has seen several rounds without work and pauses between rounds
  std::mutex wake_mu_;
  std::condition_variable wake_cv_;
  bool wake_pending_ = false;          // under wake_mu_
  std::function<void()> doorbell_;     // under wake_mu_
  std::chrono::steady_clock::time_point last_ring_{};  // under wake_mu_
  void local_update();                 // wake + doorbell if the engine was idle
  void idle_pause(uint64_t us);
  std::atomic<uint64_t> launches_{0};
  std::atomic<uint64_t> epoch_{1};
  std::string error_;
};

}  // namespace st
