#include "engine.hpp"

#include <cuda_runtime_api.h>
#include <sys/prctl.h>
#include <unistd.h>

#include <chrono>

#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace st {

namespace {
cudaStream_t S(void* p) { return static_cast<cudaStream_t>(p); }
cudaEvent_t E(void* p) { return static_cast<cudaEvent_t>(p); }
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};
}  // namespace

void GpuReplica::check(int e, const char* what) {
  if (e != int(cudaSuccess)) {
    std::string msg = std::string(what) + ": " + cudaGetErrorString(cudaError_t(e));
    error_ = msg;
    throw std::runtime_error("sharedtensor GPU engine: " + msg);
  }
}

GpuReplica::GpuReplica(int device, int64_t n, const GpuConfig& cfg) : device_(device), n_(n), cfg_(cfg) {
  if (n <= 0) throw std::invalid_argument("shared tensor needs at least one element");
  if (cfg.block < 32 || cfg.block > 4096 || (cfg.block & (cfg.block - 1)))
    throw std::invalid_argument("block must be a power of two in 32..4096");
  if (cfg.ring_slots < 2 || cfg.ring_slots > 64 || (cfg.ring_slots & (cfg.ring_slots - 1)))
    throw std::invalid_argument("ring_slots must be a power of two in 2..64");
  if (cfg.bits != 1 && cfg.bits != 2 && cfg.bits != 4 && cfg.bits != 8)
    throw std::invalid_argument("bits per element must be 1, 2, 4 or 8");
  DeviceGuard g(device_);
  n_tiles_ = int((n + kTile - 1) / kTile);
  n_padded_ = int64_t(n_tiles_) * kTile;
  int lb = 0;
  while ((1 << lb) < cfg.block) lb++;
  const int spt = kTile >> lb;
  const int pb = cfg.bits * 4 * kWordsPerTile + (spt < 16 ? 16 : spt);
  // an edge block: canary, ring payload slots, sequence flags, credit words, canary
  layout_.off_payload = kGuardBytes;
  layout_.off_flags = layout_.off_payload + align_up(size_t(cfg.ring_slots) * n_tiles_ * pb, 256);
  layout_.off_credit = layout_.off_flags + align_up(size_t(cfg.ring_slots) * n_tiles_ * 4, 256);
  layout_.bytes = layout_.off_credit + align_up(size_t(n_tiles_) * 4, 256) + kGuardBytes;

  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  cudaStream_t s;
  // The comm stream runs at the priority of ordinary streams unless asked otherwise.  A round kernel that has
  // given up its SMs for a waiting update is relaunched at once; at a higher priority those relaunches would be
  // scheduled ahead of the update for ever, so the two options exclude each other.
  if (cfg_.comm_high_priority) cfg_.yield_to_updates = false;
  check(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, cfg_.comm_high_priority ? hi : lo), "cudaStreamCreate");
  comm_ = s;

  std::string err;
  values_ = vmm_alloc(device_, size_t(n_padded_) * 4 + 2 * kGuardBytes, cfg.shareable, &err);
  if (!values_.ptr) throw std::runtime_error("sharedtensor GPU engine: cannot allocate values: " + err);
  fill_guards(values_, size_t(n_padded_) * 4 + 2 * kGuardBytes);
  links_.resize(kMaxLinks);
  blocks_.resize(kMaxRings);
  peers_.resize(kMaxRings);

  // Everything is zeroed on the comm stream, the stream that uses it (a plain cudaMemset would run on the legacy
  // default stream, which nothing here is ordered against).
  check(cudaMalloc(reinterpret_cast<void**>(&tile_state_), size_t(n_tiles_) * 4), "cudaMalloc tile_state");
  check(cudaMalloc(reinterpret_cast<void**>(&status_), kDsTotalWords * 8), "cudaMalloc status");
  check(cudaMallocHost(reinterpret_cast<void**>(&status_host_), (kDsTotalWords + 16) * 8), "cudaMallocHost status");
  check(cudaMalloc(reinterpret_cast<void**>(&yield_flag_), 4), "cudaMalloc yield flag");
  check(cudaMemsetAsync(yield_flag_, 0, 4, s), "memset");
  check(launch_fill_state(tile_state_, n_tiles_, 1u, comm_), "fill_state");
  check(cudaMemsetAsync(status_, 0, kDsTotalWords * 8, s), "memset");
  std::memset(status_host_, 0, (kDsTotalWords + 16) * 8);
  cudaEvent_t e1, e2;
  check(cudaEventCreateWithFlags(&e1, cudaEventDisableTiming), "cudaEventCreate");
  check(cudaEventCreateWithFlags(&e2, cudaEventDisableTiming), "cudaEventCreate");
  ev_user_ = e1;
  ev_comm_ = e2;
  for (int i = 0; i < (cfg.rounds_in_flight < 1 ? 1 : (cfg.rounds_in_flight > 4 ? 4 : cfg.rounds_in_flight)); i++) {
    cudaEvent_t e;
    check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    ev_round_.push_back(e);
    check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    ev_kernel_.push_back(e);
  }
  {
    cudaStream_t st;
    check(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "cudaStreamCreate");
    stat_ = st;
  }
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_);
  sms_ = sms;
  ctas_ = cfg.comm_ctas > 0 ? cfg.comm_ctas : sms;
  if (const char* e = ::getenv("SHAREDTENSOR_ROUND_SHAPE")) cfg_.shape = std::atoi(e);
  if (const char* e = ::getenv("SHAREDTENSOR_CHUNK_TILES")) cfg_.chunk_tiles = std::atoi(e);
  if (cfg_.shape < 0 || cfg_.shape > 1) throw std::invalid_argument("round kernel shape must be 0 or 1");

  params_.values = values();
  params_.n = n_;
  params_.n_tiles = n_tiles_;
  params_.ring_slots = cfg.ring_slots;
  params_.log2_block = lb;
  params_.scales_per_tile = spt;
  params_.bits = cfg.bits;
  params_.payload_bytes = pb;
  params_.min_exp = cfg.min_exp;
  params_.rel_bits = cfg.rel_bits;
  params_.tile_state = tile_state_;
  params_.status = status_;
  params_.sweeps = 1;
  params_.wait_ns = uint32_t(cfg.poll_deadline_us < 1 ? 1 : (cfg.poll_deadline_us > 2000000 ? 2000000 : cfg.poll_deadline_us)) * 1000u;
  params_.stall_tile = -1;
  params_.yield_flag = cfg_.yield_to_updates ? yield_flag_ : nullptr;
  params_.dbg = nullptr;
  if (::getenv("SHAREDTENSOR_DEBUG_CRUMBS")) {
    void* h = nullptr;
    if (cudaHostAlloc(&h, 4096 * 8 * 4, cudaHostAllocMapped) == cudaSuccess) {
      std::memset(h, 0, 4096 * 8 * 4);
      dbg_host_ = static_cast<uint32_t*>(h);
      void* d = nullptr;
      cudaHostGetDevicePointer(&d, h, 0);
      params_.dbg = static_cast<uint32_t*>(d);
    }
  }
  check(cudaDeviceSynchronize(), "init");
}

GpuReplica::~GpuReplica() {
  stop_engine();
  DeviceGuard g(device_);
  if (comm_) cudaStreamSynchronize(S(comm_));
  for (auto& p : peers_) {
    if (p.rx_seq) cudaFree(p.rx_seq);
    if (p.tx_seq) cudaFree(p.tx_seq);
  }
  for (auto& l : links_) vmm_free(&l.mirror);
  for (auto& b : blocks_) vmm_free(&b.mem);
  vmm_free(&values_);
  cudaFree(tile_state_);
  cudaFree(status_);
  cudaFree(yield_flag_);
  if (status_host_) cudaFreeHost(status_host_);
  if (tcp_words_dev_) cudaFree(tcp_words_dev_);
  if (tcp_stat_dev_) cudaFree(tcp_stat_dev_);
  if (tcp_pinned_) cudaFreeHost(tcp_pinned_);
  for (void* e : ev_round_) cudaEventDestroy(E(e));
  for (void* e : ev_kernel_) cudaEventDestroy(E(e));
  if (stat_) cudaStreamDestroy(S(stat_));
  if (ev_user_) cudaEventDestroy(E(ev_user_));
  if (ev_comm_) cudaEventDestroy(E(ev_comm_));
  if (comm_) cudaStreamDestroy(S(comm_));
}

// ---------------------------------------------------------------------------------------------
// topology
// ---------------------------------------------------------------------------------------------
int GpuReplica::add_link() {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  for (int i = 0; i < kMaxLinks; i++) {
    if (!links_[i].used) {
      std::string err;
      publish_pending();
      links_[i].mirror = vmm_alloc(device_, size_t(n_padded_) * 4 + 2 * kGuardBytes, false, &err);
      if (!links_[i].mirror.ptr) throw std::runtime_error("sharedtensor GPU engine: cannot allocate mirror: " + err);
      fill_guards(links_[i].mirror, size_t(n_padded_) * 4 + 2 * kGuardBytes);
      links_[i].used = true;
      rebuild_params();
      return i;
    }
  }
  return -1;
}

void GpuReplica::remove_link(int link) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (link < 0 || link >= kMaxLinks || !links_[link].used) return;
  publish_pending();
  for (auto& p : peers_) {
    if (p.used && p.link == link) {
      p.used = false;
      cudaFree(p.rx_seq);
      cudaFree(p.tx_seq);
      p.rx_seq = p.tx_seq = nullptr;
    }
  }
  vmm_free(&links_[link].mirror);
  links_[link].used = false;
  rebuild_params();
}

int GpuReplica::alloc_edge_block() {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  for (int i = 0; i < kMaxRings; i++) {
    if (!blocks_[i].used) {
      std::string err;
      blocks_[i].mem = vmm_alloc(device_, layout_.bytes, cfg_.shareable, &err);
      if (!blocks_[i].mem.ptr) throw std::runtime_error("sharedtensor GPU engine: cannot allocate edge block: " + err);
      fill_guards(blocks_[i].mem, layout_.bytes);
      blocks_[i].used = true;
      return i;
    }
  }
  return -1;
}

void GpuReplica::free_edge_block(int id) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (id < 0 || id >= kMaxRings || !blocks_[id].used) return;
  cudaStreamSynchronize(S(comm_));
  vmm_free(&blocks_[id].mem);
  blocks_[id].used = false;
}

int GpuReplica::attach_peer(int link, int local_block, void* remote_base) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (link < 0 || link >= kMaxLinks || !links_[link].used) throw std::invalid_argument("attach_peer: no such link");
  if (local_block < 0 || local_block >= kMaxRings || !blocks_[local_block].used)
    throw std::invalid_argument("attach_peer: no such edge block");
  for (int i = 0; i < kMaxRings; i++) {
    if (!peers_[i].used) {
      Peer& p = peers_[i];
      publish_pending();
      check(cudaMalloc(reinterpret_cast<void**>(&p.rx_seq), size_t(n_tiles_) * 4), "cudaMalloc rx_seq");
      check(cudaMalloc(reinterpret_cast<void**>(&p.tx_seq), size_t(n_tiles_) * 4), "cudaMalloc tx_seq");
      check(cudaMemsetAsync(p.rx_seq, 0, size_t(n_tiles_) * 4, S(comm_)), "memset");
      check(cudaMemsetAsync(p.tx_seq, 0, size_t(n_tiles_) * 4, S(comm_)), "memset");
      p.link = link;
      p.local_block = local_block;
      p.remote = static_cast<uint8_t*>(remote_base);
      p.used = true;
      // whatever the link still had to say must be looked at again
      launch_fill_state(tile_state_, n_tiles_, 1u, comm_);
      rebuild_params();
      return i;
    }
  }
  return -1;
}

uint64_t GpuReplica::unsend_unacknowledged(int peer) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (peer < 0 || peer >= kMaxRings || !peers_[peer].used) return 0;
  publish_pending();
  Peer& p = peers_[peer];
  uint8_t* local = static_cast<uint8_t*>(blocks_[p.local_block].mem.ptr);
  uint64_t* dev_count = nullptr;
  check(cudaMalloc(reinterpret_cast<void**>(&dev_count), 8), "cudaMalloc");
  check(cudaMemsetAsync(dev_count, 0, 8, S(comm_)), "memset");
  check(launch_unsend(mirror(p.link), p.remote + layout_.off_payload, p.tx_seq, reinterpret_cast<const uint32_t*>(local + layout_.off_credit),
                      n_tiles_, cfg_.ring_slots, params_.payload_bytes, params_.log2_block, cfg_.bits, n_, dev_count, comm_),
        "unsend kernel");
  check(launch_fill_state(tile_state_, n_tiles_, 1u, comm_), "fill_state");  // the link has something to hear again
  uint64_t host = 0;
  check(cudaMemcpyAsync(status_host_ + kDsTotalWords + 8, dev_count, 8, cudaMemcpyDeviceToHost, S(comm_)), "cudaMemcpyAsync");
  check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
  host = status_host_[kDsTotalWords + 8];
  cudaFree(dev_count);
  launches_ += 1;
  return host;
}

void GpuReplica::detach_peer(int peer) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (peer < 0 || peer >= kMaxRings || !peers_[peer].used) return;
  publish_pending();
  Peer& p = peers_[peer];
  p.used = false;
  cudaFree(p.rx_seq);
  cudaFree(p.tx_seq);
  p.rx_seq = p.tx_seq = nullptr;
  rebuild_params();
}

int GpuReplica::n_links() const {
  std::lock_guard<std::mutex> lk(mu_);
  int c = 0;
  for (auto& l : links_) c += l.used;
  return c;
}
int GpuReplica::n_peers() const {
  std::lock_guard<std::mutex> lk(mu_);
  int c = 0;
  for (auto& p : peers_) c += p.used;
  return c;
}

void GpuReplica::publish_pending() {
  // Ring numbering is about to change.  Every round ends with its publish kernel, so once the
  // stream has drained nothing refers to the old numbering any more.
  cudaStreamSynchronize(S(comm_));
}

void GpuReplica::rebuild_params() {
  int dense = 0;
  for (int i = 0; i < kMaxLinks; i++) {
    map_link_[i] = -1;
    params_.mirror[i] = nullptr;
  }
  // only links that have at least one peer take part in rounds
  for (int i = 0; i < kMaxLinks; i++) {
    if (!links_[i].used) continue;
    bool has_peer = false;
    for (auto& p : peers_) has_peer |= p.used && p.link == i;
    if (!has_peer) continue;
    map_link_[i] = dense;
    params_.mirror[dense] = mirror(i);
    dense++;
  }
  params_.n_links = dense;
  int r = 0;
  for (auto& p : peers_) {
    if (!p.used) continue;
    uint8_t* local = static_cast<uint8_t*>(blocks_[p.local_block].mem.ptr);
    InRing& in = params_.in[r];
    in.payload = local + layout_.off_payload;
    in.flags = reinterpret_cast<const uint32_t*>(local + layout_.off_flags);
    in.rx_seq = p.rx_seq;
    in.credit_remote = reinterpret_cast<uint32_t*>(p.remote + layout_.off_credit);
    in.link = map_link_[p.link];
    OutRing& out = params_.out[r];
    out.payload_remote = p.remote + layout_.off_payload;
    out.flags_remote = reinterpret_cast<uint32_t*>(p.remote + layout_.off_flags);
    out.tx_seq = p.tx_seq;
    out.credit = reinterpret_cast<const uint32_t*>(local + layout_.off_credit);
    out.link = map_link_[p.link];
    r++;
  }
  params_.n_in = r;
  params_.n_out = r;
}

// ---------------------------------------------------------------------------------------------
// data path
// ---------------------------------------------------------------------------------------------
void GpuReplica::order_after_user(void* user_stream) {
  if (user_stream == comm_) return;
  check(cudaEventRecord(E(ev_user_), S(user_stream)), "cudaEventRecord");
  check(cudaStreamWaitEvent(S(comm_), E(ev_user_), 0), "cudaStreamWaitEvent");
}
void GpuReplica::order_user_after(void* user_stream) {
  if (user_stream == comm_) return;
  check(cudaEventRecord(E(ev_comm_), S(comm_)), "cudaEventRecord");
  check(cudaStreamWaitEvent(S(user_stream), E(ev_comm_), 0), "cudaStreamWaitEvent");
}

void GpuReplica::gate_lock() {
  gate_mu_.lock();
  // updates already issued on user streams have to be in the values before the holder looks at them
  DeviceGuard g(device_);
  cudaDeviceSynchronize();
}

// canaries at both ends of the used part of a block (the mapped size may be larger: it is rounded to the granularity)
void GpuReplica::fill_guards(const VmmBlock& b, size_t used_bytes) {
  uint8_t* base = static_cast<uint8_t*>(b.ptr);
  cudaMemsetAsync(base, 0xA5, kGuardBytes, S(comm_));
  cudaMemsetAsync(base + used_bytes - kGuardBytes, 0xA5, kGuardBytes, S(comm_));
}

int GpuReplica::check_guards() {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
  std::vector<uint8_t> host(kGuardBytes);
  int bad = 0;
  auto look = [&](const uint8_t* p) {
    if (cudaMemcpy(host.data(), p, kGuardBytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
      cudaGetLastError();
      bad++;
      return;
    }
    for (size_t i = 0; i < kGuardBytes; i++)
      if (host[i] != 0xA5) {
        bad++;
        return;
      }
  };
  const size_t arr = size_t(n_padded_) * 4;
  look(static_cast<const uint8_t*>(values_.ptr));
  look(static_cast<const uint8_t*>(values_.ptr) + kGuardBytes + arr);
  for (auto& l : links_)
    if (l.used) {
      look(static_cast<const uint8_t*>(l.mirror.ptr));
      look(static_cast<const uint8_t*>(l.mirror.ptr) + kGuardBytes + arr);
    }
  for (auto& b : blocks_)
    if (b.used) {
      look(static_cast<const uint8_t*>(b.mem.ptr));
      look(static_cast<const uint8_t*>(b.mem.ptr) + layout_.bytes - kGuardBytes);
    }
  return bad;
}

void GpuReplica::set_test_stall_tile(int tile) {
  std::lock_guard<std::mutex> lk(mu_);
  params_.stall_tile = tile;
}

void GpuReplica::load_values(const float* src, void* user_stream) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> gate(gate_mu_);
  {
    std::lock_guard<std::mutex> lk(mu_);
    order_after_user(user_stream);
    check(cudaMemcpyAsync(values(), src, size_t(n_) * 4, cudaMemcpyDeviceToDevice, S(comm_)), "cudaMemcpyAsync");
    check(launch_fill_state(tile_state_, n_tiles_, 1u, comm_), "fill_state");
    launches_ += 1;
    epoch_++;
    order_user_after(user_stream);
  }
  local_update();
}

// Around an update, in the order of the caller's stream: a word that asks the round kernel to give up its SMs (it
// holds all of them, for as long as a pass over the tensor takes), then the update, then the change marks, then the
// word is cleared.  The update itself never waits for a round; it only wants somewhere to run.
void GpuReplica::ask_for_sms(void* user_stream, bool on) {
  if (!cfg_.yield_to_updates) return;
  if (!stream_write_u32(user_stream, yield_flag_, on ? 1u : 0u)) check(launch_set_word(yield_flag_, on ? 1u : 0u, user_stream), "set_word");
}

void GpuReplica::add(const float* delta, void* user_stream) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> gate(gate_mu_);
  ask_for_sms(user_stream, true);
  check(launch_add(values(), delta, n_, 1, user_stream), "add kernel");
  check(launch_fill_state(tile_state_, n_tiles_, 1u, user_stream), "fill_state");  // marks after the data, in stream order
  ask_for_sms(user_stream, false);
  epoch_++;
  launches_ += 2;
  local_update();
}

void GpuReplica::sub_add(const float* neu, const float* old, void* user_stream) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> gate(gate_mu_);
  ask_for_sms(user_stream, true);
  check(launch_sub_add(values(), neu, old, n_, 1, user_stream), "sub_add kernel");
  check(launch_fill_state(tile_state_, n_tiles_, 1u, user_stream), "fill_state");
  ask_for_sms(user_stream, false);
  epoch_++;
  launches_ += 2;
  local_update();
}

void GpuReplica::add_scaled_bf16(const void* g, float alpha, void* user_stream) {
  DeviceGuard gd(device_);
  std::lock_guard<std::mutex> gate(gate_mu_);
  ask_for_sms(user_stream, true);
  check(launch_add_scaled_bf16(values(), g, alpha, n_, 1, user_stream), "add_scaled_bf16 kernel");
  check(launch_fill_state(tile_state_, n_tiles_, 1u, user_stream), "fill_state");
  ask_for_sms(user_stream, false);
  epoch_++;
  launches_ += 2;
  local_update();
}

void GpuReplica::add_gate_held(const float* delta) {
  DeviceGuard g(device_);
  check(launch_add(values(), delta, n_, 1, comm_), "add kernel");
  check(launch_fill_state(tile_state_, n_tiles_, 1u, comm_), "fill_state");
  epoch_++;
  launches_ += 2;
}

// A snapshot sits on the training loop's critical path like an update does: it asks for the SMs too.
void GpuReplica::snapshot(float* out, void* user_stream) {
  DeviceGuard g(device_);
  ask_for_sms(user_stream, true);
  check(launch_snapshot_f32(values(), out, n_, user_stream), "snapshot kernel");
  ask_for_sms(user_stream, false);
  launches_ += 1;
}

void GpuReplica::snapshot_bf16(void* out, void* user_stream) {
  DeviceGuard g(device_);
  ask_for_sms(user_stream, true);
  check(launch_snapshot_bf16(values(), out, n_, user_stream), "snapshot kernel");
  ask_for_sms(user_stream, false);
  launches_ += 1;
}

void GpuReplica::copy_mirror_from_values(int link) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (link < 0 || link >= kMaxLinks || !links_[link].used) throw std::invalid_argument("no such link");
  check(cudaMemcpyAsync(mirror(link), values(), size_t(n_padded_) * 4, cudaMemcpyDeviceToDevice, S(comm_)), "cudaMemcpyAsync");
}

void GpuReplica::push_snapshot(int link, float* remote_values) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (link < 0 || link >= kMaxLinks || !links_[link].used) throw std::invalid_argument("no such link");
  check(launch_snapshot_join(values(), remote_values, mirror(link), n_padded_, comm_), "snapshot_join kernel");
  launches_ += 1;
  check(cudaStreamSynchronize(S(comm_)), "snapshot_join");
}

// A long pass would hold every SM for its whole duration; the tensor is therefore covered in windows, one launch
// each, so that kernels of other streams get their turn between two launches.
int GpuReplica::window_tiles() const {
  if (cfg_.window_tiles > 0) return cfg_.window_tiles < n_tiles_ ? cfg_.window_tiles : n_tiles_;
  return n_tiles_ > 8192 ? 6144 : n_tiles_;   // 25 M elements, about 0.15 ms of a one-link pass
}
int GpuReplica::n_windows() const {
  const int w = window_tiles();
  return (n_tiles_ + w - 1) / w;
}

// How a launch covers its window: the grid, and how many consecutive tiles a group owns (0: every n-th tile).
void GpuReplica::grid_for_launch(int tiles, int* grid, int* chunk, int* tiles_per_group) const {
  const int groups_per_cta = round_shape_groups(cfg_.shape);
  if (cfg_.chunk_tiles > 0) {
    // many short-lived CTAs: a group takes a run of `chunk_tiles` consecutive tiles and leaves
    const int t = cfg_.chunk_tiles;
    *chunk = t;
    *grid = (tiles + t * groups_per_cta - 1) / (t * groups_per_cta);
    *tiles_per_group = t;
  } else {
    // one CTA per SM for the whole launch, a group walks through every n-th tile of the window
    const int needed = (tiles + groups_per_cta - 1) / groups_per_cta;
    const int g = ctas_ < needed ? ctas_ : needed;
    *chunk = 0;
    *grid = g < 1 ? 1 : g;
    *tiles_per_group = (tiles + *grid * groups_per_cta - 1) / (*grid * groups_per_cta);
  }
}

int GpuReplica::auto_sweeps() const {
  if (cfg_.sweeps > 0) return cfg_.sweeps > 64 ? 64 : cfg_.sweeps;
  // One pass per launch.  The kernel can make several (a launch then sends the second and third frame of an update
  // right behind the first, and an idle launch keeps looking for a while), which saves launches; measured on 2 GPUs
  // one pass per launch delivered a single update sooner at every size from 1 Ki to 64 Mi elements (16 Mi: 0.17 ms
  // against 0.23 ms with two passes and 0.30 ms with four), because the first frames of all tiles go out, and the
  // launch ends, before anything else is done.
  return 1;
}

// One launch: window `next_window_` of the current cycle.
void GpuReplica::launch(bool do_rx, bool do_tx, int sweeps) {
  const int wt = window_tiles(), nw = n_windows();
  const int w = next_window_;
  params_.tile_begin = w * wt;
  params_.tile_count = (w == nw - 1) ? n_tiles_ - w * wt : wt;
  params_.round = round_no_++;
  params_.parity = cycle_no_ & 1;
  params_.zero_other = w == 0 ? 1 : 0;
  params_.do_rx = do_rx ? 1 : 0;
  params_.do_tx = do_tx ? 1 : 0;
  params_.sweeps = sweeps < 1 ? 1 : sweeps;
  int grid, chunk, per_group;
  grid_for_launch(params_.tile_count, &grid, &chunk, &per_group);
  params_.chunk = chunk;
  check(launch_round(params_, cfg_.shape, grid, comm_), "round kernel");
  last_parity_ = params_.parity;
  next_window_ = (w + 1) % nw;
  if (next_window_ == 0) cycle_no_++;
  launches_ += 1;
  epoch_++;
}

void GpuReplica::round(bool do_rx, bool do_tx, int sweeps) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (params_.n_in == 0 && params_.n_out == 0) return;
  // one pass over the whole tensor: the rest of the cycle in progress (if the engine thread left one), or a full cycle
  do {
    launch(do_rx, do_tx, sweeps);
  } while (next_window_ != 0);
}

float GpuReplica::tcp_encode(int link, uint32_t* words, float min_scale_abs, float min_scale_rel) {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (link < 0 || link >= kMaxLinks || !links_[link].used) throw std::invalid_argument("no such link");
  const size_t n_words = size_t((n_ + 31) / 32);
  if (!tcp_words_dev_) {
    check(cudaMalloc(reinterpret_cast<void**>(&tcp_words_dev_), n_words * 4), "cudaMalloc tcp words");
    check(cudaMalloc(reinterpret_cast<void**>(&tcp_stat_dev_), 8), "cudaMalloc tcp stat");
    check(cudaMallocHost(reinterpret_cast<void**>(&tcp_pinned_), 8 + n_words * 4), "cudaMallocHost tcp staging");
  }
  float* k = mirror(link);
  check(cudaMemsetAsync(tcp_stat_dev_, 0, 8, S(comm_)), "memset");
  check(launch_tensor_maxabs(values(), k, n_, tcp_stat_dev_, comm_), "tensor_maxabs kernel");
  check(cudaMemcpyAsync(tcp_pinned_, tcp_stat_dev_, 8, cudaMemcpyDeviceToHost, S(comm_)), "cudaMemcpyAsync");
  check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
  float xmax, vmax;
  std::memcpy(&xmax, tcp_pinned_, 4);
  std::memcpy(&vmax, tcp_pinned_ + 1, 4);
  // bisection rule of the host codec: power-of-two floor of two thirds of the largest residual
  float scaled = xmax * 0.6666667f, scale = 0.f;
  uint32_t sb;
  std::memcpy(&sb, &scaled, 4);
  if ((sb >> 23) != 0 && (sb >> 23) != 0xff) {
    sb &= 0x7f800000u;
    std::memcpy(&scale, &sb, 4);
  }
  float min_scale = min_scale_abs;
  if (vmax * min_scale_rel > min_scale) min_scale = vmax * min_scale_rel;
  if (scale < min_scale) scale = 0.f;
  check(launch_tensor_encode(values(), k, n_, scale, tcp_words_dev_, comm_), "tensor_encode kernel");
  check(cudaMemcpyAsync(tcp_pinned_ + 2, tcp_words_dev_, n_words * 4, cudaMemcpyDeviceToHost, S(comm_)), "cudaMemcpyAsync");
  check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
  std::memcpy(words, tcp_pinned_ + 2, n_words * 4);
  launches_ += 2;
  return scale;
}

void GpuReplica::tcp_decode(int link, const uint32_t* words, float scale) {
  if (scale == 0.f) return;
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> gate(gate_mu_);
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (link < 0 || link >= kMaxLinks || !links_[link].used) throw std::invalid_argument("no such link");
    const size_t n_words = size_t((n_ + 31) / 32);
    if (!tcp_words_dev_) {
      check(cudaMalloc(reinterpret_cast<void**>(&tcp_words_dev_), n_words * 4), "cudaMalloc tcp words");
      check(cudaMalloc(reinterpret_cast<void**>(&tcp_stat_dev_), 8), "cudaMalloc tcp stat");
      check(cudaMallocHost(reinterpret_cast<void**>(&tcp_pinned_), 8 + n_words * 4), "cudaMallocHost tcp staging");
    }
    std::memcpy(tcp_pinned_ + 2, words, n_words * 4);
    check(cudaMemcpyAsync(tcp_words_dev_, tcp_pinned_ + 2, n_words * 4, cudaMemcpyHostToDevice, S(comm_)), "cudaMemcpyAsync");
    check(launch_tensor_decode(tcp_words_dev_, scale, n_, values(), mirror(link), 1, comm_), "tensor_decode kernel");
    check(launch_fill_state(tile_state_, n_tiles_, 1u, comm_), "fill_state");
    check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
    launches_ += 2;
    epoch_++;
  }
  local_update();  // the frame has to travel on over the other links
}

void GpuReplica::tcp_unsend(int link, const uint32_t* words, float scale) {
  if (scale == 0.f) return;
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  if (link < 0 || link >= kMaxLinks || !links_[link].used || !tcp_words_dev_) return;
  const size_t n_words = size_t((n_ + 31) / 32);
  std::memcpy(tcp_pinned_ + 2, words, n_words * 4);
  check(cudaMemcpyAsync(tcp_words_dev_, tcp_pinned_ + 2, n_words * 4, cudaMemcpyHostToDevice, S(comm_)), "cudaMemcpyAsync");
  // the mirror steps back by exactly what tcp_encode stepped it forward: the frame counts as never made
  check(launch_tensor_decode(tcp_words_dev_, -scale, n_, mirror(link), nullptr, 0, comm_), "tensor_decode kernel");
  check(launch_fill_state(tile_state_, n_tiles_, 1u, comm_), "fill_state");
  check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
  launches_ += 2;
}

void GpuReplica::sync() {
  DeviceGuard g(device_);
  check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
}

std::vector<uint64_t> GpuReplica::status() {
  DeviceGuard g(device_);
  std::lock_guard<std::mutex> lk(mu_);
  std::vector<uint64_t> dev(kDsTotalWords);
  check(cudaMemcpyAsync(status_host_, status_, kDsTotalWords * 8, cudaMemcpyDeviceToHost, S(comm_)), "cudaMemcpyAsync");
  check(cudaStreamSynchronize(S(comm_)), "cudaStreamSynchronize");
  std::memcpy(dev.data(), status_host_, kDsTotalWords * 8);
  // the counters of the last cycle that is complete (a cycle in progress has only seen some windows)
  const int par = next_window_ == 0 ? last_parity_ : (last_parity_ ^ 1);
  const uint64_t* lw = dev.data() + (par ? kDsLaunch1 : kDsLaunch0);
  std::vector<uint64_t> out(kStTotalWords, 0);
  out[kStRounds] = dev[kDsSweeps];
  out[kStTilesProcessed] = dev[kDsTilesProcessed];
  out[kStFramesSent] = dev[kDsFramesSent];
  out[kStFramesRecv] = dev[kDsFramesRecv];
  out[kStBlockedNoCredit] = dev[kDsBlockedNoCredit];
  out[kStErrors] = dev[kDsErrors];
  out[kStLastWorkCount] = lw[kDlWork];
  out[kStResidualMax0] = lw[kDlResMax + 0];
  out[kStResidualMax1] = lw[kDlResMax + 1];
  out[kStResidualMax2] = lw[kDlResMax + 2];
  out[kStPendingTiles] = lw[kDlPending];
  out[kStWaitTimeouts] = dev[kDsWaitTimeouts];
  std::memcpy(out.data() + kStWords, dev.data() + kDsTrace, size_t(kTraceEntries) * kTraceWords * 8);
  return out;
}

std::vector<uint32_t> GpuReplica::debug_crumbs() const {
  std::vector<uint32_t> out;
  if (dbg_host_) out.assign(dbg_host_, dbg_host_ + 2048);
  return out;
}

std::string GpuReplica::last_error() const {
  std::lock_guard<std::mutex> lk(mu_);
  return error_;
}

// ---------------------------------------------------------------------------------------------
// engine thread
// ---------------------------------------------------------------------------------------------
void GpuReplica::start_engine() {
  std::lock_guard<std::mutex> g(engine_mu_);
  if (engine_on_.load()) return;
  engine_stop_.store(false);
  engine_ = std::thread([this] { engine_loop(); });
  engine_on_.store(true);
}

void GpuReplica::stop_engine() {
  std::lock_guard<std::mutex> g(engine_mu_);
  if (!engine_on_.load()) return;
  engine_stop_.store(true);
  if (engine_.joinable()) engine_.join();
  engine_on_.store(false);
}

static uint64_t steady_ns() {
  return uint64_t(std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}

bool GpuReplica::wake(bool from_neighbour) {
  (void)from_neighbour;
  last_wake_ns_.store(steady_ns());
  const bool was_idle = idle_.exchange(false);
  {
    std::lock_guard<std::mutex> g(wake_mu_);
    wake_pending_ = true;
  }
  wake_cv_.notify_all();
  return was_idle;
}

void GpuReplica::set_doorbell(std::function<void()> fn) {
  std::lock_guard<std::mutex> g(wake_mu_);
  doorbell_ = std::move(fn);
}

void GpuReplica::local_update() {
  const bool was_idle = wake(false);
  // Ring the neighbours when this engine had been pausing (theirs then are, too) or when there is no engine thread
  // here at all (rounds driven by the caller): at most one doorbell per 200 us.
  if (!was_idle && engine_on_.load()) return;
  const auto now = std::chrono::steady_clock::now();
  std::function<void()> fn;
  {
    std::lock_guard<std::mutex> g(wake_mu_);
    if (now - last_ring_ < std::chrono::microseconds(200)) return;
    last_ring_ = now;
    fn = doorbell_;
  }
  if (fn) fn();
}

void GpuReplica::idle_pause(uint64_t us) {
  std::unique_lock<std::mutex> lk(wake_mu_);
  if (!wake_pending_) wake_cv_.wait_for(lk, std::chrono::microseconds(us), [this] { return wake_pending_ || engine_stop_.load(); });
  wake_pending_ = false;
}

void GpuReplica::engine_loop() {
  cudaSetDevice(device_);
  ::prctl(PR_SET_TIMERSLACK, 1000UL, 0, 0, 0);  // 1 us instead of the default 50 us: the idle pauses start at 10 us
  const size_t depth = ev_round_.size();
  // One pinned word per launch in flight: tiles handled so far, read once that launch has finished.  The read runs on
  // a stream of its own behind an event, so that the comm stream goes from one launch straight to the next; a later
  // launch may already have added to the count by then, which only moves work from one difference to the next.
  uint64_t* work_host = status_host_ + kDsTotalWords;  // behind the part status() uses
  uint64_t work_seen = 0;
  uint64_t r = 0;
  uint64_t idle_rounds = 0;
  uint64_t quiet_launches = 0;   // launches in a row that found nothing to do
  while (!engine_stop_.load()) {
    bool launched = false;
    int windows = 1;
    try {
      std::lock_guard<std::mutex> lk(mu_);
      if (params_.n_in + params_.n_out > 0) {
        // One launch makes several passes over a small tensor and returns; nothing on the device waits for this
        // thread, which only starts the next launch and reads how much the last one found to do.
        windows = n_windows();
        launch(true, true, auto_sweeps());
        cudaEventRecord(E(ev_kernel_[r % depth]), S(comm_));
        cudaStreamWaitEvent(S(stat_), E(ev_kernel_[r % depth]), 0);
        cudaMemcpyAsync(work_host + (r % depth), status_ + kDsTilesProcessed, 8, cudaMemcpyDeviceToHost, S(stat_));
        cudaEventRecord(E(ev_round_[r % depth]), S(stat_));
        launched = true;
      }
    } catch (const std::exception&) {
      break;  // error_ holds the reason; the API surfaces it on the next call
    }
    if (!launched) {
      ::usleep(1000);
      continue;
    }
    r++;
    uint64_t work = 1;
    if (r >= depth) {
      cudaEventSynchronize(E(ev_round_[(r - depth) % depth]));
      const uint64_t now = work_host[(r - depth) % depth];
      work = now > work_seen ? now - work_seen : 0;
      work_seen = now > work_seen ? now : work_seen;
    }
    if (work != 0) epoch_++;
    quiet_launches = work == 0 ? quiet_launches + 1 : 0;
    if (work == 0 && quiet_launches < uint64_t(windows)) continue;  // the other windows of the tensor have not been looked at yet
    if (work == 0) {
      // nothing moved: back off from 10 us up to idle_sleep_us, so that a fresh update is picked up quickly after a
      // burst and an idle replica costs next to nothing
      idle_rounds++;
      if (idle_rounds > 2 && cfg_.idle_sleep_us > 0) {
        uint64_t shift = idle_rounds - 3 > 10 ? 10 : idle_rounds - 3;
        uint64_t us = 10ull << shift;
        if (us > uint64_t(cfg_.idle_sleep_us)) us = uint64_t(cfg_.idle_sleep_us);
        // A local update or a neighbour's doorbell announces work that is still on its way (the update's kernel has
        // to run first, the neighbour's frames have to cross the link): keep looking often for a few milliseconds.
        if (steady_ns() - last_wake_ns_.load() < 5000000ull && us > 20) us = 20;
        idle_.store(true);
        idle_pause(us);  // a local update or a neighbour's doorbell ends it early
        if (!idle_.load()) idle_rounds = 0;
        quiet_launches = 0;  // after a pause the whole tensor is looked at again before the next one
      }
    } else {
      idle_.store(false);
      idle_rounds = 0;
      // pacing: a training job can cap how often rounds run, leaving the GPU to its own kernels in between
      if (cfg_.round_interval_us > 0) ::usleep(useconds_t(cfg_.round_interval_us));
    }
  }
  cudaStreamSynchronize(S(comm_));
  cudaStreamSynchronize(S(stat_));
}

}  // namespace st
