// Parameter blocks and launch entry points of the sync-round kernel (host-visible, no CUDA syntax).
//
// One replica on one GPU holds `values` and, per link, a mirror (see ../core/codec.hpp for the
// state model).  A *link* is a set of neighbours that share one mirror: a tree edge is a link with
// one inbound and one outbound ring; a mesh group is a single link whose outbound frames are pushed
// to every peer and whose inbound rings (one per peer) are not forwarded to the other peers.
//
// A *ring* carries frames in one direction.  Its payload slots and per-tile sequence flags live in the
// RECEIVER's memory (the sender writes them with peer stores over NVLink), its per-tile credit words
// live in the SENDER's memory (the receiver writes them).  Every poll is therefore a local load and
// only stores cross the link.  Each 4096-element tile of the tensor is an independent stream with its
// own sequence number, so no kernel ever waits for another GPU: a tile whose ring is full or whose
// frame has not arrived is simply handled in a later sweep.
//
// A frame carries, per tile, `bits` bits per element (1: the sign of the residual, the reference's
// format, src/sharedtensor.c:166-174; 2, 4, 8: the residual as a small integer times the block's
// power-of-two step) and one exponent byte per block of `1 << log2_block` elements.
//
// One launch of the round kernel makes up to `sweeps` passes over the tensor.  In a pass every group of
// the grid looks at its own tiles' flags and credits, and for each tile that has something to do
//   - stages values and mirrors with TMA bulk copies,
//   - decodes the frames that arrived, accumulates them into the values (a bulk reduce-add, so that
//     updates made by other streams at the same time are kept) and into the mirror of the link they
//     came from (reference hot loops src/sharedtensor.c:106-111, 124-127),
//   - quantises values - mirror for every link, steps the mirror and pushes the packed codes and
//     scales straight into the neighbours' ring slots (156-177),
//   - and, once the stores have landed, publishes sequence flags to the receivers and credits to the
//     senders.
#pragma once
#include <cstdint>

namespace st {

constexpr int kTile = 4096;         // elements per tile (= per independent stream)
constexpr int kMaxLinks = 3;        // mirrors per replica
constexpr int kMaxRings = 8;        // inbound rings, and outbound rings, per replica
constexpr int kRxMax = 3;           // frames taken per ring per tile per sweep
constexpr int kWordsPerTile = kTile / 32;

struct InRing {
  const uint8_t* payload;   // local: [slot][tile][payload_bytes]
  const uint32_t* flags;    // local: [slot][tile], written by the sender: seq + 1
  uint32_t* rx_seq;         // local: [tile], frames consumed so far
  uint32_t* credit_remote;  // sender's memory: [tile], = rx_seq after consumption
  int link;
};

struct OutRing {
  uint8_t* payload_remote;      // receiver's memory
  uint32_t* flags_remote;       // receiver's memory
  uint32_t* tx_seq;             // local: [tile], frames produced so far
  const uint32_t* credit;       // local: [tile], written by the receiver
  int link;
};

struct RoundParams {
  float* values;                 // padded to a multiple of kTile, padding is zero
  float* mirror[kMaxLinks];
  int64_t n;                     // valid elements
  int32_t n_tiles;
  int32_t n_links;
  int32_t n_in, n_out;
  InRing in[kMaxRings];
  OutRing out[kMaxRings];
  int32_t ring_slots;            // power of two, at most 64
  int32_t log2_block;            // 5..12
  int32_t scales_per_tile;       // kTile >> log2_block
  int32_t bits;                  // 1, 2, 4 or 8 bits per element
  int32_t payload_bytes;         // bits * 4 * kWordsPerTile + max(16, scales_per_tile)
  int32_t min_exp, rel_bits;     // gate, see BlockGate
  uint32_t* tile_state;          // [tile]: non-zero = the values of the tile may have changed since its last visit
  uint64_t* status;              // see DevStatus
  int32_t round;                 // number of this launch's first sweep (bookkeeping only)
  int32_t tile_begin, tile_count; // the window of the tensor this launch covers
  int32_t parity;                // which half of the per-cycle counters this launch uses (a cycle = one pass over all windows)
  int32_t zero_other;            // first launch of a cycle: clear the other half for the cycle after this one
  int32_t do_rx, do_tx;          // receiver-only / sender-only launches
  int32_t sweeps;                // passes over the tensor in this launch (>= 1)
  uint32_t wait_ns;              // upper bound of every wait on one of the kernel's own copies
  int32_t stall_tile;            // test hook: the copy barrier of this tile expects more bytes than are copied (-1: none)
  int32_t chunk;                 // > 0: a group owns this many consecutive tiles; 0: every (groups in the grid)-th tile
  const uint32_t* yield_flag;    // non-zero while an update is waiting for SMs: groups hand out no more tiles and leave
  uint32_t* dbg;                 // debug builds: progress marks in mapped host memory, 8 words per CTA (else null)
};

// Layout of the device status block (uint64 each).  Counters are cumulative; the per-cycle words exist twice, the
// launches of a cycle (one launch per window of the tensor) use the half given by RoundParams::parity and the first of
// them clears the other half for the cycle after it.
enum DevStatus : int {
  kDsSweeps = 0,
  kDsTilesProcessed,
  kDsFramesSent,       // tile-frames written to out-rings
  kDsFramesRecv,       // tile-frames decoded from in-rings
  kDsBlockedNoCredit,  // tile-links that had something to send but no ring space
  kDsErrors,           // bit mask, see kErr*
  kDsWaitTimeouts,
  kDsYields,           // groups that left early because an update was waiting
  kDsLaunch0 = 8,      // per-launch words of parity 0: work, pending tiles, residual maxima of links 0..2 (fp32 bits)
  kDsLaunch1 = 16,     // ... of parity 1
  kDsTrace = 24,       // ring of kTraceEntries records {globaltimer ns, round, tiles handled by group 0, frames sent so far}
  kTraceEntries = 64,
  kTraceWords = 4,
  kDsTotalWords = kDsTrace + kTraceEntries * kTraceWords
};
constexpr int kDlWork = 0, kDlPending = 1, kDlResMax = 2;  // offsets inside a per-launch half
constexpr uint64_t kErrBarrierTimeout = 1, kErrBadCtrl = 2;

// What GpuReplica::status() hands out: the counters in this order, then the trace ring.
enum StatusWord : int {
  kStRounds = 0,
  kStTilesProcessed,
  kStFramesSent,
  kStFramesRecv,
  kStBlockedNoCredit,
  kStErrors,
  kStLastWorkCount,   // tiles handled by the last launch
  kStResidualMax0,    // per link: bits of the largest |values - mirror| (fp32) the last launch saw
  kStResidualMax1,
  kStResidualMax2,
  kStPendingTiles,    // tiles still marked pending after the last launch
  kStWaitTimeouts,
  kStWords = 16,
  kStTotalWords = kStWords + kTraceEntries * kTraceWords
};

// Launchers.  `stream` is a cudaStream_t passed as void*.  Return a cudaError_t as int.
// `shape` picks the CTA's make-up: 0 = 3 groups x 2 staging slots, 1 = 2 groups x 3 slots (one CTA per SM either way).
// A group is 4 compute warps and one I/O warp; a CTA has one more warp that publishes flags and credits.
int launch_round(const RoundParams& p, int shape, int ctas, void* stream);
int round_shape_groups(int shape);
// Takes back the frames of one out-ring that the receiver never acknowledged: their steps are subtracted from the
// link's mirror and the ring's send counters fall back to the credits.  *taken_back (device) counts the tile-frames.
int launch_unsend(float* mirror, const uint8_t* payload_remote, uint32_t* tx_seq, const uint32_t* credit, int n_tiles, int ring_slots,
                  int payload_bytes, int log2_block, int bits, int64_t n, uint64_t* taken_back, void* stream);
int round_smem_bytes(int groups, int slots, int payload_bytes);

// Element-wise kernels (copyToTensor / addFromTensor / pushUpdate; src/sharedtensor.c:435-446, 334-344).
int launch_snapshot_f32(const float* values, float* out, int64_t n, void* stream);
int launch_snapshot_bf16(const float* values, void* out_bf16, int64_t n, void* stream);
// atomic != 0: every element is added with a reduction at the L2, so the add commutes with whatever else adds into
// `values` at the same time (the round kernel, other streams).
int launch_add(float* values, const float* delta, int64_t n, int atomic, void* stream);
int launch_sub_add(float* values, const float* neu, const float* old, int64_t n, int atomic, void* stream);
int launch_add_scaled_bf16(float* values, const void* g_bf16, float alpha, int64_t n, int atomic, void* stream);
// Marks every tile as changed.  Launched behind an update on the same stream, so the marks become visible after the data.
int launch_fill_state(uint32_t* tile_state, int n_tiles, uint32_t value, void* stream);
int launch_set_word(uint32_t* word, uint32_t value, void* stream);  // one thread; stands in for a stream memory write
// Per-segment sum of squares (table sync).  partials: scratch of table_scales_scratch_doubles(...) doubles.
int64_t table_scales_scratch_doubles(int n_seg, int64_t n_total);
int launch_table_scales(const float* x, const int64_t* seg_offsets_dev, int n_seg, int64_t n_total, double* partials,
                        double* out_sumsq, int8_t* out_exp, void* stream);
// sum((a[i*stride] - b[i])^2) over count samples, into out[0] (double); out[1] counts NaNs.  Zeroes nothing.
int launch_sample_sqerr(const float* a, int64_t stride, const float* b, int64_t count, double* out, void* stream);
// The same sampled error, compared on the device: the first launch that finds it at or below `threshold` writes the
// GPU's %globaltimer into *stamp.  scratch: 16 zeroed bytes, reused by every launch; last_err: the error it saw.
int launch_probe_converged(const float* a, int64_t stride, const float* b, int64_t count, double threshold, double* scratch,
                           uint64_t* stamp, double* last_err, void* stream);
int launch_stamp(uint64_t* out, void* stream);  // *out = %globaltimer
// Busy-waits `ns` nanoseconds on the device with one thread (models "compute between updates").
int launch_delay(uint64_t ns, void* stream);
// values -> dst (peer or local) and mirror <- values in one pass; used for snapshot-on-join.
int launch_snapshot_join(const float* values, float* dst_values, float* mirror, int64_t n_padded, void* stream);
// Tensor-scale frames for TCP edges, encoded/decoded on the device (wire format of the reference).
int launch_tensor_maxabs(const float* v, const float* k, int64_t n, uint32_t* out2, void* stream);  // bits of max|v-k|, max|v|
int launch_tensor_encode(const float* v, float* k, int64_t n, float scale, uint32_t* words, void* stream);
// v += step (with L2 reductions if atomic_v, for the values) and k += step (plain; k may be null)
int launch_tensor_decode(const uint32_t* words, float scale, int64_t n, float* v, float* k, int atomic_v, void* stream);

}  // namespace st
