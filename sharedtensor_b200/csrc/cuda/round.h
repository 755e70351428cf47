// Parameter blocks and launch entry points of the sync-round kernels (host-visible, no CUDA syntax).
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
// frame has not arrived is simply handled in a later round.
//
// A round is three launches on one stream:
//   round_begin   – per tile: look at flags/credits once and build the work list;
//   round_main    – per listed tile: stage values, mirrors and arrived frames with TMA bulk copies,
//                   decode + accumulate + forward + re-quantise + push packed words and scales to the
//                   neighbours' rings (reference hot loops src/sharedtensor.c:106-111, 124-127, 156-177);
//   round_publish – per tile: sequence flags for the frames written (to receivers), credits for the
//                   frames consumed (to senders).
#pragma once
#include <cstdint>

namespace st {

constexpr int kTile = 4096;         // elements per tile (= per independent stream)
constexpr int kMaxLinks = 3;        // mirrors per replica
constexpr int kMaxRings = 8;        // inbound rings, and outbound rings, per replica
constexpr int kRxMax = 3;           // frames taken per ring per tile per round
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
  int32_t ring_slots;
  int32_t log2_block;            // 5..12
  int32_t scales_per_tile;       // kTile >> log2_block
  int32_t payload_bytes;         // 4*kWordsPerTile + max(16, scales_per_tile)
  int32_t min_exp, rel_bits;     // gate, see BlockGate
  // per-round scratch (all local)
  uint8_t* ctrl;                 // [tile][16]: bytes 0..7 in-rings (avail<<6 | first slot), 8..15 out-rings (free slots, up to 3, <<6 | slot)
  uint8_t* sent;                 // [tile][8]: number of frames round_main wrote for out-ring r
  uint8_t* tile_state;           // [tile]: 1 = something may be left to send
  int32_t* worklist;             // [n_tiles]
  int32_t* work_count;           // [2], double buffered by round parity
  uint64_t* status;              // see StatusWord
  int32_t round;
  int32_t do_rx, do_tx;          // receiver-only / sender-only rounds
  int32_t frames_per_round;      // 1..3 successive 1-bit frames per link, tile and round
};

// indices into the status block (uint64 each)
enum StatusWord : int {
  kStRounds = 0,
  kStTilesProcessed,
  kStFramesSent,      // tile-frames written to out-rings
  kStFramesRecv,      // tile-frames decoded from in-rings
  kStBlockedNoCredit, // tile-links that had something to send but no ring space
  kStErrors,          // bit mask, see kErr*
  kStLastWorkCount,
  kStResidualMax0,    // per link: bits of the largest |values - mirror| (fp32) the last round saw
  kStResidualMax1,
  kStResidualMax2,
  kStPendingTiles,    // tiles still marked pending after the last round
  kStWaitTimeouts,
  kStWords = 16,
  // after the counters: a ring of kTraceEntries records {globaltimer ns, round, listed tiles, frames sent so far}
  kTraceEntries = 64,
  kTraceWords = 4,
  kStTotalWords = kStWords + kTraceEntries * kTraceWords
};
constexpr uint64_t kErrBarrierTimeout = 1, kErrBadCtrl = 2;

// Launchers.  `stream` is a cudaStream_t passed as void*.  Return a cudaError_t as int.
int launch_round_begin(const RoundParams& p, void* stream);
int launch_round_publish(const RoundParams& p, void* stream);
int launch_round_main(const RoundParams& p, int ctas, void* stream);
// `count` rounds chained into one executable graph (a cudaGraphExec_t), built without stream capture.
int build_round_graph(const RoundParams* rounds, int count, int ctas, void** exec_out);
int round_main_smem_bytes(int n_links, int n_in, int payload_bytes, int* stages_out);

// Element-wise kernels (copyToTensor / addFromTensor / pushUpdate; src/sharedtensor.c:435-446, 334-344).
int launch_snapshot_f32(const float* values, float* out, int64_t n, void* stream);
int launch_snapshot_bf16(const float* values, void* out_bf16, int64_t n, void* stream);
int launch_add(float* values, const float* delta, int64_t n, uint8_t* tile_state, int n_tiles, int atomic, void* stream);
int launch_sub_add(float* values, const float* neu, const float* old, int64_t n, uint8_t* tile_state, int n_tiles,
                   int atomic, void* stream);
int launch_add_scaled_bf16(float* values, const void* g_bf16, float alpha, int64_t n, uint8_t* tile_state, int n_tiles,
                           void* stream);
int launch_fill_state(uint8_t* tile_state, int n_tiles, int value, void* stream);
// Per-segment sum of squares (table sync).  partials: scratch of table_scales_scratch_doubles(...) doubles.
int64_t table_scales_scratch_doubles(int n_seg, int64_t n_total);
int launch_table_scales(const float* x, const int64_t* seg_offsets_dev, int n_seg, int64_t n_total, double* partials,
                        double* out_sumsq, int8_t* out_exp, void* stream);
// sum((a[i*stride] - b[i])^2) over count samples, into out[0] (double); out[1] counts NaNs.  Zeroes nothing.
int launch_sample_sqerr(const float* a, int64_t stride, const float* b, int64_t count, double* out, void* stream);
// Busy-waits `ns` nanoseconds on the device with one thread (models "compute between updates").
int launch_delay(uint64_t ns, void* stream);
// values -> dst (peer or local) and mirror <- values in one pass; used for snapshot-on-join.
int launch_snapshot_join(const float* values, float* dst_values, float* mirror, int64_t n_padded, void* stream);
// Tensor-scale frames for TCP edges, encoded/decoded on the device (wire format of the reference).
int launch_tensor_maxabs(const float* v, const float* k, int64_t n, uint32_t* out2, void* stream);  // bits of max|v-k|, max|v|
int launch_tensor_encode(const float* v, float* k, int64_t n, float scale, uint32_t* words, void* stream);
int launch_tensor_decode(const uint32_t* words, float scale, int64_t n, float* v, float* k, uint8_t* tile_state,
                         void* stream);

}  // namespace st
