// gtk_device.cuh -- device-side view of the merge table and the launchers the
// host API calls.  Kernels live in gtk_kernels.cu.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>
#include <string>

struct gtk_tokenizer;

namespace gtk {

// Tile geometry of the segment-parallel kernel: a CTA owns the segments that
// start inside TILE consecutive bytes and sees HALO more bytes so that the
// last owned segment can finish inside shared memory.
#ifndef GTK_TILE
#define GTK_TILE 4096
#endif
#ifndef GTK_OPT_THREADS
#define GTK_OPT_THREADS 256
#endif
constexpr int kTile = GTK_TILE;
constexpr int kHalo = 256;
constexpr int kWindow = kTile + kHalo;
constexpr int kOptThreads = GTK_OPT_THREADS;
constexpr int kBaseThreads = 512;
constexpr int kBaseSmemTokens = 8192;  // chunks up to this length stay in shared memory in the local-minimum and allocation-free kernels
constexpr int kBaseSmemMaxTokens = 49152;  // one-CTA-per-chunk kernel: longest chunk held in (dynamic) shared memory, 4 bytes per slot
constexpr int kThreadSegMax = 32;      // longest segment a single thread merges on its own

// Pointers into HBM, passed by value to every kernel.
struct DeviceTable {
  const uint4* pair_buckets;       // PairBucket[65536]: four words low16(key * kPairMul) << 16 | rank, empty = all ones
  const uint2* pair_overflow;      // {key, rank} open addressing, or nullptr when no bucket overflowed
  uint32_t pair_overflow_mask;     // capacity - 1
  const uint16_t* byte_pair_rank;  // [65536]
  const uint16_t* byte_pair_info;  // [65536]: 0xFFFF cut, 0xFFFE mergeable boundary without a byte-pair rank, else rank
  const uint32_t* merged_of_rank;  // [max_rank+1]
  const uint8_t* same_of_rank;     // [max_rank+1]
  const uint32_t* adj;             // [2048]
  const uint16_t* byte_to_id;      // [256]
  const uint4* word_slots;         // WordSlot[word capacity]: {k0, k1, k2, length << 16 | id}, two-choice cuckoo
  uint32_t word_log2_capacity;
  const uint4* wide_slots;         // tables beyond 16 bits: HashSlot[1 << wide_log2] {right, left, rank, merged id}
  uint32_t wide_log2;
  uint32_t wide_max_probe;         // longest displacement of a stored key
  int monotone;
  int merged_is_256_plus_rank;
  int byte_ids_identity;
};

// Status word written by kernels instead of trapping: 0 = fine.
enum : int {
  kStatusOk = 0,
  kStatusLongQueueOverflow = 1,
  kStatusScratchTooSmall = 2,
  kStatusBadSegment = 3,
  kStatusBadOffsets = 4,  // caller-provided chunk offsets point outside the text or decrease
};

struct EncodeBuffers {
  const uint8_t* bytes;      // input text, n_bytes
  int64_t n_bytes;
  const int64_t* text_off;   // [n_texts+1]
  int64_t* text_off_copy;    // small-batch kernel only: device copy of text_off when that lives in host memory
  int64_t n_texts;
  int chunk_bytes;
  // chunker outputs
  int64_t* text_chunk_base;  // [n_texts+1] exclusive scan of chunks per text
  int64_t* chunk_off;        // [chunk_cap+1] start byte of each chunk, chunk_off[C] = n_bytes
  int64_t chunk_cap;         // upper bound on the number of chunks
  int32_t* tile_chunk0;      // [n_tiles] chunk that contains the first byte of the tile
  int64_t n_tiles;
  // merge outputs
  uint16_t* staging;         // [n_bytes] tokens of a unit, compacted at the unit's first byte
  int64_t* unit_first;       // [n_tiles] byte position where the unit's tokens start in staging (opt mode)
  int32_t* unit_cnt;         // [n_tiles] tokens produced by the unit (opt mode)
  int32_t* chunk_cnt;        // [chunk_cap] tokens per chunk
  // scan outputs
  int64_t* unit_base;        // [n_tiles+1]
  int64_t* chunk_id_off;     // [chunk_cap+1] packed id offset of each chunk (caller visible)
  int64_t* text_id_off;      // [n_texts+1] or nullptr
  int64_t* chunk_id_mirror;  // single-CTA and finish kernels: device copy of chunk_id_off when that lives in host memory
  int64_t small_seq;         // small-batch kernel only: call number, written to totals[3] as the last store of the kernel
  int32_t* out_ids;
  const uint16_t* low_id_map;  // nullptr, or 256 entries: output id of every id < 256 (GPT-2 id space)
  int64_t out_capacity;
  // scratch
  uint16_t* seg_scratch;     // per-CTA workspace for segments that do not fit in shared memory
  uint32_t* seg_scratch32;   // the same for the 32-bit kernel (tables beyond 16 bits)
  int32_t* staging32;        // [n_bytes] 32-bit kernel: tokens of a chunk, compacted at the chunk's first byte
  int64_t seg_scratch_tokens;  // tokens per CTA (two arrays of this length per CTA)
  int64_t* scan_block_sums;  // workspace of the multi-block scan
  int32_t* counters;         // [0] tile ticket, [1] status word, [2] base-mode chunk ticket
  int64_t* totals;           // device: [0] n_chunks, [1] n_ids
};

// Launchers (all asynchronous on `stream`; return the number of kernels launched).
int launch_chunker(const EncodeBuffers& b, cudaStream_t stream);
bool chunker_resets_counters(const EncodeBuffers& b);
int launch_merge_opt(const EncodeBuffers& b, const DeviceTable& t, int grid, cudaStream_t stream);
int launch_merge_base(const EncodeBuffers& b, const DeviceTable& t, int grid, int block_threads, cudaStream_t stream);
int launch_merge_wide(const EncodeBuffers& b, const DeviceTable& t, int grid, cudaStream_t stream);
int launch_pack_wide(const EncodeBuffers& b, int grid, cudaStream_t stream);
int wide_kernel_max_blocks_per_sm();
int launch_merge_localmin(const EncodeBuffers& b, const DeviceTable& t, int grid, int max_iters, cudaStream_t stream);
int launch_output_scans(const EncodeBuffers& b, int mode_base, cudaStream_t stream);
int launch_pack(const EncodeBuffers& b, int mode_base, int grid, cudaStream_t stream);
// totals[0..1] and counters[0..3] to `mapped` (page-locked host memory as the device sees it), laid out as 4 x int64
int launch_publish_totals(const EncodeBuffers& b, int64_t* mapped, cudaStream_t stream);
// a batch of at most kFinishMaxTiles tiles with a host-made chunk table (chunk_off, tile_chunk0, text_chunk_base):
// scans, pack and results into mapped host memory, then totals and the call number into mapped[0..3], in one launch
// (one CTA per tile) behind the tile kernel; uses counters[8] (zero at the start of the call) and chunk_id_mirror
int launch_finish_small_batch(const EncodeBuffers& b, int64_t* mapped, int64_t seq, cudaStream_t stream);
// the device result arena of a single-piece batch into mapped host memory, then totals {n_chunks, n_ids, status} and,
// last, the call number into mapped[0..3]; uses counters[8] (zero at the start of the call)
int launch_results_to_host(const EncodeBuffers& b, const void* src, void* dst, int64_t prefix_bytes, int64_t* mapped,
                           int64_t seq, cudaStream_t stream);
// Whole pipeline in one single-CTA kernel for small batches; totals[0..2] receive n_chunks, n_ids, status,
// totals[4] the kernel's own duration in nanoseconds and, as the very last store, totals[3] the call number.
int launch_encode_small(const EncodeBuffers& b, const DeviceTable& t, cudaStream_t stream);
#ifndef GTK_SMALL_MAX_BYTES
#define GTK_SMALL_MAX_BYTES 8192
#endif
// two tiles one after the other in one CTA (57 us) still beat the two-launch path's 58..64 us; three (75 us) do not
constexpr int64_t kSmallMaxBytes = GTK_SMALL_MAX_BYTES;
constexpr int64_t kSmallMaxTexts = 1024;
constexpr int kFinishMaxTiles = 32;  // batches through launch_finish_small_batch: at most this many tiles
// What the allocation-free entry point needs from a handle (defined in gtk_api.cu).
struct HandleView {
  int device;
  cudaStream_t stream;
  DeviceTable table;
  const uint16_t* low_id_map;  // nullptr, or the 256-entry remap of ids < 256 (GPT-2 id space selected)
  bool wide;                   // table beyond 16 bits (the allocation-free kernel is 16-bit only)
  int32_t* pinned_words;  // 8 ints of page-locked host memory owned by the handle
  std::mutex* mu;
  std::string* last_error;
};
bool handle_view(gtk_tokenizer* h, HandleView* out);

int opt_kernel_max_blocks_per_sm();
int base_kernel_max_blocks_per_sm(int chunk_bytes, int block_threads);
int localmin_kernel_max_blocks_per_sm();
void base_kernel_geometry(int chunk_bytes, int block_threads, int* warps, int* smem_tokens);

}  // namespace gtk
