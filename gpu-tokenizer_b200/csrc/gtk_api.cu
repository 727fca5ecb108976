// gtk_api.cu -- the C ABI declared in include/gputok_b200.h.
//
// One handle = one device, one stream, one merge table in HBM and a set of
// grow-only arenas (device and pinned host), so a call allocates nothing once
// the arenas have reached the working size.  The reference allocates and
// frees five device buffers inside every call (gputok_binding.cu:906-910,
// 981-986), which its own profile shows to be 70-95 % of the API time.
#include "../../include/gputok_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "gtk_device.cuh"
#include "gtk_table.hpp"

namespace {

thread_local std::string g_global_error;

struct CudaFail {
  std::string what;
};

#define GTK_CUDA(expr)                                                                              \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess) {                                                                       \
      throw CudaFail{std::string(#expr) + ": " + cudaGetErrorString(e__)};                          \
    }                                                                                               \
  } while (0)

// grow-only device / pinned-host buffers
struct DevBuf {
  void* p = nullptr;
  size_t cap = 0;
  void reserve(size_t bytes)
  {
    if (bytes <= cap) return;
    if (p) GTK_CUDA(cudaFree(p));
    p = nullptr;
    cap = 0;
    size_t want = std::max(bytes + bytes / 4, size_t(4096));
    GTK_CUDA(cudaMalloc(&p, want));
    cap = want;
  }
  void release()
  {
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
  }
  template <class T>
  T* as() const { return static_cast<T*>(p); }
};

struct PinBuf {
  void* p = nullptr;
  size_t cap = 0;
  void reserve(size_t bytes)
  {
    if (bytes <= cap) return;
    if (p) GTK_CUDA(cudaFreeHost(p));
    p = nullptr;
    cap = 0;
    size_t want = std::max(bytes + bytes / 4, size_t(4096));
    GTK_CUDA(cudaHostAlloc(&p, want, cudaHostAllocDefault));
    cap = want;
  }
  // page-locked memory that kernels write directly (dp = the address as the device sees it)
  void* dp = nullptr;
  void reserve_mapped(size_t bytes)
  {
    if (bytes <= cap && dp) return;
    if (p) GTK_CUDA(cudaFreeHost(p));
    p = dp = nullptr;
    cap = 0;
    size_t want = std::max(bytes, size_t(4096));
    GTK_CUDA(cudaHostAlloc(&p, want, cudaHostAllocMapped));
    GTK_CUDA(cudaHostGetDevicePointer(&dp, p, 0));
    cap = want;
  }
  void release()
  {
    if (p) cudaFreeHost(p);
    p = dp = nullptr;
    cap = 0;
  }
  template <class T>
  T* as() const { return static_cast<T*>(p); }
};

}  // namespace

// Buffers of one in-flight slice of a large host batch (kSliceArenas sets rotate).
constexpr int kSliceArenas = 4;
struct SliceArena {
  DevBuf text_chunk_base, chunk_off, tile_chunk0, unit_first, unit_cnt, chunk_cnt, unit_base, scan_sums, counters,
      totals;
  PinBuf h_totals;  // mapped: written by a kernel
  cudaEvent_t ev[6] = {};          // stage timing
  cudaEvent_t ev_in = nullptr;     // slice text is in HBM
  cudaEvent_t ev_front = nullptr;  // totals of the slice are on the host
  cudaEvent_t ev_packed = nullptr; // ids of the slice are packed
  cudaEvent_t ev_out = nullptr;    // results of the slice are on the host
  void release()
  {
    for (DevBuf* b : {&text_chunk_base, &chunk_off, &tile_chunk0, &unit_first, &unit_cnt, &chunk_cnt, &unit_base,
                      &scan_sums, &counters, &totals})
      b->release();
    h_totals.release();
    for (auto& e : ev)
      if (e) cudaEventDestroy(e);
    for (cudaEvent_t* e : {&ev_in, &ev_front, &ev_packed, &ev_out})
      if (*e) cudaEventDestroy(*e);
  }
};

struct gtk_tokenizer {
  std::unique_ptr<gtk::HostTable> table;
  int chunk_tokens = 2048;
  int max_iters = 50;
  int device = -1;
  int sm_count = 0;
  int opt_grid = 0, base_grid = 0, localmin_grid = 0, wide_grid = 0;
  int base_block = 0;  // threads per CTA of the one-CTA-per-chunk kernel, 0 = from the chunk size
  bool stage_timing = false;  // events between the stages of a batch that runs in one piece (gtk_set_stage_timing)
  float front_ms = -1.f;      // chunker + merge + scans of the last such batch when timed as one interval
  bool wide = false;  // ids or ranks beyond 16 bits: every GPU mode runs the 32-bit one-CTA-per-chunk kernel
  cudaStream_t stream = nullptr;      // stream in use
  cudaStream_t own_stream = nullptr;  // created by gtk_create
  cudaEvent_t ev[6] = {};
  std::mutex mu;
  mutable std::string last_error;

  // table in HBM
  DevBuf d_bpi;
  DevBuf d_slots, d_overflow, d_bpr, d_mor, d_sor, d_adj, d_b2i, d_words, d_low_map, d_wide_slots;
  DevBuf d_staging32, d_seg_scratch32;  // 32-bit kernel
  int id_space = GTK_IDS_REFERENCE;
  gtk::DeviceTable dtab{};

  // arenas
  DevBuf d_bytes, d_text_off, d_text_chunk_base, d_chunk_off, d_tile_chunk0, d_staging, d_unit_first, d_unit_cnt,
      d_chunk_cnt, d_unit_base, d_chunk_id_off, d_text_id_off, d_out_ids, d_seg_scratch, d_scan_sums,
      d_totals;  // d_totals also holds the counters (plan_batch)
  PinBuf h_ids, h_text_id_off, h_chunk_id_off, h_totals;
  // sliced host batches: offsets of all slices, moved once per batch
  DevBuf d_piece_off, d_piece_id_off, d_chunk_id_all;
  PinBuf h_piece_off, h_piece_id_off, h_chunk_id_all;
  // small batches: input and results live in mapped page-locked memory, one kernel per call
  uint8_t* small_in_h = nullptr;   // [text offsets | bytes]
  uint8_t* small_in_d = nullptr;
  uint8_t* small_out_h = nullptr;  // [totals | text id offsets | chunk id offsets | ids]
  uint8_t* small_out_d = nullptr;
  bool result_is_small = false;
  // batches below the slicing threshold: one arena [text id offsets | chunk id offsets | ids] on both sides
  DevBuf d_out_pack;
  PinBuf h_out_pack;
  bool result_is_packed = false;
  size_t pack_text_bytes = 0, pack_chunk_bytes = 0;
  const uint8_t* pack_base = nullptr;  // h_out_pack, or the mapped block below behind its 64-byte header
  // batches of up to 256 KiB: a kernel writes the results into this mapped block and the host polls its header
  uint8_t* mid_out_h = nullptr;
  uint8_t* mid_out_d = nullptr;
  int64_t mid_seq = 0;
  // one text of up to 64 KiB: chunk table, zeroed counters and the text travel in one copy (encode_host_one_text)
  PinBuf h_fast_in;
  DevBuf d_fast_in;
  int64_t small_seq = 0;  // calls of the small-batch kernel so far (the kernel echoes it as its completion mark)
  // sliced host path: copy streams and two slice arenas
  cudaStream_t in_stream = nullptr, out_stream = nullptr, pack_stream = nullptr;
  SliceArena slice[kSliceArenas];
  // host-side result of gtk_encode_cpu
  std::vector<int32_t> cpu_ids;
  std::vector<int64_t> cpu_text_off, cpu_chunk_off;
  bool result_is_cpu = false;
  int64_t res_n_ids = 0, res_n_chunks = 0, res_n_texts = 0;
  float stage_ms[5] = {0, 0, 0, 0, 0};
  int32_t last_launches = 0;

  int fail(int code, const std::string& msg) const
  {
    last_error = msg;
    return code;
  }
};

namespace {

void upload(DevBuf& buf, const void* src, size_t bytes, cudaStream_t s)
{
  buf.reserve(bytes);
  GTK_CUDA(cudaMemcpyAsync(buf.p, src, bytes, cudaMemcpyHostToDevice, s));
}

void upload_table(gtk_tokenizer* h)
{
  const gtk::HostTable& t = *h->table;
  upload(h->d_slots, t.pair_buckets.data(), t.pair_buckets.size() * sizeof(gtk::PairBucket), h->stream);
  if (!t.pair_overflow.empty())
    upload(h->d_overflow, t.pair_overflow.data(), t.pair_overflow.size() * sizeof(gtk::PairSlot), h->stream);
  upload(h->d_bpr, t.byte_pair_rank.data(), t.byte_pair_rank.size() * sizeof(uint16_t), h->stream);
  upload(h->d_bpi, t.byte_pair_info.data(), t.byte_pair_info.size() * sizeof(uint16_t), h->stream);
  upload(h->d_mor, t.merged_of_rank.data(), t.merged_of_rank.size() * sizeof(uint32_t), h->stream);
  upload(h->d_sor, t.same_of_rank.data(), t.same_of_rank.size(), h->stream);
  upload(h->d_adj, t.adj, sizeof(t.adj), h->stream);
  upload(h->d_b2i, t.byte_to_id, sizeof(t.byte_to_id), h->stream);
  upload(h->d_low_map, t.gpt2_low_id, sizeof(t.gpt2_low_id), h->stream);
  upload(h->d_words, t.word_slots.data(), t.word_slots.size() * sizeof(gtk::WordSlot), h->stream);
  if (h->wide) upload(h->d_wide_slots, t.slots.data(), t.slots.size() * sizeof(gtk::HashSlot), h->stream);
  GTK_CUDA(cudaStreamSynchronize(h->stream));
  h->dtab.pair_buckets = h->d_slots.as<uint4>();
  h->dtab.pair_overflow = t.pair_overflow.empty() ? nullptr : h->d_overflow.as<uint2>();
  h->dtab.pair_overflow_mask = t.pair_overflow.empty() ? 0u : uint32_t(t.pair_overflow.size() - 1);
  h->dtab.byte_pair_rank = h->d_bpr.as<uint16_t>();
  h->dtab.byte_pair_info = h->d_bpi.as<uint16_t>();
  h->dtab.merged_of_rank = h->d_mor.as<uint32_t>();
  h->dtab.same_of_rank = h->d_sor.as<uint8_t>();
  h->dtab.adj = h->d_adj.as<uint32_t>();
  h->dtab.byte_to_id = h->d_b2i.as<uint16_t>();
  h->dtab.word_slots = h->d_words.as<uint4>();
  h->dtab.word_log2_capacity = t.word_log2_capacity;
  h->dtab.wide_slots = h->wide ? h->d_wide_slots.as<uint4>() : nullptr;
  h->dtab.wide_log2 = t.log2_capacity;
  h->dtab.wide_max_probe = t.max_probe;
  h->dtab.monotone = t.monotone ? 1 : 0;
  h->dtab.merged_is_256_plus_rank = t.merged_is_256_plus_rank ? 1 : 0;
  h->dtab.byte_ids_identity = t.byte_ids_identity ? 1 : 0;
}

// Upper bound on the number of chunks without touching the device: every text
// contributes its full chunks plus at most one partial chunk.
int64_t chunk_upper_bound(int64_t n_bytes, int64_t n_texts, int chunk_tokens)
{
  return n_bytes / chunk_tokens + n_texts + 1;
}

struct Plan {
  gtk::EncodeBuffers b{};
  int64_t chunk_cap = 0;
};

// Size the arenas for a batch and fill the kernel argument block.
Plan plan_batch(gtk_tokenizer* h, const uint8_t* d_bytes, int64_t n_bytes, const int64_t* d_text_off,
                int64_t n_texts, int32_t* d_out_ids, int64_t out_capacity, int64_t* d_chunk_id_off,
                bool want_text_id_off)
{
  Plan p;
  gtk::EncodeBuffers& b = p.b;
  const int64_t chunk_cap = chunk_upper_bound(n_bytes, n_texts, h->chunk_tokens);
  const int64_t n_tiles = (n_bytes + gtk::kTile - 1) / gtk::kTile;
  p.chunk_cap = chunk_cap;
  h->d_text_chunk_base.reserve(size_t(n_texts + 1) * 8);
  h->d_chunk_off.reserve(size_t(chunk_cap + 1) * 8);
  h->d_tile_chunk0.reserve(size_t(n_tiles + 1) * 4);
  h->d_staging.reserve(size_t(n_bytes + 16) * 2);
  h->d_unit_first.reserve(size_t(n_tiles + 1) * 8);
  h->d_unit_cnt.reserve(size_t(n_tiles + 1) * 4);
  h->d_chunk_cnt.reserve(size_t(chunk_cap + 1) * 4);
  h->d_unit_base.reserve(size_t(n_tiles + 2) * 8);
  if (!d_chunk_id_off) {
    h->d_chunk_id_off.reserve(size_t(chunk_cap + 1) * 8);
    d_chunk_id_off = h->d_chunk_id_off.as<int64_t>();
  }
  if (want_text_id_off) h->d_text_id_off.reserve(size_t(n_texts + 1) * 8);
  const int64_t scan_items = std::max<int64_t>(std::max(chunk_cap, n_tiles), n_texts);
  h->d_scan_sums.reserve(size_t(scan_items / 4096 + 2) * 8);
  h->d_totals.reserve(128);  // [0] n_chunks, [1] n_ids as int64, then the 16 int32 counters: one copy brings both
  // workspace for segments / chunks that do not fit in shared memory
  const int64_t longest = std::min<int64_t>(h->chunk_tokens, n_bytes);
  int64_t scratch_tokens = 0;
  if (longest > gtk::kHalo) scratch_tokens = (longest + 63) & ~int64_t(63);
  const int ctas = std::max(h->opt_grid, std::max(h->base_grid, h->localmin_grid));
  if (scratch_tokens && !h->wide) h->d_seg_scratch.reserve(size_t(ctas) * 2 * size_t(scratch_tokens) * 2);
  if (h->wide) {
    h->d_staging32.reserve(size_t(n_bytes + 16) * 4);
    if (scratch_tokens) h->d_seg_scratch32.reserve(size_t(h->wide_grid) * 2 * size_t(scratch_tokens) * 4);
  }

  b.bytes = d_bytes;
  b.n_bytes = n_bytes;
  b.text_off = d_text_off;
  b.n_texts = n_texts;
  b.chunk_bytes = h->chunk_tokens;
  b.text_chunk_base = h->d_text_chunk_base.as<int64_t>();
  b.chunk_off = h->d_chunk_off.as<int64_t>();
  b.chunk_cap = chunk_cap;
  b.tile_chunk0 = h->d_tile_chunk0.as<int32_t>();
  b.n_tiles = n_tiles;
  b.staging = h->d_staging.as<uint16_t>();
  b.unit_first = h->d_unit_first.as<int64_t>();
  b.unit_cnt = h->d_unit_cnt.as<int32_t>();
  b.chunk_cnt = h->d_chunk_cnt.as<int32_t>();
  b.unit_base = h->d_unit_base.as<int64_t>();
  b.chunk_id_off = d_chunk_id_off;
  b.text_id_off = want_text_id_off ? h->d_text_id_off.as<int64_t>() : nullptr;
  b.out_ids = d_out_ids;
  b.out_capacity = out_capacity;
  b.seg_scratch = (scratch_tokens && !h->wide) ? h->d_seg_scratch.as<uint16_t>() : nullptr;
  b.seg_scratch32 = (scratch_tokens && h->wide) ? h->d_seg_scratch32.as<uint32_t>() : nullptr;
  b.staging32 = h->wide ? h->d_staging32.as<int32_t>() : nullptr;
  b.seg_scratch_tokens = scratch_tokens;
  b.scan_block_sums = h->d_scan_sums.as<int64_t>();
  b.totals = h->d_totals.as<int64_t>();
  b.counters = reinterpret_cast<int32_t*>(b.totals + 2);
  b.low_id_map = (h->id_space == GTK_IDS_GPT2) ? h->d_low_map.as<uint16_t>() : nullptr;
  return p;
}

const char* status_text(int s)
{
  switch (s) {
    case gtk::kStatusLongQueueOverflow: return "long-segment queue overflow";
    case gtk::kStatusScratchTooSmall: return "segment workspace too small";
    case gtk::kStatusBadSegment: return "merge pass made no progress";
    case gtk::kStatusBadOffsets: return "chunk offsets outside the text";
    default: return "unknown kernel status";
  }
}

// Chunker -> merge -> scans.  Leaves totals (n_chunks, n_ids) and the status
// word in the pinned totals buffer; the caller synchronises and then packs.
// n_chunks, n_ids and the status word to the host: totals and counters are adjacent in the handle's own arena
void copy_totals(gtk_tokenizer* h, const gtk::EncodeBuffers& b, int64_t* pinned_totals, cudaStream_t s)
{
  int64_t* ht = pinned_totals ? pinned_totals : h->h_totals.as<int64_t>();
  if (reinterpret_cast<const int64_t*>(b.counters) == b.totals + 2) {
    GTK_CUDA(cudaMemcpyAsync(ht, b.totals, 32, cudaMemcpyDeviceToHost, s));
  } else {
    GTK_CUDA(cudaMemcpyAsync(ht, b.totals, 16, cudaMemcpyDeviceToHost, s));
    GTK_CUDA(cudaMemcpyAsync(ht + 2, b.counters, 16, cudaMemcpyDeviceToHost, s));
  }
}

// chained: the pack follows on the same stream without a host round trip, so that one event pair around both
// times the pipeline when the stages are not timed one by one.
void run_front(gtk_tokenizer* h, const gtk::EncodeBuffers& b, int mode, int* launches, cudaEvent_t* ev = nullptr,
               int64_t* pinned_totals = nullptr, int64_t* mapped_totals = nullptr, bool chained = false)
{
  cudaStream_t s = h->stream;
  const bool stages = ev != nullptr || h->stage_timing;  // sliced batches always time their stages
  if (!ev) ev = h->ev;
  if (!gtk::chunker_resets_counters(b)) {
    GTK_CUDA(cudaMemsetAsync(b.counters, 0, 64, s));
    GTK_CUDA(cudaMemsetAsync(b.chunk_cnt, 0, size_t(b.chunk_cap + 1) * 4, s));
  }
  GTK_CUDA(cudaEventRecord(ev[0], s));
  *launches += gtk::launch_chunker(b, s);
  if (stages) GTK_CUDA(cudaEventRecord(ev[1], s));
  if (h->wide) *launches += gtk::launch_merge_wide(b, h->dtab, h->wide_grid, s);
  else if (mode == GTK_MODE_BASE) *launches += gtk::launch_merge_base(b, h->dtab, h->base_grid, h->base_block, s);
  else if (mode == GTK_MODE_LOCALMIN) *launches += gtk::launch_merge_localmin(b, h->dtab, h->localmin_grid, h->max_iters, s);
  else *launches += gtk::launch_merge_opt(b, h->dtab, h->opt_grid, s);
  if (stages) GTK_CUDA(cudaEventRecord(ev[2], s));
  *launches += gtk::launch_output_scans(b, mode != GTK_MODE_OPT || h->wide, s);
  if (stages || !chained) GTK_CUDA(cudaEventRecord(ev[3], s));
  GTK_CUDA(cudaGetLastError());
  if (mapped_totals) {  // one small kernel writes the four words into mapped host memory: no copy-engine round trips
    *launches += gtk::launch_publish_totals(b, mapped_totals, s);
    return;
  }
  if (chained) return;  // the totals travel behind the pack (run_pack), which does not have to wait for them
  copy_totals(h, b, pinned_totals, s);
}

void run_pack(gtk_tokenizer* h, const gtk::EncodeBuffers& b, int mode, int* launches, cudaEvent_t* ev = nullptr,
              cudaStream_t on = nullptr, bool chained = false, bool totals_by_copy = true)
{
  cudaStream_t s = on ? on : h->stream;
  const bool stages = ev != nullptr || h->stage_timing;
  if (!ev) ev = h->ev;
  if (stages || !chained) GTK_CUDA(cudaEventRecord(ev[5], s));
  if (h->wide) *launches += gtk::launch_pack_wide(b, h->sm_count * 8, s);
  else *launches += gtk::launch_pack(b, mode != GTK_MODE_OPT, h->sm_count * 8, s);
  GTK_CUDA(cudaEventRecord(ev[4], s));
  GTK_CUDA(cudaGetLastError());
  if (chained && totals_by_copy) copy_totals(h, b, nullptr, s);
}

// Adds the stage times of one pipeline run (one batch, or one slice) to h->stage_ms.  The events must have
// completed and must not have been recorded again since: the sliced path therefore reads the front events
// of a slice as soon as its front has finished (its arena's events are recorded again for a later slice
// soon after) and the pack events when its ids have arrived.
void collect_front_times(gtk_tokenizer* h, cudaEvent_t* ev = nullptr)
{
  const bool stages = ev != nullptr || h->stage_timing;
  if (!ev) ev = h->ev;
  float ms = 0;
  if (!stages) {  // chunker, merge and scans as one interval
    GTK_CUDA(cudaEventElapsedTime(&ms, ev[0], ev[3]));
    h->front_ms = ms;
    return;
  }
  h->front_ms = -1.f;
  for (int i = 0; i < 3; ++i) {
    GTK_CUDA(cudaEventElapsedTime(&ms, ev[i], ev[i + 1]));
    h->stage_ms[i] += ms;
  }
}

void collect_pack_time(gtk_tokenizer* h, cudaEvent_t* ev = nullptr)
{
  if (!ev) ev = h->ev;
  float ms = 0;
  GTK_CUDA(cudaEventElapsedTime(&ms, ev[5], ev[4]));
  // the pipeline time excludes the host round trip between scans and pack
  if (h->front_ms >= 0.f) {
    h->stage_ms[4] = h->front_ms + ms;
    return;
  }
  h->stage_ms[3] += ms;
  h->stage_ms[4] = h->stage_ms[0] + h->stage_ms[1] + h->stage_ms[2] + h->stage_ms[3];
}

void collect_stage_times(gtk_tokenizer* h, bool chained = false)
{
  if (chained && !h->stage_timing) {  // one event pair around the whole pipeline
    GTK_CUDA(cudaEventElapsedTime(&h->stage_ms[4], h->ev[0], h->ev[4]));
    return;
  }
  collect_front_times(h);
  collect_pack_time(h);
}


// ------------------------------------------------------------------------------------------------
// Large host batches: cut the batch into slices of whole chunks and overlap, per slice, the
// host->device copy, the kernel pipeline and the device->host copy of the results on three
// streams.  A slice is an independent sub-batch (its pieces are texts or chunk-aligned parts of a
// text), so the per-chunk results are exactly those of the unsliced batch.
// ------------------------------------------------------------------------------------------------
const char* const kWideNoLocalmin =
    "the local-minimum mode is not offered for merge tables with ids >= 65535 or ranks >= 65534";
// smaller batches take the single-shot path; from 8 MiB on the overlap of a few slices (6 + 2 MiB at the least) wins:
// 8 / 16 / 23 MiB in 0.50 / 0.88 / 1.11 ms against 0.56 / 0.97 / 1.33 ms unsliced
constexpr int64_t kSliceThresholdBytes = int64_t(8) << 20;
constexpr int64_t kSliceTargetBytes    = int64_t(24) << 20;  // measured best of 16..40 MiB on config 2 (256 MiB)

struct SlicePlan {
  int64_t byte_lo = 0, byte_hi = 0;
  std::vector<int64_t> piece_off;    // [P+1], relative to byte_lo
  std::vector<int64_t> first_text;   // [P]: text index if the piece starts a text, else -1
};

// Size of the slice that starts at byte `lo` of a batch of `total` bytes: full-size slices in the middle,
// smaller ones at both ends (a quarter, then half; for batches of two full slices and more an eighth first), because
// the first slice's upload and kernels and the last slice's download are the part of the call that nothing overlaps.
int64_t slice_target(int64_t lo, int64_t total, int64_t full)
{
  if (total >= 2 * full) {  // large batches: three steps at both ends, an eighth, a quarter, a half (256 MiB: 8.03 against 8.11 ms)
    const int64_t e = full / 8, rem = total - lo;
    int64_t t = (lo < e) ? e : (lo < 3 * e) ? 2 * e : (lo < 7 * e) ? 4 * e : full;
    if (rem <= e) t = rem;
    else if (rem <= 3 * e) t = std::min(t, rem - e);
    else if (rem <= 7 * e) t = std::min(t, rem - 3 * e);
    else if (rem <= 7 * e + full) t = std::min(t, std::max(rem - 7 * e, e));
    return std::max<int64_t>(t, 1);
  }
  const int64_t q = full / 4, rem = total - lo;
  int64_t t = (lo < q) ? q : (lo < 3 * q) ? 2 * q : full;
  if (rem <= q) t = rem;
  else if (rem <= 3 * q) t = std::min(t, rem - q);
  else if (rem <= 3 * q + full) t = std::min(t, std::max(rem - 3 * q, q));
  return std::max<int64_t>(t, 1);
}

std::vector<SlicePlan> plan_slices(const int64_t* text_off, int64_t n_texts, int chunk, int64_t full)
{
  const int64_t total = n_texts > 0 ? text_off[n_texts] : 0;
  int64_t target = slice_target(0, total, full);
  std::vector<SlicePlan> out;
  SlicePlan cur;
  cur.piece_off.push_back(0);
  auto close = [&](int64_t at) {
    cur.byte_hi = at;
    out.push_back(std::move(cur));
    cur = SlicePlan();
    cur.byte_lo = at;
    cur.piece_off.push_back(0);
    target = slice_target(at, total, full);
  };
  for (int64_t t = 0; t < n_texts; ++t) {
    int64_t pos = text_off[t];
    const int64_t end = text_off[t + 1];
    bool first = true;
    do {
      const int64_t used = pos - cur.byte_lo;
      int64_t take = end - pos;
      if (used + take > target && take > 0) {
        const int64_t room_chunks = (target - used) / chunk;
        if (room_chunks <= 0 && used > 0) {  // slice is full: start a new one and retry
          close(pos);
          continue;
        }
        take = std::min<int64_t>(take, std::max<int64_t>(room_chunks, 1) * chunk);
      }
      cur.piece_off.push_back(pos + take - cur.byte_lo);
      cur.first_text.push_back(first ? t : -1);
      first = false;
      pos += take;
      if (pos - cur.byte_lo >= target) close(pos);
    } while (pos < end);
  }
  if (cur.piece_off.size() > 1) close(text_off[n_texts]);
  return out;
}

void slice_arena_prepare(gtk_tokenizer* h, SliceArena& a, int64_t max_bytes, int64_t max_pieces)
{
  const int64_t chunk_cap = chunk_upper_bound(max_bytes, max_pieces, h->chunk_tokens);
  const int64_t n_tiles   = (max_bytes + gtk::kTile - 1) / gtk::kTile;
  a.text_chunk_base.reserve(size_t(max_pieces + 1) * 8);
  a.chunk_off.reserve(size_t(chunk_cap + 1) * 8);
  a.tile_chunk0.reserve(size_t(n_tiles + 1) * 4);
  a.unit_first.reserve(size_t(n_tiles + 1) * 8);
  a.unit_cnt.reserve(size_t(n_tiles + 1) * 4);
  a.chunk_cnt.reserve(size_t(chunk_cap + 1) * 4);
  a.unit_base.reserve(size_t(n_tiles + 2) * 8);
  a.scan_sums.reserve(size_t(std::max<int64_t>(std::max(chunk_cap, n_tiles), max_pieces) / 4096 + 2) * 8);
  a.counters.reserve(64);
  a.totals.reserve(64);
  a.h_totals.reserve_mapped(64);
  for (auto& e : a.ev)
    if (!e) GTK_CUDA(cudaEventCreate(&e));
  for (cudaEvent_t* e : {&a.ev_in, &a.ev_front, &a.ev_packed, &a.ev_out})
    if (!*e) GTK_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
}

// Device offset of slice i inside the batch-wide byte / staging / id buffers: 16-element aligned
// (vector loads) and spaced so that neighbouring slices never share an element.
inline int64_t slice_dev_offset(const SlicePlan& sp, int index) { return (sp.byte_lo + 16 * int64_t(index) + 15) & ~int64_t(15); }

gtk::EncodeBuffers slice_buffers(gtk_tokenizer* h, SliceArena& a, const SlicePlan& sp, int index, int64_t max_bytes)
{
  gtk::EncodeBuffers b{};
  const int64_t dev_off = slice_dev_offset(sp, index);
  const int64_t n_bytes = sp.byte_hi - sp.byte_lo;
  const int64_t pieces  = int64_t(sp.piece_off.size()) - 1;
  b.bytes = h->d_bytes.as<uint8_t>() + dev_off;
  b.n_bytes = n_bytes;
  b.text_off = nullptr;  // the three offset arrays are set by the caller (batch-wide buffers)
  b.n_texts = pieces;
  b.chunk_bytes = h->chunk_tokens;
  b.text_chunk_base = a.text_chunk_base.as<int64_t>();
  b.chunk_off = a.chunk_off.as<int64_t>();
  b.chunk_cap = chunk_upper_bound(n_bytes, pieces, h->chunk_tokens);
  b.tile_chunk0 = a.tile_chunk0.as<int32_t>();
  b.n_tiles = (n_bytes + gtk::kTile - 1) / gtk::kTile;
  b.staging = h->d_staging.as<uint16_t>() + dev_off;
  b.unit_first = a.unit_first.as<int64_t>();
  b.unit_cnt = a.unit_cnt.as<int32_t>();
  b.chunk_cnt = a.chunk_cnt.as<int32_t>();
  b.unit_base = a.unit_base.as<int64_t>();
  b.chunk_id_off = nullptr;
  b.text_id_off = nullptr;
  b.out_ids = h->d_out_ids.as<int32_t>() + dev_off;  // worst case one id per byte: slices never overlap
  b.out_capacity = n_bytes;
  const int64_t longest = std::min<int64_t>(h->chunk_tokens, n_bytes);
  const int64_t scratch_tokens = longest > gtk::kHalo ? ((longest + 63) & ~int64_t(63)) : 0;
  b.seg_scratch = (scratch_tokens && !h->wide) ? h->d_seg_scratch.as<uint16_t>() : nullptr;
  b.seg_scratch32 = (scratch_tokens && h->wide) ? h->d_seg_scratch32.as<uint32_t>() : nullptr;
  b.staging32 = h->wide ? h->d_staging32.as<int32_t>() + dev_off : nullptr;
  b.seg_scratch_tokens = scratch_tokens;
  b.scan_block_sums = a.scan_sums.as<int64_t>();
  b.counters = a.counters.as<int32_t>();
  b.totals = a.totals.as<int64_t>();
  b.low_id_map = (h->id_space == GTK_IDS_GPT2) ? h->d_low_map.as<uint16_t>() : nullptr;
  return b;
}


int encode_host_sliced(gtk_tokenizer* h, int mode, const uint8_t* bytes, const int64_t* text_offsets,
                       int64_t n_texts, int64_t n_bytes, float* kernel_ms)
{
  const std::vector<SlicePlan> slices = plan_slices(text_offsets, n_texts, h->chunk_tokens, kSliceTargetBytes);
  const int ns     = int(slices.size());
  const size_t nsz = size_t(ns);
  // Offsets travel once per batch, not once per slice: the piece offsets of all slices go up in one copy
  // before the first slice, the per-piece and per-chunk id offsets of all slices come back in two copies
  // after the last one.  Slice i owns entries [piece_at[i], piece_at[i+1]) and [chunk_at[i], chunk_at[i+1]).
  std::vector<int64_t> piece_at(nsz + 1, 0), chunk_at(nsz + 1, 0);
  int64_t max_bytes = 0, max_pieces = 0;
  for (int i = 0; i < ns; ++i) {
    const SlicePlan& sp  = slices[size_t(i)];
    const int64_t pieces = int64_t(sp.piece_off.size()) - 1;
    max_bytes  = std::max(max_bytes, sp.byte_hi - sp.byte_lo);
    max_pieces = std::max(max_pieces, pieces);
    piece_at[size_t(i) + 1] = piece_at[size_t(i)] + pieces + 1;
    chunk_at[size_t(i) + 1] = chunk_at[size_t(i)] + chunk_upper_bound(sp.byte_hi - sp.byte_lo, pieces, h->chunk_tokens) + 1;
  }
  const int64_t total_pieces = piece_at[nsz] - ns;
  // everything is sized before the first copy is issued: nothing may be reallocated in flight
  const size_t span = size_t(n_bytes) + 16 * size_t(ns) + 64;  // slices sit at 16-aligned, disjoint offsets
  h->d_bytes.reserve(span);
  h->d_staging.reserve(span * 2);
  h->d_out_ids.reserve(span * 4);
  {
    const int64_t longest = std::min<int64_t>(h->chunk_tokens, max_bytes);
    if (h->wide) {
      h->d_staging32.reserve(span * 4);
      if (longest > gtk::kHalo)
        h->d_seg_scratch32.reserve(size_t(h->wide_grid) * 2 * size_t((longest + 63) & ~int64_t(63)) * 4);
    } else if (longest > gtk::kHalo)
      h->d_seg_scratch.reserve(size_t(std::max(h->opt_grid, std::max(h->base_grid, h->localmin_grid))) * 2 * size_t((longest + 63) & ~int64_t(63)) * 2);
  }
  h->d_piece_off.reserve(size_t(piece_at[nsz]) * 8);
  h->d_piece_id_off.reserve(size_t(piece_at[nsz]) * 8);
  h->d_chunk_id_all.reserve(size_t(chunk_at[nsz]) * 8);
  h->h_piece_off.reserve(size_t(piece_at[nsz]) * 8);
  h->h_piece_id_off.reserve(size_t(piece_at[nsz]) * 8);
  h->h_chunk_id_all.reserve(size_t(chunk_at[nsz]) * 8);
  h->h_text_id_off.reserve(size_t(n_texts + 1) * 8);
  h->h_chunk_id_off.reserve(size_t(chunk_upper_bound(n_bytes, total_pieces, h->chunk_tokens) + 2) * 8);
  h->h_ids.reserve(size_t(n_bytes) * 2);  // grown below if the batch yields more than one id per two bytes
  if (!h->in_stream) GTK_CUDA(cudaStreamCreateWithFlags(&h->in_stream, cudaStreamNonBlocking));
  if (!h->out_stream) GTK_CUDA(cudaStreamCreateWithFlags(&h->out_stream, cudaStreamNonBlocking));
  if (!h->pack_stream) GTK_CUDA(cudaStreamCreateWithFlags(&h->pack_stream, cudaStreamNonBlocking));
  for (auto& a : h->slice) slice_arena_prepare(h, a, max_bytes, max_pieces);
  GTK_CUDA(cudaStreamSynchronize(h->stream));

  for (int i = 0; i < ns; ++i) {
    const SlicePlan& sp = slices[size_t(i)];
    std::memcpy(h->h_piece_off.as<int64_t>() + piece_at[size_t(i)], sp.piece_off.data(), sp.piece_off.size() * 8);
  }
  GTK_CUDA(cudaMemcpyAsync(h->d_piece_off.p, h->h_piece_off.p, size_t(piece_at[nsz]) * 8, cudaMemcpyHostToDevice,
                           h->in_stream));

  std::vector<gtk::EncodeBuffers> bufs(nsz);
  std::vector<int64_t> sl_c(nsz), sl_r(nsz), sl_cbase(nsz);
  int launches = 0;
  int64_t R = 0, Cbase = 0;

  auto issue_front = [&](int i) {
    SliceArena& a = h->slice[i % kSliceArenas];
    const SlicePlan& sp = slices[size_t(i)];
    GTK_CUDA(cudaMemcpyAsync(h->d_bytes.as<uint8_t>() + slice_dev_offset(sp, i), bytes + sp.byte_lo, size_t(sp.byte_hi - sp.byte_lo),
                             cudaMemcpyHostToDevice, h->in_stream));
    GTK_CUDA(cudaEventRecord(a.ev_in, h->in_stream));
    GTK_CUDA(cudaStreamWaitEvent(h->stream, a.ev_in, 0));
    if (i >= kSliceArenas) GTK_CUDA(cudaStreamWaitEvent(h->stream, a.ev_out, 0));  // its previous slice has left this arena
    gtk::EncodeBuffers& b = bufs[size_t(i)];
    b = slice_buffers(h, a, sp, i, max_bytes);
    b.text_off     = h->d_piece_off.as<int64_t>() + piece_at[size_t(i)];
    b.text_id_off  = h->d_piece_id_off.as<int64_t>() + piece_at[size_t(i)];
    b.chunk_id_off = h->d_chunk_id_all.as<int64_t>() + chunk_at[size_t(i)];
    // the four result words of the front are written into mapped host memory by a one-thread kernel
    run_front(h, b, mode, &launches, a.ev, nullptr, static_cast<int64_t*>(a.h_totals.dp));
    GTK_CUDA(cudaEventRecord(a.ev_front, h->stream));
  };
  auto finish = [&](int i) {  // the ids of slice i are on the host
    SliceArena& a = h->slice[i % kSliceArenas];
    GTK_CUDA(cudaEventSynchronize(a.ev_out));
    collect_pack_time(h, a.ev);
  };
  auto sync_all = [&] {
    cudaStreamSynchronize(h->in_stream);
    cudaStreamSynchronize(h->stream);
    cudaStreamSynchronize(h->pack_stream);
    cudaStreamSynchronize(h->out_stream);
  };

  constexpr int kAhead = kSliceArenas - 1;  // fronts queued ahead of the slice being packed
  for (int i = 0; i < std::min(ns, kAhead); ++i) issue_front(i);
  for (int i = 0; i < ns; ++i) {
    SliceArena& a = h->slice[i % kSliceArenas];
    if (i >= 2) finish(i - 2);
    GTK_CUDA(cudaEventSynchronize(a.ev_front));
    collect_front_times(h, a.ev);
    const int64_t* ht = a.h_totals.as<int64_t>();
    const int64_t C = ht[0], N = ht[1];
    const int status = reinterpret_cast<const int32_t*>(ht + 2)[1];
    if (status != gtk::kStatusOk) {
      sync_all();
      return h->fail(GTK_ERR_KERNEL, status_text(status));
    }
    if (size_t(R + N + 1) * 4 > h->h_ids.cap) {  // grow the pinned id buffer, keeping what has arrived
      GTK_CUDA(cudaStreamSynchronize(h->out_stream));
      PinBuf bigger;
      bigger.reserve(std::max(size_t(R + N + 1) * 4 * 2, h->h_ids.cap * 2));
      std::memcpy(bigger.p, h->h_ids.p, size_t(R) * 4);
      h->h_ids.release();
      h->h_ids = bigger;
    }
    // the pack runs on a stream of its own: the compute stream already holds the fronts of later slices
    GTK_CUDA(cudaStreamWaitEvent(h->pack_stream, a.ev_front, 0));
    run_pack(h, bufs[size_t(i)], mode, &launches, a.ev, h->pack_stream);
    GTK_CUDA(cudaEventRecord(a.ev_packed, h->pack_stream));
    GTK_CUDA(cudaStreamWaitEvent(h->out_stream, a.ev_packed, 0));
    GTK_CUDA(cudaMemcpyAsync(h->h_ids.as<int32_t>() + R, bufs[size_t(i)].out_ids, size_t(N) * 4, cudaMemcpyDeviceToHost,
                             h->out_stream));
    GTK_CUDA(cudaEventRecord(a.ev_out, h->out_stream));
    sl_c[size_t(i)]     = C;
    sl_r[size_t(i)]     = R;
    sl_cbase[size_t(i)] = Cbase;
    R += N;
    Cbase += C;
    if (i + kAhead < ns) issue_front(i + kAhead);
  }
  // offsets of all slices in two copies behind the last ids
  GTK_CUDA(cudaMemcpyAsync(h->h_piece_id_off.p, h->d_piece_id_off.p, size_t(piece_at[nsz]) * 8, cudaMemcpyDeviceToHost,
                           h->out_stream));
  GTK_CUDA(cudaMemcpyAsync(h->h_chunk_id_all.p, h->d_chunk_id_all.p, size_t(chunk_at[nsz]) * 8, cudaMemcpyDeviceToHost,
                           h->out_stream));
  for (int i = std::max(0, ns - 2); i < ns; ++i) finish(i);
  GTK_CUDA(cudaStreamSynchronize(h->out_stream));
  GTK_CUDA(cudaStreamSynchronize(h->stream));
  // per-slice offsets start at 0: add the ids that precede the slice.  A text that starts exactly where the
  // previous slice ended belongs to the slice that holds its first piece.
  int64_t* h_text  = h->h_text_id_off.as<int64_t>();
  int64_t* h_chunk = h->h_chunk_id_off.as<int64_t>();
  for (int i = 0; i < ns; ++i) {
    const SlicePlan& sp = slices[size_t(i)];
    const int64_t base  = sl_r[size_t(i)];
    const int64_t* pid  = h->h_piece_id_off.as<int64_t>() + piece_at[size_t(i)];
    for (size_t p = 0; p < sp.first_text.size(); ++p)
      if (sp.first_text[p] >= 0) h_text[sp.first_text[p]] = base + pid[p];
    const int64_t* src = h->h_chunk_id_all.as<int64_t>() + chunk_at[size_t(i)];
    int64_t* dst       = h_chunk + sl_cbase[size_t(i)];
    for (int64_t c = 0; c < sl_c[size_t(i)]; ++c) dst[c] = src[c] + base;
  }
  h_chunk[Cbase] = R;
  h_text[n_texts] = R;
  h->last_launches = launches;
  h->res_n_ids = R;
  h->res_n_chunks = Cbase;
  if (kernel_ms) *kernel_ms = h->stage_ms[4];
  return GTK_OK;
}


// ------------------------------------------------------------------------------------------------
// Small host batches (latency mode): the text is copied into mapped page-locked memory, one
// single-CTA kernel reads it over PCIe and writes ids and offsets straight back into mapped
// memory; the call is one launch plus one stream synchronisation.
// ------------------------------------------------------------------------------------------------
constexpr size_t kSmallInOff    = 0;
constexpr size_t kSmallInBytes  = ((size_t(gtk::kSmallMaxTexts) + 1) * 8 + 63) & ~size_t(63);
constexpr size_t kSmallInSize   = kSmallInBytes + size_t(gtk::kSmallMaxBytes) + 64;
constexpr int64_t kSmallChunkCap = gtk::kSmallMaxBytes + gtk::kSmallMaxTexts + 2;
constexpr size_t kSmallOutTotals = 0;
constexpr size_t kSmallOutText   = 64;
constexpr size_t kSmallOutChunk  = kSmallOutText + (((size_t(gtk::kSmallMaxTexts) + 1) * 8 + 63) & ~size_t(63));
constexpr size_t kSmallOutIds    = kSmallOutChunk + (((size_t(kSmallChunkCap) + 1) * 8 + 63) & ~size_t(63));
constexpr size_t kSmallOutSize   = kSmallOutIds + size_t(gtk::kSmallMaxBytes) * 4 + 64;
constexpr size_t kMappedResultBytes        = size_t(2) << 20;    // mapped result block of the next size class
constexpr int64_t kResultsByKernelMaxBytes = int64_t(256) << 10;  // batches up to this size use it

void small_path_init(gtk_tokenizer* h)
{
  void *ih = nullptr, *oh = nullptr, *id = nullptr, *od = nullptr;
  GTK_CUDA(cudaHostAlloc(&ih, kSmallInSize, cudaHostAllocMapped));
  GTK_CUDA(cudaHostAlloc(&oh, kSmallOutSize, cudaHostAllocMapped));
  GTK_CUDA(cudaHostGetDevicePointer(&id, ih, 0));
  GTK_CUDA(cudaHostGetDevicePointer(&od, oh, 0));
  std::memset(oh, 0, 64);  // the completion mark of the result block starts at call number 0
  h->small_in_h = static_cast<uint8_t*>(ih);
  h->small_out_h = static_cast<uint8_t*>(oh);
  h->small_in_d = static_cast<uint8_t*>(id);
  h->small_out_d = static_cast<uint8_t*>(od);
  void *mh = nullptr, *md = nullptr;
  GTK_CUDA(cudaHostAlloc(&mh, kMappedResultBytes, cudaHostAllocMapped));
  GTK_CUDA(cudaHostGetDevicePointer(&md, mh, 0));
  std::memset(mh, 0, 64);
  h->mid_out_h = static_cast<uint8_t*>(mh);
  h->mid_out_d = static_cast<uint8_t*>(md);
}

// Waits for a kernel's completion mark (the call number, its last store behind a system-wide fence) in a mapped
// result block: returns as soon as the results are on the host, several microseconds before a stream
// synchronisation would.  The stream is asked now and then so that a failed launch or a fault ends the wait
// with its error.  false: the stream went idle without the mark.
bool wait_for_mark(volatile const int64_t* mark, int64_t seq, cudaStream_t s, const char* what)
{
  for (unsigned spin = 1; *mark != seq; ++spin) {
    if ((spin & 0xFFFFu) == 0u) {
      const cudaError_t q = cudaStreamQuery(s);
      if (q == cudaSuccess) return *mark == seq;
      if (q != cudaErrorNotReady) throw CudaFail{std::string(what) + ": " + cudaGetErrorString(q)};
    }
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#endif
  }
  std::atomic_thread_fence(std::memory_order_acquire);
  return true;
}

int encode_host_small(gtk_tokenizer* h, const uint8_t* bytes, const int64_t* text_offsets, int64_t n_texts,
                      int64_t n_bytes, float* kernel_ms)
{
  std::memcpy(h->small_in_h + kSmallInOff, text_offsets, size_t(n_texts + 1) * 8);
  std::memcpy(h->small_in_h + kSmallInBytes, bytes, size_t(n_bytes));
  Plan p = plan_batch(h, h->small_in_d + kSmallInBytes, n_bytes,
                      reinterpret_cast<const int64_t*>(h->small_in_d + kSmallInOff), n_texts,
                      reinterpret_cast<int32_t*>(h->small_out_d + kSmallOutIds), gtk::kSmallMaxBytes,
                      reinterpret_cast<int64_t*>(h->small_out_d + kSmallOutChunk), false);
  p.b.text_id_off = reinterpret_cast<int64_t*>(h->small_out_d + kSmallOutText);
  p.b.totals      = reinterpret_cast<int64_t*>(h->small_out_d + kSmallOutTotals);
  h->d_text_off.reserve((size_t(gtk::kSmallMaxTexts) + 1) * 8);
  p.b.text_off_copy = h->d_text_off.as<int64_t>();
  h->d_chunk_id_off.reserve(size_t(kSmallChunkCap + 1) * 8);
  p.b.chunk_id_mirror = h->d_chunk_id_off.as<int64_t>();
  cudaStream_t s = h->stream;
  p.b.small_seq = ++h->small_seq;
  const int launches = gtk::launch_encode_small(p.b, h->dtab, s);
  GTK_CUDA(cudaGetLastError());
  // The kernel's last store is the call number, behind a system-wide fence: polling it in the mapped result block
  // returns as soon as the results are on the host, several microseconds before a stream synchronisation would.
  // The stream is asked now and then so that a failed launch or a fault ends the wait with its error.
  volatile const int64_t* tot = reinterpret_cast<volatile const int64_t*>(h->small_out_h + kSmallOutTotals);
  if (!wait_for_mark(tot + 3, p.b.small_seq, s, "small-batch kernel"))
    return h->fail(GTK_ERR_KERNEL, "small-batch kernel ended without publishing its results");
  if (tot[2] != gtk::kStatusOk) return h->fail(GTK_ERR_KERNEL, status_text(int(tot[2])));
  h->stage_ms[1] = h->stage_ms[4] = float(double(tot[4]) * 1e-6);  // the kernel's own globaltimer span
  h->last_launches = launches;
  h->result_is_small = true;
  h->res_n_chunks = tot[0];
  h->res_n_ids = tot[1];
  if (kernel_ms) *kernel_ms = h->stage_ms[4];
  return GTK_OK;
}

// Batches of up to 64 KiB and 1024 texts (GTK_MODE_OPT, 16-bit table): two launches.  The host lays out the chunk
// table (a few thousand entries at most) and sends it with zeroed counters and the text in ONE copy; the tile kernel
// runs as for any batch; one more kernel (a CTA per tile) does the scans and the pack and writes the results into
// mapped host memory, where the host polls the call number.  No chunker launch, no copy back, no synchronisation.
constexpr int64_t kTwoLaunchMaxBytes  = int64_t(gtk::kFinishMaxTiles / 2) * gtk::kTile;  // 64 KiB
constexpr int64_t kTwoLaunchMaxChunks = 4096;

// number of chunks of the batch, or -1 when it does not qualify for the two-launch path
int64_t two_launch_chunks(const gtk_tokenizer* h, int mode, const int64_t* text_offsets, int64_t n_texts, int64_t n_bytes)
{
  if (h->wide || mode != GTK_MODE_OPT || !h->mid_out_h || h->stage_timing) return -1;
  if (n_bytes > kTwoLaunchMaxBytes || n_texts > gtk::kSmallMaxTexts) return -1;
  const int64_t chunk = h->chunk_tokens;
  int64_t C = 0;
  for (int64_t t = 0; t < n_texts; ++t) C += (text_offsets[t + 1] - text_offsets[t] + chunk - 1) / chunk;
  return C <= kTwoLaunchMaxChunks ? C : -1;
}

int encode_host_two_launches(gtk_tokenizer* h, const uint8_t* bytes, const int64_t* text_offsets, int64_t n_texts,
                             int64_t n_bytes, int64_t C, float* kernel_ms)
{
  auto up = [](size_t x) { return (x + 63) & ~size_t(63); };
  const int64_t chunk = h->chunk_tokens;
  const int64_t K     = (n_bytes + gtk::kTile - 1) / gtk::kTile;
  const size_t o_cnt = 128, o_coff = up(o_cnt + size_t(C + 1) * 4), o_tile = up(o_coff + size_t(C + 1) * 8);
  const size_t o_tbase = up(o_tile + size_t(K) * 4), o_bytes = up(o_tbase + size_t(n_texts + 1) * 8);
  const size_t total = o_bytes + size_t(n_bytes) + 32;
  h->h_fast_in.reserve(total);
  h->d_fast_in.reserve(total);
  uint8_t* hp = static_cast<uint8_t*>(h->h_fast_in.p);
  std::memset(hp, 0, o_coff);  // totals, counters, per-chunk counts
  reinterpret_cast<int64_t*>(hp)[0] = C;
  int64_t* coff  = reinterpret_cast<int64_t*>(hp + o_coff);
  int64_t* tbase = reinterpret_cast<int64_t*>(hp + o_tbase);
  int64_t c = 0;
  for (int64_t t = 0; t < n_texts; ++t) {
    tbase[t] = c;
    for (int64_t pos = text_offsets[t]; pos < text_offsets[t + 1]; pos += chunk) coff[c++] = pos;
  }
  tbase[n_texts] = c;
  coff[c]        = n_bytes;
  int32_t* tile0 = reinterpret_cast<int32_t*>(hp + o_tile);
  for (int64_t k = 0, cc = 0; k < K; ++k) {  // last chunk that starts at or before the tile's first byte
    while (cc + 1 < C && coff[cc + 1] <= k * gtk::kTile) ++cc;
    tile0[k] = int32_t(cc);
  }
  std::memcpy(hp + o_bytes, bytes, size_t(n_bytes));
  std::memset(hp + o_bytes + n_bytes, 0, 32);
  cudaStream_t s = h->stream;
  uint8_t* dp = h->d_fast_in.as<uint8_t>();
  GTK_CUDA(cudaMemcpyAsync(dp, hp, total, cudaMemcpyHostToDevice, s));

  const size_t text_b = up(size_t(n_texts + 1) * 8), chunk_b = up(size_t(C + 1) * 8);
  uint8_t* md = h->mid_out_d;  // [64-byte header | text id offsets | chunk id offsets | ids]
  Plan p = plan_batch(h, dp + o_bytes, n_bytes, nullptr, n_texts, reinterpret_cast<int32_t*>(md + 64 + text_b + chunk_b),
                      n_bytes, reinterpret_cast<int64_t*>(md + 64 + text_b), false);
  p.b.text_id_off     = reinterpret_cast<int64_t*>(md + 64);
  p.b.totals          = reinterpret_cast<int64_t*>(dp);
  p.b.counters        = reinterpret_cast<int32_t*>(dp + 16);
  p.b.chunk_cnt       = reinterpret_cast<int32_t*>(dp + o_cnt);
  p.b.chunk_off       = reinterpret_cast<int64_t*>(dp + o_coff);
  p.b.tile_chunk0     = reinterpret_cast<int32_t*>(dp + o_tile);
  p.b.text_chunk_base = reinterpret_cast<int64_t*>(dp + o_tbase);
  h->d_chunk_id_off.reserve(size_t(kTwoLaunchMaxChunks + 1) * 8);
  p.b.chunk_id_mirror = h->d_chunk_id_off.as<int64_t>();  // the scan's own copy in HBM: the text offsets index it
  const int64_t seq = ++h->mid_seq;
  GTK_CUDA(cudaEventRecord(h->ev[0], s));
  int launches = gtk::launch_merge_opt(p.b, h->dtab, h->opt_grid, s);
  launches += gtk::launch_finish_small_batch(p.b, reinterpret_cast<int64_t*>(md), seq, s);
  GTK_CUDA(cudaEventRecord(h->ev[4], s));
  GTK_CUDA(cudaGetLastError());
  volatile const int64_t* tot = reinterpret_cast<volatile const int64_t*>(h->mid_out_h);
  if (!wait_for_mark(tot + 3, seq, s, "finish kernel"))
    return h->fail(GTK_ERR_KERNEL, "finish kernel ended without publishing its results");
  if (tot[2] != gtk::kStatusOk) return h->fail(GTK_ERR_KERNEL, status_text(int(tot[2])));
  if (tot[0] != C || tot[1] > n_bytes) return h->fail(GTK_ERR_KERNEL, "inconsistent totals");
  GTK_CUDA(cudaEventSynchronize(h->ev[4]));  // completes a moment after the mark
  GTK_CUDA(cudaEventElapsedTime(&h->stage_ms[4], h->ev[0], h->ev[4]));
  h->result_is_packed = true;
  h->pack_base        = h->mid_out_h + 64;
  h->pack_text_bytes  = text_b;
  h->pack_chunk_bytes = chunk_b;
  h->last_launches    = launches;
  h->res_n_chunks     = C;
  h->res_n_ids        = tot[1];
  if (kernel_ms) *kernel_ms = h->stage_ms[4];
  return GTK_OK;
}

// frees every device / pinned buffer, stream and event of a handle (also used when gtk_create fails half way)
void release_handle(gtk_tokenizer* h)
{
  if (h->device >= 0) {
    cudaSetDevice(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    for (DevBuf* b : {&h->d_bpi, &h->d_slots, &h->d_overflow, &h->d_bpr, &h->d_mor, &h->d_sor, &h->d_adj, &h->d_b2i, &h->d_words, &h->d_low_map, &h->d_wide_slots, &h->d_staging32, &h->d_seg_scratch32, &h->d_bytes, &h->d_text_off,
                      &h->d_text_chunk_base, &h->d_chunk_off, &h->d_tile_chunk0, &h->d_staging, &h->d_unit_first,
                      &h->d_unit_cnt, &h->d_chunk_cnt, &h->d_unit_base, &h->d_chunk_id_off, &h->d_text_id_off,
                      &h->d_out_ids, &h->d_seg_scratch, &h->d_scan_sums, &h->d_totals, &h->d_out_pack, &h->d_fast_in})
      b->release();
    for (PinBuf* b : {&h->h_ids, &h->h_text_id_off, &h->h_chunk_id_off, &h->h_totals, &h->h_piece_off, &h->h_piece_id_off, &h->h_chunk_id_all, &h->h_out_pack, &h->h_fast_in}) b->release();
    for (DevBuf* b : {&h->d_piece_off, &h->d_piece_id_off, &h->d_chunk_id_all}) b->release();
    if (h->small_in_h) cudaFreeHost(h->small_in_h);
    if (h->small_out_h) cudaFreeHost(h->small_out_h);
    if (h->mid_out_h) cudaFreeHost(h->mid_out_h);
    for (auto& sl : h->slice) sl.release();
    if (h->in_stream) cudaStreamDestroy(h->in_stream);
    if (h->out_stream) cudaStreamDestroy(h->out_stream);
    if (h->pack_stream) cudaStreamDestroy(h->pack_stream);
    for (auto& ev : h->ev)
      if (ev) cudaEventDestroy(ev);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
  }
}

int validate_offsets(gtk_tokenizer* h, const int64_t* text_offsets, int64_t n_texts)
{
  if (n_texts < 0) return h->fail(GTK_ERR_INVALID_ARG, "n_texts must be >= 0");
  if (n_texts > 0 && !text_offsets) return h->fail(GTK_ERR_INVALID_ARG, "text_offsets is null");
  if (n_texts > 0 && text_offsets[0] != 0) return h->fail(GTK_ERR_INVALID_ARG, "text_offsets[0] must be 0");
  for (int64_t t = 0; t < n_texts; ++t)
    if (text_offsets[t + 1] < text_offsets[t]) return h->fail(GTK_ERR_INVALID_ARG, "text_offsets must be non-decreasing");
  return GTK_OK;
}

}  // namespace

namespace gtk {
bool handle_view(gtk_tokenizer* h, HandleView* out)
{
  if (!h || !out) return false;
  out->device = h->device;
  out->stream = h->stream;
  out->table = h->dtab;
  out->wide = h->wide;
  out->low_id_map = (h->device >= 0 && h->id_space == GTK_IDS_GPT2) ? h->d_low_map.as<uint16_t>() : nullptr;
  out->pinned_words = h->device >= 0 ? h->h_totals.as<int32_t>() + 8 : nullptr;
  out->mu = &h->mu;
  out->last_error = &h->last_error;
  return true;
}
}  // namespace gtk

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------

extern "C" {

GTK_API const char* gtk_version(void) { return "gputok_b200 0.1 (sm_100a)"; }

GTK_API const char* gtk_global_error(void) { return g_global_error.c_str(); }

GTK_API int gtk_create(const char* merges_path, int chunk_tokens, int max_iters, int device, gtk_tokenizer** out)
{
  if (!out) {
    g_global_error = "out is null";
    return GTK_ERR_INVALID_ARG;
  }
  *out = nullptr;
  if (!merges_path) {
    g_global_error = "merges_path is null";
    return GTK_ERR_INVALID_ARG;
  }
  if (chunk_tokens <= 0) {
    g_global_error = "chunk_tokens must be > 0";
    return GTK_ERR_INVALID_ARG;
  }
  if (max_iters <= 0) max_iters = 50;
  gtk_tokenizer* h = nullptr;
  try {
    h = new gtk_tokenizer();
    h->chunk_tokens = chunk_tokens;
    h->max_iters = max_iters;
    h->device = device;
    try {
      h->table.reset(new gtk::HostTable(merges_path));
    } catch (const std::runtime_error& e) {
      g_global_error = e.what();
      delete h;
      return GTK_ERR_IO;
    }
    if (device >= 0) {
      h->wide = !h->table->fits_u16;  // ids >= 65535 or ranks >= 65534: served by the 32-bit kernel
      int count = 0;
      cudaError_t e = cudaGetDeviceCount(&count);
      if (e != cudaSuccess || device >= count) {
        g_global_error = std::string("CUDA device ") + std::to_string(device) + " not available: " +
                         (e != cudaSuccess ? cudaGetErrorString(e) : "ordinal out of range");
        delete h;
        return GTK_ERR_NO_DEVICE;
      }
      GTK_CUDA(cudaSetDevice(device));
      GTK_CUDA(cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, device));
      GTK_CUDA(cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking));
      h->stream = h->own_stream;
      for (auto& ev : h->ev) GTK_CUDA(cudaEventCreate(&ev));
      upload_table(h);
      h->opt_grid = h->sm_count * std::max(1, gtk::opt_kernel_max_blocks_per_sm());
      h->base_grid = h->sm_count * std::max(1, gtk::base_kernel_max_blocks_per_sm(chunk_tokens, 0));
      h->localmin_grid = h->sm_count * std::max(1, gtk::localmin_kernel_max_blocks_per_sm());
      h->wide_grid = h->sm_count * std::max(1, gtk::wide_kernel_max_blocks_per_sm());
      h->h_totals.reserve(64);
      small_path_init(h);
    }
    *out = h;
    return GTK_OK;
  } catch (const CudaFail& f) {
    g_global_error = f.what;
    if (h) release_handle(h);
    delete h;
    return GTK_ERR_CUDA;
  } catch (const std::bad_alloc&) {
    g_global_error = "out of host memory";
    if (h) release_handle(h);
    delete h;
    return GTK_ERR_INVALID_ARG;
  }
}

GTK_API void gtk_destroy(gtk_tokenizer* h)
{
  if (!h) return;
  release_handle(h);
  delete h;
}

GTK_API const char* gtk_last_error(const gtk_tokenizer* h) { return h ? h->last_error.c_str() : "null handle"; }

GTK_API int gtk_table_info_get(const gtk_tokenizer* h, gtk_table_info* out)
{
  if (!h || !out) return GTK_ERR_INVALID_ARG;
  const gtk::HostTable& t = *h->table;
  out->vocab_size = int32_t(t.id_to_symbols.size());
  out->num_merges = int32_t(t.rows.size());
  out->max_rank = t.max_rank;
  out->hash_capacity = uint32_t(t.pair_buckets.size() * 4);
  out->hash_overflow_entries = t.pair_overflow_count;
  out->hash_bytes = uint32_t(t.pair_buckets.size() * sizeof(gtk::PairBucket) + t.pair_overflow.size() * sizeof(gtk::PairSlot));
  out->monotone = t.monotone;
  out->merged_is_256_plus_rank = t.merged_is_256_plus_rank;
  out->byte_ids_identity = t.byte_ids_identity;
  out->adj_bigrams = t.adj_count;
  out->chunk_tokens = h->chunk_tokens;
  out->max_iters = h->max_iters;
  out->device = h->device;
  out->sm_count = h->sm_count;
  out->whole_segment_entries = int32_t(t.word_count);
  out->whole_segment_dropped = t.word_dropped;
  return GTK_OK;
}

GTK_API int gtk_encode_device(gtk_tokenizer* h, int mode, const uint8_t* d_bytes, int64_t n_bytes,
                              const int64_t* d_text_offsets, int64_t n_texts, int32_t* d_out_ids,
                              int64_t out_capacity, int64_t* d_out_chunk_offsets, int64_t chunk_capacity,
                              int64_t* n_ids, int64_t* n_chunks, float* kernel_ms)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(h->mu);
  if (h->device < 0) return h->fail(GTK_ERR_NO_DEVICE, "host-only handle: no GPU entry points");
  if (mode != GTK_MODE_OPT && mode != GTK_MODE_BASE && mode != GTK_MODE_LOCALMIN) return h->fail(GTK_ERR_INVALID_ARG, "unknown mode");
  if (n_bytes < 0 || n_texts < 0) return h->fail(GTK_ERR_INVALID_ARG, "negative size");
  if (n_ids) *n_ids = 0;
  if (n_chunks) *n_chunks = 0;
  if (kernel_ms) *kernel_ms = 0.f;
  h->last_launches = 0;
  std::fill(h->stage_ms, h->stage_ms + 5, 0.f);
  h->front_ms = -1.f;
  if (n_texts == 0 || n_bytes == 0) return GTK_OK;
  if (!d_bytes || !d_text_offsets || !d_out_ids) return h->fail(GTK_ERR_INVALID_ARG, "null device pointer");
  if (h->wide && mode == GTK_MODE_LOCALMIN) return h->fail(GTK_ERR_TABLE, kWideNoLocalmin);
  try {
    GTK_CUDA(cudaSetDevice(h->device));
    const int64_t need_chunks = chunk_upper_bound(n_bytes, n_texts, h->chunk_tokens);
    int64_t* chunk_dst = d_out_chunk_offsets;
    if (chunk_dst && chunk_capacity < need_chunks + 1) chunk_dst = nullptr;  // scan into the arena, copy what fits
    Plan p = plan_batch(h, d_bytes, n_bytes, d_text_offsets, n_texts, d_out_ids, out_capacity, chunk_dst, false);
    int launches = 0;
    // When the chunk offsets are scanned straight into the caller's buffer (or not wanted), the pack follows
    // the front without a host round trip: the pack kernel itself never writes past out_capacity, and the
    // totals are checked once at the end.
    const bool one_sync = !d_out_chunk_offsets || chunk_dst;
    run_front(h, p.b, mode, &launches, nullptr, nullptr, nullptr, one_sync);
    if (one_sync) run_pack(h, p.b, mode, &launches, nullptr, nullptr, true);
    GTK_CUDA(cudaStreamSynchronize(h->stream));
    const int64_t* ht = h->h_totals.as<int64_t>();
    const int64_t C = ht[0], N = ht[1];
    const int status = reinterpret_cast<const int32_t*>(ht + 2)[1];
    if (status != gtk::kStatusOk) return h->fail(GTK_ERR_KERNEL, status_text(status));
    if (N > out_capacity) return h->fail(GTK_ERR_CAPACITY, "d_out_ids too small: need " + std::to_string(N) + " ids");
    if (one_sync) {
      collect_stage_times(h, true);
      h->last_launches = launches;
      if (n_ids) *n_ids = N;
      if (n_chunks) *n_chunks = C;
      if (kernel_ms) *kernel_ms = h->stage_ms[4];
      return GTK_OK;
    }
    if (d_out_chunk_offsets && !chunk_dst) {
      if (chunk_capacity < C + 1)
        return h->fail(GTK_ERR_CAPACITY, "d_out_chunk_offsets too small: need " + std::to_string(C + 1));
      GTK_CUDA(cudaMemcpyAsync(d_out_chunk_offsets, p.b.chunk_id_off, size_t(C + 1) * 8, cudaMemcpyDeviceToDevice,
                               h->stream));
    }
    run_pack(h, p.b, mode, &launches);
    GTK_CUDA(cudaStreamSynchronize(h->stream));
    collect_stage_times(h);
    h->last_launches = launches;
    if (n_ids) *n_ids = N;
    if (n_chunks) *n_chunks = C;
    if (kernel_ms) *kernel_ms = h->stage_ms[4];
    return GTK_OK;
  } catch (const CudaFail& f) {
    return h->fail(GTK_ERR_CUDA, f.what);
  }
}

GTK_API int gtk_encode(gtk_tokenizer* h, int mode, const uint8_t* bytes, const int64_t* text_offsets,
                       int64_t n_texts, float* kernel_ms)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(h->mu);
  if (h->device < 0) return h->fail(GTK_ERR_NO_DEVICE, "host-only handle: no GPU entry points");
  if (mode != GTK_MODE_OPT && mode != GTK_MODE_BASE && mode != GTK_MODE_LOCALMIN) return h->fail(GTK_ERR_INVALID_ARG, "unknown mode");
  if (int rc = validate_offsets(h, text_offsets, n_texts)) return rc;
  if (kernel_ms) *kernel_ms = 0.f;
  h->result_is_cpu = false;
  h->result_is_small = false;
  h->result_is_packed = false;
  h->res_n_ids = h->res_n_chunks = 0;
  h->res_n_texts = n_texts;
  h->last_launches = 0;
  std::fill(h->stage_ms, h->stage_ms + 5, 0.f);
  h->front_ms = -1.f;
  try {
    GTK_CUDA(cudaSetDevice(h->device));
    const int64_t n_bytes = n_texts ? text_offsets[n_texts] : 0;
    h->h_text_id_off.reserve(size_t(n_texts + 1) * 8);
    if (n_bytes == 0) {  // empty batch or only empty texts: ([], 0.0) in the reference
      std::memset(h->h_text_id_off.p, 0, size_t(n_texts + 1) * 8);
      h->h_chunk_id_off.reserve(8);
      h->h_chunk_id_off.as<int64_t>()[0] = 0;
      return GTK_OK;
    }
    if (!bytes) return h->fail(GTK_ERR_INVALID_ARG, "bytes is null");
    if (h->wide && mode == GTK_MODE_LOCALMIN) return h->fail(GTK_ERR_TABLE, kWideNoLocalmin);
    if (!h->wide && mode == GTK_MODE_OPT && n_bytes <= gtk::kSmallMaxBytes && n_texts <= gtk::kSmallMaxTexts)
      return encode_host_small(h, bytes, text_offsets, n_texts, n_bytes, kernel_ms);
    if (const int64_t C2 = two_launch_chunks(h, mode, text_offsets, n_texts, n_bytes); C2 >= 0)
      return encode_host_two_launches(h, bytes, text_offsets, n_texts, n_bytes, C2, kernel_ms);
    if (n_bytes >= kSliceThresholdBytes) return encode_host_sliced(h, mode, bytes, text_offsets, n_texts, n_bytes, kernel_ms);
    cudaStream_t s = h->stream;
    h->d_bytes.reserve(size_t(n_bytes) + 32);
    h->d_text_off.reserve(size_t(n_texts + 1) * 8);
    GTK_CUDA(cudaMemcpyAsync(h->d_bytes.p, bytes, size_t(n_bytes), cudaMemcpyHostToDevice, s));
    GTK_CUDA(cudaMemcpyAsync(h->d_text_off.p, text_offsets, size_t(n_texts + 1) * 8, cudaMemcpyHostToDevice, s));
    // Everything that goes back lives in one arena, [text id offsets | chunk id offsets | ids], each sized by its
    // bound (a batch of this path is below 8 MiB, so 4 bytes per input byte for the ids is little): the pack
    // follows the front without a host round trip and one copy brings the results.
    const size_t text_b  = ((size_t(n_texts) + 1) * 8 + 63) & ~size_t(63);
    const size_t chunk_b = ((size_t(chunk_upper_bound(n_bytes, n_texts, h->chunk_tokens)) + 1) * 8 + 63) & ~size_t(63);
    h->d_out_pack.reserve(text_b + chunk_b + size_t(n_bytes) * 4 + 64);
    uint8_t* dp = h->d_out_pack.as<uint8_t>();
    Plan p = plan_batch(h, h->d_bytes.as<uint8_t>(), n_bytes, h->d_text_off.as<int64_t>(), n_texts,
                        reinterpret_cast<int32_t*>(dp + text_b + chunk_b), n_bytes,
                        reinterpret_cast<int64_t*>(dp + text_b), true);
    p.b.text_id_off = reinterpret_cast<int64_t*>(dp);
    int launches = 0;
    // Up to 256 KiB of text a kernel behind the pack writes the results into mapped host memory and the host polls
    // its completion mark: no copy of the totals, no second copy sized by them, no stream synchronisation.
    const bool by_kernel = h->mid_out_h != nullptr && n_bytes <= kResultsByKernelMaxBytes &&
                           64 + text_b + chunk_b + size_t(n_bytes) * 4 + 64 <= kMappedResultBytes;
    run_front(h, p.b, mode, &launches, nullptr, nullptr, nullptr, true);
    run_pack(h, p.b, mode, &launches, nullptr, nullptr, true, !by_kernel);
    int64_t C = 0, N = 0;
    int status = gtk::kStatusOk;
    if (by_kernel) {
      const int64_t seq = ++h->mid_seq;
      launches += gtk::launch_results_to_host(p.b, dp, h->mid_out_d + 64, int64_t(text_b + chunk_b),
                                              reinterpret_cast<int64_t*>(h->mid_out_d), seq, s);
      GTK_CUDA(cudaGetLastError());
      volatile const int64_t* tot = reinterpret_cast<volatile const int64_t*>(h->mid_out_h);
      if (!wait_for_mark(tot + 3, seq, s, "result kernel"))
        return h->fail(GTK_ERR_KERNEL, "result kernel ended without publishing its results");
      C = tot[0], N = tot[1], status = int(tot[2]);
      h->pack_base = h->mid_out_h + 64;
    } else {
      GTK_CUDA(cudaStreamSynchronize(s));
      const int64_t* ht = h->h_totals.as<int64_t>();
      C = ht[0], N = ht[1];
      status = reinterpret_cast<const int32_t*>(ht + 2)[1];
    }
    if (status != gtk::kStatusOk) return h->fail(GTK_ERR_KERNEL, status_text(status));
    if (N > n_bytes) return h->fail(GTK_ERR_KERNEL, "more ids than input bytes");
    if (!by_kernel) {
      h->h_out_pack.reserve(text_b + chunk_b + size_t(N) * 4 + 64);
      GTK_CUDA(cudaMemcpyAsync(h->h_out_pack.p, dp, text_b + chunk_b + size_t(N) * 4, cudaMemcpyDeviceToHost, s));
      GTK_CUDA(cudaStreamSynchronize(s));
      h->pack_base = h->h_out_pack.as<uint8_t>();
    }
    collect_stage_times(h, true);
    h->result_is_packed = true;
    h->pack_text_bytes  = text_b;
    h->pack_chunk_bytes = chunk_b;
    h->last_launches = launches;
    h->res_n_ids = N;
    h->res_n_chunks = C;
    if (kernel_ms) *kernel_ms = h->stage_ms[4];
    return GTK_OK;
  } catch (const CudaFail& f) {
    return h->fail(GTK_ERR_CUDA, f.what);
  }
}

GTK_API int gtk_encode_cpu(gtk_tokenizer* h, int rule, const uint8_t* bytes, const int64_t* text_offsets,
                           int64_t n_texts)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(h->mu);
  if (rule != GTK_RULE_GREEDY && rule != GTK_RULE_LOCALMIN) return h->fail(GTK_ERR_INVALID_ARG, "unknown rule");
  if (int rc = validate_offsets(h, text_offsets, n_texts)) return rc;
  if (n_texts > 0 && text_offsets[n_texts] > 0 && !bytes) return h->fail(GTK_ERR_INVALID_ARG, "bytes is null");
  h->cpu_ids.clear();
  h->cpu_text_off.assign(1, 0);
  h->cpu_chunk_off.assign(1, 0);
  for (int64_t t = 0; t < n_texts; ++t) {
    const int64_t s = text_offsets[t], e = text_offsets[t + 1];
    if (rule == GTK_RULE_LOCALMIN) {
      if (e > s) {
        h->table->localmin_text(bytes + s, e - s, h->max_iters, h->cpu_ids);
        h->cpu_chunk_off.push_back(int64_t(h->cpu_ids.size()));
      }
    } else {
      for (int64_t pos = s; pos < e; pos += h->chunk_tokens) {
        const int64_t len = std::min<int64_t>(h->chunk_tokens, e - pos);
        h->table->greedy_chunk(bytes + pos, len, h->cpu_ids);
        h->cpu_chunk_off.push_back(int64_t(h->cpu_ids.size()));
      }
    }
    h->cpu_text_off.push_back(int64_t(h->cpu_ids.size()));
  }
  h->result_is_cpu = true;
  h->result_is_small = false;
  h->result_is_packed = false;
  h->res_n_ids = int64_t(h->cpu_ids.size());
  h->res_n_chunks = int64_t(h->cpu_chunk_off.size()) - 1;
  h->res_n_texts = n_texts;
  return GTK_OK;
}

GTK_API int gtk_result_sizes(const gtk_tokenizer* h, int64_t* n_ids, int64_t* n_chunks, int64_t* n_texts)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  if (n_ids) *n_ids = h->res_n_ids;
  if (n_chunks) *n_chunks = h->res_n_chunks;
  if (n_texts) *n_texts = h->res_n_texts;
  return GTK_OK;
}

GTK_API int gtk_result_view(const gtk_tokenizer* h, const int32_t** ids, const int64_t** text_id_offsets,
                            const int64_t** chunk_id_offsets)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  if (h->result_is_cpu) {
    if (ids) *ids = h->cpu_ids.data();
    if (text_id_offsets) *text_id_offsets = h->cpu_text_off.data();
    if (chunk_id_offsets) *chunk_id_offsets = h->cpu_chunk_off.data();
  } else if (h->result_is_small) {
    if (ids) *ids = reinterpret_cast<const int32_t*>(h->small_out_h + kSmallOutIds);
    if (text_id_offsets) *text_id_offsets = reinterpret_cast<const int64_t*>(h->small_out_h + kSmallOutText);
    if (chunk_id_offsets) *chunk_id_offsets = reinterpret_cast<const int64_t*>(h->small_out_h + kSmallOutChunk);
  } else if (h->result_is_packed) {
    const uint8_t* base = h->pack_base;
    if (ids) *ids = reinterpret_cast<const int32_t*>(base + h->pack_text_bytes + h->pack_chunk_bytes);
    if (text_id_offsets) *text_id_offsets = reinterpret_cast<const int64_t*>(base);
    if (chunk_id_offsets) *chunk_id_offsets = reinterpret_cast<const int64_t*>(base + h->pack_text_bytes);
  } else {
    if (ids) *ids = h->h_ids.as<int32_t>();
    if (text_id_offsets) *text_id_offsets = h->h_text_id_off.as<int64_t>();
    if (chunk_id_offsets) *chunk_id_offsets = h->h_chunk_id_off.as<int64_t>();
  }
  return GTK_OK;
}

GTK_API int gtk_result_copy(const gtk_tokenizer* h, int32_t* ids, int64_t ids_capacity, int64_t* text_id_offsets,
                            int64_t* chunk_id_offsets, int64_t chunk_capacity)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  const int32_t* src_ids;
  const int64_t *src_text, *src_chunk;
  gtk_result_view(h, &src_ids, &src_text, &src_chunk);
  if (ids) {
    if (ids_capacity < h->res_n_ids) return h->fail(GTK_ERR_CAPACITY, "ids buffer too small");
    if (h->res_n_ids) std::memcpy(ids, src_ids, size_t(h->res_n_ids) * 4);
  }
  if (text_id_offsets && src_text) std::memcpy(text_id_offsets, src_text, size_t(h->res_n_texts + 1) * 8);
  if (chunk_id_offsets) {
    if (chunk_capacity < h->res_n_chunks + 1) return h->fail(GTK_ERR_CAPACITY, "chunk offset buffer too small");
    if (src_chunk) std::memcpy(chunk_id_offsets, src_chunk, size_t(h->res_n_chunks + 1) * 8);
  }
  return GTK_OK;
}

GTK_API int gtk_last_stage_ms(const gtk_tokenizer* h, float stage_ms[5], int32_t* kernel_launches)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  if (stage_ms) std::memcpy(stage_ms, h->stage_ms, sizeof(h->stage_ms));
  if (kernel_launches) *kernel_launches = h->last_launches;
  return GTK_OK;
}

GTK_API int gtk_decode(const gtk_tokenizer* h, const int32_t* ids, int64_t n_ids, uint8_t* out, int64_t out_capacity,
                       int64_t* n_out)
{
  if (!h || (n_ids > 0 && !ids)) return GTK_ERR_INVALID_ARG;
  const gtk::HostTable& t = *h->table;
  int64_t k = 0;
  for (int64_t i = 0; i < n_ids; ++i) {
    const int32_t id = ids[i];
    if (id < 0 || size_t(id) >= t.id_to_bytes.size() || !t.decodable[size_t(id)])
      return h->fail(GTK_ERR_INVALID_ARG, "id " + std::to_string(id) + " has no byte string");
    const std::string& s = t.id_to_bytes[size_t(id)];
    if (out) {
      if (k + int64_t(s.size()) > out_capacity) return h->fail(GTK_ERR_CAPACITY, "decode buffer too small");
      std::memcpy(out + k, s.data(), s.size());
    }
    k += int64_t(s.size());
  }
  if (n_out) *n_out = k;
  return GTK_OK;
}

GTK_API int32_t gtk_token_symbols(const gtk_tokenizer* h, int32_t id, char* buf, int32_t capacity)
{
  if (!h || id < 0 || size_t(id) >= h->table->id_to_symbols.size()) return -1;
  const std::string& s = h->table->id_to_symbols[size_t(id)];
  if (buf && capacity >= int32_t(s.size())) std::memcpy(buf, s.data(), s.size());
  return int32_t(s.size());
}

GTK_API int gtk_set_stream(gtk_tokenizer* h, void* cuda_stream)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(h->mu);
  if (h->device < 0) return h->fail(GTK_ERR_NO_DEVICE, "host-only handle: no GPU entry points");
  cudaSetDevice(h->device);
  cudaStreamSynchronize(h->stream);
  h->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : h->own_stream;
  return GTK_OK;
}

GTK_API int gtk_set_stage_timing(gtk_tokenizer* h, int per_stage)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(h->mu);
  h->stage_timing = per_stage != 0;
  return GTK_OK;
}

GTK_API int gtk_set_base_block_size(gtk_tokenizer* h, int threads)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(h->mu);
  if (h->device < 0) return h->fail(GTK_ERR_NO_DEVICE, "host-only handle: no GPU entry points");
  if (threads != 0 && threads != 64 && threads != 128 && threads != 256 && threads != 512 && threads != 1024)
    return h->fail(GTK_ERR_INVALID_ARG, "block size must be 0 (automatic), 64, 128, 256, 512 or 1024");
  try {
    GTK_CUDA(cudaSetDevice(h->device));
    h->base_block = threads;
    h->base_grid  = h->sm_count * std::max(1, gtk::base_kernel_max_blocks_per_sm(h->chunk_tokens, threads));
    GTK_CUDA(cudaGetLastError());
  } catch (const CudaFail& f) {
    return h->fail(GTK_ERR_CUDA, f.what);
  }
  return GTK_OK;
}

GTK_API int gtk_set_id_space(gtk_tokenizer* h, int id_space)
{
  if (!h) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(h->mu);
  if (id_space != GTK_IDS_REFERENCE && id_space != GTK_IDS_GPT2) return h->fail(GTK_ERR_INVALID_ARG, "unknown id space");
  h->id_space = id_space;
  return GTK_OK;
}

GTK_API int gtk_write_token_strings(const gtk_tokenizer* h, const char* path, const int32_t* ids,
                                    const int64_t* chunk_id_offsets, int64_t n_chunks)
{
  if (!h || !path || n_chunks < 0 || (n_chunks > 0 && (!ids || !chunk_id_offsets))) return GTK_ERR_INVALID_ARG;
  FILE* f = std::fopen(path, "wb");
  if (!f) return h->fail(GTK_ERR_IO, std::string("Failed to open output file for writing: ") + path);
  const auto& sym = h->table->id_to_symbols;
  std::string line;
  for (int64_t c = 0; c < n_chunks; ++c) {
    line.clear();
    for (int64_t i = chunk_id_offsets[c]; i < chunk_id_offsets[c + 1]; ++i) {
      const int32_t id = ids[i];
      if (id < 0 || size_t(id) >= sym.size()) line += std::to_string(id);  // raw id, as the reference's fallback
      else line += sym[size_t(id)];
      if (i + 1 < chunk_id_offsets[c + 1]) line += ' ';
    }
    line += '\n';
    std::fwrite(line.data(), 1, line.size(), f);
  }
  std::fclose(f);
  return GTK_OK;
}

GTK_API void* gtk_pinned_alloc(size_t bytes)
{
  void* p = nullptr;
  if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) return nullptr;
  return p;
}

GTK_API void gtk_pinned_free(void* p)
{
  if (p) cudaFreeHost(p);
}

}  // extern "C"
