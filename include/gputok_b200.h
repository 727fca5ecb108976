/*
 * gputok_b200.h -- C ABI of the B200-native greedy byte-level BPE tokenizer.
 *
 * This is the drop-in boundary for the reference's `GpuTokenizer` class
 * (gputok_binding.cu:650-1011, exported to Python at :1015-1065).  Every entry
 * point is `extern "C"`, takes plain pointers and sizes, returns an `int`
 * status (GTK_OK == 0) and never throws or exits; the message of the last
 * failure is available from gtk_last_error() / gtk_global_error().
 *
 * Semantics shared by all encode entry points (reference:
 * gputok_binding.cu:704-752, 823-836):
 *   - a batch is `n_texts` byte strings laid back to back in one buffer;
 *     text t is bytes[text_offsets[t] .. text_offsets[t+1]), text_offsets[0]
 *     must be 0 and the array non-decreasing;
 *   - every text is cut into chunks of `chunk_tokens` bytes (the last chunk of
 *     a text may be shorter, an empty text has no chunk); chunks are tokenised
 *     independently with the greedy rule (globally lowest merge rank, left-most
 *     occurrence, one merge at a time until no adjacent pair is mergeable:
 *     bpe_merge_cpu_greedy, gputok_blockbpe.cu:248-300);
 *   - token ids live in the reference's id space: ids 0..255 are the byte
 *     values, merge number r (0-based line of merges.txt after the header)
 *     creates id 256+r for a well-formed table (build_vocab_and_merges,
 *     gputok_blockbpe.cu:178-236);
 *   - the result is packed: all ids of the batch back to back in chunk order,
 *     int64 offsets per chunk and per text.
 */
#ifndef GPUTOK_B200_H
#define GPUTOK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define GTK_API __attribute__((visibility("default")))
#else
#define GTK_API
#endif

/* status codes */
enum {
  GTK_OK               = 0,
  GTK_ERR_INVALID_ARG  = 1, /* e.g. chunk_tokens <= 0 (std::invalid_argument, gputok_binding.cu:661-663) */
  GTK_ERR_IO           = 2, /* merges file unreadable or empty (std::runtime_error, :153-161) */
  GTK_ERR_CUDA         = 3, /* a CUDA runtime call failed (the reference prints and exit()s, :24-30) */
  GTK_ERR_CAPACITY     = 4, /* a caller-provided output buffer is too small */
  GTK_ERR_TABLE        = 5, /* the entry point does not serve this merge table (see gtk_create) */
  GTK_ERR_NO_DEVICE    = 6, /* GPU entry point called on a host-only handle */
  GTK_ERR_KERNEL       = 7  /* a kernel reported an internal inconsistency through its status word */
};

/* which merge kernel serves the call */
enum {
  GTK_MODE_OPT  = 0, /* GpuTokenizer::tokenize_batch               (gputok_binding.cu:704-846) */
  GTK_MODE_BASE = 1, /* GpuTokenizer::tokenize_batch_blockbpe_base (gputok_binding.cu:850-989) */
  GTK_MODE_LOCALMIN = 2 /* the reference's OTHER rule on the GPU: bpe_merge_kernel_optimized (gputok_binding.cu:290-414),
                           per chunk, at most max_iters passes; not greedy Algorithm 1 -- offered for timing and
                           behaviour comparisons with the reference's tokenize_batch only */
};

/* merge rule of the host reference entry point */
enum {
  GTK_RULE_GREEDY   = 0, /* bpe_merge_cpu_greedy, per chunk (gputok_blockbpe.cu:248-300) */
  GTK_RULE_LOCALMIN = 1  /* bpe_merge_cpu, whole text, max_iters passes (gputok_binding.cu:200-270, 992-1003) */
};

typedef struct gtk_tokenizer gtk_tokenizer;

typedef struct gtk_table_info {
  int32_t  vocab_size;       /* number of token ids (50 256 for GPT-2 merges.txt) */
  int32_t  num_merges;       /* distinct (left,right) pairs in the table */
  uint32_t max_rank;         /* highest rank present */
  uint32_t hash_capacity;    /* slots of the pair table: 65 536 buckets of four */
  uint32_t hash_overflow_entries; /* pairs whose bucket was full (side table, second load) */
  uint32_t hash_bytes;       /* bytes of the pair table in HBM */
  int32_t  monotone;         /* 1: every merge has a higher rank than the merges that create its parts */
  int32_t  merged_is_256_plus_rank; /* 1: merged id == 256 + rank for every merge */
  int32_t  byte_ids_identity;       /* 1: id of byte b == b for all 256 bytes */
  int32_t  adj_bigrams;      /* byte bigrams that occur inside at least one merge result */
  int32_t  chunk_tokens;
  int32_t  max_iters;
  int32_t  device;           /* CUDA device ordinal, -1 for a host-only handle */
  int32_t  sm_count;
  int32_t  whole_segment_entries;   /* vocabulary strings (2..12 bytes) answered by one table probe */
  uint32_t whole_segment_dropped; /* qualifying strings that found no place (they are merged instead) */
} gtk_table_info;

/* Library version string. */
GTK_API const char* gtk_version(void);

/* Message of the last failure that had no handle to attach to (gtk_create). Thread-local. */
GTK_API const char* gtk_global_error(void);

/* Replaces GpuTokenizer::GpuTokenizer(merges_path, chunk_tokens, max_iters)
 * (gputok_binding.cu:652-701): parses merges.txt, rebuilds the vocabulary,
 * builds the merge-rank hash table, the byte-pair rank table and the
 * never-merge bigram bitmap and uploads them to `device`.
 * chunk_tokens <= 0 -> GTK_ERR_INVALID_ARG; max_iters <= 0 -> 50 (as :664-666).
 * device == -1 builds a host-only handle: the GPU entry points then return
 * GTK_ERR_NO_DEVICE (there is no CPU fallback); gtk_encode_cpu still works.
 * Any merges file the reference accepts is accepted (it carries int32 ids and a 64-bit pair key,
 * gputok_blockbpe.cu:139-157).  The fast kernels hold ids and ranks in 16 bits; a table with ids
 * >= 65535 or ranks >= 65534 (beyond roughly 65 000 merges; GPT-2 has 50 000) is served, for both
 * GTK_MODE_OPT and GTK_MODE_BASE, by a 32-bit one-CTA-per-chunk kernel with the same results at
 * the speed of the literal design.  For such a table GTK_MODE_LOCALMIN and
 * gtk_encode_chunks_noalloc return GTK_ERR_TABLE. */
GTK_API int gtk_create(const char* merges_path, int chunk_tokens, int max_iters, int device,
                       gtk_tokenizer** out);

/* Replaces the destructor of GpuTokenizer (frees the table and all arenas). */
GTK_API void gtk_destroy(gtk_tokenizer* h);

GTK_API const char* gtk_last_error(const gtk_tokenizer* h);

GTK_API int gtk_table_info_get(const gtk_tokenizer* h, gtk_table_info* out);

/* Replaces tokenize_batch (mode GTK_MODE_OPT, gputok_binding.cu:704-846) and
 * tokenize_batch_blockbpe_base (mode GTK_MODE_BASE, :850-989) for HOST input.
 * Copies the batch to the device (fastest from pinned memory, see
 * gtk_pinned_alloc), runs chunker -> merge kernel -> output scan/pack, copies
 * ids and offsets back into pinned buffers owned by the handle.
 * *kernel_ms (optional) receives the device time of the kernel pipeline
 * (cudaEvent pair, as :790-805).  Results stay valid until the next call on
 * the handle; read them with gtk_result_sizes/_view/_copy.
 * An empty batch or a batch of empty texts is not an error: 0 ids, 0 chunks.
 * Small batches (up to 8 KiB and 1024 texts, GTK_MODE_OPT) run as one kernel that reads the text from and
 * writes the results to mapped page-locked memory; the call returns when the kernel's completion mark has
 * arrived there (its last store, behind a system-wide fence), which is when the results are complete -- the
 * stream may still be retiring the kernel for a few microseconds.  *kernel_ms is then the kernel's own
 * measurement of its duration. */
GTK_API int gtk_encode(gtk_tokenizer* h, int mode, const uint8_t* bytes, const int64_t* text_offsets,
                       int64_t n_texts, float* kernel_ms);

/* Replaces tokenize_batch_cpu (gputok_binding.cu:992-1003): host-only
 * reference tokenizer.  GTK_RULE_GREEDY (default of the Python surface) runs
 * the greedy rule per chunk; GTK_RULE_LOCALMIN reproduces the reference
 * method's own rule on the un-chunked text.  Never used as a fallback. */
GTK_API int gtk_encode_cpu(gtk_tokenizer* h, int rule, const uint8_t* bytes, const int64_t* text_offsets,
                           int64_t n_texts);

/* Sizes of the result of the last gtk_encode / gtk_encode_cpu. */
GTK_API int gtk_result_sizes(const gtk_tokenizer* h, int64_t* n_ids, int64_t* n_chunks, int64_t* n_texts);

/* Zero-copy view of the last result (replaces the unflatten loop,
 * gputok_binding.cu:823-836): ids[n_ids], text_id_offsets[n_texts+1]
 * (text t owns ids[text_id_offsets[t] .. text_id_offsets[t+1])),
 * chunk_id_offsets[n_chunks+1].  Pointers are owned by the handle. */
GTK_API int gtk_result_view(const gtk_tokenizer* h, const int32_t** ids, const int64_t** text_id_offsets,
                            const int64_t** chunk_id_offsets);

/* Copy of the last result into caller buffers (any of them may be NULL). */
GTK_API int gtk_result_copy(const gtk_tokenizer* h, int32_t* ids, int64_t ids_capacity,
                            int64_t* text_id_offsets, int64_t* chunk_id_offsets, int64_t chunk_capacity);

/* Device-resident variant of gtk_encode for callers that keep text and ids in
 * HBM (replaces the kernel launch section, gputok_binding.cu:790-805, together
 * with the host chunk/flatten loops :718-752 that now run on the device).
 * d_bytes (16-byte aligned for full speed), d_text_offsets[n_texts+1] (int64),
 * d_out_ids[out_capacity] and d_out_chunk_offsets[chunk_capacity] (>= number
 * of chunks + 1, may be NULL) are device pointers on the handle's device.
 * *n_ids / *n_chunks are host outputs.  Synchronous on return.  GTK_ERR_CAPACITY
 * if a buffer is too small: nothing is written past a capacity, what was
 * written before the error is unspecified. */
GTK_API int gtk_encode_device(gtk_tokenizer* h, int mode, const uint8_t* d_bytes, int64_t n_bytes,
                              const int64_t* d_text_offsets, int64_t n_texts, int32_t* d_out_ids,
                              int64_t out_capacity, int64_t* d_out_chunk_offsets, int64_t chunk_capacity,
                              int64_t* n_ids, int64_t* n_chunks, float* kernel_ms);

/* Device time of the stages of the last GPU encode, in milliseconds:
 * [0] chunker, [1] merge kernel, [2] output scans, [3] pack, [4] whole pipeline.
 * Also the number of kernels launched by that call (for launch accounting).
 * [4] is always measured (it is the kernel_ms the encode entry points return, the reference's one event pair,
 * gputok_binding.cu:790-805).  [0]..[3] are measured for batches that the host path cuts into slices, and for
 * batches that run in one piece only after gtk_set_stage_timing(h, 1); otherwise they are 0.  The events between
 * the stages cost a call of a few hundred KiB to a few MiB about a tenth of its time, which is why they are off
 * by default. */
GTK_API int gtk_last_stage_ms(const gtk_tokenizer* h, float stage_ms[5], int32_t* kernel_launches);
GTK_API int gtk_set_stage_timing(gtk_tokenizer* h, int per_stage);

/* ids -> bytes (inverse of the byte encoder + merges); the token-string writer
 * of gputok_blockbpe.cu:841-865 builds on this.  *n_out receives the byte count. */
GTK_API int gtk_decode(const gtk_tokenizer* h, const int32_t* ids, int64_t n_ids, uint8_t* out,
                       int64_t out_capacity, int64_t* n_out);

/* The symbol string the reference prints for a token (id_to_token,
 * gputok_blockbpe.cu:857).  Returns the length, -1 for an unknown id. */
GTK_API int32_t gtk_token_symbols(const gtk_tokenizer* h, int32_t id, char* buf, int32_t capacity);

/* Run all later GPU work of this handle on the caller's CUDA stream (a cudaStream_t passed as
 * void*).  NULL restores the handle's own stream, which is created non-blocking: work on it is NOT
 * ordered against the legacy default stream.  To run on the legacy default stream itself -- the
 * stream the reference always uses (gputok_binding.cu:794-799) and the one a framework reports as
 * handle 0 -- pass cudaStreamLegacy, i.e. (void*)0x1; cudaStreamPerThread is (void*)0x2.
 * Ordering contract of the device-pointer entry points (gtk_encode_device,
 * gtk_encode_chunks_noalloc): the kernels read d_bytes / offsets and write the outputs on the
 * handle's current stream; whatever produces the inputs or reuses the outputs must be ordered
 * against that stream (same stream, an event, or a synchronisation before the call).  The entry
 * points stay synchronous on return. */
GTK_API int gtk_set_stream(gtk_tokenizer* h, void* cuda_stream);

/* Threads per CTA of the one-CTA-per-chunk kernel (GTK_MODE_BASE).  Replaces the reference's compile-time
 * BLOCK_SIZE (gputok_blockbpe.cu:313-315, swept by profile_blockbpe_block_sizes.sh:9,22-25 over 128..1024):
 * 0 (default) = one warp per KiB of chunk, 64 / 128 / 256 / 512 / 1024 = that many threads whatever the chunk
 * size; anything else is GTK_ERR_INVALID_ARG.  Results never depend on it. */
GTK_API int gtk_set_base_block_size(gtk_tokenizer* h, int threads);

/* Id space of the ids returned by the GPU encode entry points (no counterpart in the reference,
 * whose ids 0..255 are the byte values -- a permutation of GPT-2's own ids for the byte tokens,
 * e.g. the space byte is 32 here and 220 in GPT-2's vocab.json; ids >= 256 coincide).
 *   GTK_IDS_REFERENCE (default)  ids as the reference produces them
 *   GTK_IDS_GPT2                 ids < 256 are remapped to their position in GPT-2's byte-symbol
 *                                order, so the ids can be fed to a GPT-2 model directly
 * gtk_decode / gtk_write_token_strings expect GTK_IDS_REFERENCE ids. */
enum { GTK_IDS_REFERENCE = 0, GTK_IDS_GPT2 = 1 };
GTK_API int gtk_set_id_space(gtk_tokenizer* h, int id_space);

/* Replaces the token-string writer of the standalone binary (gputok_blockbpe.cu:841-865): writes
 * the chunks' tokens as GPT-2 symbol strings, separated by one space, one chunk per line -- the
 * format of the reference's data/output/gpu_tokens_blockbpe.txt.  chunk_id_offsets[n_chunks+1]
 * delimits the chunks inside ids (as returned by gtk_result_view). */
GTK_API int gtk_write_token_strings(const gtk_tokenizer* h, const char* path, const int32_t* ids,
                                    const int64_t* chunk_id_offsets, int64_t n_chunks);

/* Longest chunk, in bytes, that gtk_encode_chunks_noalloc accepts. */
#define GTK_NOALLOC_MAX_CHUNK_BYTES 16384

/* No counterpart in the reference (which allocates five device buffers inside every call).
 *
 * For callers that must not allocate while they tokenise: code running inside a serving loop
 * with a frozen memory budget, under a framework whose caching allocator owns all of HBM, or
 * anywhere a cudaMalloc -- which synchronises the whole device -- would stall other streams.
 * Once the handle exists this call performs no cudaMalloc/cudaFree and calls no allocating
 * library routine: one kernel (the one-CTA-per-chunk greedy merge kernel) runs with its work
 * queue, status word and long-chunk workspace in a fixed array that is part of the library
 * image (8 MiB + 256 B of device memory on every GPU that loads the library, held until the
 * process exits).
 *
 *   d_bytes[n_bytes]              text on the handle's device
 *   d_chunk_offsets[n_chunks+1]   int64, on the device: chunk c is bytes[off[c] .. off[c+1]);
 *                                 non-decreasing, 0 <= off[c] <= n_bytes.  A chunk that breaks this is
 *                                 not touched (its count is 0) and the call returns GTK_ERR_INVALID_ARG
 *   max_chunk_bytes               the caller's bound on off[c+1]-off[c]; values above
 *                                 GTK_NOALLOC_MAX_CHUNK_BYTES are rejected with GTK_ERR_CAPACITY
 *                                 before anything is launched; a chunk that breaks the bound is
 *                                 reported as GTK_ERR_CAPACITY after the kernel (its count is 0)
 *   d_out_ids[n_bytes]            int32; the ids of chunk c start at d_out_ids[off[c]] (the layout
 *                                 of the reference kernel's d_tokens_out, gputok_blockbpe.cu:530-537)
 *   d_out_counts[n_chunks]        int32 ids produced per chunk
 * The ids follow gtk_set_id_space like those of the other GPU entry points.
 *
 * The first call on a device looks up the device address of the fixed array
 * (cudaGetSymbolAddress); make that first call before any stream capture.  All calls on a
 * device share the array, which keeps the previous call's contents: the queue and status words
 * are cleared at the start of every call, the workspace is fully rewritten per chunk.  Two calls
 * that overlap on the same GPU (different handles or streams) race on it -- serialise them.
 * Synchronous on return. */
GTK_API int gtk_encode_chunks_noalloc(gtk_tokenizer* h, const uint8_t* d_bytes, int64_t n_bytes,
                                      const int64_t* d_chunk_offsets, int64_t n_chunks, int32_t max_chunk_bytes,
                                      int32_t* d_out_ids, int32_t* d_out_counts);

/* Page-locked host memory for inputs (cudaHostAlloc / cudaFreeHost). */
GTK_API void* gtk_pinned_alloc(size_t bytes);
GTK_API void  gtk_pinned_free(void* p);

#ifdef __cplusplus
}
#endif
#endif /* GPUTOK_B200_H */
