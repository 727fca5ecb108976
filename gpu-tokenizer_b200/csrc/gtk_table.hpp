// gtk_table.hpp -- host side of the merge table: byte encoder, merges.txt
// parser, vocabulary, and the flat arrays the kernels read from HBM.
//
// Behaviour follows the reference's ByteEncoder / BPEVocab /
// build_vocab_and_merges (gputok_blockbpe.cu:64-236); the data layout is new:
// an open-addressing table with 16-byte slots for host lookups, and for the
// kernels a bucketed pair table answered by one 128-bit load, a dense 256x256
// table for byte pairs, per-rank merged ids, a never-merge bigram bitmap and a
// two-choice cuckoo table of vocabulary strings that are their own tokenisation.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace gtk {

constexpr uint32_t kNoRank16 = 0xFFFFu;  // "pair not mergeable" in the 16-bit rank arrays
constexpr uint32_t kSelRank16 = 0xFFFEu; // transient "selected for this pass" marker
constexpr uint32_t kDeadTok16 = 0xFFFFu; // tombstone in the 16-bit token arrays
constexpr uint64_t kEmptyKey = 0xFFFFFFFFFFFFFFFFull;

// One slot of the device hash table: 64-bit (left,right) key, 32-bit rank,
// 32-bit merged id.  16 bytes so a probe is a single 128-bit load.
struct alignas(16) HashSlot {
  uint32_t key_lo;  // right id
  uint32_t key_hi;  // left id
  uint32_t rank;
  uint32_t merged;
};

// Device form of the pair table when ids and ranks fit 16 bits.  key = left << 16 | right; h = key * kPairMul is a
// bijection on 32 bits, so inside bucket (h >> 16) the low 16 bits of h identify the key exactly.  A bucket is
// four 32-bit words (low16(h) << 16 | rank), filled front to back, 0xFFFFFFFF = empty: one 128-bit load answers
// a probe, found or not.  Keys whose bucket already holds four entries go to a small open-addressing overflow
// table of {key, rank} (empty = all ones), looked at only when the home bucket is full and has no match.
constexpr uint32_t kPairMul = 0x9E3779B1u;
constexpr uint32_t kPairBuckets = 65536;
struct alignas(16) PairBucket {
  uint32_t w[4];
};
struct alignas(8) PairSlot {
  uint32_t key;
  uint32_t rank;
};

// One slot of the whole-segment table: a byte string of 2..12 bytes (zero padded to three
// words) whose greedy tokenisation is the single id in `meta` (length << 16 | id); meta 0 = empty.
struct alignas(16) WordSlot {
  uint32_t k0, k1, k2;
  uint32_t meta;
};
constexpr int kWordMaxBytes = 12;

// The whole-segment table is a two-choice cuckoo table: a string sits at word_hash_a or word_hash_b of its
// key, so a lookup is two independent 128-bit loads and no loop, found or not.
inline uint32_t word_mix(uint32_t k0, uint32_t k1, uint32_t k2)
{
  uint32_t h = (k0 * 0x9E3779B1u) ^ (k1 * 0x85EBCA77u) ^ (k2 * 0xC2B2AE3Du);
  h ^= h >> 15;
  return h * 0x2C1B3C6Du;
}
inline uint32_t word_hash_a(uint32_t m, uint32_t log2_capacity) { return m >> (32 - log2_capacity); }
inline uint32_t word_hash_b(uint32_t m, uint32_t log2_capacity)
{
  return ((m ^ (m >> 13)) * 0x165667B1u) >> (32 - log2_capacity);
}

struct MergeRow {
  int32_t  left, right;
  uint32_t rank;
  int32_t  merged;
};

inline uint64_t pair_key(uint32_t left, uint32_t right) { return (uint64_t(left) << 32) | uint64_t(right); }

// Hash shared by host and device (probe_rank in gtk_kernels.cu): the pair folded into 32 bits
// (exact for 16-bit ids), one 32-bit multiply, top bits.  Three integer instructions on the GPU.
inline uint32_t pair_hash(uint64_t key, uint32_t log2_capacity)
{
  const uint32_t left = uint32_t(key >> 32), right = uint32_t(key);
  return (((left << 16) ^ right) * 0x9E3779B1u) >> (32 - log2_capacity);
}

class HostTable {
 public:
  // Throws std::runtime_error for an unreadable / empty file (as the reference does).
  explicit HostTable(const std::string& merges_path);

  // vocabulary
  std::vector<std::string> id_to_symbols;               // token id -> GPT-2 symbol string
  std::unordered_map<std::string, int32_t> symbols_to_id;
  std::vector<std::string> id_to_bytes;                 // token id -> raw bytes ("" + !decodable if impossible)
  std::vector<uint8_t> decodable;
  uint16_t byte_to_id[256];
  uint16_t gpt2_low_id[256];  // id < 256 (reference id space) -> id of the same byte token in GPT-2's own vocabulary

  // merges, unique pairs in rank order
  std::vector<MergeRow> rows;
  uint32_t max_rank = 0;

  // flat arrays for the device
  std::vector<HashSlot> slots;
  std::vector<PairBucket> pair_buckets;    // device form (only when fits_u16)
  std::vector<PairSlot> pair_overflow;     // power-of-two capacity, or empty when nothing overflowed
  uint32_t pair_overflow_count = 0;
  uint32_t log2_capacity = 0;
  uint32_t max_probe = 0;                  // longest displacement of a stored key
  std::vector<uint16_t> byte_pair_rank;    // [256*256], index (u<<8|v) on raw bytes, kNoRank16 if none
  std::vector<uint16_t> byte_pair_info;    // [256*256]: 0xFFFF bigram never inside a merge result (cut), 0xFFFE inside
                                           // one but not itself a merge, else the rank of the byte pair
  std::vector<uint32_t> merged_of_rank;    // [max_rank+1]
  std::vector<uint8_t> same_of_rank;       // [max_rank+1]: 1 if left == right
  uint32_t adj[2048];                      // bit (u<<8|v): bigram occurs inside a merge result
  int adj_count = 0;

  // whole-segment fast path: every vocabulary string of 2..12 bytes that the greedy rule turns
  // into exactly its own id (verified one by one with greedy_chunk at build time)
  std::vector<WordSlot> word_slots;
  uint32_t word_log2_capacity = 0;
  uint32_t word_count = 0;    // strings that qualify
  uint32_t word_dropped = 0;  // of those, not placed (they take the merge path instead)

  // properties the kernels rely on
  bool monotone = false;        // rank(m) > rank of every merge producing one of m's parts
  bool merged_is_256_plus_rank = false;
  bool byte_ids_identity = false;
  bool fits_u16 = false;        // ids < 0xFFFF and ranks < 0xFFFE

  // host lookup through the same hash layout the device uses
  bool find(int32_t left, int32_t right, uint32_t* rank, int32_t* merged) const;

  bool can_merge_across(uint8_t u, uint8_t v) const
  {
    uint32_t bit = (uint32_t(u) << 8) | v;
    return (adj[bit >> 5] >> (bit & 31)) & 1u;
  }

  // Host reference tokenizers (serve GpuTokenizer.tokenize_batch_cpu; never a fallback).
  // Greedy rule on one chunk of raw bytes; appends ids to out.
  void greedy_chunk(const uint8_t* bytes, int64_t n, std::vector<int32_t>& out) const;
  // The binding's local-minimum rule with a pass cap, on one text.
  void localmin_text(const uint8_t* bytes, int64_t n, int max_iters, std::vector<int32_t>& out) const;

 private:
  int32_t add_token(const std::string& symbols);
  void build_hash();
  void build_derived();
  void build_words();
  void build_pair_buckets();
  void verify_device_tables() const;
};

}  // namespace gtk
