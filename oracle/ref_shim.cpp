// ref_shim.cpp -- C-ABI wrapper around the REFERENCE's own host functions.
//
// TEST INFRASTRUCTURE ONLY.  This file is never compiled on its own: the
// Makefile beside it pipes the reference's host-only line ranges
// (gputok_blockbpe.cu: includes, ByteEncoder, BPEVocab, build_vocab_and_merges,
// bpe_merge_cpu_greedy, encode_text_to_tokens; gputok_binding.cu: bpe_merge_cpu)
// straight from the reference tree into the compiler, followed by this file,
// and writes only the resulting shared object to oracle/_ref/.  No reference
// source text is stored in this repository.
//
// The wrapper adds nothing to the algorithm: it owns the reference objects,
// splits the byte buffer into the caller's chunks, calls the reference
// functions per chunk (optionally from several std::threads, one chunk per
// task) and packs the results.
#include <atomic>
#include <cstring>
#include <thread>

struct RefHandle {
  ByteEncoder enc;
  BPEVocab    vocab;
};

extern "C" {

__attribute__((visibility("default"))) void* ref_create(const char* merges_path, char* err, int errlen)
{
  try {
    auto* h = new RefHandle();
    build_vocab_and_merges(merges_path, h->vocab, h->enc);
    return h;
  } catch (std::exception const& ex) {
    if (err && errlen > 0) std::snprintf(err, static_cast<size_t>(errlen), "%s", ex.what());
    return nullptr;
  }
}

__attribute__((visibility("default"))) void ref_destroy(void* p) { delete static_cast<RefHandle*>(p); }

__attribute__((visibility("default"))) int32_t ref_vocab_size(void* p)
{
  return static_cast<int32_t>(static_cast<RefHandle*>(p)->vocab.id_to_token.size());
}

__attribute__((visibility("default"))) int64_t ref_num_pairs(void* p)
{
  return static_cast<int64_t>(static_cast<RefHandle*>(p)->vocab.cpu_pairs.size());
}

__attribute__((visibility("default"))) int ref_pair_lookup(void* p, int32_t a, int32_t b, uint32_t* rank,
                                                           int32_t* new_token)
{
  auto& m = static_cast<RefHandle*>(p)->vocab.cpu_pairs;
  auto it = m.find(pack_pair(a, b));
  if (it == m.end()) return 0;
  *rank      = it->second.rank;
  *new_token = it->second.new_token;
  return 1;
}

__attribute__((visibility("default"))) int64_t ref_dump_pairs(void* p, int32_t* rows, int64_t max_rows)
{
  auto& m   = static_cast<RefHandle*>(p)->vocab.cpu_pairs;
  int64_t k = 0;
  for (auto const& kv : m) {
    if (k >= max_rows) break;
    rows[4 * k + 0] = static_cast<int32_t>(kv.first >> 32);
    rows[4 * k + 1] = static_cast<int32_t>(kv.first & 0xFFFFFFFFu);
    rows[4 * k + 2] = static_cast<int32_t>(kv.second.rank);
    rows[4 * k + 3] = kv.second.new_token;
    ++k;
  }
  return k;
}

__attribute__((visibility("default"))) int32_t ref_token_symbols(void* p, int32_t id, char* buf, int32_t cap)
{
  auto& v = static_cast<RefHandle*>(p)->vocab.id_to_token;
  if (id < 0 || static_cast<size_t>(id) >= v.size()) return -1;
  int32_t n = static_cast<int32_t>(v[id].size());
  if (buf && cap >= n) std::memcpy(buf, v[id].data(), static_cast<size_t>(n));
  return n;
}

// mode 0: bpe_merge_cpu_greedy per chunk; mode 2: bpe_merge_cpu (local-min, max_iters) per chunk.
__attribute__((visibility("default"))) int64_t ref_encode_chunks(void* p, const uint8_t* bytes,
                                                                 const int64_t* chunk_off, int64_t n_chunks,
                                                                 int32_t* out_ids, int64_t* out_off, int mode,
                                                                 int max_iters, int n_threads)
{
  auto* h = static_cast<RefHandle*>(p);
  std::vector<std::vector<std::int32_t>> res(static_cast<size_t>(n_chunks > 0 ? n_chunks : 0));
  std::atomic<int64_t> next{0};
  auto work = [&]() {
    for (;;) {
      int64_t c = next.fetch_add(1);
      if (c >= n_chunks) break;
      std::string text(reinterpret_cast<const char*>(bytes) + chunk_off[c],
                       static_cast<size_t>(chunk_off[c + 1] - chunk_off[c]));
      auto tok = encode_text_to_tokens(text, h->enc, h->vocab);
      if (mode == 0) bpe_merge_cpu_greedy(tok, h->vocab.cpu_pairs);
      else bpe_merge_cpu(tok, h->vocab.cpu_pairs, max_iters);
      res[static_cast<size_t>(c)] = std::move(tok);
    }
  };
  if (n_threads <= 1) {
    work();
  } else {
    std::vector<std::thread> th;
    for (int t = 0; t < n_threads; ++t) th.emplace_back(work);
    for (auto& t : th) t.join();
  }
  int64_t k = 0;
  for (int64_t c = 0; c < n_chunks; ++c) {
    out_off[c] = k;
    auto& r    = res[static_cast<size_t>(c)];
    if (!r.empty()) std::memcpy(out_ids + k, r.data(), r.size() * sizeof(std::int32_t));
    k += static_cast<int64_t>(r.size());
  }
  out_off[n_chunks] = k;
  return k;
}

}  // extern "C"
