// gtk_table.cpp -- see gtk_table.hpp.
#include "gtk_table.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace gtk {

namespace {

// GPT-2 bytes_to_unicode (reference: ByteEncoder, gputok_blockbpe.cu:86-126):
// '!'..'~', 0xA1..0xAC and 0xAE..0xFF keep their code point, every other byte
// gets U+0100 + (its index among the remaining bytes).
void byte_symbol_codepoints(int cp_of_byte[256])
{
  int next = 0;
  for (int b = 0; b < 256; ++b) {
    bool keeps = (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
    cp_of_byte[b] = keeps ? b : 256 + next++;
  }
}

std::string utf8_of(int cp)
{
  std::string s;
  if (cp < 0x80) {
    s += char(cp);
  } else if (cp < 0x800) {
    s += char(0xC0 | (cp >> 6));
    s += char(0x80 | (cp & 0x3F));
  } else if (cp < 0x10000) {
    s += char(0xE0 | (cp >> 12));
    s += char(0x80 | ((cp >> 6) & 0x3F));
    s += char(0x80 | (cp & 0x3F));
  } else {
    s += char(0xF0 | (cp >> 18));
    s += char(0x80 | ((cp >> 12) & 0x3F));
    s += char(0x80 | ((cp >> 6) & 0x3F));
    s += char(0x80 | (cp & 0x3F));
  }
  return s;
}

// istream >> string field separators in the "C" locale
inline bool is_field_space(unsigned char c)
{
  return c == ' ' || c == '\t' || c == '\n' || c == '\v' || c == '\f' || c == '\r';
}

// symbol string -> raw bytes; false if a character is not a byte symbol
bool symbols_to_bytes(const std::string& sym, const std::unordered_map<int, int>& byte_of_cp, std::string& out)
{
  out.clear();
  size_t i = 0;
  while (i < sym.size()) {
    unsigned char c = (unsigned char)sym[i];
    int cp, len;
    if (c < 0x80) { cp = c; len = 1; }
    else if ((c & 0xE0) == 0xC0) { cp = c & 0x1F; len = 2; }
    else if ((c & 0xF0) == 0xE0) { cp = c & 0x0F; len = 3; }
    else if ((c & 0xF8) == 0xF0) { cp = c & 0x07; len = 4; }
    else return false;
    if (i + len > sym.size()) return false;
    for (int j = 1; j < len; ++j) {
      unsigned char cc = (unsigned char)sym[i + j];
      if ((cc & 0xC0) != 0x80) return false;
      cp = (cp << 6) | (cc & 0x3F);
    }
    auto it = byte_of_cp.find(cp);
    if (it == byte_of_cp.end()) return false;
    out += char(it->second);
    i += len;
  }
  return true;
}

}  // namespace

int32_t HostTable::add_token(const std::string& symbols)
{
  auto it = symbols_to_id.find(symbols);
  if (it != symbols_to_id.end()) return it->second;
  int32_t id = int32_t(id_to_symbols.size());
  id_to_symbols.push_back(symbols);
  symbols_to_id.emplace(symbols, id);
  return id;
}

HostTable::HostTable(const std::string& merges_path)
{
  int cp_of_byte[256];
  byte_symbol_codepoints(cp_of_byte);
  for (int b = 0; b < 256; ++b) byte_to_id[b] = uint16_t(add_token(utf8_of(cp_of_byte[b])));
  // GPT-2's vocabulary lists the byte symbols in bytes_to_unicode order: the 188 bytes that keep
  // their code point first (in byte order), then the 68 remapped bytes (in byte order).
  {
    int next_kept = 0, next_moved = 188;
    for (int b = 0; b < 256; ++b) {
      const bool keeps = cp_of_byte[b] == b;
      for (int id = 0; id < 256; ++id)
        if (byte_to_id[b] == id) gpt2_low_id[id] = uint16_t(keeps ? next_kept : next_moved);
      if (keeps) ++next_kept; else ++next_moved;
    }
  }

  FILE* f = std::fopen(merges_path.c_str(), "rb");
  if (!f) throw std::runtime_error("Failed to open merges file: " + merges_path);
  std::string data;
  {
    char buf[1 << 16];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof(buf), f)) > 0) data.append(buf, n);
    std::fclose(f);
  }
  if (data.empty()) throw std::runtime_error("Empty merges file");

  // Line 1 is a header.  Each later non-empty line with at least two
  // whitespace-separated fields is one merge; its rank is its index among such
  // lines (lines with fewer fields do not consume a rank).
  size_t pos = data.find('\n');
  pos = (pos == std::string::npos) ? data.size() : pos + 1;
  std::unordered_map<uint64_t, size_t> seen;
  uint32_t rank = 0;
  while (pos < data.size()) {
    size_t eol = data.find('\n', pos);
    if (eol == std::string::npos) eol = data.size();
    size_t i = pos;
    auto skip_space = [&] { while (i < eol && is_field_space((unsigned char)data[i])) ++i; };
    auto skip_field = [&] { while (i < eol && !is_field_space((unsigned char)data[i])) ++i; };
    skip_space();
    size_t a0 = i;
    skip_field();
    size_t a1 = i;
    skip_space();
    size_t b0 = i;
    skip_field();
    size_t b1 = i;
    pos = eol + 1;
    if (a1 == a0 || b1 == b0) continue;
    int32_t left = add_token(data.substr(a0, a1 - a0));
    int32_t right = add_token(data.substr(b0, b1 - b0));
    int32_t merged = add_token(id_to_symbols[left] + id_to_symbols[right]);
    uint64_t key = pair_key(uint32_t(left), uint32_t(right));
    if (seen.emplace(key, rows.size()).second) rows.push_back({left, right, rank, merged});  // first entry wins
    ++rank;
  }
  build_hash();
  build_derived();
  build_words();
  if (fits_u16) verify_device_tables();
}

void HostTable::build_hash()
{
  log2_capacity = 10;
  while ((size_t(1) << log2_capacity) < rows.size() * 2 + 1) ++log2_capacity;
  const uint32_t cap = 1u << log2_capacity, mask = cap - 1;
  HashSlot empty{0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
  slots.assign(cap, empty);
  max_probe = 0;
  max_rank = 0;
  for (const MergeRow& r : rows) {
    uint64_t key = pair_key(uint32_t(r.left), uint32_t(r.right));
    uint32_t h = pair_hash(key, log2_capacity), d = 0;
    while (!(slots[h].key_lo == 0xFFFFFFFFu && slots[h].key_hi == 0xFFFFFFFFu)) { h = (h + 1) & mask; ++d; }
    slots[h] = {uint32_t(r.right), uint32_t(r.left), r.rank, uint32_t(r.merged)};
    max_probe = std::max(max_probe, d);
    max_rank = std::max(max_rank, r.rank);
  }
}

// A segment whose bytes equal a vocabulary string that the greedy rule collapses to that one id
// needs no merging at all.  The entries are checked here, one by one, with the same greedy routine
// that defines the result, so the shortcut cannot change any output.
void HostTable::build_words()
{
  std::vector<std::pair<std::string, int32_t>> words;
  std::vector<int32_t> out;
  for (size_t id = 0; id < id_to_bytes.size(); ++id) {
    const std::string& bs = id_to_bytes[id];
    if (!decodable[id] || bs.size() < 2 || bs.size() > size_t(kWordMaxBytes) || id >= 0xFFFFu) continue;
    out.clear();
    greedy_chunk(reinterpret_cast<const uint8_t*>(bs.data()), int64_t(bs.size()), out);
    if (out.size() == 1 && out[0] == int32_t(id)) words.emplace_back(bs, int32_t(id));
  }
  word_count = uint32_t(words.size());
  word_log2_capacity = 10;
  while ((size_t(1) << word_log2_capacity) < words.size() * 2 + 1) ++word_log2_capacity;
  word_slots.assign(size_t(1) << word_log2_capacity, WordSlot{0, 0, 0, 0});
  word_dropped = 0;
  auto home = [&](const WordSlot& w, int which) {
    const uint32_t m = word_mix(w.k0, w.k1, w.k2);
    return which ? word_hash_b(m, word_log2_capacity) : word_hash_a(m, word_log2_capacity);
  };
  for (auto& w : words) {
    uint32_t k[3] = {0, 0, 0};
    for (size_t i = 0; i < w.first.size(); ++i) k[i >> 2] |= uint32_t((unsigned char)w.first[i]) << (8 * (i & 3));
    WordSlot cur{k[0], k[1], k[2], (uint32_t(w.first.size()) << 16) | uint32_t(w.second)};
    // cuckoo insertion: take the first free choice, else evict from alternating choices
    bool placed = false;
    int which   = 0;
    for (int kick = 0; kick < 500 && !placed; ++kick) {
      const uint32_t ha = home(cur, 0), hb = home(cur, 1);
      if (word_slots[ha].meta == 0) { word_slots[ha] = cur; placed = true; break; }
      if (word_slots[hb].meta == 0) { word_slots[hb] = cur; placed = true; break; }
      const uint32_t at = which ? hb : ha;
      std::swap(cur, word_slots[at]);
      // the evicted entry must move to its other choice next
      which = (home(cur, 0) == at) ? 1 : 0;
    }
    if (!placed) ++word_dropped;  // `cur` (some entry) is left out: it only loses the shortcut
  }
}

void HostTable::build_pair_buckets()
{
  pair_buckets.assign(kPairBuckets, PairBucket{{0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu}});
  std::vector<PairSlot> spilled;
  for (const MergeRow& r : rows) {
    const uint32_t key = (uint32_t(r.left) << 16) | uint32_t(r.right);
    const uint32_t h   = key * kPairMul;
    PairBucket& b      = pair_buckets[h >> 16];
    int i = 0;
    while (i < 4 && b.w[i] != 0xFFFFFFFFu) ++i;
    if (i < 4) b.w[i] = (h << 16) | r.rank;
    else spilled.push_back(PairSlot{key, r.rank});
  }
  pair_overflow_count = uint32_t(spilled.size());
  pair_overflow.clear();
  if (!spilled.empty()) {
    size_t cap = 16;
    while (cap < spilled.size() * 4) cap <<= 1;
    pair_overflow.assign(cap, PairSlot{0xFFFFFFFFu, 0xFFFFFFFFu});
    for (const PairSlot& e : spilled) {
      size_t h = (e.key * 0x85EBCA77u) >> 7 & (cap - 1);
      while (pair_overflow[h].key != 0xFFFFFFFFu) h = (h + 1) & (cap - 1);
      pair_overflow[h] = e;
    }
  }
}

// The kernels' probe sequences, replayed on the host over the arrays that will be uploaded: every merge
// must come back with its rank, every placed string with its id.
void HostTable::verify_device_tables() const
{
  for (const MergeRow& r : rows) {
    const uint32_t key = (uint32_t(r.left) << 16) | uint32_t(r.right);
    const uint32_t h   = key * kPairMul;
    const PairBucket& b = pair_buckets[h >> 16];
    uint32_t got = 0xFFFFFFFFu;
    for (int i = 0; i < 4; ++i) got = std::min(got, b.w[i] ^ (h << 16));
    if (got >= kSelRank16 && b.w[3] != 0xFFFFFFFFu && !pair_overflow.empty()) {
      const size_t mask = pair_overflow.size() - 1;
      size_t at = ((key * 0x85EBCA77u) >> 7) & mask;
      for (size_t d = 0; d <= mask && pair_overflow[at].key != 0xFFFFFFFFu; ++d, at = (at + 1) & mask)
        if (pair_overflow[at].key == key) { got = pair_overflow[at].rank; break; }
    }
    if (got != r.rank) throw std::runtime_error("internal error: device pair table does not return a merge's rank");
  }
  uint32_t found = 0;
  for (const WordSlot& w : word_slots) {
    if (w.meta == 0) continue;
    const uint32_t m = word_mix(w.k0, w.k1, w.k2);
    const WordSlot& a = word_slots[word_hash_a(m, word_log2_capacity)];
    const WordSlot& c = word_slots[word_hash_b(m, word_log2_capacity)];
    const bool at_a = a.k0 == w.k0 && a.k1 == w.k1 && a.k2 == w.k2 && a.meta == w.meta;
    const bool at_c = c.k0 == w.k0 && c.k1 == w.k1 && c.k2 == w.k2 && c.meta == w.meta;
    if (!at_a && !at_c) throw std::runtime_error("internal error: whole-segment table entry is not at either of its slots");
    ++found;
  }
  if (found + word_dropped != word_count) throw std::runtime_error("internal error: whole-segment table lost entries");
}

bool HostTable::find(int32_t left, int32_t right, uint32_t* rank, int32_t* merged) const
{
  const uint32_t mask = (1u << log2_capacity) - 1;
  uint64_t key = pair_key(uint32_t(left), uint32_t(right));
  uint32_t h = pair_hash(key, log2_capacity);
  for (uint32_t d = 0; d <= max_probe; ++d) {
    const HashSlot& s = slots[h];
    if (s.key_lo == uint32_t(right) && s.key_hi == uint32_t(left)) {
      if (rank) *rank = s.rank;
      if (merged) *merged = int32_t(s.merged);
      return true;
    }
    if (s.key_lo == 0xFFFFFFFFu && s.key_hi == 0xFFFFFFFFu) return false;
    h = (h + 1) & mask;
  }
  return false;
}

void HostTable::build_derived()
{
  const size_t nt = id_to_symbols.size();
  // raw bytes of every token
  int cp_of_byte[256];
  byte_symbol_codepoints(cp_of_byte);
  std::unordered_map<int, int> byte_of_cp;
  for (int b = 0; b < 256; ++b) byte_of_cp[cp_of_byte[b]] = b;
  id_to_bytes.assign(nt, std::string());
  decodable.assign(nt, 0);
  for (size_t i = 0; i < nt; ++i) decodable[i] = symbols_to_bytes(id_to_symbols[i], byte_of_cp, id_to_bytes[i]);

  // dense byte-pair rank table
  byte_pair_rank.assign(65536, uint16_t(kNoRank16));
  merged_of_rank.assign(size_t(max_rank) + 1, 0xFFFFFFFFu);
  same_of_rank.assign(size_t(max_rank) + 1, 0);
  merged_is_256_plus_rank = !rows.empty();
  int32_t max_id = int32_t(nt) - 1;
  for (const MergeRow& r : rows) {
    merged_of_rank[r.rank] = uint32_t(r.merged);
    same_of_rank[r.rank] = (r.left == r.right);
    if (uint32_t(r.merged) != 256u + r.rank) merged_is_256_plus_rank = false;
  }
  fits_u16 = (max_id < int32_t(kDeadTok16)) && (max_rank < kSelRank16);
  byte_ids_identity = true;
  for (int b = 0; b < 256; ++b) byte_ids_identity = byte_ids_identity && (byte_to_id[b] == b);
  if (fits_u16) {
    build_pair_buckets();
    for (int u = 0; u < 256; ++u)
      for (int v = 0; v < 256; ++v) {
        uint32_t rk;
        if (find(byte_to_id[u], byte_to_id[v], &rk, nullptr)) byte_pair_rank[(u << 8) | v] = uint16_t(rk);
      }
  }

  // monotone: a merge outranks every merge that produces one of its parts, so
  // merging at the current minimum rank can never expose a lower rank.
  std::vector<int64_t> last_producer(nt, -1);
  for (const MergeRow& r : rows) last_producer[r.merged] = std::max<int64_t>(last_producer[r.merged], r.rank);
  monotone = true;
  for (const MergeRow& r : rows)
    if (int64_t(r.rank) <= last_producer[r.left] || int64_t(r.rank) <= last_producer[r.right]) monotone = false;

  // never-merge analysis: the boundary between bytes u,v can only disappear
  // if some merge result contains the bigram (u,v).  Undecodable merge results
  // cannot be reached from byte input and are ignored.
  std::memset(adj, 0, sizeof(adj));
  for (const MergeRow& r : rows) {
    if (!decodable[r.merged]) continue;
    const std::string& s = id_to_bytes[r.merged];
    for (size_t j = 0; j + 1 < s.size(); ++j) {
      uint32_t bit = (uint32_t((unsigned char)s[j]) << 8) | (unsigned char)s[j + 1];
      adj[bit >> 5] |= 1u << (bit & 31);
    }
  }
  adj_count = 0;
  for (uint32_t w : adj) adj_count += __builtin_popcount(w);
  // one lookup answers both "may this boundary ever merge" and "rank of this byte pair"
  byte_pair_info.assign(65536, uint16_t(0xFFFF));
  for (uint32_t bit = 0; bit < 65536; ++bit) {
    const bool inside = (adj[bit >> 5] >> (bit & 31)) & 1u;
    const uint16_t rk = byte_pair_rank[bit];
    if (rk != uint16_t(kNoRank16)) byte_pair_info[bit] = rk;  // a merge pair is inside its own result
    else if (inside) byte_pair_info[bit] = uint16_t(0xFFFE);
  }
}

// Greedy rule on one chunk.  The chunk is cut at never-merge boundaries (the
// pieces are independent, so the result equals the rule applied to the whole
// chunk); each piece keeps a rank per adjacent pair and, per step, merges the
// left-most pair of lowest rank and refreshes the two ranks next to it.
void HostTable::greedy_chunk(const uint8_t* bytes, int64_t n, std::vector<int32_t>& out) const
{
  std::vector<int32_t> tok;
  std::vector<uint32_t> rk;
  int64_t s = 0;
  while (s < n) {
    int64_t e = s + 1;
    while (e < n && can_merge_across(bytes[e - 1], bytes[e])) ++e;
    const size_t len0 = size_t(e - s);
    tok.resize(len0);
    rk.assign(len0, 0xFFFFFFFFu);
    for (size_t i = 0; i < len0; ++i) tok[i] = byte_to_id[bytes[s + int64_t(i)]];
    for (size_t i = 0; i + 1 < len0; ++i) {
      uint32_t r;
      if (find(tok[i], tok[i + 1], &r, nullptr)) rk[i] = r;
    }
    size_t len = len0;
    for (;;) {
      uint32_t best = 0xFFFFFFFFu;
      size_t at = 0;
      for (size_t i = 0; i + 1 < len; ++i)
        if (rk[i] < best) { best = rk[i]; at = i; }
      if (best == 0xFFFFFFFFu) break;
      int32_t merged = 0;
      find(tok[at], tok[at + 1], nullptr, &merged);
      tok[at] = merged;
      tok.erase(tok.begin() + at + 1);
      rk.erase(rk.begin() + at + 1);
      --len;
      uint32_t r;
      rk[at] = (at + 1 < len && find(tok[at], tok[at + 1], &r, nullptr)) ? r : 0xFFFFFFFFu;
      if (at > 0) rk[at - 1] = find(tok[at - 1], tok[at], &r, nullptr) ? r : 0xFFFFFFFFu;
    }
    out.insert(out.end(), tok.begin(), tok.begin() + len);
    s = e;
  }
}

// Local-minimum rule of the reference's tokenize_batch_cpu
// (bpe_merge_cpu, gputok_binding.cu:200-270): per pass, a mergeable pair is
// merged unless its left neighbour ranks strictly lower or its right neighbour
// ranks lower or equal; at most max_iters passes.
void HostTable::localmin_text(const uint8_t* bytes, int64_t n, int max_iters, std::vector<int32_t>& out) const
{
  std::vector<int32_t> tok, next;
  tok.resize(size_t(n));
  for (int64_t i = 0; i < n; ++i) tok[size_t(i)] = byte_to_id[bytes[i]];
  std::vector<uint32_t> rk;
  for (int pass = 0; pass < max_iters && tok.size() >= 2; ++pass) {
    const size_t len = tok.size();
    rk.assign(len - 1, 0xFFFFFFFFu);
    for (size_t i = 0; i + 1 < len; ++i) {
      uint32_t r;
      if (find(tok[i], tok[i + 1], &r, nullptr)) rk[i] = r;
    }
    next.clear();
    bool any = false;
    size_t i = 0;
    while (i < len) {
      bool here = false;
      if (i + 1 < len && rk[i] != 0xFFFFFFFFu) {
        here = !(i > 0 && rk[i - 1] < rk[i]) && !(i + 2 < len && rk[i + 1] <= rk[i]);
      }
      if (here) {
        int32_t merged = 0;
        find(tok[i], tok[i + 1], nullptr, &merged);
        next.push_back(merged);
        i += 2;
        any = true;
      } else {
        next.push_back(tok[i++]);
      }
    }
    if (!any) break;
    tok.swap(next);
  }
  out.insert(out.end(), tok.begin(), tok.end());
}

}  // namespace gtk
