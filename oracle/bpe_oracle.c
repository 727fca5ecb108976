/*
 * bpe_oracle.c -- CPU restatement of the reference's greedy byte-level BPE path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker for the CUDA
 * tokenizer: the test-suite, the smoke check and the benchmark's CPU-baseline
 * legs load it; the shipped library never does.
 *
 * Parity status: PINNED.  The restatement is checked (tests/test_oracle.py)
 *   - against the reference's committed output data/output/gpu_tokens_blockbpe.txt
 *     (348 chunks of 2048 bytes of data/input/pride_and_prejudice.txt), and
 *   - against the reference's own host functions compiled in place from
 *     gputok_blockbpe.cu (oracle/Makefile -> oracle/_ref/libref_greedy.so).
 *
 * Every function names the reference lines it follows (paths are relative to
 * the reference project root).  Plain C, no dependencies beyond libc/pthreads.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Byte encoder: gputok_blockbpe.cu:64-126 (codepoint_to_utf8, ByteEncoder).   */
/* 188 "printable" bytes map to the code point equal to the byte, the other   */
/* 68 bytes map, in increasing byte order, to U+0100, U+0101, ...             */
/* ------------------------------------------------------------------------- */

static int cp_to_utf8(int cp, char out[4])
{
  if (cp <= 0x7F) { out[0] = (char)cp; return 1; }
  if (cp <= 0x7FF) {
    out[0] = (char)(0xC0 | ((cp >> 6) & 0x1F));
    out[1] = (char)(0x80 | (cp & 0x3F));
    return 2;
  }
  if (cp <= 0xFFFF) {
    out[0] = (char)(0xE0 | ((cp >> 12) & 0x0F));
    out[1] = (char)(0x80 | ((cp >> 6) & 0x3F));
    out[2] = (char)(0x80 | (cp & 0x3F));
    return 3;
  }
  out[0] = (char)(0xF0 | ((cp >> 18) & 0x07));
  out[1] = (char)(0x80 | ((cp >> 12) & 0x3F));
  out[2] = (char)(0x80 | ((cp >> 6) & 0x3F));
  out[3] = (char)(0x80 | (cp & 0x3F));
  return 4;
}

static void byte_encoder_codepoints(int cp_of_byte[256])
{
  int printable[256];
  int n = 0;
  memset(printable, 0, sizeof(printable));
  for (int c = '!'; c <= '~'; ++c) printable[c] = 1;
  for (int c = 0xA1; c <= 0xAC; ++c) printable[c] = 1;
  for (int c = 0xAE; c <= 0xFF; ++c) printable[c] = 1;
  for (int b = 0; b < 256; ++b) {
    if (printable[b]) cp_of_byte[b] = b;
    else cp_of_byte[b] = 256 + n++;
  }
}

/* ------------------------------------------------------------------------- */
/* Vocabulary: gputok_blockbpe.cu:159-176 (BPEVocab::add_token).              */
/* token string -> id (first insertion wins), id -> token string.             */
/* ------------------------------------------------------------------------- */

typedef struct {
  char*    str;
  uint32_t len;
} tokstr_t;

typedef struct {
  tokstr_t* id_to_token;
  int32_t   n_tokens, cap_tokens;
  int32_t*  slots; /* open addressing over ids, -1 empty */
  uint32_t  slot_mask;
} vocab_t;

static uint64_t fnv1a(const char* s, uint32_t n)
{
  uint64_t h = 1469598103934665603ull;
  for (uint32_t i = 0; i < n; ++i) { h ^= (unsigned char)s[i]; h *= 1099511628211ull; }
  return h;
}

static void vocab_init(vocab_t* v)
{
  v->cap_tokens  = 1 << 16;
  v->n_tokens    = 0;
  v->id_to_token = (tokstr_t*)malloc(sizeof(tokstr_t) * (size_t)v->cap_tokens);
  v->slot_mask   = (1u << 18) - 1;
  v->slots       = (int32_t*)malloc(sizeof(int32_t) * ((size_t)v->slot_mask + 1));
  for (uint32_t i = 0; i <= v->slot_mask; ++i) v->slots[i] = -1;
}

static void vocab_rehash(vocab_t* v)
{
  uint32_t new_mask = v->slot_mask * 2 + 1;
  int32_t* ns       = (int32_t*)malloc(sizeof(int32_t) * ((size_t)new_mask + 1));
  for (uint32_t i = 0; i <= new_mask; ++i) ns[i] = -1;
  for (int32_t id = 0; id < v->n_tokens; ++id) {
    uint32_t h = (uint32_t)fnv1a(v->id_to_token[id].str, v->id_to_token[id].len) & new_mask;
    while (ns[h] >= 0) h = (h + 1) & new_mask;
    ns[h] = id;
  }
  free(v->slots);
  v->slots     = ns;
  v->slot_mask = new_mask;
}

static int32_t vocab_find(const vocab_t* v, const char* s, uint32_t n)
{
  uint32_t h = (uint32_t)fnv1a(s, n) & v->slot_mask;
  while (v->slots[h] >= 0) {
    const tokstr_t* t = &v->id_to_token[v->slots[h]];
    if (t->len == n && memcmp(t->str, s, n) == 0) return v->slots[h];
    h = (h + 1) & v->slot_mask;
  }
  return -1;
}

/* add_token: return the existing id of an equal string, else append. */
static int32_t vocab_add(vocab_t* v, const char* s, uint32_t n)
{
  int32_t id = vocab_find(v, s, n);
  if (id >= 0) return id;
  if (v->n_tokens == v->cap_tokens) {
    v->cap_tokens *= 2;
    v->id_to_token = (tokstr_t*)realloc(v->id_to_token, sizeof(tokstr_t) * (size_t)v->cap_tokens);
  }
  if ((uint32_t)v->n_tokens * 2 > v->slot_mask) vocab_rehash(v);
  id                     = v->n_tokens++;
  v->id_to_token[id].str = (char*)malloc(n ? n : 1);
  memcpy(v->id_to_token[id].str, s, n);
  v->id_to_token[id].len = n;
  uint32_t h             = (uint32_t)fnv1a(s, n) & v->slot_mask;
  while (v->slots[h] >= 0) h = (h + 1) & v->slot_mask;
  v->slots[h] = id;
  return id;
}

/* ------------------------------------------------------------------------- */
/* Pair map: gputok_blockbpe.cu:130-157 (PairInfo, pack_pair).                 */
/* key = uint32(a) << 32 | uint32(b); value = (rank, new_token).              */
/* emplace semantics: the first insertion of a key wins (:229).               */
/* ------------------------------------------------------------------------- */

typedef struct {
  uint64_t key;
  uint32_t rank;
  int32_t  new_token;
} pairslot_t;

#define PAIR_EMPTY 0xFFFFFFFFFFFFFFFFull

typedef struct {
  pairslot_t* slots;
  uint64_t    mask;
  uint64_t    count;
} pairmap_t;

static inline uint64_t pack_pair(int32_t a, int32_t b)
{
  return ((uint64_t)(uint32_t)a << 32) | (uint64_t)(uint32_t)b;
}

static inline uint64_t pair_hash(uint64_t k)
{
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  return k;
}

static void pairmap_init(pairmap_t* m, uint64_t expected)
{
  uint64_t cap = 1024;
  while (cap < expected * 4) cap <<= 1;
  m->mask  = cap - 1;
  m->count = 0;
  m->slots = (pairslot_t*)malloc(sizeof(pairslot_t) * cap);
  for (uint64_t i = 0; i < cap; ++i) m->slots[i].key = PAIR_EMPTY;
}

static const pairslot_t* pairmap_find(const pairmap_t* m, uint64_t key)
{
  uint64_t h = pair_hash(key) & m->mask;
  while (m->slots[h].key != PAIR_EMPTY) {
    if (m->slots[h].key == key) return &m->slots[h];
    h = (h + 1) & m->mask;
  }
  return NULL;
}

static void pairmap_grow(pairmap_t* m)
{
  pairmap_t n;
  pairmap_init(&n, m->count * 2);
  for (uint64_t i = 0; i <= m->mask; ++i) {
    if (m->slots[i].key == PAIR_EMPTY) continue;
    uint64_t h = pair_hash(m->slots[i].key) & n.mask;
    while (n.slots[h].key != PAIR_EMPTY) h = (h + 1) & n.mask;
    n.slots[h] = m->slots[i];
    n.count++;
  }
  free(m->slots);
  *m = n;
}

static void pairmap_emplace(pairmap_t* m, uint64_t key, uint32_t rank, int32_t new_token)
{
  if (pairmap_find(m, key)) return; /* first wins */
  if ((m->count + 1) * 2 > m->mask) pairmap_grow(m);
  uint64_t h = pair_hash(key) & m->mask;
  while (m->slots[h].key != PAIR_EMPTY) h = (h + 1) & m->mask;
  m->slots[h].key       = key;
  m->slots[h].rank      = rank;
  m->slots[h].new_token = new_token;
  m->count++;
}

/* ------------------------------------------------------------------------- */
/* The oracle object.                                                          */
/* ------------------------------------------------------------------------- */

typedef struct bpe_oracle {
  vocab_t   vocab;
  pairmap_t pairs;
  int       cp_of_byte[256];
  int32_t   id_of_byte[256]; /* encode_text_to_tokens: gputok_blockbpe.cu:557-573 */
  /* derived, used by the segmented variant and by the property tests */
  uint8_t*  tok_bytes;     /* raw bytes of every decodable token, concatenated */
  int64_t*  tok_bytes_off; /* [n_tokens+1]; an undecodable token has length 0 and tok_decodable 0 */
  uint8_t*  tok_decodable;
  uint32_t  adj[2048]; /* bit (u<<8|v): byte bigram (u,v) occurs inside a merge result */
} bpe_oracle;

static int is_stream_space(unsigned char c)
{
  /* std::istream >> std::string skips/stops at isspace() in the "C" locale */
  return c == ' ' || c == '\t' || c == '\n' || c == '\v' || c == '\f' || c == '\r';
}

/* decode a token's symbol string back to raw bytes; returns -1 if a symbol is
 * not one of the 256 byte-encoder symbols */
static int64_t decode_symbols(const bpe_oracle* o, const char* s, uint32_t n, uint8_t* out)
{
  static const int8_t inv_ready = 0;
  (void)inv_ready;
  int64_t k = 0;
  uint32_t i = 0;
  while (i < n) {
    unsigned char c = (unsigned char)s[i];
    int cp, len;
    if (c < 0x80) { cp = c; len = 1; }
    else if ((c & 0xE0) == 0xC0) { cp = c & 0x1F; len = 2; }
    else if ((c & 0xF0) == 0xE0) { cp = c & 0x0F; len = 3; }
    else if ((c & 0xF8) == 0xF0) { cp = c & 0x07; len = 4; }
    else return -1;
    if (i + (uint32_t)len > n) return -1;
    for (int j = 1; j < len; ++j) {
      unsigned char cc = (unsigned char)s[i + j];
      if ((cc & 0xC0) != 0x80) return -1;
      cp = (cp << 6) | (cc & 0x3F);
    }
    int b = -1;
    if (cp < 256 && o->cp_of_byte[cp] == cp) b = cp;
    else if (cp >= 256 && cp < 256 + 68) {
      for (int t = 0; t < 256; ++t)
        if (o->cp_of_byte[t] == cp) { b = t; break; }
    }
    if (b < 0) return -1;
    out[k++] = (uint8_t)b;
    i += (uint32_t)len;
  }
  return k;
}

static void build_derived(bpe_oracle* o)
{
  int32_t nt = o->vocab.n_tokens;
  size_t total = 0;
  for (int32_t i = 0; i < nt; ++i) total += o->vocab.id_to_token[i].len;
  o->tok_bytes     = (uint8_t*)malloc(total ? total : 1);
  o->tok_bytes_off = (int64_t*)malloc(sizeof(int64_t) * ((size_t)nt + 1));
  o->tok_decodable = (uint8_t*)malloc((size_t)nt ? (size_t)nt : 1);
  int64_t off = 0;
  for (int32_t i = 0; i < nt; ++i) {
    o->tok_bytes_off[i] = off;
    int64_t k = decode_symbols(o, o->vocab.id_to_token[i].str, o->vocab.id_to_token[i].len,
                               o->tok_bytes + off);
    o->tok_decodable[i] = (k >= 0);
    if (k > 0) off += k;
  }
  o->tok_bytes_off[nt] = off;
  /* never-merge analysis: a boundary between bytes u,v can only ever be merged
   * across if some merge result contains the bigram (u,v) */
  memset(o->adj, 0, sizeof(o->adj));
  for (uint64_t s = 0; s <= o->pairs.mask; ++s) {
    if (o->pairs.slots[s].key == PAIR_EMPTY) continue;
    int32_t id = o->pairs.slots[s].new_token;
    if (id < 0 || id >= nt || !o->tok_decodable[id]) continue;
    const uint8_t* p = o->tok_bytes + o->tok_bytes_off[id];
    int64_t len      = o->tok_bytes_off[id + 1] - o->tok_bytes_off[id];
    for (int64_t j = 0; j + 1 < len; ++j) {
      uint32_t bit = ((uint32_t)p[j] << 8) | p[j + 1];
      o->adj[bit >> 5] |= 1u << (bit & 31);
    }
  }
}

/* build_vocab_and_merges: gputok_blockbpe.cu:178-236.
 *  - ids 0..255 = byte-encoder symbols in byte order (:181-184)
 *  - first line of the file is skipped (:192-196), an unreadable file or a
 *    file without a first line is an error (:188-196)
 *  - empty lines and lines with fewer than two whitespace-separated fields are
 *    skipped WITHOUT consuming a rank (:200-205)
 *  - unknown components are appended to the vocabulary (:207-215)
 *  - merged string = concatenation, id via add_token (existing string keeps
 *    its id) (:221-222); pair map emplace keeps the first entry (:229)       */
ORACLE_API bpe_oracle* bpe_oracle_create(const char* merges_path, char* err, int errlen)
{
  FILE* f = fopen(merges_path, "rb");
  if (!f) {
    if (err) snprintf(err, (size_t)errlen, "Failed to open merges file: %s", merges_path);
    return NULL;
  }
  bpe_oracle* o = (bpe_oracle*)calloc(1, sizeof(bpe_oracle));
  vocab_init(&o->vocab);
  pairmap_init(&o->pairs, 1 << 16);
  byte_encoder_codepoints(o->cp_of_byte);
  for (int b = 0; b < 256; ++b) {
    char u[4];
    int n            = cp_to_utf8(o->cp_of_byte[b], u);
    o->id_of_byte[b] = vocab_add(&o->vocab, u, (uint32_t)n);
  }

  char*   line = NULL;
  size_t  cap  = 0;
  ssize_t n;
  n = getline(&line, &cap, f);
  if (n < 0) {
    if (err) snprintf(err, (size_t)errlen, "Empty merges file");
    fclose(f);
    free(line);
    /* leak of the small tables on this error path is accepted in test code */
    return NULL;
  }
  uint32_t rank = 0;
  char*    merged = NULL;
  size_t   merged_cap = 0;
  while ((n = getline(&line, &cap, f)) >= 0) {
    size_t len = (size_t)n;
    if (len && line[len - 1] == '\n') --len; /* std::getline strips the newline only */
    if (len == 0) continue;
    size_t i = 0;
    while (i < len && is_stream_space((unsigned char)line[i])) ++i;
    size_t a0 = i;
    while (i < len && !is_stream_space((unsigned char)line[i])) ++i;
    size_t a1 = i;
    while (i < len && is_stream_space((unsigned char)line[i])) ++i;
    size_t b0 = i;
    while (i < len && !is_stream_space((unsigned char)line[i])) ++i;
    size_t b1 = i;
    if (a1 == a0 || b1 == b0) continue;
    int32_t id_a = vocab_add(&o->vocab, line + a0, (uint32_t)(a1 - a0));
    int32_t id_b = vocab_add(&o->vocab, line + b0, (uint32_t)(b1 - b0));
    uint32_t la = o->vocab.id_to_token[id_a].len, lb = o->vocab.id_to_token[id_b].len;
    if (merged_cap < (size_t)la + lb + 1) {
      merged_cap = (size_t)la + lb + 64;
      merged     = (char*)realloc(merged, merged_cap);
    }
    memcpy(merged, o->vocab.id_to_token[id_a].str, la);
    memcpy(merged + la, o->vocab.id_to_token[id_b].str, lb);
    int32_t new_id = vocab_add(&o->vocab, merged, la + lb);
    pairmap_emplace(&o->pairs, pack_pair(id_a, id_b), rank, new_id);
    ++rank;
  }
  free(merged);
  free(line);
  fclose(f);
  build_derived(o);
  return o;
}

ORACLE_API void bpe_oracle_destroy(bpe_oracle* o)
{
  if (!o) return;
  for (int32_t i = 0; i < o->vocab.n_tokens; ++i) free(o->vocab.id_to_token[i].str);
  free(o->vocab.id_to_token);
  free(o->vocab.slots);
  free(o->pairs.slots);
  free(o->tok_bytes);
  free(o->tok_bytes_off);
  free(o->tok_decodable);
  free(o);
}

ORACLE_API int32_t bpe_oracle_vocab_size(const bpe_oracle* o) { return o->vocab.n_tokens; }
ORACLE_API int64_t bpe_oracle_num_pairs(const bpe_oracle* o) { return (int64_t)o->pairs.count; }
ORACLE_API int32_t bpe_oracle_byte_id(const bpe_oracle* o, int b) { return o->id_of_byte[b & 255]; }

ORACLE_API int bpe_oracle_pair_lookup(const bpe_oracle* o, int32_t a, int32_t b, uint32_t* rank,
                                      int32_t* new_token)
{
  const pairslot_t* s = pairmap_find(&o->pairs, pack_pair(a, b));
  if (!s) return 0;
  if (rank) *rank = s->rank;
  if (new_token) *new_token = s->new_token;
  return 1;
}

/* dump all pairs as (a, b, rank, new_token) rows; returns the number written */
ORACLE_API int64_t bpe_oracle_dump_pairs(const bpe_oracle* o, int32_t* rows, int64_t max_rows)
{
  int64_t k = 0;
  for (uint64_t s = 0; s <= o->pairs.mask && k < max_rows; ++s) {
    if (o->pairs.slots[s].key == PAIR_EMPTY) continue;
    rows[4 * k + 0] = (int32_t)(o->pairs.slots[s].key >> 32);
    rows[4 * k + 1] = (int32_t)(o->pairs.slots[s].key & 0xFFFFFFFFu);
    rows[4 * k + 2] = (int32_t)o->pairs.slots[s].rank;
    rows[4 * k + 3] = o->pairs.slots[s].new_token;
    ++k;
  }
  return k;
}

/* token symbol string (as the reference writes it, gputok_blockbpe.cu:852-858) */
ORACLE_API int32_t bpe_oracle_token_symbols(const bpe_oracle* o, int32_t id, char* buf, int32_t cap)
{
  if (id < 0 || id >= o->vocab.n_tokens) return -1;
  int32_t n = (int32_t)o->vocab.id_to_token[id].len;
  if (buf && cap >= n) memcpy(buf, o->vocab.id_to_token[id].str, (size_t)n);
  return n;
}

ORACLE_API int32_t bpe_oracle_token_id(const bpe_oracle* o, const char* symbols, int32_t n)
{
  return vocab_find(&o->vocab, symbols, (uint32_t)n);
}

/* raw bytes a token stands for; -1 if the token is not decodable */
ORACLE_API int32_t bpe_oracle_token_bytes(const bpe_oracle* o, int32_t id, uint8_t* buf, int32_t cap)
{
  if (id < 0 || id >= o->vocab.n_tokens || !o->tok_decodable[id]) return -1;
  int32_t n = (int32_t)(o->tok_bytes_off[id + 1] - o->tok_bytes_off[id]);
  if (buf && cap >= n) memcpy(buf, o->tok_bytes + o->tok_bytes_off[id], (size_t)n);
  return n;
}

/* ids -> bytes; returns the number of bytes, or -1 on an undecodable id / overflow */
ORACLE_API int64_t bpe_oracle_decode(const bpe_oracle* o, const int32_t* ids, int64_t n, uint8_t* out,
                                     int64_t cap)
{
  int64_t k = 0;
  for (int64_t i = 0; i < n; ++i) {
    int32_t id = ids[i];
    if (id < 0 || id >= o->vocab.n_tokens || !o->tok_decodable[id]) return -1;
    int64_t len = o->tok_bytes_off[id + 1] - o->tok_bytes_off[id];
    if (k + len > cap) return -1;
    memcpy(out + k, o->tok_bytes + o->tok_bytes_off[id], (size_t)len);
    k += len;
  }
  return k;
}

ORACLE_API void bpe_oracle_adj_bitmap(const bpe_oracle* o, uint32_t out[2048])
{
  memcpy(out, o->adj, sizeof(o->adj));
}

/* ------------------------------------------------------------------------- */
/* Algorithm 1, literal: bpe_merge_cpu_greedy, gputok_blockbpe.cu:248-300.     */
/* Each pass: scan all adjacent pairs, keep the strictly lowest rank (so the  */
/* left-most occurrence wins, :271), merge that single occurrence, repeat     */
/* until no adjacent pair is in the table.  In place; returns the new length. */
/* ------------------------------------------------------------------------- */
ORACLE_API int64_t bpe_oracle_greedy(const bpe_oracle* o, int32_t* tokens, int64_t n)
{
  while (n >= 2) {
    uint32_t best_rank = 0xFFFFFFFFu;
    int64_t  best_pos  = -1;
    int32_t  best_new  = 0;
    for (int64_t i = 0; i + 1 < n; ++i) {
      const pairslot_t* s = pairmap_find(&o->pairs, pack_pair(tokens[i], tokens[i + 1]));
      if (!s) continue;
      if (s->rank < best_rank) {
        best_rank = s->rank;
        best_pos  = i;
        best_new  = s->new_token;
      }
    }
    if (best_pos < 0) break;
    tokens[best_pos] = best_new;
    memmove(tokens + best_pos + 1, tokens + best_pos + 2, sizeof(int32_t) * (size_t)(n - best_pos - 2));
    --n;
  }
  return n;
}

/* The binding's other rule, bpe_merge_cpu, gputok_binding.cu:200-270: a
 * mergeable position is kept if its left neighbour's rank is not strictly
 * lower (:234) and its right neighbour's rank is strictly higher (:236); all
 * kept positions merge in the same pass; at most max_iters passes (:210).
 * NOT the greedy rule and never used as the parity target; provided so the
 * difference can be demonstrated in the tests. */
ORACLE_API int64_t bpe_oracle_localmin(const bpe_oracle* o, int32_t* tokens, int64_t n, int max_iters)
{
  if (n <= 0) return n;
  uint32_t* ranks = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)n);
  char*     here  = (char*)malloc((size_t)n);
  int32_t*  tmp   = (int32_t*)malloc(sizeof(int32_t) * (size_t)n);
  int changed = 1, iter = 0;
  while (changed && iter < max_iters) {
    if (n < 2) break;
    for (int64_t i = 0; i + 1 < n; ++i) {
      const pairslot_t* s = pairmap_find(&o->pairs, pack_pair(tokens[i], tokens[i + 1]));
      ranks[i]            = s ? s->rank : 0xFFFFFFFFu;
    }
    changed = 0;
    for (int64_t i = 0; i + 1 < n; ++i) {
      here[i]    = 0;
      uint32_t r = ranks[i];
      if (r == 0xFFFFFFFFu) continue;
      if (i > 0 && ranks[i - 1] < r) continue;
      if (i + 1 < n - 1 && ranks[i + 1] <= r) continue;
      here[i] = 1;
      changed = 1;
    }
    if (!changed) break;
    int64_t k = 0, i = 0;
    while (i < n) {
      if (i < n - 1 && here[i]) {
        const pairslot_t* s = pairmap_find(&o->pairs, pack_pair(tokens[i], tokens[i + 1]));
        tmp[k++]            = s->new_token;
        i += 2;
      } else {
        tmp[k++] = tokens[i++];
      }
    }
    memcpy(tokens, tmp, sizeof(int32_t) * (size_t)k);
    n = k;
    ++iter;
  }
  free(ranks);
  free(here);
  free(tmp);
  return n;
}

/* Segmented variant (the repo's own fast checker, NOT in the reference): cut
 * the chunk wherever the byte bigram across the boundary occurs in no merge
 * result, run the literal greedy loop on every piece, concatenate.  Proven
 * equal to the literal loop by tests/test_oracle.py on real and adversarial
 * inputs; used to check full-size configurations in seconds. */
static int64_t greedy_segmented(const bpe_oracle* o, const uint8_t* bytes, int64_t n, int32_t* out)
{
  int64_t k = 0, s = 0;
  while (s < n) {
    int64_t e = s + 1;
    while (e < n) {
      uint32_t bit = ((uint32_t)bytes[e - 1] << 8) | bytes[e];
      if (!((o->adj[bit >> 5] >> (bit & 31)) & 1)) break;
      ++e;
    }
    for (int64_t i = s; i < e; ++i) out[k + (i - s)] = o->id_of_byte[bytes[i]];
    k += bpe_oracle_greedy(o, out + k, e - s);
    s = e;
  }
  return k;
}

/* ------------------------------------------------------------------------- */
/* Chunked driver: mirrors the per-chunk loop of gputok_blockbpe.cu:722-729    */
/* (encode bytes -> ids, :557-573; greedy per chunk).  Output is packed:      */
/* out_ids holds the chunks' ids back to back, out_off[c]..out_off[c+1].      */
/* mode 0 = literal greedy, 1 = segmented greedy, 2 = local-min (max_iters).  */
/* Threads split the chunk list; each chunk is written to a private region    */
/* (worst case one id per byte) and compacted afterwards.                     */
/* ------------------------------------------------------------------------- */

typedef struct {
  const bpe_oracle* o;
  const uint8_t*    bytes;
  const int64_t*    chunk_off;
  int64_t           n_chunks;
  int32_t*          scratch; /* one id per input byte, addressed by byte offset - base */
  int64_t*          counts;
  int64_t           base;
  int               mode, max_iters;
  volatile int64_t* next;
} job_t;

static void* worker(void* arg)
{
  job_t* j = (job_t*)arg;
  for (;;) {
    int64_t c = __sync_fetch_and_add(j->next, 1);
    if (c >= j->n_chunks) break;
    int64_t s = j->chunk_off[c], e = j->chunk_off[c + 1];
    int32_t* dst = j->scratch + (s - j->base);
    if (j->mode == 1) {
      j->counts[c] = greedy_segmented(j->o, j->bytes + s, e - s, dst);
    } else {
      for (int64_t i = s; i < e; ++i) dst[i - s] = j->o->id_of_byte[j->bytes[i]];
      j->counts[c] = (j->mode == 0) ? bpe_oracle_greedy(j->o, dst, e - s)
                                    : bpe_oracle_localmin(j->o, dst, e - s, j->max_iters);
    }
  }
  return NULL;
}

ORACLE_API int64_t bpe_oracle_encode_chunks(const bpe_oracle* o, const uint8_t* bytes,
                                            const int64_t* chunk_off, int64_t n_chunks, int32_t* out_ids,
                                            int64_t* out_off, int mode, int max_iters, int n_threads)
{
  if (n_chunks <= 0) {
    if (out_off) out_off[0] = 0;
    return 0;
  }
  int64_t base = chunk_off[0], total = chunk_off[n_chunks] - base;
  int32_t* scratch = (int32_t*)malloc(sizeof(int32_t) * (size_t)(total ? total : 1));
  int64_t* counts  = (int64_t*)malloc(sizeof(int64_t) * (size_t)n_chunks);
  volatile int64_t next = 0;
  job_t job = {o, bytes, chunk_off, n_chunks, scratch, counts, base, mode, max_iters, &next};
  if (n_threads < 1) n_threads = 1;
  if (n_threads > 256) n_threads = 256;
  if (n_threads == 1) {
    worker(&job);
  } else {
    pthread_t th[256];
    for (int t = 0; t < n_threads; ++t) pthread_create(&th[t], NULL, worker, &job);
    for (int t = 0; t < n_threads; ++t) pthread_join(th[t], NULL);
  }
  int64_t k = 0;
  for (int64_t c = 0; c < n_chunks; ++c) {
    out_off[c] = k;
    memmove(out_ids + k, scratch + (chunk_off[c] - base), sizeof(int32_t) * (size_t)counts[c]);
    k += counts[c];
  }
  out_off[n_chunks] = k;
  free(scratch);
  free(counts);
  return k;
}
