/*
 * gtk_textgen.c -- seeded synthetic text for the tokenizer's tests and benchmark.
 *
 * The reference benchmarks on WikiText-103 and ships one novel as sample input;
 * neither a dataset download nor the reference tree is available where the
 * benchmark runs, so this generator stands in for them.  It is deterministic
 * in (seed, stream, mix): the CPU checkers and the GPU path always see the
 * same bytes.  CPU only, no dependencies beyond libc/libm/pthreads.
 *
 * Text model
 *   - lexicon: 20 000 lowercase ASCII words of length 1..12.  The 160 most
 *     frequent ranks are common English function words (fixed list, order
 *     shuffled by the seed inside groups of 16); every other word is derived
 *     from the seed as a concatenation of common English letter groups cut to
 *     a length drawn from a fixed histogram peaking at 4..6.
 *   - word choice: Zipf(s = 1.1) over ranks 1..20 000 (inverse-CDF lookup).
 *   - 10 % of words get an upper-case first letter; one of ". , ; : ! ?"
 *     follows a word with p = 0.08; words are separated by one space, or by a
 *     newline with p = 1/80.
 *   - mix GTK_MIX_STRESS additionally replaces 20 % of the words by 1..8
 *     multi-byte UTF-8 characters (class chosen uniformly: U+00C0..U+024F,
 *     U+4E00..U+9FFF, U+1F600..U+1F64F; character uniform inside the class)
 *     and turns 5 % of the word slots into a run of 8..256 copies of a space
 *     (half of the runs) or of one lowercase letter.
 *   - a text is a sequence of independent blocks; block b of a seed is
 *     generated from stream (seed, b) and cut to exactly block_bytes, so any
 *     block range can be produced on its own (each GPU rank generates only its
 *     shard) and by several threads.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GTK_TG_API __attribute__((visibility("default")))

#define LEX_WORDS 20000
#define MAX_WORD 12

enum { GTK_MIX_PLAIN = 0, GTK_MIX_STRESS = 1 };

typedef struct gtk_textgen {
  uint64_t seed;
  uint8_t  word[LEX_WORDS][MAX_WORD];
  uint8_t  word_len[LEX_WORDS];
  uint64_t cdf[LEX_WORDS]; /* cumulative Zipf mass scaled to 2^64-1 */
} gtk_textgen;

static inline uint64_t splitmix64(uint64_t* s)
{
  uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

static inline uint64_t stream_state(uint64_t seed, uint64_t stream)
{
  uint64_t s = seed * 0xD1342543DE82EF95ull + 0x2545F4914F6CDD1Dull;
  (void)splitmix64(&s);
  s ^= stream * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull;
  (void)splitmix64(&s);
  return s;
}

/* uniform integer in [0, n) */
static inline uint32_t rnd_below(uint64_t* s, uint32_t n)
{
  return (uint32_t)(((splitmix64(s) >> 32) * (uint64_t)n) >> 32);
}

/* true with probability num/den */
static inline int rnd_chance(uint64_t* s, uint32_t num, uint32_t den) { return rnd_below(s, den) < num; }

static const char* const FRAG[] = {
  "th", "he", "in", "er", "an", "re", "on", "at", "en", "nd", "ti", "es", "or", "te", "of", "ed",
  "is", "it", "al", "ar", "st", "to", "nt", "ng", "se", "ha", "as", "ou", "io", "le", "ve", "co",
  "me", "de", "hi", "ri", "ro", "ic", "ne", "ea", "ra", "ce", "li", "ch", "ll", "be", "ma", "si",
  "ing", "ion", "ent", "and", "the", "tio", "for", "ate", "ous", "ver", "con", "pro", "com", "ment",
  "a", "e", "i", "o", "u", "s", "t", "r", "n", "l", "d", "c", "m", "p", "b", "g", "w", "y", "f", "k", "v", "h",
  "x", "q", "z", "j"};
#define N_FRAG ((int)(sizeof(FRAG) / sizeof(FRAG[0])))

static const char* const COMMON[] = {
  "the", "of", "and", "to", "a", "in", "is", "that", "it", "was", "for", "on", "with", "he", "be", "as",
  "by", "at", "you", "are", "his", "had", "not", "this", "have", "from", "but", "which", "she", "they", "or", "an",
  "her", "were", "there", "we", "their", "been", "has", "will", "one", "all", "would", "can", "if", "who", "more", "when",
  "said", "do", "what", "about", "its", "so", "up", "into", "them", "no", "time", "only", "could", "new", "than", "some",
  "these", "other", "may", "then", "me", "my", "out", "first", "two", "also", "after", "did", "over", "such", "made", "any",
  "most", "people", "should", "very", "our", "like", "many", "him", "how", "before", "must", "through", "years", "where", "much", "your",
  "way", "well", "down", "because", "each", "just", "those", "now", "see", "between", "being", "under", "never", "same", "another", "know",
  "while", "last", "might", "us", "great", "old", "year", "off", "come", "since", "against", "go", "came", "right", "used", "take",
  "three", "states", "himself", "few", "house", "use", "during", "without", "again", "place", "around", "however", "home", "small", "found", "thought",
  "went", "say", "part", "once", "general", "high", "upon", "school", "every", "still", "world", "little", "long", "good", "own", "work"};
#define N_COMMON ((int)(sizeof(COMMON) / sizeof(COMMON[0])))

/* length histogram (per mille) for lengths 1..12 */
static const int LEN_PM[MAX_WORD] = {30, 90, 150, 170, 150, 120, 100, 70, 50, 35, 20, 15};

GTK_TG_API gtk_textgen* gtk_textgen_create(uint64_t seed)
{
  gtk_textgen* g = (gtk_textgen*)calloc(1, sizeof(gtk_textgen));
  if (!g) return NULL;
  g->seed    = seed;
  uint64_t s = stream_state(seed, 0xFFFFFFFFFFFFFF01ull);
  /* ranks 0..N_COMMON-1: the fixed list, shuffled inside groups of 16 */
  int order[N_COMMON];
  for (int k = 0; k < N_COMMON; ++k) order[k] = k;
  for (int g0 = 0; g0 < N_COMMON; g0 += 16) {
    for (int i = 15; i > 0; --i) {
      int j = (int)rnd_below(&s, (uint32_t)(i + 1));
      int t = order[g0 + i];
      order[g0 + i] = order[g0 + j];
      order[g0 + j] = t;
    }
  }
  for (int k = 0; k < N_COMMON; ++k) {
    const char* w = COMMON[order[k]];
    int len = (int)strlen(w);
    if (len > MAX_WORD) len = MAX_WORD;
    memcpy(g->word[k], w, (size_t)len);
    g->word_len[k] = (uint8_t)len;
  }
  for (int k = N_COMMON; k < LEX_WORDS; ++k) {
    int len;
    {
      int r = (int)rnd_below(&s, 1000), acc = 0;
      len = MAX_WORD;
      for (int l = 0; l < MAX_WORD; ++l) {
        acc += LEN_PM[l];
        if (r < acc) { len = l + 1; break; }
      }
    }
    int n = 0;
    while (n < len) {
      /* the first 62 groups (multi-letter) are drawn twice as often as single letters */
      int f = rnd_chance(&s, 2, 3) ? (int)rnd_below(&s, 62) : (int)rnd_below(&s, (uint32_t)N_FRAG);
      const char* fr = FRAG[f];
      for (int j = 0; fr[j] && n < len; ++j) g->word[k][n++] = (uint8_t)fr[j];
    }
    g->word_len[k] = (uint8_t)len;
  }
  /* Zipf(1.1) cumulative table */
  double total = 0.0;
  for (int k = 0; k < LEX_WORDS; ++k) total += pow((double)(k + 1), -1.1);
  double acc = 0.0;
  for (int k = 0; k < LEX_WORDS; ++k) {
    acc += pow((double)(k + 1), -1.1);
    double f  = acc / total;
    g->cdf[k] = (f >= 1.0) ? UINT64_MAX : (uint64_t)(f * 18446744073709551615.0);
  }
  g->cdf[LEX_WORDS - 1] = UINT64_MAX;
  return g;
}

GTK_TG_API void gtk_textgen_destroy(gtk_textgen* g) { free(g); }

static inline int zipf_rank(const gtk_textgen* g, uint64_t u)
{
  int lo = 0, hi = LEX_WORDS - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (g->cdf[mid] >= u) hi = mid; else lo = mid + 1;
  }
  return lo;
}

static int put_utf8(uint32_t cp, uint8_t out[4])
{
  if (cp <= 0x7F) { out[0] = (uint8_t)cp; return 1; }
  if (cp <= 0x7FF) { out[0] = (uint8_t)(0xC0 | (cp >> 6)); out[1] = (uint8_t)(0x80 | (cp & 0x3F)); return 2; }
  if (cp <= 0xFFFF) {
    out[0] = (uint8_t)(0xE0 | (cp >> 12));
    out[1] = (uint8_t)(0x80 | ((cp >> 6) & 0x3F));
    out[2] = (uint8_t)(0x80 | (cp & 0x3F));
    return 3;
  }
  out[0] = (uint8_t)(0xF0 | (cp >> 18));
  out[1] = (uint8_t)(0x80 | ((cp >> 12) & 0x3F));
  out[2] = (uint8_t)(0x80 | ((cp >> 6) & 0x3F));
  out[3] = (uint8_t)(0x80 | (cp & 0x3F));
  return 4;
}

/* Fill out[0..n) from stream (seed, stream).  The last word is cut at n. */
GTK_TG_API void gtk_textgen_fill(const gtk_textgen* g, uint64_t stream, int mix, uint8_t* out, int64_t n)
{
  static const char PUNCT[6] = {'.', ',', ';', ':', '!', '?'};
  uint64_t s = stream_state(g->seed, stream);
  int64_t  k = 0;
  uint8_t  buf[320];
  while (k < n) {
    int m = 0;
    int want_sep = 1;
    int kind = 0; /* 0 word, 1 multibyte, 2 run */
    if (mix == GTK_MIX_STRESS) {
      uint32_t r = rnd_below(&s, 100);
      if (r < 5) kind = 2;
      else if (r < 25) kind = 1;
    }
    if (kind == 2) {
      int len = 8 + (int)rnd_below(&s, 249);
      uint8_t c;
      if (rnd_chance(&s, 1, 2)) { c = ' '; want_sep = 0; }
      else c = (uint8_t)('a' + rnd_below(&s, 26));
      memset(buf, c, (size_t)len);
      m = len;
    } else if (kind == 1) {
      int cls    = (int)rnd_below(&s, 3);
      int nchars = 1 + (int)rnd_below(&s, 8);
      for (int i = 0; i < nchars; ++i) {
        uint32_t cp;
        if (cls == 0) cp = 0x00C0 + rnd_below(&s, 0x024F - 0x00C0 + 1);
        else if (cls == 1) cp = 0x4E00 + rnd_below(&s, 0x9FFF - 0x4E00 + 1);
        else cp = 0x1F600 + rnd_below(&s, 0x1F64F - 0x1F600 + 1);
        m += put_utf8(cp, buf + m);
      }
    } else {
      int w = zipf_rank(g, splitmix64(&s));
      m     = g->word_len[w];
      memcpy(buf, g->word[w], (size_t)m);
      if (rnd_chance(&s, 10, 100)) buf[0] = (uint8_t)(buf[0] - 'a' + 'A');
    }
    if (kind != 2 && rnd_chance(&s, 8, 100)) buf[m++] = (uint8_t)PUNCT[rnd_below(&s, 6)];
    if (want_sep) buf[m++] = rnd_chance(&s, 1, 80) ? '\n' : ' ';
    int64_t take = (n - k < m) ? (n - k) : m;
    memcpy(out + k, buf, (size_t)take);
    k += take;
  }
}

typedef struct {
  const gtk_textgen* g;
  int                mix;
  int64_t            block_bytes, first_block, n_blocks;
  uint8_t*           out;
  volatile int64_t*  next;
} tg_job;

static void* tg_worker(void* arg)
{
  tg_job* j = (tg_job*)arg;
  for (;;) {
    int64_t b = __sync_fetch_and_add(j->next, 1);
    if (b >= j->n_blocks) break;
    gtk_textgen_fill(j->g, (uint64_t)(j->first_block + b), j->mix, j->out + b * j->block_bytes, j->block_bytes);
  }
  return NULL;
}

/* Blocks first_block .. first_block+n_blocks-1, block_bytes each, back to back into out. */
GTK_TG_API void gtk_textgen_blocks(const gtk_textgen* g, int mix, int64_t block_bytes, int64_t first_block,
                                   int64_t n_blocks, uint8_t* out, int n_threads)
{
  volatile int64_t next = 0;
  tg_job job = {g, mix, block_bytes, first_block, n_blocks, out, &next};
  if (n_threads < 1) n_threads = 1;
  if (n_threads > 128) n_threads = 128;
  if (n_threads == 1 || n_blocks < 2) { tg_worker(&job); return; }
  pthread_t th[128];
  for (int t = 0; t < n_threads; ++t) pthread_create(&th[t], NULL, tg_worker, &job);
  for (int t = 0; t < n_threads; ++t) pthread_join(th[t], NULL);
}

/* Log-normal piece lengths (median, sigma of the underlying normal), clipped
 * to [lo, hi], until total_bytes are covered (the last piece is cut short).
 * Writes offsets[0..count]; returns count, or -1 if cap is too small. */
GTK_TG_API int64_t gtk_textgen_lognormal_offsets(uint64_t seed, double median, double sigma, int64_t lo,
                                                 int64_t hi, int64_t total_bytes, int64_t* offsets, int64_t cap)
{
  uint64_t s = stream_state(seed, 0xFFFFFFFFFFFFFF02ull);
  int64_t pos = 0, c = 0;
  const double mu = log(median);
  if (cap < 1) return -1;
  offsets[0] = 0;
  while (pos < total_bytes) {
    double u1 = ((double)(splitmix64(&s) >> 11) + 1.0) / 9007199254740993.0;
    double u2 = (double)(splitmix64(&s) >> 11) / 9007199254740992.0;
    double z  = sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
    double v  = exp(mu + sigma * z);
    int64_t len = (int64_t)v;
    if (len < lo) len = lo;
    if (len > hi) len = hi;
    if (pos + len > total_bytes) len = total_bytes - pos;
    pos += len;
    if (c + 1 >= cap) return -1;
    offsets[++c] = pos;
  }
  return c;
}
