// gtk_kernels.cu -- sm_100a kernels of the greedy byte-level BPE path.
//
//   chunker      text lengths -> chunk counts -> exclusive scan -> chunk start
//                offsets (replaces the host chunk/flatten loops of the
//                reference, gputok_binding.cu:718-752)
//   merge (opt)  persistent CTAs walk the byte stream in tiles; a tile is cut
//                into never-merge segments; a segment that is a vocabulary
//                string of its own is answered by a table lookup, the other
//                short segments are merged by one thread each, long ones by a
//                warp, oversize ones by the CTA in an HBM workspace; the
//                segment-start bitmap ends up as the bitmap of live tokens
//                that drives compaction (replaces bpe_merge_kernel_optimized's
//                role as the fast entry point, gputok_binding.cu:704-846, with
//                the greedy rule of gputok_blockbpe.cu:248-300)
//   merge (base) one CTA per chunk runs Algorithm 1 pass by pass on the whole
//                chunk, held in dynamic shared memory sized by the chunk length
//                (replaces bpe_merge_kernel_blockbpe, gputok_blockbpe.cu:328-538)
//   merge (wide) the same for merge tables whose ids or ranks need more than
//                16 bits: 32-bit tokens and ranks, 16-byte-slot pair table
//   local-min    the reference's other rule (bpe_merge_kernel_optimized,
//                gputok_binding.cu:290-414), one CTA per chunk
//   small        chunker, tiles, scans and pack of a small batch in one
//                single-CTA launch (latency mode)
//   output       exclusive scans over per-unit and per-chunk token counts and
//                a pack kernel that writes int32 ids back to back (replaces
//                the padded D2H + host unflatten, gputok_binding.cu:807-836)
//
// Nothing here is a dense contraction: the kernels are integer/byte work bound
// by shared-memory and issue throughput, so there is no tensor-core code.
// Kernels report trouble through a status word and never trap; every loop is
// bounded.  -DGTK_CHECKED adds range checks on every data-dependent index.
#include "gtk_device.cuh"

#include <algorithm>
#include <cstddef>

namespace gtk {
namespace {

#ifdef GTK_PHASE_TIMING
__device__ unsigned long long g_phase_cycles[32];
#endif

// Checked build (-DGTK_CHECKED): every index into shared memory, the lane scratch, the staging buffer and the
// per-chunk / per-unit arrays that is computed from data is compared with its limit before it is used.  A
// violation is recorded (first failing check, offending value, limit, number of violations) and the access is
// skipped, so a wrong index shows up as a report, never as a fault; read the record with
// gtk_debug_check_words.  Without the flag the checks compile to nothing.
#ifdef GTK_CHECKED
__device__ int g_check_words[4];
__device__ __noinline__ bool check_failed(int id, long long value, long long limit)
{
  if (atomicAdd(&g_check_words[3], 1) == 0) {
    g_check_words[0] = id;
    g_check_words[1] = int(value);
    g_check_words[2] = int(limit);
  }
  return false;
}
#define GTK_IN(value, limit, id) \
  ((static_cast<unsigned long long>(value) < static_cast<unsigned long long>(limit)) || check_failed((id), (long long)(value), (long long)(limit)))
#else
#define GTK_IN(value, limit, id) true
#endif

constexpr uint32_t NONE = 0xFFFFu;  // pair not mergeable
constexpr uint32_t SEL  = 0xFFFEu;  // pair selected for the current pass
constexpr uint32_t DEAD = 0xFFFFu;  // token slot holds nothing

// ------------------------------------------------------------------------------------------------
// merge table probes
// ------------------------------------------------------------------------------------------------

// What a probe of the pair table needs, small enough to travel in registers.
struct PairTable {
  const uint4* buckets;
  const uint2* overflow;           // nullptr when no bucket overflowed
  const uint32_t* merged_of_rank;  // nullptr when merged id = 256 + rank
  uint32_t overflow_mask;
};

__device__ __forceinline__ PairTable pair_table(const DeviceTable& T)
{
  return PairTable{T.pair_buckets, T.pair_overflow, T.merged_is_256_plus_rank ? nullptr : T.merged_of_rank,
                   T.pair_overflow_mask};
}

// keys of a full bucket that has no match may live in the overflow table
__device__ __noinline__ uint32_t probe_overflow(const uint2* overflow, uint32_t mask, uint32_t key)
{
  uint32_t h = ((key * 0x85EBCA77u) >> 7) & mask;
  for (uint32_t d = 0; d <= mask; ++d) {
    const uint2 s = __ldg(overflow + h);
    if (s.x == key) return s.y;
    if (s.x == 0xFFFFFFFFu) return NONE;
    h = (h + 1u) & mask;
  }
  return NONE;
}

// Rank of the key whose hash is h in its home bucket v.  An entry is low16(h) << 16 | rank, so XOR with
// low16(h) << 16 leaves the bare rank (< 65536) for the key's own entry and something larger for every other
// entry: the minimum over the four words is the rank, or a value >= 65536 when the key is not there (an empty
// word can only "match" with rank 0xFFFF, which is the right answer for a bucket that is not full).
__device__ __forceinline__ uint32_t bucket_rank(const uint4& v, uint32_t h)
{
  const uint32_t f = h << 16;
  return min(min(v.x ^ f, v.y ^ f), min(v.z ^ f, v.w ^ f));
}

// any value >= SEL means "no such merge"
__device__ __forceinline__ uint32_t resolve_rank_raw(const uint4& v, uint32_t key, const uint2* overflow,
                                                     uint32_t mask)
{
  uint32_t r = bucket_rank(v, key * 0x9E3779B1u);
  if (r >= SEL && overflow != nullptr && v.w != 0xFFFFFFFFu) r = probe_overflow(overflow, mask, key);
  return r;
}

__device__ __forceinline__ uint32_t resolve_rank(const uint4& v, uint32_t key, const uint2* overflow, uint32_t mask)
{
  return min(resolve_rank_raw(v, key, overflow, mask), NONE);
}

__device__ __forceinline__ uint32_t probe_rank(const DeviceTable& T, uint32_t left, uint32_t right)
{
  const uint32_t key = (left << 16) | right;
  const uint4 v      = __ldg(T.pair_buckets + ((key * 0x9E3779B1u) >> 16));
  return resolve_rank(v, key, T.pair_overflow, T.pair_overflow_mask);
}

// Tables whose ids or ranks do not fit 16 bits are served from the 16-byte-slot open-addressing table
// ({right, left, rank, merged id}, linear probing, empty = all ones): rank of the pair, 0xFFFFFFFF if none.
__device__ __forceinline__ uint32_t probe_rank_wide(const DeviceTable& T, uint32_t left, uint32_t right)
{
  const uint32_t mask = (1u << T.wide_log2) - 1u;
  uint32_t h = (((left << 16) ^ right) * 0x9E3779B1u) >> (32u - T.wide_log2);
  for (uint32_t d = 0; d <= T.wide_max_probe; ++d) {
    const uint4 v = __ldg(T.wide_slots + h);
    if (v.x == right && v.y == left) return v.z;
    if ((v.x & v.y) == 0xFFFFFFFFu) return 0xFFFFFFFFu;
    h = (h + 1u) & mask;
  }
  return 0xFFFFFFFFu;
}

// rank of a pair in the marker convention of the element type (16-bit: 0xFFFF = none, 32-bit: all ones = none)
template <typename TT>
__device__ __forceinline__ uint32_t probe_rank_t(const DeviceTable& T, uint32_t left, uint32_t right)
{
  if (sizeof(TT) == 2) return probe_rank(T, left, right);
  return probe_rank_wide(T, left, right);
}

// Whole-segment table: id of the vocabulary string (k0,k1,k2 = bytes zero padded, L = length)
// if the greedy rule turns exactly that string into one token, else 0xFFFFFFFF.  Two-choice cuckoo
// table: both candidate slots are loaded at once.
__device__ __forceinline__ uint32_t word_lookup(const uint4* word_slots, uint32_t sh, uint32_t k0, uint32_t k1,
                                                uint32_t k2, uint32_t L)
{
  uint32_t m = (k0 * 0x9E3779B1u) ^ (k1 * 0x85EBCA77u) ^ (k2 * 0xC2B2AE3Du);
  m ^= m >> 15;
  m *= 0x2C1B3C6Du;
  const uint4 a = __ldg(word_slots + (m >> sh));
  const uint4 c = __ldg(word_slots + (((m ^ (m >> 13)) * 0x165667B1u) >> sh));
  const uint32_t meta = (L << 16);
  if (a.x == k0 && a.y == k1 && a.z == k2 && (a.w & 0xFFFF0000u) == meta) return a.w & 0xFFFFu;
  if (c.x == k0 && c.y == k1 && c.z == k2 && (c.w & 0xFFFF0000u) == meta) return c.w & 0xFFFFu;
  return 0xFFFFFFFFu;
}

// segment bytes at shared-memory offset `at` (any alignment), zero padded to three words
__device__ __forceinline__ void segment_key(const uint8_t* bytes, int at, int LL, uint32_t& k0, uint32_t& k1,
                                            uint32_t& k2)
{
  const uint32_t* wp = reinterpret_cast<const uint32_t*>(bytes + (at & ~3));
  const uint32_t sh  = uint32_t(at & 3) * 8u;
  const uint32_t a0 = wp[0], a1 = wp[1], a2 = wp[2], a3 = wp[3];
  k0 = __funnelshift_r(a0, a1, sh);
  k1 = __funnelshift_r(a1, a2, sh);
  k2 = __funnelshift_r(a2, a3, sh);
  k0 &= (LL >= 4) ? 0xFFFFFFFFu : ((1u << (8 * LL)) - 1u);
  k1 &= (LL >= 8) ? 0xFFFFFFFFu : ((LL <= 4) ? 0u : ((1u << (8 * (LL - 4))) - 1u));
  k2 &= (LL >= 12) ? 0xFFFFFFFFu : ((LL <= 8) ? 0u : ((1u << (8 * (LL - 8))) - 1u));
}

__device__ __forceinline__ uint32_t merged_id(const DeviceTable& T, uint32_t rank)
{
  return T.merged_is_256_plus_rank ? 256u + rank : __ldg(T.merged_of_rank + rank);
}

__device__ __forceinline__ bool adj_bit(const uint32_t* adj, uint32_t u, uint32_t v)
{
  const uint32_t bit = (u << 8) | v;
  return (__ldg(adj + (bit >> 5)) >> (bit & 31u)) & 1u;
}

__device__ __forceinline__ uint32_t lanemask_lt()
{
  uint32_t m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// ------------------------------------------------------------------------------------------------
// One short segment (<= 32 tokens) merged by a single thread.
//
// tok[0..L) / rk[0..L) live in shared memory; rk[i] is the rank of the pair
// (token i, next live token), NONE for dead slots and for the last live one.
// Dead slots become DEAD tombstones and stay where they are; the alive set is
// a 32-bit register mask.  `best` = (rank << 16 | position) of the left-most
// pair of lowest rank -- the pair Algorithm 1 restricted to the segment merges
// next.  A step merges it, starts the two table probes for the pairs next to
// the new token, scans the cached ranks of all other pairs while the probes are
// in flight, and folds the two new ranks into the next `best`.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t segment_argmin(const uint16_t* rk_all, int s, int L)
{
  // two ranks per 32-bit load.  The words may reach one slot before the segment (when s is odd) and the
  // segment's own last slot: both always hold NONE, so they never win.
  uint32_t best         = 0xFFFFFFFFu;
  const uint32_t* words = reinterpret_cast<const uint32_t*>(rk_all);
  const int w_last      = (s + L - 2) >> 1;
  uint32_t rel          = uint32_t(((s >> 1) << 1) - s);  // index of the low half relative to s: 0 or -1
  for (int w = s >> 1; w <= w_last; ++w, rel += 2) {
    const uint32_t x = words[w];
    best = min(best, min((x << 16) | (rel & 0xFFFFu), (x & 0xFFFF0000u) | ((rel + 1u) & 0xFFFFu)));
  }
  return best;
}

// Returns false (and changes nothing) when no pair of the segment is mergeable any more.
__device__ __forceinline__ bool thread_merge_step(uint16_t* tok_all, uint16_t* rk_all, int s, int L,
                                                  uint32_t& alive, uint32_t& best, const PairTable& P)
{
  const uint32_t r = best >> 16;
  if (r >= SEL) return false;
  uint16_t* tok = tok_all + s;
  uint16_t* rk  = rk_all + s;
  const int j   = int(best & 0xFFFFu);
  const int q   = j + __ffs(int(alive >> (j + 1)));  // next live slot after j (j <= 30)
  if (!(GTK_IN(j, L - 1, 12) && GTK_IN(q - j - 1, L - j - 1, 13))) {
    best = 0xFFFFFFFFu;
    return false;
  }
  const uint32_t c = P.merged_of_rank ? __ldg(P.merged_of_rank + r) : 256u + r;
  alive &= ~(1u << q);
  const uint32_t right = (q >= 31) ? 0u : (alive >> (q + 1));
  const uint32_t left  = alive & ((1u << j) - 1u);
  const int p          = left ? 31 - __clz(int(left)) : j;  // j itself when there is no left neighbour
  // both probes leave before anything waits for them; an absent neighbour reads as an empty slot
  uint32_t keyR = 0xFFFFFFFFu, keyL = 0xFFFFFFFFu;
  uint4 vR = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu), vL = vR;
  if (right) {
    keyR = (c << 16) | uint32_t(tok[q + __ffs(int(right))]);
    vR   = __ldg(P.buckets + ((keyR * 0x9E3779B1u) >> 16));
  }
  if (left) {
    keyL = (uint32_t(tok[p]) << 16) | c;
    vL   = __ldg(P.buckets + ((keyL * 0x9E3779B1u) >> 16));
  }
  tok[j] = uint16_t(c);
  tok[q] = uint16_t(DEAD);
  rk[q]  = uint16_t(NONE);
  rk[j]  = uint16_t(NONE);
  rk[p]  = uint16_t(NONE);
  best   = segment_argmin(rk_all, s, L);  // every pair but the two new ones
  const uint32_t rr = resolve_rank_raw(vR, keyR, P.overflow, P.overflow_mask);
  const uint32_t rl = resolve_rank_raw(vL, keyL, P.overflow, P.overflow_mask);
  if (rr < SEL) {
    rk[j] = uint16_t(rr);
    best  = min(best, (rr << 16) | uint32_t(j));
  }
  if (rl < SEL) {
    rk[p] = uint16_t(rl);
    best  = min(best, (rl << 16) | uint32_t(p));
  }
  return true;
}

// ------------------------------------------------------------------------------------------------
// A group of NW warps (one warp, or the whole CTA) merges one sequence pass by
// pass.  tok/rk may point to shared memory or to an HBM workspace.
//
// Slots: tok[i] is a token id or the DEAD tombstone; for a live slot rk[i] is the
// cached rank of the pair (tok[i], next live token), NONE when there is none; a
// dead slot has rk NONE.  Tombstones stay where they are and the slots are
// compacted only when an eighth of them is dead, so a pass costs two sweeps over
// the cached ranks plus work proportional to the number of merges:
//   (1) group-wide minimum of the cached ranks (four ranks per 64-bit load when
//       VEC, i.e. when rk is 8-byte aligned; warp redux + cross-warp exchange);
//   (2) selection of the occurrences of that pair;
//   (3) every selected occurrence writes the merged id and a tombstone and
//       remembers its slot;
//   (4) the two pairs next to every new token are probed again (only those);
//   (5) in-place compaction when due -- each thread keeps its elements in
//       registers between the read and the write, offsets come from warp ballots
//       and popc plus a cross-warp sum.
//
// With a monotone table all non-overlapping occurrences of the winning pair,
// taken left to right, are merged in one pass; this is what Algorithm 1 does
// over consecutive passes because no merge at the minimum rank can expose a
// lower rank.  Otherwise only the left-most occurrence is merged.
// ------------------------------------------------------------------------------------------------
constexpr int kMergeList = 64;  // merges of one pass that are re-probed from a list; more fall back to a sweep
struct GroupScratch {
  uint32_t red[2][32];
  uint32_t wsum[32];
  int dead;  // tombstones since the last compaction (CTA-wide groups)
  int list[kMergeList];  // slots merged in the current pass (CTA-wide groups)
};

template <int NW>
__device__ __forceinline__ void gsync()
{
  if (NW == 1) __syncwarp();
  else __syncthreads();
}

template <int NW>
__device__ __forceinline__ uint32_t group_min(uint32_t v, GroupScratch* gs, int& parity, int lane, int warp)
{
  v = __reduce_min_sync(0xFFFFFFFFu, v);
  if (NW > 1) {
    if (lane == 0) gs->red[parity][warp] = v;
    __syncthreads();
    uint32_t x = (lane < NW) ? gs->red[parity][lane] : 0xFFFFFFFFu;
    v          = __reduce_min_sync(0xFFFFFFFFu, x);
    parity ^= 1;
  }
  return v;
}

// first live slot after i (n when there is none) / before i (-1 when there is none)
__device__ __forceinline__ int next_live(const uint16_t* tok, int i, int n)
{
  int j = i + 1;
  while (j < n && tok[j] == DEAD) ++j;
  return j;
}
__device__ __forceinline__ int prev_live(const uint16_t* tok, int i)
{
  int p = i - 1;
  while (p >= 0 && tok[p] == DEAD) --p;
  return p;
}

// VEC sweeps read the cached ranks four at a time (one 64-bit load) and reduce them with the packed 16-bit
// three-input minimum; the up to three slots between n and the next multiple of four hold NONE (pad_ranks).
__device__ __forceinline__ void pad_ranks(uint16_t* rk, int n, int tid)
{
  if (tid < ((4 - (n & 3)) & 3)) rk[n + tid] = uint16_t(NONE);
}

// calls f(i) for every slot i < n whose cached rank equals `pick`
template <int NW, bool VEC, class F>
__device__ __forceinline__ void for_each_rank(const uint16_t* rk, int n, int tid, uint32_t pick, F f)
{
  constexpr int G = NW * 32;
  if (VEC) {
    const int nw      = (n + 3) >> 2;
    const uint32_t p2 = pick | (pick << 16);
    for (int w = tid; w < nw; w += G) {
      const uint2 x = reinterpret_cast<const uint2*>(rk)[w];
      // a half-word of z is zero exactly when one of the four ranks equals pick
      const uint32_t z = __vimin3_u16x2(x.x ^ p2, x.y ^ p2, 0xFFFFFFFFu);
      if ((z & 0xFFFFu) == 0u || (z >> 16) == 0u) {
        const uint32_t q[4] = {x.x & 0xFFFFu, x.x >> 16, x.y & 0xFFFFu, x.y >> 16};
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (q[k] == pick) f(4 * w + k);
      }
    }
  } else {
    for (int i = tid; i < n; i += G)
      if (rk[i] == pick) f(i);
  }
}

// In-place compaction of tok/rk[0..n): returns the number of live slots, which end up at the front in order.
template <int NW>
__device__ __forceinline__ int group_compact(uint16_t* tok, uint16_t* rk, int n, GroupScratch* gs, int lane, int warp,
                                             uint32_t lt)
{
  constexpr int G = NW * 32;
  constexpr int E = 4;
  int out = 0;
  for (int base = 0; base < n; base += G * E) {
    uint16_t t[E], q[E];
    uint32_t bal[E];
    int wt = 0;
#pragma unroll
    for (int k = 0; k < E; ++k) {
      const int i  = base + warp * 32 * E + k * 32 + lane;
      const bool v = i < n;
      t[k]   = v ? tok[i] : uint16_t(DEAD);
      q[k]   = v ? rk[i] : uint16_t(NONE);
      bal[k] = __ballot_sync(0xFFFFFFFFu, t[k] != DEAD);
      wt += __popc(bal[k]);
    }
    int pre = 0, tot = wt;
    if (NW > 1) {
      if (lane == 0) gs->wsum[warp] = uint32_t(wt);
      __syncthreads();  // all loads of the batch are done, warp totals visible
      tot = 0;
      for (int w = 0; w < NW; ++w) {
        const int x = int(gs->wsum[w]);
        if (w < warp) pre += x;
        tot += x;
      }
    } else {
      __syncwarp();
    }
    int o = out + pre;
#pragma unroll
    for (int k = 0; k < E; ++k) {
      if (t[k] != DEAD) {
        const int d = o + __popc(bal[k] & lt);
        tok[d] = t[k];
        rk[d]  = q[k];
      }
      o += __popc(bal[k]);
    }
    out += tot;
    gsync<NW>();
  }
  return out;
}

template <int NW, bool VEC>
__device__ int group_merge(uint16_t* tok, uint16_t* rk, int L, const DeviceTable& T, GroupScratch* gs,
                           int* status)
{
  constexpr int G    = NW * 32;
  constexpr int kMem = 4;  // merged slots a thread remembers per pass; more fall back to a sweep
  const int lane  = threadIdx.x & 31;
  const int warp  = (NW == 1) ? 0 : (threadIdx.x >> 5);
  const int tid   = (NW == 1) ? lane : int(threadIdx.x);
  const uint32_t lt = lanemask_lt();
  const bool batch  = T.monotone != 0;
  int parity = 0;
  int n      = L;  // slots in use
  int dead   = 0;  // tombstones among them
  if (VEC) pad_ranks(rk, n, tid);
  if (NW > 1) {
    if (tid == 0) gs->dead = 0;
    __syncthreads();
  } else {
    __syncwarp();
  }
  for (int pass = 0; pass < L && n - dead >= 2; ++pass) {
    // (1) lowest cached rank
    uint32_t m = NONE;
    if (VEC) {
      const int nw = (n + 3) >> 2;
      uint32_t m2  = 0xFFFFFFFFu;
      for (int w = tid; w < nw; w += G) {
        const uint2 x = reinterpret_cast<const uint2*>(rk)[w];
        m2 = __vimin3_u16x2(m2, x.x, x.y);
      }
      m = min(m2 & 0xFFFFu, m2 >> 16);
    } else {
      for (int i = tid; i < n; i += G) m = min(m, uint32_t(rk[i]));
    }
    m = group_min<NW>(m, gs, parity, lane, warp);
    if (m >= SEL) break;
    const uint32_t r = m;
    const uint32_t c = merged_id(T, r);
    const bool same  = batch && (__ldg(T.same_of_rank + r) != 0);
    // (2) selection
    if (!batch) {
      uint32_t p = 0xFFFFFFFFu;
      for_each_rank<NW, VEC>(rk, n, tid, r, [&](int i) { p = min(p, uint32_t(i)); });
      p = group_min<NW>(p, gs, parity, lane, warp);
      gsync<NW>();
      if (tid == 0) rk[p] = uint16_t(SEL);
      gsync<NW>();
    } else if (same) {
      // occurrences of (a,a) overlap inside a run a a a ...; left to right
      // selection keeps the even offsets of every maximal run of matches
      for_each_rank<NW, VEC>(rk, n, tid, r, [&](int i) {
        const int pl = prev_live(tok, i);
        if (pl >= 0) {
          const uint32_t pv = rk[pl];
          if (pv == r || pv == SEL) return;  // not the first match of its run
        }
        int j = i;
        for (;;) {
          rk[j] = uint16_t(SEL);
          const int j1 = next_live(tok, j, n);
          if (j1 >= n || rk[j1] != r) break;
          const int j2 = next_live(tok, j1, n);
          if (j2 >= n || rk[j2] != r) break;
          j = j2;
        }
      });
      gsync<NW>();
    }
    const uint32_t pick = (!batch || same) ? SEL : r;
    // (3) apply: the selected occurrences never share a slot, so the writes are disjoint.  A CTA-wide group
    // collects the merged slots in a shared list (the tombstone counter hands out the places), a single warp
    // keeps them in registers
    int mine = 0;
    int at[kMem];
    for_each_rank<NW, VEC>(rk, n, tid, pick, [&](int i) {
      const int j = next_live(tok, i, n);  // exists: the pair has a cached rank
      if (!GTK_IN(i, n, 30)) return;
      tok[i] = uint16_t(c);
      rk[i]  = uint16_t(NONE);
      if (j < n) {
        tok[j] = uint16_t(DEAD);
        rk[j]  = uint16_t(NONE);
      }
      if (NW > 1) {
        const int place = atomicAdd(&gs->dead, 1) - dead;
        if (place < kMergeList) gs->list[place] = i;
      } else {
#pragma unroll
        for (int k = 0; k < kMem; ++k)
          if (mine == k) at[k] = i;
        ++mine;
      }
    });
    // (4) ranks of the two pairs next to every new token
    auto refresh = [&](int i) {
      const int jn = next_live(tok, i, n);
      rk[i] = uint16_t((jn < n) ? probe_rank(T, c, tok[jn]) : NONE);
      const int pl = prev_live(tok, i);
      if (pl >= 0) rk[pl] = uint16_t(probe_rank(T, tok[pl], c));
    };
    if (NW > 1) {
      __syncthreads();
      const int now = gs->dead;
      if (now == dead) {  // a pass must remove at least one token
        if (tid == 0 && status) atomicMax(status, int(kStatusBadSegment));
        break;
      }
      const int merged = now - dead;
      dead = now;
      if (merged <= kMergeList) {  // the first threads take one merged slot each: one or two warps do the probes
        if (tid < merged) refresh(gs->list[tid]);
      } else {
        for (int i = tid; i < n; i += G)
          if (tok[i] == c) refresh(i);
      }
    } else {
      const int wsum   = __reduce_add_sync(0xFFFFFFFFu, mine);
      const bool sweep = __any_sync(0xFFFFFFFFu, mine > kMem) != 0;
      if (wsum == 0) {
        if (tid == 0 && status) atomicMax(status, int(kStatusBadSegment));
        break;
      }
      dead += wsum;
      if (!sweep) {
#pragma unroll
        for (int k = 0; k < kMem; ++k)
          if (k < mine) refresh(at[k]);
      } else {
        for (int i = tid; i < n; i += G)
          if (tok[i] == c) refresh(i);
      }
    }
    gsync<NW>();
    // (5) compaction when an eighth of the slots is dead
    if (dead * 8 >= n) {
      n    = group_compact<NW>(tok, rk, n, gs, lane, warp, lt);
      dead = 0;
      if (VEC) pad_ranks(rk, n, tid);
      if (NW > 1) {
        if (tid == 0) gs->dead = 0;
        __syncthreads();
      } else {
        __syncwarp();
      }
    }
  }
  if (dead) n = group_compact<NW>(tok, rk, n, gs, lane, warp, lt);
  return n;
}

// The same merge with a compaction in every pass: cheaper for the short sequences a single warp handles
// inside a tile (a few dozen to a few hundred tokens), where a sweep costs little and the tombstone searches of
// the lazy variant do not pay.
template <int NW, typename TT>
__device__ int group_merge_dense(TT* tok, TT* rk, int L, const DeviceTable& T, GroupScratch* gs,
                           int* status)
{
  constexpr int G = NW * 32;
  constexpr int E = 4;
  // markers in the element type: all ones = no rank / tombstone, all ones minus one = selected
  constexpr uint32_t kNone = uint32_t(TT(~TT(0))), kSel = kNone - 1u, kDead = kNone;
  const int lane  = threadIdx.x & 31;
  const int warp  = (NW == 1) ? 0 : (threadIdx.x >> 5);
  const int tid   = (NW == 1) ? lane : int(threadIdx.x);
  const uint32_t lt = lanemask_lt();
  int parity = 0;
  int len    = L;
  for (int pass = 0; pass < L && len >= 2; ++pass) {
    // (1) lowest cached rank
    uint32_t m = kNone;
    for (int i = tid; i < len - 1; i += G) m = min(m, uint32_t(rk[i]));
    m = group_min<NW>(m, gs, parity, lane, warp);
    if (m >= kSel) break;
    const uint32_t r = m;
    const uint32_t c = merged_id(T, r);
    const bool batch = T.monotone != 0;
    const bool same  = batch && (__ldg(T.same_of_rank + r) != 0);
    // (2) selection
    if (!batch) {
      uint32_t p = 0xFFFFFFFFu;
      for (int i = tid; i < len - 1; i += G)
        if (rk[i] == r) { p = uint32_t(i); break; }
      p = group_min<NW>(p, gs, parity, lane, warp);
      gsync<NW>();
      if (tid == 0) rk[p] = TT(kSel);
      gsync<NW>();
    } else if (same && NW == 1) {
      // occurrences of (a,a) overlap inside a run a a a ...; left to right selection keeps the even offsets of
      // every maximal run of matches.  One warp, 32 slots per round: a ballot gives the matches, the distance of a
      // match to the start of its run is the distance to the nearest non-match below it (the run may reach back
      // into earlier rounds: `before` carries the parity of the matches that directly precede this round)
      uint32_t before = 0;
      for (int base = 0; base < len - 1; base += 32) {
        const int i       = base + lane;
        const bool match  = (i < len - 1) && (rk[i] == r);
        const uint32_t mm = __ballot_sync(0xFFFFFFFFu, match);
        if (match) {
          const uint32_t gaps = ~mm & lt;  // non-matches below this lane
          const uint32_t off  = gaps ? uint32_t(lane) - (32u - uint32_t(__clz(int(gaps)))) : uint32_t(lane) + before;
          if ((off & 1u) == 0u) rk[i] = TT(kSel);
        }
        const uint32_t tail = uint32_t(__clz(int(~mm)));  // matches at the top of this round
        before = (tail == 32u) ? ((before + 32u) & 1u) : (tail & 1u);
      }
      __syncwarp();
    } else if (same) {
      // the same selection for a CTA-wide group: the first match of every run walks its run
      for (int i = tid; i < len - 1; i += G) {
        if (rk[i] != r) continue;
        if (i > 0) {
          const uint32_t pv = rk[i - 1];
          if (pv == r || pv == kSel) continue;  // not the first match of its run
        }
        int j = i;
        for (;;) {
          rk[j] = TT(kSel);
          if (j + 2 < len - 1 && rk[j + 1] == r && rk[j + 2] == r) j += 2;
          else break;
        }
      }
      gsync<NW>();
    }
    const uint32_t pick = (!batch || same) ? kSel : r;
    // (3) apply
    for (int i = tid; i < len - 1; i += G) {
      if (rk[i] == pick) {
        tok[i]     = TT(c);
        tok[i + 1] = TT(kDead);
      }
    }
    gsync<NW>();
    // (4) in-place compaction, batch by batch, registers as the second buffer
    int out = 0;
    for (int base = 0; base < len; base += G * E) {
      TT t[E], q[E];
      uint32_t bal[E];
      int wt = 0;
#pragma unroll
      for (int k = 0; k < E; ++k) {
        const int i = base + warp * 32 * E + k * 32 + lane;
        const bool v = i < len;
        t[k]   = v ? tok[i] : TT(kDead);
        q[k]   = v ? rk[i] : TT(kNone);
        bal[k] = __ballot_sync(0xFFFFFFFFu, t[k] != kDead);
        wt += __popc(bal[k]);
      }
      int pre = 0, tot = wt;
      if (NW > 1) {
        if (lane == 0) gs->wsum[warp] = uint32_t(wt);
        __syncthreads();  // all loads of the batch are done, warp totals visible
        tot = 0;
        for (int w = 0; w < NW; ++w) {
          const int x = int(gs->wsum[w]);
          if (w < warp) pre += x;
          tot += x;
        }
      } else {
        __syncwarp();
      }
      int o = out + pre;
#pragma unroll
      for (int k = 0; k < E; ++k) {
        if (t[k] != kDead) {
          const int d = o + __popc(bal[k] & lt);
          tok[d] = t[k];
          rk[d]  = q[k];
        }
        o += __popc(bal[k]);
      }
      out += tot;
      gsync<NW>();
    }
    if (!GTK_IN(out, L + 1, 29)) break;
    if (out >= len) {  // a pass must remove at least one token
      if (tid == 0 && status) atomicMax(status, int(kStatusBadSegment));
      break;
    }
    len = out;
    // (5) refresh ranks next to new tokens
    for (int d = tid; d < len; d += G) {
      if (tok[d] == c) {
        rk[d] = TT((d + 1 < len) ? probe_rank_t<TT>(T, c, tok[d + 1]) : kNone);
        if (d > 0) rk[d - 1] = TT(probe_rank_t<TT>(T, tok[d - 1], c));
      }
    }
    gsync<NW>();
  }
  return len;
}

// ------------------------------------------------------------------------------------------------
// block-wide helpers
// ------------------------------------------------------------------------------------------------

// exclusive scan of one int per thread over the CTA; *total receives the sum.
// `buf` must hold 33 ints of shared memory; contains two barriers.
__device__ __forceinline__ int block_exclusive_scan(int v, int* buf, int* total)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int y = __shfl_up_sync(0xFFFFFFFFu, inc, d);
    if (lane >= d) inc += y;
  }
  if (lane == 31) buf[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = (lane < nw) ? buf[lane] : 0;
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int y = __shfl_up_sync(0xFFFFFFFFu, winc, d);
      if (lane >= d) winc += y;
    }
    buf[lane] = winc - w;
    if (lane == 31) buf[32] = winc;
  }
  __syncthreads();
  *total = buf[32];
  return buf[warp] + inc - v;
}

// ------------------------------------------------------------------------------------------------
// multi-block exclusive scan: counts (int32 array, or chunks-per-text computed
// on the fly) -> int64 offsets[n+1].  Three kernels: per-block sums, scan of
// the block sums by one CTA, final pass.  n may live on the device.
// ------------------------------------------------------------------------------------------------
constexpr int kScanThreads = 256;
constexpr int kScanItems   = 16;
constexpr int kScanBlock   = kScanThreads * kScanItems;

struct CountsI32 {
  const int32_t* p;
  __device__ int64_t operator()(int64_t i) const { return p[i]; }
};
struct ChunksPerText {
  const int64_t* off;
  int chunk;
  __device__ int64_t operator()(int64_t i) const
  {
    const int64_t len = off[i + 1] - off[i];
    if (len <= 0) return 0;
    if (len < (int64_t(1) << 31)) return int64_t((uint32_t(len) + uint32_t(chunk) - 1u) / uint32_t(chunk));  // the usual case, a 32-bit division
    return (len + chunk - 1) / chunk;
  }
};

__device__ __forceinline__ int64_t block_sum_i64(int64_t v, int64_t* buf)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  int64_t s = 0;
  for (int w = 0; w < kScanThreads / 32; ++w) s += buf[w];
  __syncthreads();
  return s;
}

template <class In>
__global__ void __launch_bounds__(kScanThreads) k_scan_partial(In in, int64_t n_imm, const int64_t* n_ptr,
                                                               int64_t* block_sums)
{
  __shared__ int64_t buf[kScanThreads / 32];
  const int64_t n    = n_ptr ? *n_ptr : n_imm;
  const int64_t base = int64_t(blockIdx.x) * kScanBlock;
  int64_t s          = 0;
  for (int e = 0; e < kScanItems; ++e) {
    const int64_t i = base + int64_t(e) * kScanThreads + threadIdx.x;
    if (i < n) s += in(i);
  }
  s = block_sum_i64(s, buf);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = s;
}

// one CTA: exclusive scan of block_sums[0..nb) in place
__global__ void __launch_bounds__(kScanThreads) k_scan_block_sums(int64_t* block_sums, int64_t nb)
{
  __shared__ int64_t wtot[kScanThreads / 32];
  __shared__ int64_t carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < nb; base += kScanThreads) {
    const int64_t i = base + threadIdx.x;
    const int64_t v = (i < nb) ? block_sums[i] : 0;
    int64_t inc     = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int64_t y = __shfl_up_sync(0xFFFFFFFFu, inc, d);
      if (lane >= d) inc += y;
    }
    if (lane == 31) wtot[warp] = inc;
    __syncthreads();
    int64_t pre = carry_s;
    for (int w = 0; w < warp; ++w) pre += wtot[w];
    if (i < nb) block_sums[i] = pre + inc - v;
    __syncthreads();
    if (threadIdx.x == kScanThreads - 1) carry_s = pre + inc;
    __syncthreads();
  }
}

template <class In>
__global__ void __launch_bounds__(kScanThreads) k_scan_final(In in, int64_t n_imm, const int64_t* n_ptr,
                                                             const int64_t* block_sums, int64_t* out,
                                                             int64_t* total_out)
{
  __shared__ int64_t wtot[kScanThreads / 32];
  const int64_t n = n_ptr ? *n_ptr : n_imm;
  if (n == 0) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      out[0] = 0;
      if (total_out) *total_out = 0;
    }
    return;
  }
  const int64_t base = int64_t(blockIdx.x) * kScanBlock;
  if (base >= n) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // blocked layout: thread t owns items base + t*kScanItems .. +kScanItems
  int64_t v[kScanItems];
  int64_t s = 0;
  const int64_t first = base + int64_t(threadIdx.x) * kScanItems;
#pragma unroll
  for (int e = 0; e < kScanItems; ++e) {
    const int64_t i = first + e;
    v[e] = (i < n) ? in(i) : 0;
    s += v[e];
  }
  int64_t inc = s;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int64_t y = __shfl_up_sync(0xFFFFFFFFu, inc, d);
    if (lane >= d) inc += y;
  }
  if (lane == 31) wtot[warp] = inc;
  __syncthreads();
  int64_t pre = block_sums[blockIdx.x];
  for (int w = 0; w < warp; ++w) pre += wtot[w];
  int64_t run = pre + inc - s;
#pragma unroll
  for (int e = 0; e < kScanItems; ++e) {
    const int64_t i = first + e;
    if (i < n) {
      out[i] = run;
      run += v[e];
      if (i == n - 1) {
        out[n] = run;
        if (total_out) *total_out = run;
      }
    }
  }
}

template <class In>
int run_scan(In in, int64_t n_upper, int64_t n_imm, const int64_t* n_ptr, int64_t* block_sums, int64_t* out,
             int64_t* total_out, cudaStream_t stream)
{
  int64_t nb = (n_upper + kScanBlock - 1) / kScanBlock;
  if (nb < 1) nb = 1;
  k_scan_partial<In><<<unsigned(nb), kScanThreads, 0, stream>>>(in, n_imm, n_ptr, block_sums);
  k_scan_block_sums<<<1, kScanThreads, 0, stream>>>(block_sums, nb);
  k_scan_final<In><<<unsigned(nb), kScanThreads, 0, stream>>>(in, n_imm, n_ptr, block_sums, out, total_out);
  return 3;
}

// ------------------------------------------------------------------------------------------------
// chunker
// ------------------------------------------------------------------------------------------------

// chunk c -> owning text by binary search over the scanned chunk counts, then
// its start byte.  Empty texts own no chunk and are skipped by the search.
__global__ void k_chunk_fill(const int64_t* __restrict__ text_off, const int64_t* __restrict__ text_chunk_base,
                             int64_t n_texts, int chunk_bytes, int64_t* __restrict__ chunk_off)
{
  const int64_t C = text_chunk_base[n_texts];
  for (int64_t c = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; c <= C; c += int64_t(gridDim.x) * blockDim.x) {
    if (c == C) {
      chunk_off[c] = text_off[n_texts];
      continue;
    }
    int64_t lo = 0, hi = n_texts;  // last t with text_chunk_base[t] <= c
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) >> 1;
      if (text_chunk_base[mid] <= c) lo = mid; else hi = mid;
    }
    chunk_off[c] = text_off[lo] + (c - text_chunk_base[lo]) * int64_t(chunk_bytes);
  }
}

// tile k -> chunk that contains byte k*kTile
__global__ void k_tile_chunk0(const int64_t* __restrict__ chunk_off, const int64_t* __restrict__ n_chunks_ptr,
                              int64_t n_tiles, int32_t* __restrict__ tile_chunk0)
{
  const int64_t C = *n_chunks_ptr;
  for (int64_t k = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; k < n_tiles; k += int64_t(gridDim.x) * blockDim.x) {
    const int64_t pos = k * kTile;
    int64_t lo = 0, hi = C;  // last c with chunk_off[c] <= pos (chunk_off[0] == 0)
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) >> 1;
      if (chunk_off[mid] <= pos) lo = mid; else hi = mid;
    }
    tile_chunk0[k] = int32_t(lo);
  }
}

// ------------------------------------------------------------------------------------------------
// merge kernel, segment-parallel ("opt")
// ------------------------------------------------------------------------------------------------

constexpr int kCutWords = kWindow / 32;  // 144
constexpr int kSegCap   = kTile / 2 + 8;
constexpr int kLongCap  = 128;

// Optional per-phase cycle accounting of k_merge_opt (build with -DGTK_PHASE_TIMING): thread 0 of
// every CTA accumulates clock64() deltas between phase boundaries; read with gtk_debug_phase_cycles.
#ifdef GTK_PHASE_TIMING
#define GTK_PHASE(k)                                              \
  do {                                                            \
    if (tid == 0) {                                               \
      const long long now__ = clock64();                          \
      atomicAdd(&g_phase_cycles[k], (unsigned long long)(now__ - phase_t0)); \
      phase_t0 = now__;                                           \
    }                                                             \
  } while (0)
#else
#define GTK_PHASE(k) do { } while (0)
#endif


struct OptSmem {
  // seg and bytes are adjacent on purpose: once the segments have been looked up, bytes and the unused tail of
  // seg (entries from kOptThreads on) are the rank scratch of the merge loop (lane_scratch below)
  alignas(16) uint16_t seg[kSegCap];  // starts of the segments that missed the lookup (length = distance to the next start)
  alignas(16) uint8_t bytes[kWindow + 32];  // [15] = byte before the window, [16+i] = window position i
  alignas(8) uint16_t tok[kWindow];
  alignas(8) uint16_t rk[kWindow];  // reused as the compacted output buffer after merging
  int hist[34];
  uint32_t cut[kCutWords + 2];  // segment-start bits; reused as the alive bitmap
  uint16_t woff[kCutWords + 2];
  uint16_t longq[kLongCap];
  GroupScratch gs;
  int scanbuf[33];
  int ticket;
  int nseg, nlong, seg_next, nmiss;
  int first_start, last_start, over_start;
  int over_len;
  long long over_end;
  long long run_base;  // single-CTA kernel: ids written by the tiles so far
  int over_chunk;
  int end_owned;
};

// One instance per CTA; the kernels below and the out-of-line merge loop name it directly.
__shared__ OptSmem g_tile;

static_assert(kSegCap % 8 == 0 && offsetof(OptSmem, bytes) == offsetof(OptSmem, seg) + kSegCap * 2,
              "seg and bytes must be adjacent");
// Rank scratch of the one-segment-per-thread merge loop: 32-bit words from seg[kOptThreads] to the end of bytes.
// Warp w owns kLaneWords words per lane at word offset w * 32 * kLaneWords, lane-interleaved (word k of lane l at
// k * 32 + l), so the 32 lanes of a rank scan hit 32 different banks.  The last warp gets what is left.
constexpr int kLaneWords        = 8;  // 16 ranks: segments of up to 16 tokens
constexpr int kLaneScratchWords = ((kSegCap - kOptThreads) * 2 + kWindow + 32) / 4;
__device__ __forceinline__ uint32_t* lane_scratch()
{
  return reinterpret_cast<uint32_t*>(g_tile.seg + kOptThreads);
}

// Every lane merges its own segment [s, s+L) to the end (s < 0: no segment).  Kept out of line so that
// the loop gets registers of its own instead of sharing them with the tile code around the call.
__device__ __noinline__ uint32_t thread_merge_segments(int s, int L, PairTable P)
{
  uint16_t* tok = g_tile.tok;  // named directly so that the accesses compile to shared-memory instructions
  uint16_t* rk  = g_tile.rk;
  uint32_t alive = 0, best = 0xFFFFFFFFu;
  if (s >= 0 && !(GTK_IN(s + L, kWindow + 1, 10) && GTK_IN(L - 2, kThreadSegMax - 1, 11))) s = -1;
  if (s >= 0) {
    alive = (L >= 32) ? 0xFFFFFFFFu : ((1u << L) - 1u);
    best  = segment_argmin(rk, s, L);
  }
#ifdef GTK_PHASE_TIMING
  if (threadIdx.x == 0) {  // in-situ latency of one table load and of one rank scan
    const long long a0 = clock64();
    const uint4 v      = __ldg(P.buckets + (uint32_t(a0) * 2654435761u >> 16));
    const long long a1 = clock64() + (v.x == 0x12345u);
    atomicAdd(&g_phase_cycles[16], (unsigned long long)(a1 - a0));
    atomicAdd(&g_phase_cycles[17], 1ull);
    if (s >= 0) {
      const long long b0 = clock64();
      const uint32_t bb  = segment_argmin(rk, s, L);
      const long long b1 = clock64() + (bb == 0x12345u);
      atomicAdd(&g_phase_cycles[18], (unsigned long long)(b1 - b0));
      atomicAdd(&g_phase_cycles[19], 1ull);
      atomicAdd(&g_phase_cycles[20], (unsigned long long)L);
    }
  }
  const long long t0 = clock64();
  int steps          = 0;
#endif
  while (__any_sync(0xFFFFFFFFu, best < (SEL << 16))) {
    if (best < (SEL << 16)) thread_merge_step(tok, rk, s, L, alive, best, P);
#ifdef GTK_PHASE_TIMING
    ++steps;
#endif
  }
#ifdef GTK_PHASE_TIMING
  if (threadIdx.x == 0) {  // warp 0: loop trips and their wall cycles
    atomicAdd(&g_phase_cycles[14], (unsigned long long)(clock64() - t0));
    atomicAdd(&g_phase_cycles[15], (unsigned long long)steps);
  }
#endif
  return alive;
}

// The same loop with the ranks of every segment copied into the lane-interleaved scratch first (WW words =
// 2 * WW ranks per lane, uniform over the warp): the rank scan is unrolled, needs no alignment handling and is
// free of bank conflicts; the tokens stay in place.
template <int WW>
__device__ __noinline__ uint32_t thread_merge_segments_lanes(int s, int L, PairTable P, int area, uint32_t alive)
{
  if (!GTK_IN(area + 32 * WW, kLaneScratchWords + 1, 14)) return alive;
  if (s >= 0 && !(GTK_IN(s + L, kWindow + 1, 15) && GTK_IN(L - 2, 2 * WW - 1, 16))) {
    s     = -1;
    alive = 0;
  }
  uint32_t* scr = lane_scratch() + area + (threadIdx.x & 31);
  uint16_t* tok = g_tile.tok + max(s, 0);
#pragma unroll
  for (int k = 0; k < WW; ++k) {
    uint32_t lo = NONE, hi = NONE;
    if (s >= 0 && 2 * k < L) lo = g_tile.rk[s + 2 * k];
    if (s >= 0 && 2 * k + 1 < L) hi = g_tile.rk[s + 2 * k + 1];
    scr[k * 32] = lo | (hi << 16);
  }
  auto scan = [&]() {
    uint32_t b = 0xFFFFFFFFu;
#pragma unroll
    for (int k = 0; k < WW; ++k) {
      const uint32_t x = scr[k * 32];
      b = min(b, min((x << 16) | uint32_t(2 * k), (x & 0xFFFF0000u) | uint32_t(2 * k + 1)));
    }
    return b;
  };
  auto set_rank = [&](int i, uint32_t v) { reinterpret_cast<uint16_t*>(scr + (i >> 1) * 32)[i & 1] = uint16_t(v); };
  uint32_t best = scan();
#ifdef GTK_PHASE_TIMING
  if (threadIdx.x == 0) {  // in-situ latency of one table load and of one rank scan
    const long long a0 = clock64();
    const uint4 v      = __ldg(P.buckets + (uint32_t(a0) * 2654435761u >> 16));
    const long long a1 = clock64() + (v.x == 0x12345u);
    atomicAdd(&g_phase_cycles[16], (unsigned long long)(a1 - a0));
    atomicAdd(&g_phase_cycles[17], 1ull);
    const long long b0 = clock64();
    const uint32_t bb  = scan();
    const long long b1 = clock64() + (bb == 0x12345u);
    atomicAdd(&g_phase_cycles[18], (unsigned long long)(b1 - b0));
    atomicAdd(&g_phase_cycles[19], 1ull);
  }
  const long long t0 = clock64();
  int steps          = 0;
#endif
  while (__any_sync(0xFFFFFFFFu, best < (SEL << 16))) {
#ifdef GTK_PHASE_TIMING
    ++steps;
    {  // merges done by this loop, all warps (each costs two bucket loads)
      const uint32_t act = __ballot_sync(0xFFFFFFFFu, best < (SEL << 16));
      if ((threadIdx.x & 31) == 0) atomicAdd(&g_phase_cycles[21], (unsigned long long)__popc(act));
    }
#endif
    if (best < (SEL << 16)) {
      const uint32_t r = best >> 16;
      const int j      = int(best & 0xFFFFu);
      const int q      = j + __ffs(int(alive >> (j + 1)));
      if (!(GTK_IN(j, L - 1, 17) && GTK_IN(q - j - 1, L - j - 1, 18))) {
        best = 0xFFFFFFFFu;
        continue;
      }
      const uint32_t c = P.merged_of_rank ? __ldg(P.merged_of_rank + r) : 256u + r;
      alive &= ~(1u << q);
      const uint32_t right = (q >= 31) ? 0u : (alive >> (q + 1));
      const uint32_t left  = alive & ((1u << j) - 1u);
      const int p          = left ? 31 - __clz(int(left)) : j;
      uint32_t keyR = 0xFFFFFFFFu, keyL = 0xFFFFFFFFu;
      uint4 vR = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu), vL = vR;
      if (right) {
        keyR = (c << 16) | uint32_t(tok[q + __ffs(int(right))]);
        vR   = __ldg(P.buckets + ((keyR * 0x9E3779B1u) >> 16));
      }
      if (left) {
        keyL = (uint32_t(tok[p]) << 16) | c;
        vL   = __ldg(P.buckets + ((keyL * 0x9E3779B1u) >> 16));
      }
      tok[j] = uint16_t(c);
      tok[q] = uint16_t(DEAD);
      set_rank(q, NONE);
      set_rank(j, NONE);
      set_rank(p, NONE);
      best = scan();  // every pair but the two new ones
      const uint32_t rr = resolve_rank_raw(vR, keyR, P.overflow, P.overflow_mask);
      const uint32_t rl = resolve_rank_raw(vL, keyL, P.overflow, P.overflow_mask);
      if (rr < SEL) {
        set_rank(j, rr);
        best = min(best, (rr << 16) | uint32_t(j));
      }
      if (rl < SEL) {
        set_rank(p, rl);
        best = min(best, (rl << 16) | uint32_t(p));
      }
    }
  }
#ifdef GTK_PHASE_TIMING
  if (threadIdx.x == 0) {  // warp 0: loop trips and their wall cycles
    atomicAdd(&g_phase_cycles[14], (unsigned long long)(clock64() - t0));
    atomicAdd(&g_phase_cycles[15], (unsigned long long)steps);
  }
#endif
  return alive;
}

// first segment start strictly after window position s (words past the window are all ones)
__device__ __forceinline__ int next_cut(const uint32_t* cut, int s)
{
  int w      = (s + 1) >> 5;
  if (!GTK_IN(w, kCutWords + 2, 1)) return kWindow;
  uint32_t x = cut[w] & (0xFFFFFFFFu << ((s + 1) & 31));
  while (!x) {
    if (!GTK_IN(w + 1, kCutWords + 2, 2)) return kWindow;
    x = cut[++w];
  }
  return w * 32 + __ffs(int(x)) - 1;
}

// One multi-byte segment that starts at window position ss: oversize and long ones are noted, a short one is
// looked up as a whole; returns true when it has to be merged (it then joins the list of misses).
__device__ __forceinline__ bool walk_one(int ss, const uint4* word_slots, uint32_t word_shift, int wlen, int* status)
{
  OptSmem& S   = g_tile;
  const int e  = next_cut(S.cut, ss);
  const int LL = e - ss;
  if (e >= kWindow && wlen == kWindow) {
    S.over_start = ss;  // runs past the window: finished in the HBM workspace
    return false;
  }
  if (LL > kThreadSegMax) {
    const int q = atomicAdd(&S.nlong, 1);
    if (q < kLongCap && GTK_IN(ss, kWindow, 3)) S.longq[q] = uint16_t(ss);
    else atomicMax(status, int(kStatusLongQueueOverflow));
    return false;
  }
  if (LL <= 12 && GTK_IN(ss, kWindow, 4)) {
    uint32_t k0, k1, k2;
    segment_key(S.bytes, 16 + ss, LL, k0, k1, k2);
    const uint32_t id = word_lookup(word_slots, word_shift, k0, k1, k2, uint32_t(LL));
    if (id != 0xFFFFFFFFu) {
      S.tok[ss] = uint16_t(id);
      return false;
    }
  }
  return true;
}

// Step D/E1 of a tile, out of line so that it gets registers of its own: every thread walks the multi-byte
// segments that start in its 16 positions (window positions [16*tid, 16*tid+16), owned ones only).
__device__ __noinline__ void walk_segments(const uint4* word_slots, uint32_t word_shift, int own, int wlen,
                                           int* status)
{
  OptSmem& S     = g_tile;
  const int tid  = threadIdx.x, lane = tid & 31;
  const uint32_t lt = lanemask_lt();
  const int base = tid * 16;
  uint32_t m16   = 0;
  if (base < own) {
    const uint32_t w32     = __funnelshift_r(S.cut[tid >> 1], S.cut[(tid >> 1) + 1], (tid & 1) * 16);
    const uint32_t ownmask = (base + 16 <= own) ? 0xFFFFu : ((1u << (own - base)) - 1u);
    m16 = w32 & ~(w32 >> 1) & ownmask;  // starts whose next position is not a start
  }
#ifdef GTK_PHASE_TIMING
  atomicAdd(&S.nseg, __popc(m16));
#endif
  while (__any_sync(0xFFFFFFFFu, m16 != 0)) {
    bool miss = false;
    int ss    = 0;
    if (m16) {
      ss = base + __ffs(int(m16)) - 1;
      m16 &= m16 - 1;
      miss = walk_one(ss, word_slots, word_shift, wlen, status);
    }
    const uint32_t bal = __ballot_sync(0xFFFFFFFFu, miss);
    if (bal) {
      int wbase = 0;
      if (lane == 0) wbase = atomicAdd(&S.nmiss, __popc(bal));
      wbase = __shfl_sync(0xFFFFFFFFu, wbase, 0);
      if (miss && GTK_IN(wbase + __popc(bal & lt), kSegCap, 5)) S.seg[wbase + __popc(bal & lt)] = uint16_t(ss);
    }
  }
}

// The same step for a CTA that has its SM to itself (small batches, one tile at a time): the segments are listed
// first (block-wide scan of the per-thread counts) and then dealt out one per thread and round.  A 512-byte text,
// whose segments all start in the positions of the first 32 threads, is then looked up in one round of table loads
// instead of one round per segment of the busiest thread.
__device__ __noinline__ void walk_segments_cta(const uint4* word_slots, uint32_t word_shift, int own, int wlen,
                                               int* status)
{
  OptSmem& S     = g_tile;
  const int tid  = threadIdx.x, lane = tid & 31;
  const uint32_t lt = lanemask_lt();
  const int base = tid * 16;
  uint32_t m16   = 0;
  if (base < own) {
    const uint32_t w32     = __funnelshift_r(S.cut[tid >> 1], S.cut[(tid >> 1) + 1], (tid & 1) * 16);
    const uint32_t ownmask = (base + 16 <= own) ? 0xFFFFu : ((1u << (own - base)) - 1u);
    m16 = w32 & ~(w32 >> 1) & ownmask;
  }
  constexpr int kListAt = kSegCap / 2, kListCap = kSegCap - kListAt;  // upper half of seg; misses fill the lower
  int total;
  int at = block_exclusive_scan(__popc(m16), S.scanbuf, &total);
  if (total > kListCap) {  // CTA-uniform: too many for the list, walk per thread
    walk_segments(word_slots, word_shift, own, wlen, status);
    return;
  }
  for (uint32_t m = m16; m; m &= m - 1) S.seg[kListAt + at++] = uint16_t(base + __ffs(int(m)) - 1);
  __syncthreads();
  for (int g0 = 0; g0 < total; g0 += kOptThreads) {
    const int g = g0 + tid;
    bool miss   = false;
    int ss      = 0;
    if (g < total) {
      ss   = S.seg[kListAt + g];
      miss = walk_one(ss, word_slots, word_shift, wlen, status);
    }
    const uint32_t bal = __ballot_sync(0xFFFFFFFFu, miss);
    if (bal) {
      int wbase = 0;
      if (lane == 0) wbase = atomicAdd(&S.nmiss, __popc(bal));
      wbase = __shfl_sync(0xFFFFFFFFu, wbase, 0);
      if (miss && GTK_IN(wbase + __popc(bal & lt), kListAt, 5)) S.seg[wbase + __popc(bal & lt)] = uint16_t(ss);
    }
  }
}

// The segment-start bitmap turns into the bitmap of live tokens as segments finish: the first token of a
// segment is always live, so a finished segment adds the bits of its other live slots (`a`, relative to
// its start s; bit 0 is ignored).  Only bits inside the segment change, so next_cut() of any other
// segment still finds the same end.
__device__ __forceinline__ void mark_alive(uint32_t* cut, int s, uint32_t a)
{
  a &= ~1u;
  if (!a) return;
  const int sh = s & 31;
  if (!GTK_IN((s >> 5) + 1, kCutWords + 2, 6)) return;
  atomicOr(&cut[s >> 5], a << sh);
  if (sh && (a >> (32 - sh))) atomicOr(&cut[(s >> 5) + 1], a >> (32 - sh));
}

// one warp: positions [lo, hi) become live
__device__ __forceinline__ void mark_alive_range(uint32_t* cut, int lo, int hi, int lane)
{
  if (hi <= lo || !GTK_IN(hi - 1, kWindow, 7) || !GTK_IN(lo, kWindow, 7)) return;
  for (int w = (lo >> 5) + lane; w <= ((hi - 1) >> 5); w += 32) {
    uint32_t x = 0xFFFFFFFFu;
    if (w == (lo >> 5)) x &= 0xFFFFFFFFu << (lo & 31);
    if (w == ((hi - 1) >> 5)) x &= 0xFFFFFFFFu >> (31 - ((hi - 1) & 31));
    atomicOr(&cut[w], x);
  }
}

// Per-CTA set-up shared by the kernels that process tiles: never-merge bitmap into shared memory and
// the all-ones sentinel words behind the segment-start bitmap.
__device__ __forceinline__ void opt_tile_setup(OptSmem& S, const DeviceTable& T)
{
  if (threadIdx.x < 2) S.cut[kCutWords + threadIdx.x] = 0xFFFFFFFFu;
}

// Reset of the per-tile words; call by one thread, then __syncthreads().
__device__ __forceinline__ void opt_tile_reset(OptSmem& S)
{
  S.nlong       = 0;
  S.nseg        = 0;
  S.seg_next    = 0;
  S.nmiss       = 0;
  S.first_start = kWindow;
  S.last_start  = -1;
  S.over_start  = -1;
  S.over_len    = 0;
  S.end_owned   = 0;
}

// One tile of the byte stream: tokenises every segment that starts in bytes [k*kTile, (k+1)*kTile),
// writes the tokens compacted to staging, the unit record and the per-chunk counts.
// SEQ: the tiles of a batch are walked in order by one CTA (small batches); the tile then writes its ids and the
// id offsets of its chunks straight to the output, at the running id count kept in S.run_base, instead of going
// through staging, counts, scans and pack.
template <bool SEQ>
__device__ __forceinline__ void opt_tile(OptSmem& S, const EncodeBuffers& b, const DeviceTable& T, int64_t k,
                                         int64_t C)
{
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lt = lanemask_lt();
  const int64_t n   = b.n_bytes;
  int* status       = b.counters + 1;
  const bool aligned = (reinterpret_cast<uintptr_t>(b.bytes) & 15u) == 0;
  const bool identity_ids = T.byte_ids_identity != 0;
#ifdef GTK_PHASE_TIMING
  long long phase_t0 = clock64();
#endif
  {
    const int64_t lo = k * kTile;
    const int wlen   = int(min(int64_t(kWindow), n - lo));
    const int own    = int(min(int64_t(kTile), n - lo));

    // ---- A. stage the window ----
    if (aligned) {
      for (int v = tid; v < kWindow / 16; v += kOptThreads) {
        const int64_t pos = lo + int64_t(v) * 16;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (pos + 16 <= n) {
          x = __ldg(reinterpret_cast<const uint4*>(b.bytes + pos));
        } else if (pos < n) {
          uint8_t tmp[16];
          for (int j = 0; j < 16; ++j) tmp[j] = (pos + j < n) ? b.bytes[pos + j] : uint8_t(0);
          x = *reinterpret_cast<uint4*>(tmp);
        }
        *reinterpret_cast<uint4*>(&S.bytes[16 + v * 16]) = x;
      }
    } else {
      for (int i = tid; i < kWindow; i += kOptThreads) S.bytes[16 + i] = (lo + i < n) ? b.bytes[lo + i] : uint8_t(0);
    }
    if (tid == 0) S.bytes[15] = (lo > 0) ? b.bytes[lo - 1] : uint8_t(0);
    __syncthreads();

    GTK_PHASE(0);
    // Only the 32-position words that hold text are processed; the words behind them are all
    // "segment start" (the window may be shorter than a tile at the end of the text or in small batches).
    const int used_words  = (wlen + 31) >> 5;
    const int used_groups = used_words * 8;
    if (tid >= used_words && tid < kCutWords) S.cut[tid] = 0xFFFFFFFFu;
    // ---- B. segment starts from the never-merge bitmap, initial ids and byte-pair ranks.
    //         Four consecutive positions per thread; eight lanes assemble one 32-bit bitmap word ----
    for (int g = tid; g < used_groups; g += kOptThreads) {
      const int i0     = g * 4;
      const uint32_t w = *reinterpret_cast<const uint32_t*>(&S.bytes[16 + i0]);
      uint32_t by[6];
      by[0] = S.bytes[15 + i0];
      by[1] = w & 0xFFu;
      by[2] = (w >> 8) & 0xFFu;
      by[3] = (w >> 16) & 0xFFu;
      by[4] = w >> 24;
      by[5] = S.bytes[20 + i0];
      // one 16-bit table entry per byte pair answers both questions: can this boundary ever merge
      // (anything but 0xFFFF), and what is the rank of the byte pair (values below 0xFFFE)
      uint32_t info[5];
#pragma unroll
      for (int k = 0; k < 5; ++k) info[k] = __ldg(T.byte_pair_info + ((by[k] << 8) | by[k + 1]));
      uint32_t nib = 0, t[4], r[4];
      if (i0 + 5 <= wlen && lo + i0 > 0) {  // the four positions and their right neighbours all hold text
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          nib |= uint32_t(info[k] == 0xFFFFu) << k;
          t[k] = identity_ids ? by[k + 1] : uint32_t(__ldg(T.byte_to_id + by[k + 1]));
          r[k] = (info[k + 1] < SEL) ? info[k + 1] : NONE;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int i      = i0 + k;
          const bool start = (i >= wlen) || (lo + i == 0) || (info[k] == 0xFFFFu);
          nib |= uint32_t(start) << k;
          t[k] = (i < wlen) ? (identity_ids ? by[k + 1] : uint32_t(__ldg(T.byte_to_id + by[k + 1]))) : DEAD;
          r[k] = ((i + 1 < wlen) && info[k + 1] < SEL) ? info[k + 1] : NONE;
        }
      }
      const uint32_t word = __reduce_or_sync(0xFFu << (lane & 24), nib << (4 * (lane & 7)));
      if ((lane & 7) == 0) S.cut[g >> 3] = word;
      *reinterpret_cast<uint2*>(&S.tok[i0]) = make_uint2(t[0] | (t[1] << 16), t[2] | (t[3] << 16));
      *reinterpret_cast<uint2*>(&S.rk[i0])  = make_uint2(r[0] | (r[1] << 16), r[2] | (r[3] << 16));
    }
    __syncthreads();

    GTK_PHASE(1);
    // ---- C. chunk boundaries are segment starts too ----
    {
      const int64_t c0 = b.tile_chunk0[k];
      for (int64_t c = c0 + tid; c <= C; c += kOptThreads) {
        const int64_t p = b.chunk_off[c] - lo;
        if (p >= wlen) break;
        if (p >= 0 && GTK_IN(p, kWindow, 28)) {
          atomicOr(&S.cut[p >> 5], 1u << (p & 31));
          if (p > 0) S.rk[p - 1] = uint16_t(NONE);
        }
      }
    }
    __syncthreads();

    GTK_PHASE(2);
    // ---- D/E1. every thread walks the multi-byte segments that start in its 16 positions.
    //      Whole-segment lookup: a segment whose bytes are a vocabulary string that the greedy rule
    //      collapses to one id is finished with two independent table loads; the others go to the
    //      list of misses (short), the warp queue (long) or the oversize slot (runs past the window) ----
    {
      if (tid < kTile / 32) {
        const int w0        = tid * 32;
        const uint32_t word = S.cut[tid];
        const uint32_t ownmask = (w0 + 32 <= own) ? 0xFFFFFFFFu : (w0 >= own ? 0u : ((1u << (own - w0)) - 1u));
        const uint32_t starts  = word & ownmask;
        if (starts) {
          const int last = w0 + 31 - __clz(int(starts));
          atomicMin(&S.first_start, w0 + __ffs(int(starts)) - 1);
          atomicMax(&S.last_start, last);
          // end of the owned region = end of the last owned segment, taken while the bitmap still holds
          // segment starts only (ends grow with starts, so the maximum is the last segment's end)
          atomicMax(&S.end_owned, next_cut(S.cut, last));
        }
      }
      if (SEQ) walk_segments_cta(T.word_slots, 32u - T.word_log2_capacity, own, wlen, status);
      else walk_segments(T.word_slots, 32u - T.word_log2_capacity, own, wlen, status);
    }
    __syncthreads();
    GTK_PHASE(3);
    const int nmiss = S.nmiss;

    // ---- E1c. the misses, sorted by length (longest first) so that the lanes of a warp work on segments of
    //           similar length in step E2: thread j keeps entry j in registers while the list is rewritten ----
    if (nmiss > 32 && nmiss <= kOptThreads) {
      if (tid < 34) S.hist[tid] = 0;
      __syncthreads();
      int ss = 0, LL = 0, slot = 0;
      if (tid < nmiss) {
        ss   = S.seg[tid];
        LL   = next_cut(S.cut, ss) - ss;
        if (!GTK_IN(LL, 33, 8)) LL = 2;
        slot = atomicAdd(&S.hist[LL], 1);
      }
      __syncthreads();
      if (warp == 0) {  // exclusive prefix over lengths 32, 31, ... 2
        const int len = 32 - lane;
        const int v   = S.hist[len];
        int inc       = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int y = __shfl_up_sync(0xFFFFFFFFu, inc, d);
          if (lane >= d) inc += y;
        }
        S.hist[len] = inc - v;
      }
      __syncthreads();
      if (tid < nmiss && GTK_IN(S.hist[LL] + slot, kSegCap, 9)) S.seg[S.hist[LL] + slot] = uint16_t(ss);
      __syncthreads();
    }

#ifdef GTK_PHASE_TIMING
    if (tid == 0) {
      atomicAdd(&g_phase_cycles[10], (unsigned long long)nmiss);
      atomicAdd(&g_phase_cycles[11], (unsigned long long)S.nseg);
    }
#endif
    // ---- E2. short segments that missed the lookup: one thread per segment (the usual case), or, when a
    //          tile has more misses than threads, every lane pulls segments from a CTA-wide list and does one
    //          merge step per loop trip ----
    GTK_PHASE(12);
    if (nmiss <= kOptThreads) {
      // at most one segment per thread (the usual case): no queue, thread t takes entry t of the sorted list
      int s = -1, L = 0;
      if (tid < nmiss) {
        s = S.seg[tid];
        L = next_cut(S.cut, s) - s;
      }
      // The ranks go to the lane-interleaved scratch when the warp's longest segment fits its area (nobody
      // needs the staged bytes any more).
      // Two sizes only: every further copy of the loop costs instruction-cache hits on text with many long runs.
      const int wmax  = __reduce_max_sync(0xFFFFFFFFu, L);
      const int words = (wmax + 1) >> 1;
      const int area  = warp * 32 * kLaneWords;
      const int room  = min(kLaneWords, (kLaneScratchWords - area) / 32);
      const uint32_t all = (s < 0) ? 0u : ((L >= 32) ? 0xFFFFFFFFu : ((1u << L) - 1u));
      uint32_t alive;
      if (words > room) alive = thread_merge_segments(s, L, pair_table(T));
      else if (words <= 4) alive = thread_merge_segments_lanes<4>(s, L, pair_table(T), area, all);
      else alive = thread_merge_segments_lanes<8>(s, L, pair_table(T), area, all);
      if (s >= 0) mark_alive(S.cut, s, alive);
    } else {
      const int nseg   = nmiss;
      int s            = -1, L = 0;
      uint32_t alive   = 0, best = 0xFFFFFFFFu;
      bool drained     = false;
      const PairTable P = pair_table(T);
      for (;;) {
        const bool need   = (s < 0) && !drained;
        const uint32_t nb = __ballot_sync(0xFFFFFFFFu, need);
        if (nb) {
          const int leader = __ffs(int(nb)) - 1;
          int base         = 0;
          if (lane == leader) base = atomicAdd(&S.seg_next, __popc(nb));
          base = __shfl_sync(0xFFFFFFFFu, base, leader);
          if (need) {
            const int j = base + __popc(nb & lt);
            if (j >= nseg) {
              drained = true;
            } else {
              const int ss0 = S.seg[j];
              const int LL0 = next_cut(S.cut, ss0) - ss0;
              s     = ss0;
              L     = LL0;
              alive = (L >= 32) ? 0xFFFFFFFFu : ((1u << L) - 1u);
              best  = segment_argmin(S.rk, s, L);
            }
          }
        }
        if (!__any_sync(0xFFFFFFFFu, s >= 0)) {
          if (__all_sync(0xFFFFFFFFu, drained)) break;
          continue;
        }
        if (s >= 0 && !thread_merge_step(S.tok, S.rk, s, L, alive, best, P)) {
          mark_alive(S.cut, s, alive);
          s = -1;
        }
      }
    }
    __syncthreads();

    GTK_PHASE(13);
    GTK_PHASE(4);
    // ---- F. one warp per long segment ----
    {
      const int nl = min(S.nlong, kLongCap);
      for (int q = warp; q < nl; q += kOptThreads / 32) {
        const int s   = S.longq[q];
        const int L   = next_cut(S.cut, s) - s;
        if (!(GTK_IN(s, kWindow, 19) && GTK_IN(s + L, kWindow + 1, 20))) continue;
        const int len = group_merge_dense<1>(S.tok + s, S.rk + s, L, T, nullptr, status);  // ids at the front
        mark_alive_range(S.cut, s + 1, s + len, lane);
        __syncwarp();
      }
    }
    __syncthreads();

    GTK_PHASE(5);
    // ---- G/H. compact the owned region [first, end) into S.rk, then to staging ----
    const int first     = S.first_start;
    const int end_owned = min((S.over_start >= 0) ? S.over_start : S.end_owned, wlen);
    int total;
    {
      int cnt = 0;
      if (tid < used_words) {  // the bitmap now marks live tokens; keep the owned range [first, end_owned)
        const int w0 = tid * 32;
        uint32_t x   = S.cut[tid];
        x &= (first <= w0) ? 0xFFFFFFFFu : ((first >= w0 + 32) ? 0u : (0xFFFFFFFFu << (first - w0)));
        x &= (end_owned >= w0 + 32) ? 0xFFFFFFFFu : ((end_owned <= w0) ? 0u : ((1u << (end_owned - w0)) - 1u));
        S.cut[tid] = x;
        cnt        = __popc(x);
      }
      const int off = block_exclusive_scan(cnt, S.scanbuf, &total);
      if (tid < used_words) S.woff[tid] = uint16_t(off);
    }
    __syncthreads();
    for (int g = tid; g < used_groups; g += kOptThreads) {
      const int i0        = g * 4;
      const int sh        = 4 * (lane & 7);
      const uint32_t word = S.cut[g >> 3];
      uint32_t nib        = (word >> sh) & 0xFu;
      if (nib) {
        int d          = S.woff[g >> 3] + __popc(word & ((1u << sh) - 1u));
        const uint2 tk = *reinterpret_cast<const uint2*>(&S.tok[i0]);
        const uint32_t t[4] = {tk.x & 0xFFFFu, tk.x >> 16, tk.y & 0xFFFFu, tk.y >> 16};
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (((nib >> k) & 1u) && GTK_IN(d, kWindow, 21)) S.rk[d++] = uint16_t(t[k]);
      }
    }
    __syncthreads();
    if (SEQ) {
      // ---- single-CTA kernel: ids and chunk offsets go straight to the output ----
      // J'. a segment that runs past the window is merged first (its tokens follow the tile's own ones)
      int over_len         = 0;
      const uint16_t* wtok = nullptr;
      if (S.over_start >= 0) {  // CTA-uniform
        const int64_t gs0 = lo + S.over_start;
        if (tid == 0) {
          int64_t c = b.tile_chunk0[k];
          while (c + 1 < C && b.chunk_off[c + 1] <= gs0) ++c;
          S.over_end = b.chunk_off[c + 1];
        }
        __syncthreads();
        const int64_t cend = S.over_end;
        int64_t ge         = cend;
        for (int64_t pos = lo + kWindow; pos < cend; pos += kOptThreads) {
          const int64_t p = pos + tid;
          const bool cutp = (p < cend) && !adj_bit(T.adj, b.bytes[p - 1], b.bytes[p]);
          if (__syncthreads_or(cutp)) {
            if (cutp) atomicMin(reinterpret_cast<unsigned long long*>(&S.over_end), (unsigned long long)p);
            __syncthreads();
            ge = S.over_end;
            break;
          }
        }
        const int64_t L64 = ge - gs0;
        if (L64 > b.seg_scratch_tokens || b.seg_scratch == nullptr) {
          if (tid == 0) atomicMax(status, int(kStatusScratchTooSmall));
        } else {
          const int L   = int(L64);
          uint16_t* wt  = b.seg_scratch + int64_t(blockIdx.x) * 2 * b.seg_scratch_tokens;
          uint16_t* wrk = wt + b.seg_scratch_tokens;
          for (int i = tid; i < L; i += kOptThreads) {
            const uint32_t cur = b.bytes[gs0 + i];
            wt[i]  = __ldg(T.byte_to_id + cur);
            wrk[i] = (i + 1 < L) ? __ldg(T.byte_pair_rank + ((cur << 8) | b.bytes[gs0 + i + 1])) : uint16_t(NONE);
          }
          __syncthreads();
          over_len = group_merge<kOptThreads / 32, true>(wt, wrk, L, T, &S.gs, status);
          wtok     = wt;
        }
        __syncthreads();
      }
      const int64_t out_base = S.run_base;  // written by thread 0 behind the barrier at the end of the last tile
      const uint16_t* map    = b.low_id_map;
      for (int j = tid; j < total; j += kOptThreads) {
        const uint32_t t = S.rk[j];
        if (out_base + j < b.out_capacity)
          b.out_ids[out_base + j] = int32_t((map && t < 256u) ? uint32_t(__ldg(map + t)) : t);
      }
      for (int j = tid; j < over_len; j += kOptThreads) {
        const uint32_t t = wtok[j];
        if (out_base + total + j < b.out_capacity)
          b.out_ids[out_base + total + j] = int32_t((map && t < 256u) ? uint32_t(__ldg(map + t)) : t);
      }
      // id offset of every chunk that starts in this tile: the ids in front of the tile plus the live tokens of the
      // tile in front of the chunk's first byte (a chunk start is a segment start, so it lies inside the owned
      // region, or is the start of the oversize segment right behind it)
      const int64_t c0 = b.tile_chunk0[k];
      for (int64_t c = c0 + tid; c < C; c += kOptThreads) {
        const int64_t p64 = b.chunk_off[c] - lo;
        if (p64 >= own) break;
        if (p64 >= 0) {
          const int p = int(p64);
          const int64_t at = out_base + S.woff[p >> 5] + __popc(S.cut[p >> 5] & ((1u << (p & 31)) - 1u));
          b.chunk_id_off[c]    = at;
          b.chunk_id_mirror[c] = at;
        }
      }
      __syncthreads();
      if (tid == 0) {
        S.run_base = out_base + total + over_len;
        if (k == b.n_tiles - 1) {  // the tile with the last byte closes the offsets
          b.chunk_id_off[C]    = S.run_base;
          b.chunk_id_mirror[C] = S.run_base;
        }
      }
      return;
    }
    const int64_t region_start = lo + ((first < kWindow) ? first : 0);
    for (int j = tid; j < total; j += kOptThreads)
      if (GTK_IN(j, kWindow, 22) && GTK_IN(region_start + j, n, 23)) b.staging[region_start + j] = S.rk[j];

    GTK_PHASE(6);
    // ---- I. per-chunk token counts from the alive bitmap ----
    {
      const int64_t region_end = lo + end_owned;
      const int64_t c0         = b.tile_chunk0[k];
      if (c0 < C && region_end <= b.chunk_off[c0 + 1]) {
        // the owned region lies inside the chunk that holds the tile's first byte (CTA-uniform test):
        // the count is the tile's total
        if (tid == 0 && total > 0 && GTK_IN(c0, b.chunk_cap, 24)) atomicAdd(b.chunk_cnt + c0, total);
      } else
      for (int64_t c = c0 + warp; c < C; c += kOptThreads / 32) {
        const int64_t cs_g = b.chunk_off[c];
        if (cs_g >= region_end) break;
        const int64_t ce_g = b.chunk_off[c + 1];
        const int cs = int(max(cs_g, region_start) - lo);
        const int ce = int(min(ce_g, region_end) - lo);
        if (ce <= cs) continue;
        int cnt = 0;
        for (int w = (cs >> 5) + lane; w <= ((ce - 1) >> 5); w += 32) {
          uint32_t x = S.cut[w];
          if (w == (cs >> 5)) x &= 0xFFFFFFFFu << (cs & 31);
          if (w == ((ce - 1) >> 5)) x &= 0xFFFFFFFFu >> (31 - ((ce - 1) & 31));
          cnt += __popc(x);
        }
        cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
        if (lane == 0 && cnt && GTK_IN(c, b.chunk_cap, 25)) atomicAdd(b.chunk_cnt + c, cnt);
      }
    }

    GTK_PHASE(7);
    // ---- J. a segment that runs past the window (rare): whole CTA, HBM workspace ----
    if (S.over_start >= 0) {  // CTA-uniform
      const int64_t gs0 = lo + S.over_start;
      if (tid == 0) {
        int64_t c = b.tile_chunk0[k];
        while (c + 1 < C && b.chunk_off[c + 1] <= gs0) ++c;
        S.over_chunk = int(c);
        S.over_end   = b.chunk_off[c + 1];
      }
      __syncthreads();
      // first never-merge boundary after the window, at most the chunk end
      const int64_t cend = S.over_end;
      int64_t ge         = cend;
      for (int64_t pos = lo + kWindow; pos < cend; pos += kOptThreads) {
        const int64_t p = pos + tid;
        const bool cutp = (p < cend) && !adj_bit(T.adj, b.bytes[p - 1], b.bytes[p]);
        if (__syncthreads_or(cutp)) {
          if (cutp) atomicMin(reinterpret_cast<unsigned long long*>(&S.over_end), (unsigned long long)p);
          __syncthreads();
          ge = S.over_end;
          break;
        }
      }
      const int64_t L64 = ge - gs0;
      if (L64 > b.seg_scratch_tokens || b.seg_scratch == nullptr) {
        if (tid == 0) atomicMax(status, int(kStatusScratchTooSmall));
      } else {
        const int L    = int(L64);
        uint16_t* wtok = b.seg_scratch + int64_t(blockIdx.x) * 2 * b.seg_scratch_tokens;
        uint16_t* wrk  = wtok + b.seg_scratch_tokens;
        for (int i = tid; i < L; i += kOptThreads) {
          const uint32_t cur = b.bytes[gs0 + i];
          wtok[i] = __ldg(T.byte_to_id + cur);
          wrk[i]  = (i + 1 < L) ? __ldg(T.byte_pair_rank + ((cur << 8) | b.bytes[gs0 + i + 1])) : uint16_t(NONE);
        }
        __syncthreads();
        const int len = group_merge<kOptThreads / 32, true>(wtok, wrk, L, T, &S.gs, status);
        for (int j = tid; j < len; j += kOptThreads)
          if (GTK_IN(region_start + total + j, n, 26)) b.staging[region_start + total + j] = wtok[j];
        if (tid == 0 && GTK_IN(S.over_chunk, b.chunk_cap, 27)) {
          atomicAdd(b.chunk_cnt + S.over_chunk, len);
          S.over_len = len;
        }
      }
      __syncthreads();
    }

    GTK_PHASE(8);
    // ---- K. unit record ----
    if (tid == 0) {
      b.unit_first[k] = region_start;
      b.unit_cnt[k]   = total + S.over_len;
    }
  }
}

// Six CTAs per SM (40 registers per thread) measured faster than eight (32 registers, 120 bytes of spills): the
// shared memory the two missing CTAs leave free becomes L1 for the table probes.
#ifndef GTK_OPT_CTAS
#define GTK_OPT_CTAS 6
#endif
__global__ void __launch_bounds__(kOptThreads, GTK_OPT_CTAS) k_merge_opt(EncodeBuffers b, DeviceTable T)
{
  OptSmem& S = g_tile;
  const int tid   = threadIdx.x;
  const int64_t C = b.totals[0];
  opt_tile_setup(S, T);
  for (;;) {
    __syncthreads();
    if (tid == 0) {
      S.ticket = atomicAdd(b.counters + 0, 1);
      opt_tile_reset(S);
    }
    __syncthreads();
    const int64_t k = S.ticket;
    if (k >= b.n_tiles) break;
    opt_tile<false>(S, b, T, k, C);
  }
}

// ------------------------------------------------------------------------------------------------
// small batches (latency mode): ONE kernel, one CTA, does the chunker, every tile, the output
// scans and the pack.  Input and output pointers may be mapped host memory, so a call is one
// launch and one stream synchronisation.
// ------------------------------------------------------------------------------------------------

// single-CTA exclusive scan of f(0..n) into out[0..n] (int64); returns the total to every thread
template <class F>
__device__ int64_t cta_exclusive_scan(F f, int64_t n, int64_t* out, int* scanbuf, int64_t* carry_s)
{
  if (threadIdx.x == 0) *carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += kOptThreads) {
    const int64_t i = base + threadIdx.x;
    const int v     = (i < n) ? int(f(i)) : 0;
    int total;
    const int off       = block_exclusive_scan(v, scanbuf, &total);
    const int64_t carry = *carry_s;
    if (i < n) out[i] = carry + off;
    __syncthreads();
    if (threadIdx.x == 0) *carry_s = carry + total;
    __syncthreads();
  }
  const int64_t total = *carry_s;
  if (threadIdx.x == 0) out[n] = total;
  __syncthreads();
  return total;
}

// The scans of a medium batch, one CTA of kMediumThreads: rounds of four items per thread.  The items are
// evaluated in lane order (coalesced loads) into shared memory and scanned in blocks of four per thread (each
// thread then writes 32 contiguous bytes of offsets).
constexpr int kMediumThreads = 1024;  // more warps hide the latency of the dependent loads of a single CTA
template <class F>
__device__ int64_t cta_exclusive_scan_medium(F f, int64_t n, int64_t* out, int* scanbuf, int64_t* carry_s, int* stage)
{
  constexpr int E = 4;
  const int tid = threadIdx.x;
  if (tid == 0) *carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += int64_t(kMediumThreads) * E) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int64_t i = base + e * kMediumThreads + tid;
      stage[e * kMediumThreads + tid] = (i < n) ? int(f(i)) : 0;
    }
    __syncthreads();
    const int4 v = reinterpret_cast<const int4*>(stage)[tid];
    int total;
    const int off       = block_exclusive_scan(v.x + v.y + v.z + v.w, scanbuf, &total);
    const int64_t first = base + int64_t(tid) * E;
    const int64_t r0    = *carry_s + off;
    const int64_t r[4]  = {r0, r0 + v.x, r0 + v.x + v.y, r0 + v.x + v.y + v.z};
#pragma unroll
    for (int e = 0; e < E; ++e)
      if (first + e < n) out[first + e] = r[e];
    __syncthreads();
    if (tid == 0) *carry_s += total;
    __syncthreads();
  }
  const int64_t total = *carry_s;
  if (tid == 0) out[n] = total;
  __syncthreads();
  return total;
}

// Medium batches (a few thousand texts, chunks and tiles at most): the whole chunker in one single-CTA launch
// instead of five, and both output scans plus the text offsets in one instead of seven -- at these sizes the
// launches, not the work, are what the multi-block kernels cost.
constexpr int64_t kMediumMaxItems = 16384;

__global__ void __launch_bounds__(kMediumThreads) k_chunker_medium(EncodeBuffers b, int per_text)
{
  __shared__ int scanbuf[33];
  __shared__ int64_t carry_s;
  __shared__ __align__(16) int stage[4 * kMediumThreads];
  const int tid = threadIdx.x;
#ifdef GTK_PHASE_TIMING
  const long long m_t0 = clock64();
#endif
  // this launch also resets the call's counters and per-chunk counts (two memsets less on the host)
  if (tid < 16) b.counters[tid] = 0;
  for (int64_t c = tid; c <= b.chunk_cap; c += kMediumThreads) b.chunk_cnt[c] = 0;
  const int64_t C = cta_exclusive_scan_medium(ChunksPerText{b.text_off, b.chunk_bytes}, b.n_texts, b.text_chunk_base,
                                              scanbuf, &carry_s, stage);
#ifdef GTK_PHASE_TIMING
  if (tid == 0) g_phase_cycles[24] = (unsigned long long)(clock64() - m_t0);
#endif
  if (tid == 0) b.totals[0] = C;
  if (per_text) {
    // many short texts: every text writes the offsets of its own chunks and the first chunk of every tile that
    // starts inside one of them (no search); a thread takes the texts of up to 32 chunks, a warp the longer ones.
    // A medium batch has at most 2048 tiles, so byte offsets and chunk numbers fit 32 bits.
    constexpr int kLongTexts = 128;
    __shared__ int n_long;
    __shared__ int long_text[kLongTexts];
    const uint32_t cb = uint32_t(b.chunk_bytes);
    auto lay_chunk = [&](uint32_t c, uint32_t start, uint32_t end) {  // chunk c covers bytes [start, end)
      b.chunk_off[c] = start;
      for (uint32_t k = (start + kTile - 1) / kTile; k * kTile < end; ++k) b.tile_chunk0[k] = int32_t(c);
    };
    if (tid == 0) {
      b.chunk_off[C] = b.text_off[b.n_texts];
      n_long         = 0;
    }
    __syncthreads();
    for (int64_t t = tid; t < b.n_texts; t += kMediumThreads) {
      const uint32_t c0 = uint32_t(b.text_chunk_base[t]), nc = uint32_t(b.text_chunk_base[t + 1]) - c0;
      const uint32_t at = uint32_t(b.text_off[t]), to = uint32_t(b.text_off[t + 1]);
      if (nc == 1) {
        lay_chunk(c0, at, to);
      } else if (nc <= 32) {
        for (uint32_t c = 0; c < nc; ++c) lay_chunk(c0 + c, at + c * cb, min(at + (c + 1) * cb, to));
      } else {
        const int q = atomicAdd(&n_long, 1);
        if (q < kLongTexts) long_text[q] = int(t);
      }
    }
    __syncthreads();
#ifdef GTK_PHASE_TIMING
    if (tid == 0) g_phase_cycles[25] = (unsigned long long)(clock64() - m_t0);
#endif
    const int lane = tid & 31, warp = tid >> 5;
    if (n_long <= kLongTexts) {  // the usual case: the few long texts come from the list
      for (int q = warp; q < n_long; q += kMediumThreads / 32) {
        const int64_t t   = long_text[q];
        const uint32_t cc = uint32_t(b.text_chunk_base[t]), nn = uint32_t(b.text_chunk_base[t + 1]) - cc;
        const uint32_t at = uint32_t(b.text_off[t]), to = uint32_t(b.text_off[t + 1]);
        for (uint32_t c = lane; c < nn; c += 32) lay_chunk(cc + c, at + c * cb, min(at + (c + 1) * cb, to));
      }
      return;
    }
    for (int64_t t0 = int64_t(warp) * 32; t0 < b.n_texts; t0 += kMediumThreads) {
      const int64_t t   = t0 + lane;
      const uint32_t c0 = (t < b.n_texts) ? uint32_t(b.text_chunk_base[t]) : 0u;
      const uint32_t nc = (t < b.n_texts) ? uint32_t(b.text_chunk_base[t + 1]) - c0 : 0u;
      for (uint32_t m = __ballot_sync(0xFFFFFFFFu, nc > 32); m; m &= m - 1) {
        const int src     = __ffs(int(m)) - 1;
        const uint32_t cc = __shfl_sync(0xFFFFFFFFu, c0, src), nn = __shfl_sync(0xFFFFFFFFu, nc, src);
        const uint32_t at = uint32_t(b.text_off[t0 + src]), to = uint32_t(b.text_off[t0 + src + 1]);
        for (uint32_t c = lane; c < nn; c += 32) lay_chunk(cc + c, at + c * cb, min(at + (c + 1) * cb, to));
      }
    }
    return;
  } else {
    for (int64_t c = tid; c <= C; c += kMediumThreads) {
      if (c == C) {
        b.chunk_off[c] = b.text_off[b.n_texts];
        continue;
      }
      int64_t lo = 0, hi = b.n_texts;  // last t with text_chunk_base[t] <= c
      while (hi - lo > 1) {
        const int64_t mid = (lo + hi) >> 1;
        if (b.text_chunk_base[mid] <= c) lo = mid; else hi = mid;
      }
      b.chunk_off[c] = b.text_off[lo] + (c - b.text_chunk_base[lo]) * int64_t(b.chunk_bytes);
    }
  }
  __syncthreads();
  for (int64_t k = tid; k < b.n_tiles; k += kMediumThreads) {
    const int64_t pos = k * kTile;
    int64_t lo = 0, hi = C;  // last c with chunk_off[c] <= pos
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) >> 1;
      if (b.chunk_off[mid] <= pos) lo = mid; else hi = mid;
    }
    b.tile_chunk0[k] = int32_t(lo);
  }
}

__global__ void __launch_bounds__(kMediumThreads) k_scans_medium(EncodeBuffers b, int with_units)
{
  __shared__ int scanbuf[33];
  __shared__ int64_t carry_s;
  __shared__ __align__(16) int stage[4 * kMediumThreads];
  const int tid   = threadIdx.x;
  const int64_t C = b.totals[0];
  const int64_t N = cta_exclusive_scan_medium(CountsI32{b.chunk_cnt}, C, b.chunk_id_off, scanbuf, &carry_s, stage);
  if (tid == 0) b.totals[1] = N;
  if (with_units) cta_exclusive_scan_medium(CountsI32{b.unit_cnt}, b.n_tiles, b.unit_base, scanbuf, &carry_s, stage);
  if (b.text_id_off)
    for (int64_t t = tid; t <= b.n_texts; t += kMediumThreads) b.text_id_off[t] = b.chunk_id_off[b.text_chunk_base[t]];
}

__global__ void __launch_bounds__(kOptThreads) k_encode_small(EncodeBuffers b, DeviceTable T)
{
  OptSmem& S = g_tile;
  __shared__ int64_t carry_s;
  const int tid = threadIdx.x;
  unsigned long long t_start = 0;
  if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
  opt_tile_setup(S, T);
  if (tid < 4) b.counters[tid] = 0;
  // One text of a few chunks (the one-string-per-call case): its chunk table is arithmetic and lives in shared
  // memory, so nothing is read over PCIe but the text itself and no search or scan runs.
  constexpr int kFastChunks = 64;
  __shared__ int64_t s_chunk_off[kFastChunks + 1];
  __shared__ int32_t s_tile_chunk0[kSmallMaxBytes / kTile + 1];
  const int64_t one_c = (b.n_bytes + b.chunk_bytes - 1) / b.chunk_bytes;
  const bool one_text = b.n_texts == 1 && one_c <= kFastChunks;  // CTA-uniform
  int64_t C;
  if (one_text) {
    C = one_c;
    for (int64_t c = tid; c <= C; c += kOptThreads) s_chunk_off[c] = min(c * int64_t(b.chunk_bytes), b.n_bytes);
    for (int64_t k = tid; k < b.n_tiles; k += kOptThreads) s_tile_chunk0[k] = int32_t((k * kTile) / b.chunk_bytes);
    b.chunk_off   = s_chunk_off;
    b.tile_chunk0 = s_tile_chunk0;
  } else {
  if (b.text_off_copy) {  // one parallel read over PCIe instead of dependent reads in the searches below
    for (int64_t t = tid; t <= b.n_texts; t += kOptThreads) b.text_off_copy[t] = b.text_off[t];
    b.text_off = b.text_off_copy;
    __syncthreads();
  }
  // chunker: chunks per text -> offsets of every chunk -> first chunk of every tile
  C = cta_exclusive_scan(ChunksPerText{b.text_off, b.chunk_bytes}, b.n_texts, b.text_chunk_base,
                         S.scanbuf, &carry_s);
  for (int64_t c = tid; c <= C; c += kOptThreads) {
    if (c == C) {
      b.chunk_off[c] = b.text_off[b.n_texts];
      continue;
    }
    int64_t lo = 0, hi = b.n_texts;
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) >> 1;
      if (b.text_chunk_base[mid] <= c) lo = mid; else hi = mid;
    }
    b.chunk_off[c] = b.text_off[lo] + (c - b.text_chunk_base[lo]) * int64_t(b.chunk_bytes);
  }
  __syncthreads();
  for (int64_t k = tid; k < b.n_tiles; k += kOptThreads) {
    const int64_t pos = k * kTile;
    int64_t lo = 0, hi = C;
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) >> 1;
      if (b.chunk_off[mid] <= pos) lo = mid; else hi = mid;
    }
    b.tile_chunk0[k] = int32_t(lo);
  }
  }
  // tiles, one after the other; each writes its ids and the id offsets of the chunks that start in it
  if (tid == 0) S.run_base = 0;
  for (int64_t k = 0; k < b.n_tiles; ++k) {
    __syncthreads();
    if (tid == 0) opt_tile_reset(S);
    __syncthreads();
    opt_tile<true>(S, b, T, k, C);
  }
  __syncthreads();
  // the offsets of the texts follow from those of their chunks; the caller-visible chunk offsets may live in
  // mapped host memory, so they are read back from the copy in device memory
  if (one_text) {
    if (tid < 2) b.text_id_off[tid] = tid ? S.run_base : 0;
  } else {
    for (int64_t t = tid; t <= b.n_texts; t += kOptThreads) b.text_id_off[t] = b.chunk_id_mirror[b.text_chunk_base[t]];
  }
  // The results may live in mapped host memory and the host may be polling totals[3] instead of waiting for the
  // stream: every store of this CTA is made visible system-wide before the call number goes out as the last one.
  __syncthreads();
  if (tid == 0) {
    unsigned long long t_end;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
    b.totals[0] = C;
    b.totals[1] = S.run_base;
    b.totals[2] = int64_t(b.counters[1]);
    b.totals[4] = int64_t(t_end - t_start);
    __threadfence_system();
    *reinterpret_cast<volatile int64_t*>(b.totals + 3) = b.small_seq;
  }
}

// ------------------------------------------------------------------------------------------------
// merge kernel, one CTA per chunk ("base")
// ------------------------------------------------------------------------------------------------
extern __shared__ __align__(16) unsigned char g_dyn_smem[];

// The chunk lives in dynamic shared memory (tokens and cached ranks, 16 bits each, `smem_tokens` slots per
// array); a chunk longer than that takes the HBM workspace.  NW warps per CTA: few for short chunks (the cost
// of a pass is dominated by its fixed part, so many small CTAs per SM give the best throughput), many for
// long ones.
template <int NW>
__global__ void __launch_bounds__(NW * 32) k_merge_base(EncodeBuffers b, DeviceTable T, int smem_tokens)
{
  constexpr int G = NW * 32;
  uint16_t* s_tok = reinterpret_cast<uint16_t*>(g_dyn_smem);
  uint16_t* s_rk  = s_tok + smem_tokens;
  __shared__ GroupScratch gs;
  __shared__ int ticket;
  const int tid   = threadIdx.x;
  const int64_t C = b.totals[0];
  int* status     = b.counters + 1;
  for (;;) {
    __syncthreads();
    if (tid == 0) ticket = atomicAdd(b.counters + 2, 1);
    __syncthreads();
    const int64_t c = ticket;
    if (c >= C) break;
    const int64_t cs  = b.chunk_off[c];
    const int64_t L64 = b.chunk_off[c + 1] - cs;
    uint16_t *tok = s_tok, *rk = s_rk;
    if (L64 > smem_tokens) {
      if (L64 > b.seg_scratch_tokens || b.seg_scratch == nullptr) {
        if (tid == 0) {
          atomicMax(status, int(kStatusScratchTooSmall));
          b.chunk_cnt[c] = 0;
        }
        continue;
      }
      tok = b.seg_scratch + int64_t(blockIdx.x) * 2 * b.seg_scratch_tokens;
      rk  = tok + b.seg_scratch_tokens;
    }
    const int L = int(L64);
    for (int i = tid; i < L; i += G) {
      const uint32_t cur = b.bytes[cs + i];
      tok[i] = __ldg(T.byte_to_id + cur);
      rk[i]  = (i + 1 < L) ? __ldg(T.byte_pair_rank + ((cur << 8) | b.bytes[cs + i + 1])) : uint16_t(NONE);
    }
    __syncthreads();
    const int len = group_merge<NW, true>(tok, rk, L, T, &gs, status);
    for (int j = tid; j < len; j += G)
      if (GTK_IN(cs + j, b.n_bytes, 31)) b.staging[cs + j] = tok[j];
    if (tid == 0) b.chunk_cnt[c] = len;
  }
}

// ------------------------------------------------------------------------------------------------
// Merge tables whose ids or ranks do not fit 16 bits (beyond roughly 65 000 merges): one CTA per chunk, 32-bit
// tokens and ranks (shared memory up to kWideSmemTokens tokens, else the HBM workspace), the pass-by-pass
// merge with a compaction in every pass, probes into the 16-byte-slot table.  The reference carries int32
// ids and a 64-bit pair key and so accepts any merges file (gputok_blockbpe.cu:139-157); this kernel keeps
// that property for the GPU entry points at the speed of the literal design.
// ------------------------------------------------------------------------------------------------
constexpr int kWideThreads    = 256;
constexpr int kWideSmemTokens = 4096;

__global__ void __launch_bounds__(kWideThreads) k_merge_wide(EncodeBuffers b, DeviceTable T)
{
  __shared__ __align__(16) uint32_t s_tok[kWideSmemTokens];
  __shared__ __align__(16) uint32_t s_rk[kWideSmemTokens];
  __shared__ GroupScratch gs;
  __shared__ int ticket;
  const int tid   = threadIdx.x;
  const int64_t C = b.totals[0];
  int* status     = b.counters + 1;
  for (;;) {
    __syncthreads();
    if (tid == 0) ticket = atomicAdd(b.counters + 2, 1);
    __syncthreads();
    const int64_t c = ticket;
    if (c >= C) break;
    const int64_t cs  = b.chunk_off[c];
    const int64_t L64 = b.chunk_off[c + 1] - cs;
    uint32_t *tok = s_tok, *rk = s_rk;
    if (L64 > kWideSmemTokens) {
      if (L64 > b.seg_scratch_tokens || b.seg_scratch32 == nullptr) {
        if (tid == 0) {
          atomicMax(status, int(kStatusScratchTooSmall));
          b.chunk_cnt[c] = 0;
        }
        continue;
      }
      tok = b.seg_scratch32 + int64_t(blockIdx.x) * 2 * b.seg_scratch_tokens;
      rk  = tok + b.seg_scratch_tokens;
    }
    const int L = int(L64);
    for (int i = tid; i < L; i += kWideThreads) {
      const uint32_t cur = __ldg(T.byte_to_id + b.bytes[cs + i]);
      tok[i] = cur;
      rk[i]  = (i + 1 < L) ? probe_rank_wide(T, cur, __ldg(T.byte_to_id + b.bytes[cs + i + 1])) : 0xFFFFFFFFu;
    }
    __syncthreads();
    const int len = group_merge_dense<kWideThreads / 32>(tok, rk, L, T, &gs, status);
    for (int j = tid; j < len; j += kWideThreads) b.staging32[cs + j] = int32_t(tok[j]);
    if (tid == 0) b.chunk_cnt[c] = len;
  }
}

// packs the staged 32-bit tokens of every chunk (one warp per chunk)
__global__ void __launch_bounds__(256) k_pack_wide(const int32_t* __restrict__ staging, const int64_t* __restrict__ first,
                                                   const int32_t* __restrict__ cnt, const int64_t* __restrict__ base,
                                                   const int64_t* n_units_ptr, int32_t* __restrict__ out,
                                                   int64_t capacity, const uint16_t* __restrict__ low_id_map)
{
  const int64_t U    = *n_units_ptr;
  const int lane     = threadIdx.x & 31;
  const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nw   = (int64_t(gridDim.x) * blockDim.x) >> 5;
  for (int64_t u = warp; u < U; u += nw) {
    const int64_t src = first[u], dst = base[u];
    int64_t m = cnt[u];
    if (dst + m > capacity) m = capacity > dst ? capacity - dst : 0;
    for (int64_t j = lane; j < m; j += 32) {
      const uint32_t t = uint32_t(staging[src + j]);
      out[dst + j] = int32_t((low_id_map && t < 256u) ? uint32_t(__ldg(low_id_map + t)) : t);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// local-minimum rule, one CTA per chunk (GTK_MODE_LOCALMIN).  The reference's tokenize_batch runs
// this rule, not Algorithm 1 (bpe_merge_kernel_optimized, gputok_binding.cu:290-414): per pass
// every adjacent pair gets its rank; a mergeable pair is merged unless its left neighbour ranks
// strictly lower or its right neighbour ranks lower or equal; all such pairs merge in the same
// pass; at most max_iters passes.  The reference compacts with one thread; here the compaction is
// the in-place ballot/popc routine.
// ------------------------------------------------------------------------------------------------
template <int NW>
__device__ int compact_tokens(uint16_t* tok, int len, GroupScratch* gs)
{
  constexpr int G = NW * 32, E = 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t lt = lanemask_lt();
  int out = 0;
  for (int base = 0; base < len; base += G * E) {
    uint16_t t[E];
    uint32_t bal[E];
    int wt = 0;
#pragma unroll
    for (int k = 0; k < E; ++k) {
      const int i = base + warp * 32 * E + k * 32 + lane;
      t[k]   = (i < len) ? tok[i] : uint16_t(DEAD);
      bal[k] = __ballot_sync(0xFFFFFFFFu, t[k] != DEAD);
      wt += __popc(bal[k]);
    }
    if (lane == 0) gs->wsum[warp] = uint32_t(wt);
    __syncthreads();
    int pre = 0, tot = 0;
    for (int w = 0; w < NW; ++w) {
      const int x = int(gs->wsum[w]);
      if (w < warp) pre += x;
      tot += x;
    }
    int o = out + pre;
#pragma unroll
    for (int k = 0; k < E; ++k) {
      if (t[k] != DEAD) tok[o + __popc(bal[k] & lt)] = t[k];
      o += __popc(bal[k]);
    }
    out += tot;
    __syncthreads();
  }
  return out;
}

__global__ void __launch_bounds__(kBaseThreads) k_merge_localmin(EncodeBuffers b, DeviceTable T, int max_iters)
{
  __shared__ __align__(16) uint16_t s_tok[kBaseSmemTokens];
  __shared__ __align__(16) uint16_t s_rk[kBaseSmemTokens];
  __shared__ GroupScratch gs;
  __shared__ int ticket;
  const int tid   = threadIdx.x;
  const int64_t C = b.totals[0];
  int* status     = b.counters + 1;
  for (;;) {
    __syncthreads();
    if (tid == 0) ticket = atomicAdd(b.counters + 2, 1);
    __syncthreads();
    const int64_t c = ticket;
    if (c >= C) break;
    const int64_t cs  = b.chunk_off[c];
    const int64_t L64 = b.chunk_off[c + 1] - cs;
    uint16_t *tok = s_tok, *rk = s_rk;
    if (L64 > kBaseSmemTokens) {
      if (L64 > b.seg_scratch_tokens || b.seg_scratch == nullptr) {
        if (tid == 0) {
          atomicMax(status, int(kStatusScratchTooSmall));
          b.chunk_cnt[c] = 0;
        }
        continue;
      }
      tok = b.seg_scratch + int64_t(blockIdx.x) * 2 * b.seg_scratch_tokens;
      rk  = tok + b.seg_scratch_tokens;
    }
    int len = int(L64);
    for (int i = tid; i < len; i += kBaseThreads) tok[i] = __ldg(T.byte_to_id + b.bytes[cs + i]);
    __syncthreads();
    for (int iter = 0; iter < max_iters && len >= 2; ++iter) {
      for (int i = tid; i < len - 1; i += kBaseThreads) rk[i] = uint16_t(probe_rank(T, tok[i], tok[i + 1]));
      __syncthreads();
      bool mine = false;
      for (int i = tid; i < len - 1; i += kBaseThreads) {
        const uint32_t r = rk[i];
        if (r == NONE) continue;
        if (i > 0 && uint32_t(rk[i - 1]) < r) continue;
        if (i + 1 < len - 1 && uint32_t(rk[i + 1]) <= r) continue;
        tok[i]     = uint16_t(merged_id(T, r));  // two kept positions are never adjacent
        tok[i + 1] = uint16_t(DEAD);
        mine       = true;
      }
      if (!__syncthreads_or(mine)) break;
      len = compact_tokens<kBaseThreads / 32>(tok, len, &gs);
    }
    for (int j = tid; j < len; j += kBaseThreads) b.staging[cs + j] = tok[j];
    if (tid == 0) b.chunk_cnt[c] = len;
  }
}

// ------------------------------------------------------------------------------------------------
// output: pack staged 16-bit tokens of every unit into the int32 id buffer
// ------------------------------------------------------------------------------------------------
// One warp per unit (a tile's or a chunk's compacted tokens): the ids of a unit are written in groups of
// four as one 16-byte store once the destination is aligned; the 16-bit source tokens are read through L1.
__global__ void __launch_bounds__(256) k_pack(const uint16_t* __restrict__ staging, const int64_t* __restrict__ first,
                                              const int32_t* __restrict__ cnt, const int64_t* __restrict__ base,
                                              int64_t n_units_imm, const int64_t* n_units_ptr,
                                              int32_t* __restrict__ out, int64_t capacity,
                                              const uint16_t* __restrict__ low_id_map)
{
  const int64_t U    = n_units_ptr ? *n_units_ptr : n_units_imm;
  const int lane     = threadIdx.x & 31;
  const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nw   = (int64_t(gridDim.x) * blockDim.x) >> 5;
  for (int64_t u = warp; u < U; u += nw) {
    const int64_t src = first[u], dst = base[u];
    int64_t m = cnt[u];
    if (dst + m > capacity) m = capacity > dst ? capacity - dst : 0;
    const uint16_t* sp = staging + src;
    int32_t* dp        = out + dst;
    auto conv = [&](uint32_t t) { return int32_t((low_id_map && t < 256u) ? uint32_t(__ldg(low_id_map + t)) : t); };
    // head: up to three ids until the destination is 16-byte aligned
    const int64_t head = min(m, int64_t(((16u - uint32_t(reinterpret_cast<uintptr_t>(dp) & 15u)) >> 2) & 3u));
    if (lane < head) dp[lane] = conv(sp[lane]);
    const int64_t quads = (m - head) >> 2;
    // four groups of four tokens per lane and trip: sixteen independent 16-bit loads in flight before the first
    // store, because this kernel lives on memory latency (one warp per unit, nothing to overlap with)
    for (int64_t q0 = lane; q0 < quads; q0 += 128) {
      uint32_t t[4][4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int64_t q = q0 + 32 * g;
        if (q < quads) {
          const uint16_t* s4 = sp + head + 4 * q;
#pragma unroll
          for (int e = 0; e < 4; ++e) t[g][e] = s4[e];
        }
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int64_t q = q0 + 32 * g;
        if (q < quads)
          *reinterpret_cast<int4*>(dp + head + 4 * q) = make_int4(conv(t[g][0]), conv(t[g][1]), conv(t[g][2]), conv(t[g][3]));
      }
    }
    const int64_t done = head + 4 * quads;
    if (done + lane < m) dp[done + lane] = conv(sp[done + lane]);
  }
}

__global__ void k_text_id_off(const int64_t* __restrict__ text_chunk_base, const int64_t* __restrict__ chunk_id_off,
                              int64_t n_texts, int64_t* __restrict__ text_id_off)
{
  for (int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; t <= n_texts; t += int64_t(gridDim.x) * blockDim.x)
    text_id_off[t] = chunk_id_off[text_chunk_base[t]];
}

inline unsigned grid_for(int64_t items, int threads, int64_t cap = 65535)
{
  int64_t g = (items + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return unsigned(g);
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------

// The scans have no dependent searches, so one CTA serves them up to a few thousand items; the chunker's binary
// searches (one per chunk and one per tile) are latency-bound in a single CTA and only pay while there are few.
static bool medium_scans(const EncodeBuffers& b)
{
  return b.n_texts <= kMediumMaxItems && b.chunk_cap <= kMediumMaxItems && b.n_tiles <= kMediumMaxItems;
}
// The single-CTA chunker finds the text of every chunk by binary search, which is cheap for a few texts and a few
// thousand chunks; a batch of many short texts (no more chunk-sized pieces than texts) is laid out per text instead.
static bool medium_chunker_by_search(const EncodeBuffers& b)
{
  return b.n_texts <= 256 && b.chunk_cap <= 2048 && b.n_tiles <= 1024;
}
static bool medium_chunker_per_text(const EncodeBuffers& b)
{
  return b.n_texts <= kMediumMaxItems && b.chunk_cap <= kMediumMaxItems && b.n_tiles <= 2048 &&
         b.chunk_cap <= 2 * b.n_texts + 1;
}

// true when the chunker is the single-CTA kernel, which also resets counters[0..16) and chunk_cnt[0..chunk_cap]
bool chunker_resets_counters(const EncodeBuffers& b)
{
  return medium_chunker_by_search(b) || medium_chunker_per_text(b);
}

int launch_chunker(const EncodeBuffers& b, cudaStream_t stream)
{
  if (medium_chunker_by_search(b) || medium_chunker_per_text(b)) {
    k_chunker_medium<<<1, kMediumThreads, 0, stream>>>(b, medium_chunker_by_search(b) ? 0 : 1);
    return 1;
  }
  int launches = run_scan(ChunksPerText{b.text_off, b.chunk_bytes}, b.n_texts, b.n_texts, nullptr,
                          b.scan_block_sums, b.text_chunk_base, b.totals + 0, stream);
  k_chunk_fill<<<grid_for(b.chunk_cap + 1, 256, 2048), 256, 0, stream>>>(b.text_off, b.text_chunk_base, b.n_texts,
                                                                         b.chunk_bytes, b.chunk_off);
  ++launches;
  if (b.n_tiles > 0) {
    k_tile_chunk0<<<grid_for(b.n_tiles, 256, 2048), 256, 0, stream>>>(b.chunk_off, b.totals + 0, b.n_tiles,
                                                                      b.tile_chunk0);
    ++launches;
  }
  return launches;
}

int launch_merge_opt(const EncodeBuffers& b, const DeviceTable& t, int grid, cudaStream_t stream)
{
  if (b.n_tiles <= 0) return 0;
  if (grid > b.n_tiles) grid = int(b.n_tiles);
  k_merge_opt<<<grid, kOptThreads, 0, stream>>>(b, t);
  return 1;
}

// Geometry of the one-CTA-per-chunk kernel for a chunk size: warps per CTA and slots of shared memory per array.
// block_threads = 0 picks the warp count from the chunk size; 64 .. 1024 (a power of two) forces it, which is what
// the reference's BLOCK_SIZE compile-time constant does (gputok_blockbpe.cu:313-315).
void base_kernel_geometry(int chunk_bytes, int block_threads, int* warps, int* smem_tokens)
{
  const int c  = std::max(chunk_bytes, 1);
  const int w  = block_threads > 0 ? block_threads / 32 : (c + 1023) >> 10;  // one warp per KiB of chunk
  *warps       = w <= 2 ? 2 : w <= 4 ? 4 : w <= 8 ? 8 : w <= 16 ? 16 : 32;
  *smem_tokens = (std::min(c, kBaseSmemMaxTokens) + 63) & ~63;
}

namespace {
template <int NW>
int base_blocks_per_sm(int smem_tokens)
{
  const int bytes = smem_tokens * 4;
  // opt in to the largest size any chunk length can ask for (a forced block size pairs any warp count with any
  // chunk length), so that handles with different chunk sizes on one device never lower each other's limit
  cudaFuncSetAttribute(k_merge_base<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBaseSmemMaxTokens * 4);
  int nb = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_merge_base<NW>, NW * 32, bytes);
  return nb;
}
}  // namespace

int launch_merge_base(const EncodeBuffers& b, const DeviceTable& t, int grid, int block_threads, cudaStream_t stream)
{
  if (b.n_bytes <= 0) return 0;
  if (grid > b.chunk_cap) grid = int(b.chunk_cap);
  if (grid < 1) grid = 1;
  int nw = 0, st = 0;
  base_kernel_geometry(b.chunk_bytes, block_threads, &nw, &st);
  const size_t bytes = size_t(st) * 4;
  switch (nw) {
    case 2: k_merge_base<2><<<grid, 64, bytes, stream>>>(b, t, st); break;
    case 4: k_merge_base<4><<<grid, 128, bytes, stream>>>(b, t, st); break;
    case 8: k_merge_base<8><<<grid, 256, bytes, stream>>>(b, t, st); break;
    case 16: k_merge_base<16><<<grid, 512, bytes, stream>>>(b, t, st); break;
    default: k_merge_base<32><<<grid, 1024, bytes, stream>>>(b, t, st); break;
  }
  return 1;
}

int launch_merge_wide(const EncodeBuffers& b, const DeviceTable& t, int grid, cudaStream_t stream)
{
  if (b.n_bytes <= 0) return 0;
  if (grid > b.chunk_cap) grid = int(b.chunk_cap);
  if (grid < 1) grid = 1;
  k_merge_wide<<<grid, kWideThreads, 0, stream>>>(b, t);
  return 1;
}

int launch_pack_wide(const EncodeBuffers& b, int grid, cudaStream_t stream)
{
  if (b.n_bytes <= 0) return 0;
  k_pack_wide<<<grid, 256, 0, stream>>>(b.staging32, b.chunk_off, b.chunk_cnt, b.chunk_id_off, b.totals + 0, b.out_ids,
                                        b.out_capacity, b.low_id_map);
  return 1;
}

int wide_kernel_max_blocks_per_sm()
{
  int nb = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_merge_wide, kWideThreads, 0);
  return nb;
}

int launch_merge_localmin(const EncodeBuffers& b, const DeviceTable& t, int grid, int max_iters, cudaStream_t stream)
{
  if (b.n_bytes <= 0) return 0;
  if (grid > b.chunk_cap) grid = int(b.chunk_cap);
  if (grid < 1) grid = 1;
  k_merge_localmin<<<grid, kBaseThreads, 0, stream>>>(b, t, max_iters);
  return 1;
}

int launch_output_scans(const EncodeBuffers& b, int mode_base, cudaStream_t stream)
{
  if (medium_scans(b)) {
    k_scans_medium<<<1, kMediumThreads, 0, stream>>>(b, (!mode_base && b.n_tiles > 0) ? 1 : 0);
    return 1;
  }
  int launches = 0;
  // per-chunk counts -> packed id offset of every chunk (+ total id count)
  launches += run_scan(CountsI32{b.chunk_cnt}, b.chunk_cap, 0, b.totals + 0, b.scan_block_sums, b.chunk_id_off,
                       b.totals + 1, stream);
  if (!mode_base && b.n_tiles > 0) {
    launches += run_scan(CountsI32{b.unit_cnt}, b.n_tiles, b.n_tiles, nullptr, b.scan_block_sums, b.unit_base,
                         nullptr, stream);
  }
  if (b.text_id_off) {
    k_text_id_off<<<grid_for(b.n_texts + 1, 256, 2048), 256, 0, stream>>>(b.text_chunk_base, b.chunk_id_off,
                                                                          b.n_texts, b.text_id_off);
    ++launches;
  }
  return launches;
}

int launch_pack(const EncodeBuffers& b, int mode_base, int grid, cudaStream_t stream)
{
  if (b.n_bytes <= 0) return 0;
  if (mode_base) {
    k_pack<<<grid, 256, 0, stream>>>(b.staging, b.chunk_off, b.chunk_cnt, b.chunk_id_off, 0, b.totals + 0, b.out_ids,
                                     b.out_capacity, b.low_id_map);
  } else {
    k_pack<<<grid, 256, 0, stream>>>(b.staging, b.unit_first, b.unit_cnt, b.unit_base, b.n_tiles, nullptr, b.out_ids,
                                     b.out_capacity, b.low_id_map);
  }
  return 1;
}

int launch_encode_small(const EncodeBuffers& b, const DeviceTable& t, cudaStream_t stream)
{
  k_encode_small<<<1, kOptThreads, 0, stream>>>(b, t);
  return 1;
}

#ifdef GTK_CHECKED
// Checked build only: the record of index checks that failed since the last reset ([0] id of the first failing
// check, [1] its value, [2] its limit, [3] number of failures), plus a self-test of the mechanism: a kernel
// evaluates one check that must fail and skips the guarded store.
__global__ void k_check_selftest(int* sink)
{
  const int bad = 5 + int(threadIdx.x);
  if (GTK_IN(bad, 4, 99)) sink[bad] = 1;
}

extern "C" __attribute__((visibility("default"))) int gtk_debug_check_words(int out[4], int reset, int selftest)
{
  if (selftest) {
    int* sink = nullptr;
    if (cudaMalloc(&sink, 64) != cudaSuccess) return -1;
    k_check_selftest<<<1, 1>>>(sink);
    cudaDeviceSynchronize();
    cudaFree(sink);
  }
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(out, g_check_words, sizeof(int) * 4) != cudaSuccess) return -1;
  if (reset) {
    const int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_check_words, z, sizeof(z));
  }
  return 0;
}
#endif

#ifdef GTK_PHASE_TIMING
extern "C" __attribute__((visibility("default"))) void gtk_debug_phase_cycles(unsigned long long out[32], int reset)
{
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, g_phase_cycles, sizeof(unsigned long long) * 32);
  if (reset) {
    unsigned long long z[32] = {};
    cudaMemcpyToSymbol(g_phase_cycles, z, sizeof(z));
  }
}
#endif

__global__ void k_publish_totals(const int64_t* totals, const int32_t* counters, int64_t* mapped)
{
  if (threadIdx.x == 0) {
    mapped[0] = totals[0];
    mapped[1] = totals[1];
    int32_t* c = reinterpret_cast<int32_t*>(mapped + 2);
    c[0] = counters[0];
    c[1] = counters[1];
    c[2] = counters[2];
    c[3] = counters[3];
    __threadfence_system();
  }
}

// Results of a batch that ran in one piece, from their device arena [text id offsets | chunk id offsets | ids] into
// mapped host memory: the first prefix_bytes (a multiple of 16) and the n_ids ids behind them, n_ids read from the
// totals on the device.  The CTA that finishes last (a counter, no waiting) publishes the totals and, as the very
// last store behind a system-wide fence, the call number that the host polls for.
__global__ void __launch_bounds__(256) k_results_to_host(const uint4* __restrict__ src, uint4* dst, int64_t prefix_bytes,
                                                         const int64_t* totals, int32_t* counters, int64_t* mapped,
                                                         int64_t seq)
{
  __shared__ int last;
  const int64_t n16 = (prefix_bytes + totals[1] * 4 + 15) / 16;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += int64_t(gridDim.x) * blockDim.x)
    dst[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) last = (atomicAdd(counters + 8, 1) == int(gridDim.x) - 1);
  __syncthreads();
  if (last && threadIdx.x == 0) {
    mapped[0] = totals[0];
    mapped[1] = totals[1];
    mapped[2] = int64_t(counters[1]);  // status word
    __threadfence_system();
    *reinterpret_cast<volatile int64_t*>(mapped + 3) = seq;
  }
}

// A batch of a few tiles whose chunk table the host has laid out (chunk_off, tile_chunk0, text_chunk_base):
// everything behind the tile kernel in one launch, one CTA per tile -- the CTA packs its tile's token run into int32
// ids (the runs' offsets are a sum over at most kFinishMaxTiles counts, which every CTA forms for itself), CTA 0
// also scans the per-chunk counts into id offsets (into chunk_id_mirror in HBM, then out) and writes the texts' id
// offsets -- straight into mapped host memory (b.chunk_id_off, b.text_id_off, b.out_ids point there).  The CTA
// that finishes last (a counter, no waiting) adds {n_chunks, n_ids, status} and, as the very last store behind a
// system-wide fence, the call number the host polls for.
__global__ void __launch_bounds__(kMediumThreads) k_finish_small_batch(EncodeBuffers b, int64_t* mapped, int64_t seq)
{
  __shared__ int scanbuf[33];
  __shared__ int64_t carry_s;
  __shared__ __align__(16) int stage[4 * kMediumThreads];
  __shared__ int64_t s_base, s_total;
  __shared__ int last;
  const int tid   = threadIdx.x;
  const int64_t u = blockIdx.x;
  const int64_t C = b.totals[0];
  if (tid == 0) {
    int64_t run = 0, base = 0;
    for (int64_t v = 0; v < b.n_tiles; ++v) {
      if (v == u) base = run;
      run += b.unit_cnt[v];
    }
    s_base  = base;
    s_total = run;
  }
  __syncthreads();
  const int64_t N = s_total;
  {
    const uint16_t* sp = b.staging + b.unit_first[u];
    int32_t* dp        = b.out_ids + s_base;
    int64_t m          = b.unit_cnt[u];
    if (s_base + m > b.out_capacity) m = b.out_capacity > s_base ? b.out_capacity - s_base : 0;
    for (int64_t i = tid; i < m; i += kMediumThreads) {
      const uint32_t t = sp[i];
      dp[i] = int32_t((b.low_id_map && t < 256u) ? uint32_t(__ldg(b.low_id_map + t)) : t);
    }
  }
  if (u == 0) {
    cta_exclusive_scan_medium(CountsI32{b.chunk_cnt}, C, b.chunk_id_mirror, scanbuf, &carry_s, stage);
    for (int64_t c = tid; c <= C; c += kMediumThreads) b.chunk_id_off[c] = b.chunk_id_mirror[c];
    for (int64_t t = tid; t <= b.n_texts; t += kMediumThreads) b.text_id_off[t] = b.chunk_id_mirror[b.text_chunk_base[t]];
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) last = (atomicAdd(b.counters + 8, 1) == int(gridDim.x) - 1);
  __syncthreads();
  if (last && tid == 0) {
    mapped[0] = C;
    mapped[1] = N;
    mapped[2] = int64_t(b.counters[1]);  // status word
    __threadfence_system();
    *reinterpret_cast<volatile int64_t*>(mapped + 3) = seq;
  }
}

int launch_finish_small_batch(const EncodeBuffers& b, int64_t* mapped, int64_t seq, cudaStream_t stream)
{
  k_finish_small_batch<<<unsigned(b.n_tiles), kMediumThreads, 0, stream>>>(b, mapped, seq);
  return 1;
}

int launch_results_to_host(const EncodeBuffers& b, const void* src, void* dst, int64_t prefix_bytes, int64_t* mapped,
                           int64_t seq, cudaStream_t stream)
{
  k_results_to_host<<<148, 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), prefix_bytes,
                                           b.totals, b.counters, mapped, seq);
  return 1;
}

int launch_publish_totals(const EncodeBuffers& b, int64_t* mapped, cudaStream_t stream)
{
  k_publish_totals<<<1, 32, 0, stream>>>(b.totals, b.counters, mapped);
  return 1;
}

int opt_kernel_max_blocks_per_sm()
{
  int nb = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_merge_opt, kOptThreads, 0);
  return nb;
}

// Call once per device and chunk size (that device current): opts the kernel in to its dynamic shared memory
// and returns the resident CTAs per SM.
int base_kernel_max_blocks_per_sm(int chunk_bytes, int block_threads)
{
  int nw = 0, st = 0;
  base_kernel_geometry(chunk_bytes, block_threads, &nw, &st);
  switch (nw) {
    case 2: return base_blocks_per_sm<2>(st);
    case 4: return base_blocks_per_sm<4>(st);
    case 8: return base_blocks_per_sm<8>(st);
    case 16: return base_blocks_per_sm<16>(st);
    default: return base_blocks_per_sm<32>(st);
  }
}

int localmin_kernel_max_blocks_per_sm()
{
  int nb = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_merge_localmin, kBaseThreads, 0);
  return nb;
}

}  // namespace gtk

// ------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in include/gputok_b200.h): the one-CTA-per-chunk merge
// kernel with its ticket counter, status word and long-chunk workspace in a fixed device array
// instead of buffers from cudaMalloc.
// ------------------------------------------------------------------------------------------------
#include "../../include/gputok_b200.h"

namespace {

constexpr int kNoAllocCtas        = 128;                          // persistent CTAs of the kernel
constexpr int kNoAllocMaxTokens   = GTK_NOALLOC_MAX_CHUNK_BYTES;  // longest chunk (one token per byte at most)
constexpr size_t kNoAllocHeader   = 256;                          // [0] chunk ticket, [1] status word
constexpr size_t kNoAllocPerCta   = size_t(2) * kNoAllocMaxTokens * sizeof(uint16_t);  // tokens + ranks
constexpr size_t kNoAllocBytes    = kNoAllocHeader + size_t(kNoAllocCtas) * kNoAllocPerCta;  // 8 MiB + 256 B
constexpr int kMaxDevices         = 64;

// Lives in the library image on every GPU that loads it.  In host code this name is only a
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

__global__ void __launch_bounds__(gtk::kBaseThreads)
k_merge_chunks_noalloc(const uint8_t* __restrict__ bytes, int64_t n_bytes, const int64_t* __restrict__ chunk_off,
                       int64_t n_chunks, int max_chunk, int32_t* __restrict__ out_ids,
                       int32_t* __restrict__ out_counts, gtk::DeviceTable T,
                       const uint16_t* __restrict__ low_id_map, unsigned char* scratch)
{
  using namespace gtk;
  __shared__ __align__(16) uint16_t s_tok[kBaseSmemTokens];
  __shared__ __align__(16) uint16_t s_rk[kBaseSmemTokens];
  __shared__ GroupScratch gs;
  __shared__ int ticket;
  const int tid   = threadIdx.x;
  int* counter    = reinterpret_cast<int*>(scratch);
  int* status     = counter + 1;
  uint16_t* w_tok = reinterpret_cast<uint16_t*>(scratch + kNoAllocHeader + size_t(blockIdx.x) * kNoAllocPerCta);
  uint16_t* w_rk  = w_tok + kNoAllocMaxTokens;
  for (;;) {
    __syncthreads();
    if (tid == 0) ticket = atomicAdd(counter, 1);
    __syncthreads();
    const int64_t c = ticket;
    if (c >= n_chunks) break;
    const int64_t cs  = chunk_off[c];
    const int64_t L64 = chunk_off[c + 1] - cs;
    // The offsets come from the caller's device memory and are used as indices below: a chunk that is not
    // inside bytes[0, n_bytes) is skipped (count 0) and reported through the status word, never touched.
    const bool outside = cs < 0 || L64 < 0 || cs > n_bytes || L64 > n_bytes - cs;
    if (outside || L64 == 0 || L64 > max_chunk) {
      if (tid == 0) {
        out_counts[c] = 0;
        if (outside) atomicMax(status, int(kStatusBadOffsets));
        else if (L64 != 0) atomicMax(status, int(kStatusScratchTooSmall));
      }
      continue;
    }
    const int L   = int(L64);
    uint16_t* tok = (L <= kBaseSmemTokens) ? s_tok : w_tok;
    uint16_t* rk  = (L <= kBaseSmemTokens) ? s_rk : w_rk;
    for (int i = tid; i < L; i += kBaseThreads) {
      const uint32_t cur = bytes[cs + i];
      tok[i] = __ldg(T.byte_to_id + cur);
      rk[i]  = (i + 1 < L) ? __ldg(T.byte_pair_rank + ((cur << 8) | bytes[cs + i + 1])) : uint16_t(NONE);
    }
    __syncthreads();
    const int len = group_merge<kBaseThreads / 32, true>(tok, rk, L, T, &gs, status);
    for (int j = tid; j < len; j += kBaseThreads) {
      const uint32_t t = tok[j];
      out_ids[cs + j]  = int32_t((low_id_map && t < 256u) ? uint32_t(__ldg(low_id_map + t)) : t);
    }
    if (tid == 0) out_counts[c] = len;
  }
}

// Device address of the fixed array, looked up once per device with that device current.
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_ptr[kMaxDevices] = {};

cudaError_t noalloc_scratch_for(int device, unsigned char** out)
{
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_noalloc_ptr[device] = static_cast<unsigned char*>(p);
  }
  *out = g_noalloc_ptr[device];
  return cudaSuccess;
}

}  // namespace

extern "C" GTK_API int gtk_encode_chunks_noalloc(gtk_tokenizer* h, const uint8_t* d_bytes, int64_t n_bytes,
                                                 const int64_t* d_chunk_offsets, int64_t n_chunks,
                                                 int32_t max_chunk_bytes, int32_t* d_out_ids, int32_t* d_out_counts)
{
  gtk::HandleView v;
  if (!gtk::handle_view(h, &v)) return GTK_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(*v.mu);
  auto fail = [&](int code, const std::string& msg) {
    *v.last_error = msg;
    return code;
  };
  if (v.device < 0) return fail(GTK_ERR_NO_DEVICE, "host-only handle: no GPU entry points");
  if (v.wide) return fail(GTK_ERR_TABLE, "the allocation-free entry point serves merge tables with ids < 65535 and ranks < 65534 only");
  if (v.device >= kMaxDevices) return fail(GTK_ERR_INVALID_ARG, "device ordinal beyond the supported range");
  if (n_chunks < 0 || n_bytes < 0 || max_chunk_bytes <= 0) return fail(GTK_ERR_INVALID_ARG, "negative or zero size");
  if (n_chunks > int64_t(0x7FFFFFF0)) return fail(GTK_ERR_INVALID_ARG, "more than 2^31 chunks in one call");
  if (max_chunk_bytes > GTK_NOALLOC_MAX_CHUNK_BYTES)
    return fail(GTK_ERR_CAPACITY, "max_chunk_bytes " + std::to_string(max_chunk_bytes) +
                                      " exceeds the allocation-free limit of " +
                                      std::to_string(GTK_NOALLOC_MAX_CHUNK_BYTES) + " bytes per chunk");
  if (n_chunks == 0) return GTK_OK;
  if (!d_bytes || !d_chunk_offsets || !d_out_ids || !d_out_counts) return fail(GTK_ERR_INVALID_ARG, "null device pointer");
  cudaError_t e = cudaSetDevice(v.device);
  unsigned char* scratch = nullptr;
  if (e == cudaSuccess) e = noalloc_scratch_for(v.device, &scratch);
  if (e != cudaSuccess) return fail(GTK_ERR_CUDA, std::string("fixed workspace lookup: ") + cudaGetErrorString(e));
  // the previous call's ticket and status words must start at zero
  e = cudaMemsetAsync(scratch, 0, kNoAllocHeader, v.stream);
  if (e != cudaSuccess) return fail(GTK_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  const int grid = int(n_chunks < kNoAllocCtas ? n_chunks : kNoAllocCtas);
  k_merge_chunks_noalloc<<<grid, gtk::kBaseThreads, 0, v.stream>>>(d_bytes, n_bytes, d_chunk_offsets, n_chunks,
                                                                   max_chunk_bytes, d_out_ids, d_out_counts, v.table,
                                                                   v.low_id_map, scratch);
  e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyAsync(v.pinned_words, scratch, 8, cudaMemcpyDeviceToHost, v.stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(v.stream);
  if (e != cudaSuccess) return fail(GTK_ERR_CUDA, std::string("allocation-free merge kernel: ") + cudaGetErrorString(e));
  const int status = v.pinned_words[1];
  if (status == gtk::kStatusBadOffsets)
    return fail(GTK_ERR_INVALID_ARG, "d_chunk_offsets must be non-decreasing and stay inside [0, n_bytes]: the "
                                     "offending chunks were skipped (count 0)");
  if (status == gtk::kStatusScratchTooSmall)
    return fail(GTK_ERR_CAPACITY, "a chunk is longer than max_chunk_bytes (" + std::to_string(max_chunk_bytes) + ")");
  if (status != gtk::kStatusOk) return fail(GTK_ERR_KERNEL, "merge pass made no progress");
  return GTK_OK;
}

