// Onesweep-style least-significant-digit radix sort (keys or key/value pairs) for sm_100a.
//
// Replaces the cub::DeviceRadixSort::SortKeys / SortPairs call of
// thrust/system/cuda/detail/sort.h:1343-1427.  Structure:
//   1. radix_hist_kernel      one read of the keys builds the 256-bin histogram of EVERY 8-bit
//                             digit place at once (shared-memory bins, then global atomics);
//   2. radix_scan_hist_kernel exclusive-scans each histogram into bucket bases and marks a digit
//                             place as skippable when one bucket holds every key;
//   3. onesweep_kernel        once per non-skipped digit place, persistent CTAs (two per SM) that take
//                             tiles by an atomic ticket: while a tile is processed the next tile's
//                             keys and values are already being loaded into registers.  A tile is
//                             ranked inside the CTA on per-warp shared-memory counters -- every lane
//                             increments its digit's counter, lanes of a warp that collide on a digit
//                             are ordered by a short ballot loop (about two ballots per 32 keys; a row
//                             with many collisions falls back to one ballot per digit bit) --, the
//                             tile's per-digit counts are published, keys and values are staged side
//                             by side in shared memory in bucket order, the counts are chained to the
//                             preceding tiles by decoupled look-back (one thread per digit, four
//                             descriptors fetched per round trip, bounded waits), and the pairs leave
//                             shared memory in one loop so that each bucket's run is written
//                             contiguously;
//   4. radix_copy_back_kernel only if an odd number of places ran: moves the result from the
//                             alternate buffer to the caller's.
// A pass therefore reads and writes each key (and value) exactly once.  The sort is stable.
// Key order is defined on an unsigned code of the key: unsigned keys unchanged, signed keys
// with the sign bit flipped, IEEE floats with all bits flipped when negative and the sign bit
// flipped otherwise (the encoders of thrust/system/detail/sequential/stable_radix_sort.inl:54-138);
// descending order complements the code.
#pragma once
#include "common.cuh"

namespace tb200 {

constexpr int RADIX_BITS = 8;
constexpr int RADIX_BINS = 256;
constexpr int RADIX_MAX_PASSES = 8;
#ifndef TB200_SWEEP_BLOCK
#define TB200_SWEEP_BLOCK 512
#endif
constexpr int ONESWEEP_BLOCK = TB200_SWEEP_BLOCK;
constexpr int ONESWEEP_CTAS_PER_SM = 1024 / ONESWEEP_BLOCK;
constexpr int HIST_BLOCK = 1024;

enum key_kind : int { KEY_UNSIGNED = 0, KEY_SIGNED = 1, KEY_FLOAT = 2 };

struct key_coding {
  int kind; int descending;
};

// Digit `shift / 8` of the key's order-preserving unsigned code.  For integer keys the code
// differs from the raw bits by a constant, so the digit is the raw byte XOR `dmask` (the matching
// byte of that constant); float keys first flip all bits of negative values.
template <class UK> __host__ __device__ __forceinline__ unsigned digit_mask(key_coding c, int shift) {
  constexpr int B = 8 * sizeof(UK);
  UK m = c.descending ? (UK)~(UK)0 : (UK)0;
  if (c.kind != KEY_UNSIGNED) m ^= (UK)1 << (B - 1);
  return (unsigned)(m >> shift) & 0xffu;
}
template <bool IS_FLOAT, class UK> __device__ __forceinline__ unsigned key_digit(UK k, int shift, unsigned dmask) {
  constexpr int B = 8 * sizeof(UK);
  if (IS_FLOAT) {
    using SK = typename std::make_signed<UK>::type;
    k ^= (UK)((SK)k >> (B - 1)) & (UK)~((UK)1 << (B - 1));   // negative: flip the non-sign bits too
  }
  return ((unsigned)(k >> shift) & 0xffu) ^ dmask;
}

// Control block in the workspace, after ws_header.
struct radix_ctrl {
  unsigned long long hist[RADIX_MAX_PASSES][RADIX_BINS];   // counts, then exclusive bases
  unsigned skip[RADIX_MAX_PASSES];                         // 1: every key shares this digit
  unsigned tickets[RADIX_MAX_PASSES];
  unsigned pad[48];
};

// ---------------------------------------------------------------- 1. histograms of all digit places
// One CTA per SM.  Shared memory holds, for every digit place, COPIES interleaved copies of the
// 256 bins; lane l only ever touches copy l % COPIES, so with 32 copies a warp's atomics never
// share a bank and a degenerate digit (every key equal) costs no more than a uniform one.
template <class UK> struct hist_tuning { static constexpr int COPIES = sizeof(UK) <= 4 ? 32 : 16; };

template <class UK, bool IS_FLOAT>
__global__ void __launch_bounds__(HIST_BLOCK)
radix_hist_kernel(const UK* keys, size_t n, key_coding coding, int first_pass, int num_passes, radix_ctrl* ctrl) {
  constexpr int NP = sizeof(UK);
  constexpr int COPIES = hist_tuning<UK>::COPIES;
  constexpr int VEC = 16 / sizeof(UK);
  extern __shared__ __align__(16) unsigned hist_bins[];   // [NP][256][COPIES]
  for (int i = threadIdx.x; i < NP * RADIX_BINS * COPIES; i += HIST_BLOCK) hist_bins[i] = 0;
  __syncthreads();
  const int col = lane_id() & (COPIES - 1);
  unsigned dmask[NP];
#pragma unroll
  for (int p = 0; p < NP; ++p) dmask[p] = digit_mask<UK>(coding, p * RADIX_BITS);
  auto account = [&](UK k) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      unsigned d = key_digit<IS_FLOAT>(k, p * RADIX_BITS, dmask[p]);
      atomicAdd(&hist_bins[(p * RADIX_BINS + d) * COPIES + col], 1u);
    }
  };
  // 16-byte loads over the aligned body; the ragged head and tail one key at a time
  const uintptr_t addr = reinterpret_cast<uintptr_t>(keys);
  size_t head = ((16 - (addr & 15)) & 15) / sizeof(UK);
  if (head > n) head = n;
  const size_t nvec = (n - head) / VEC;
  const vec16* vkeys = reinterpret_cast<const vec16*>(keys + head);
  const size_t gtid = (size_t)blockIdx.x * HIST_BLOCK + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * HIST_BLOCK;
  constexpr int U = 4;
  size_t v = gtid;
  for (; v + (U - 1) * stride < nvec; v += U * stride) {
    vec16 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) r[u] = load_stream16(vkeys + v + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const UK* e = reinterpret_cast<const UK*>(&r[u]);
#pragma unroll
      for (int k = 0; k < VEC; ++k) account(e[k]);
    }
  }
  for (; v < nvec; v += stride) {
    vec16 r = load_stream16(vkeys + v);
    const UK* e = reinterpret_cast<const UK*>(&r);
#pragma unroll
    for (int k = 0; k < VEC; ++k) account(e[k]);
  }
  if (gtid < head) account(keys[gtid]);
  const size_t tail0 = head + nvec * VEC;
  if (tail0 + gtid < n) account(keys[tail0 + gtid]);
  __syncthreads();
  for (int j = threadIdx.x; j < NP * RADIX_BINS; j += HIST_BLOCK) {
    const int p = j / RADIX_BINS;
    unsigned c = 0;
#pragma unroll
    for (int q = 0; q < COPIES; ++q) c += hist_bins[j * COPIES + ((q + threadIdx.x) & (COPIES - 1))];
    if (c && p >= first_pass && p < first_pass + num_passes) atomicAdd(&ctrl->hist[p][j % RADIX_BINS], (unsigned long long)c);
  }
}

// ---------------------------------------------------------------- 2. bucket bases + skip flags
template <int UNUSED = 0>   // a template only so that the header can be included in several translation units
__global__ void __launch_bounds__(RADIX_BINS)
radix_scan_hist_kernel(radix_ctrl* ctrl, size_t n, int first_pass) {
  const int p = first_pass + blockIdx.x;
  __shared__ unsigned long long warp_tot[RADIX_BINS / 32];
  __shared__ unsigned degenerate;
  if (threadIdx.x == 0) degenerate = 0;
  __syncthreads();
  unsigned long long c = ctrl->hist[p][threadIdx.x];
  if (c == n) degenerate = 1;
  unsigned long long incl = warp_inclusive_scan(c, plus_op());
  if (lane_id() == 31) warp_tot[threadIdx.x >> 5] = incl;
  __syncthreads();
  unsigned long long base = 0;
  for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) base += warp_tot[w];
  ctrl->hist[p][threadIdx.x] = base + incl - c;
  if (threadIdx.x == 0) ctrl->skip[p] = degenerate;
}

// ---------------------------------------------------------------- 3. one digit place
#ifndef TB200_SWEEP_IPT_44
#define TB200_SWEEP_IPT_44 16
#endif
#ifndef TB200_SWEEP_MATCH_EVERY
#define TB200_SWEEP_MATCH_EVERY 0
#endif
#ifndef TB200_SWEEP_IPT_84
#define TB200_SWEEP_IPT_84 12
#endif
template <int KB, int VB> struct onesweep_tuning {
  // items per thread; two 512-thread CTAs per SM (64 registers per thread, ~80 KB of staging each)
  static constexpr int IPT = KB <= 4 ? (VB == 0 ? 18 : VB <= 4 ? TB200_SWEEP_IPT_44 : 12) : (VB == 0 ? 12 : VB <= 4 ? TB200_SWEEP_IPT_84 : 8);
};

// What distinguishes a radix digit pass from the multi-GPU bucket scatter: how a key maps to one of
// up to 256 bins and where a bin's items go.
template <class UK, class UV, bool IS_FLOAT> struct radix_pass_policy {
  static constexpr int BITS = RADIX_BITS;       // ballots per key
  static constexpr int MATCH_EVERY = TB200_SWEEP_MATCH_EVERY;   // n > 0: every n-th row is ranked with match.any instead (0: never)
  UK* dst; UV* vdst; int shift; unsigned dmask;
  __device__ __forceinline__ unsigned digit(UK k) const { return key_digit<IS_FLOAT>(k, shift, dmask); }
  __device__ __forceinline__ UK* keys_of(unsigned) const { return dst; }
  __device__ __forceinline__ UV* vals_of(unsigned) const { return vdst; }
};

// Order-preserving unsigned code of a key (see the file header).
template <class UK> __host__ __device__ __forceinline__ UK key_code(UK k, key_coding c) {
  constexpr int B = 8 * sizeof(UK);
  const UK sign = (UK)1 << (B - 1);
  if (c.kind == KEY_SIGNED) k ^= sign;
  else if (c.kind == KEY_FLOAT) k ^= (k & sign) ? (UK)~(UK)0 : sign;
  return c.descending ? (UK)~k : k;
}

constexpr int MAX_BUCKETS = 16;
// bin = number of splitters whose code is <= the key's code; bin b goes to destination b, which
// may be a buffer in another GPU's memory (ordinary stores over NVLink)
template <class UK, class UV> struct bucket_policy {
  static constexpr int BITS = 4;
  static constexpr int MATCH_EVERY = 0;
  key_coding coding; int buckets;
  const UK* split_code;      // shared memory: buckets - 1 codes, ascending
  UK* const* dst_k; UV* const* dst_v;   // shared memory tables of destination pointers
  __device__ __forceinline__ unsigned digit(UK k) const {
    const UK c = key_code(k, coding);
    unsigned d = 0;
    for (int i = 0; i < buckets - 1; ++i) d += (c >= split_code[i]) ? 1u : 0u;
    return d;
  }
  __device__ __forceinline__ UK* keys_of(unsigned d) const { return dst_k[d]; }
  __device__ __forceinline__ UV* vals_of(unsigned d) const { return dst_v[d]; }
};

// Tunables of the tile routine (overridable on the compiler's command line for experiments).
// Tunables of the tile routine (overridable on the compiler's command line for experiments).
#ifndef TB200_SWEEP_LATE_CLAIM
#define TB200_SWEEP_LATE_CLAIM 0    // 1: the next tile is claimed after the staging instead of after the ranking
#endif
#ifndef TB200_SWEEP_LB_BATCH
#define TB200_SWEEP_LB_BATCH 4      // descriptors fetched per round trip of the look-back
#endif
#ifndef TB200_SWEEP_LOOP_MAX
#define TB200_SWEEP_LOOP_MAX 6      // rows with more colliding lanes than this are ranked with ballots
#endif

// Staged item: a key and its value side by side, so that one shared-memory store / load moves both.
template <class UK, class UV, bool HAS_V, bool PACKED> struct sweep_stage;
template <class UK, class UV> struct sweep_stage<UK, UV, true, true> {   // sizeof(UK) == sizeof(UV)
  struct __align__(2 * sizeof(UK)) item { UK k; UV v; };
  item* slots;
  __device__ __forceinline__ sweep_stage(unsigned char* base, int) : slots(reinterpret_cast<item*>(base)) {}
  __device__ __forceinline__ void put(unsigned p, UK k, UV v) const { item it; it.k = k; it.v = v; slots[p] = it; }
  __device__ __forceinline__ void get(unsigned p, UK& k, UV& v) const { const item it = slots[p]; k = it.k; v = it.v; }
};
template <class UK, class UV> struct sweep_stage<UK, UV, true, false> {
  UK* ks; UV* vs;
  __device__ __forceinline__ sweep_stage(unsigned char* base, int tile_items)
      : ks(reinterpret_cast<UK*>(sizeof(UK) >= sizeof(UV) ? base : base + (size_t)tile_items * sizeof(UV))),
        vs(reinterpret_cast<UV*>(sizeof(UK) >= sizeof(UV) ? base + (size_t)tile_items * sizeof(UK) : base)) {}
  __device__ __forceinline__ void put(unsigned p, UK k, UV v) const { ks[p] = k; vs[p] = v; }
  __device__ __forceinline__ void get(unsigned p, UK& k, UV& v) const { k = ks[p]; v = vs[p]; }
};
template <class UK, class UV, bool PACKED> struct sweep_stage<UK, UV, false, PACKED> {
  UK* ks;
  __device__ __forceinline__ sweep_stage(unsigned char* base, int) : ks(reinterpret_cast<UK*>(base)) {}
  __device__ __forceinline__ void put(unsigned p, UK k, UV) const { ks[p] = k; }
  __device__ __forceinline__ void get(unsigned p, UK& k, UV&) const { k = ks[p]; }
};

// A tile's items in registers, lane-interleaved inside each warp's chunk (item i of lane l is element
// warp * 32 * IPT + i * 32 + l of the tile, so a warp-wide load instruction is contiguous).
template <class UK, class UV, bool HAS_V, int IPT> struct sweep_regs { UK key[IPT]; UV val[HAS_V ? IPT : 1]; };

template <class UK, class UV, bool HAS_V, int IPT, bool FULL>
__device__ __forceinline__ void sweep_load(sweep_regs<UK, UV, HAS_V, IPT>& r, const UK* __restrict__ src, const UV* __restrict__ vsrc, unsigned n,
                                           unsigned tile) {
  constexpr int TILE = ONESWEEP_BLOCK * IPT;
  const unsigned tile_base = tile * (unsigned)TILE;
  const unsigned tile_n = FULL ? (unsigned)TILE : n - tile_base;
  const unsigned wofs = (threadIdx.x >> 5) * (32 * IPT) + (threadIdx.x & 31);
  const UK* ks = src + tile_base + wofs;
#pragma unroll
  for (int i = 0; i < IPT; ++i) r.key[i] = (FULL || wofs + i * 32 < tile_n) ? __ldcs(ks + i * 32) : (UK)0;
  if constexpr (HAS_V) {
    const UV* vs = vsrc + tile_base + wofs;
#pragma unroll
    for (int i = 0; i < IPT; ++i) r.val[i] = (FULL || wofs + i * 32 < tile_n) ? __ldcs(vs + i * 32) : (UV)0;
  }
}
template <class UK, class UV, bool HAS_V, int IPT>
__device__ __forceinline__ void sweep_load_any(sweep_regs<UK, UV, HAS_V, IPT>& r, const UK* __restrict__ src, const UV* __restrict__ vsrc, unsigned n,
                                               unsigned tile) {
  if ((unsigned long long)(tile + 1) * (ONESWEEP_BLOCK * IPT) <= n) sweep_load<UK, UV, HAS_V, IPT, true>(r, src, vsrc, n, tile);
  else sweep_load<UK, UV, HAS_V, IPT, false>(r, src, vsrc, n, tile);
}

// One tile of a digit pass: ranks the tile's keys (held in `r`) by digit, chains the per-digit
// counts to the preceding tiles and writes keys and values to their buckets.  Once the items are
// staged in shared memory the registers are free, so the NEXT tile of this CTA (`next`, if
// `next < num_tiles`) is loaded into them while this one is chained and written out.
//
// Ranking.  Every lane adds 1 to its warp's private counter of its digit and then reads the counter
// back: `old` is some slot of the digit's group in this row, `now - old > 1` tells all members of a
// group of two or more lanes, except the one that drew the last slot, that they collided.  Lanes
// that did not collide are done (rank = old).  Groups are then put in lane order one at a time: the
// highest colliding lane announces its digit, one ballot finds its group, each member takes
// base + (members in lower lanes).  With 256 bins and 32 lanes a row has about two groups, which
// costs half the instructions of finding every lane's peers with one ballot per digit bit; rows
// with more than TB200_SWEEP_LOOP_MAX colliding lanes (skewed digits, the padded last tile) take
// the ballots.  The result does not depend on the order in which the hardware serves the atomics.
template <class UK, class UV, bool HAS_V, class Policy, class LB, int IPT, bool FULL>
__device__ __forceinline__ void onesweep_tile(sweep_regs<UK, UV, HAS_V, IPT>& r, const UK* __restrict__ src, const UV* __restrict__ vsrc, unsigned n,
                                              unsigned tile, unsigned num_tiles, unsigned* next_ticket, unsigned& next, const Policy policy,
                                              unsigned my_bin_base, LB* lookback, unsigned* err, unsigned* warp_hist, unsigned* s_goff,
                                              unsigned* s_scan, unsigned* s_next, unsigned char* stage_raw) {
  constexpr int NWARPS = ONESWEEP_BLOCK / 32;
  constexpr int TILE = ONESWEEP_BLOCK * IPT;
  constexpr int WCHUNK = 32 * IPT;
  constexpr int LB_BITS = 8 * sizeof(LB) - 2;
  constexpr LB LB_MASK = ((LB)1 << LB_BITS) - 1;
  constexpr LB F_VALID = (LB)1 << LB_BITS, F_INC = (LB)2 << LB_BITS;   // a tile's count: valid; an inclusive prefix: valid | inc
  constexpr int PAD_DIGIT = (1 << Policy::BITS) - 1;
  constexpr bool PACKED = HAS_V && sizeof(UK) == sizeof(UV);
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const unsigned tile_base = tile * (unsigned)TILE;
  const unsigned tile_n = FULL ? (unsigned)TILE : n - tile_base;
  const unsigned wofs = warp * WCHUNK + lane;   // this lane's first item inside the tile

  // ---- rank inside the warp
  unsigned pd[IPT];   // low 16 bits: position, bits 16..23: digit
  unsigned* my_hist = warp_hist + warp * RADIX_BINS;
  const unsigned lanemask_lt = (1u << lane) - 1, lanemask_ge = ~lanemask_lt;
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    // a partial tile pads with pseudo-keys of the highest digit: ranked after every real key of the tile
    const unsigned d = (FULL || wofs + i * 32 < tile_n) ? policy.digit(r.key[i]) : (unsigned)PAD_DIGIT;
    unsigned rank;
    if (Policy::MATCH_EVERY != 0 && (i + 1) % (Policy::MATCH_EVERY != 0 ? Policy::MATCH_EVERY : 1) == 0) {
      // the match unit runs beside the ALU pipe, but at a small fraction of its rate on sm_100
      const unsigned peers = __match_any_sync(FULL_MASK, d);
      const unsigned ahead = __popc(peers & lanemask_lt);
      unsigned before = 0;
      if (ahead == 0) before = atomicAdd(&my_hist[d], (unsigned)__popc(peers));
      rank = __shfl_sync(FULL_MASK, before, __ffs(peers) - 1) + ahead;
    } else {
      const unsigned old = atomicAdd(&my_hist[d], 1u);
      __syncwarp();   // every lane's increment precedes every lane's read
      const unsigned now = *reinterpret_cast<volatile unsigned*>(&my_hist[d]);
      unsigned pending = __ballot_sync(FULL_MASK, now - old > 1u);
      rank = old;
      if (Policy::BITS > 4 && __popc(pending) <= TB200_SWEEP_LOOP_MAX) {
        while (pending) {
          const unsigned dsrc = __shfl_sync(FULL_MASK, d, 31 - __clz(pending));
          const unsigned peers = __ballot_sync(FULL_MASK, d == dsrc);
          if (d == dsrc) rank = now - __popc(peers & lanemask_ge);   // base + members in lower lanes
          pending &= ~peers;
        }
      } else if (pending) {
        unsigned peers = FULL_MASK;
#pragma unroll
        for (int b = 0; b < Policy::BITS; ++b) {
          const bool bit = (d >> b) & 1;
          const unsigned vote = __ballot_sync(FULL_MASK, bit);
          peers &= bit ? vote : ~vote;
        }
        rank = now - __popc(peers & lanemask_ge);
      }
    }
    pd[i] = rank | (d << 16);
  }
  __syncthreads();

  // ---- per digit: stack the warps' counts, scan the digits
  if (!TB200_SWEEP_LATE_CLAIM && threadIdx.x == 0) *s_next = atomicAdd(next_ticket, 1u);
  unsigned my_count = 0, digit_off = 0;
  LB* const slot = lookback + (size_t)tile * RADIX_BINS + (threadIdx.x & (RADIX_BINS - 1));
  if (threadIdx.x < RADIX_BINS) {
    unsigned run = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) { unsigned c = warp_hist[w * RADIX_BINS + threadIdx.x]; warp_hist[w * RADIX_BINS + threadIdx.x] = run; run += c; }
    my_count = run;
    if (!FULL && threadIdx.x == PAD_DIGIT) my_count -= (unsigned)TILE - tile_n;
    // the tile's own count is visible to its successors before anything else happens
    *reinterpret_cast<volatile LB*>(slot) = (tile == 0 ? (F_VALID | F_INC) : F_VALID) | (LB)my_count;
    const unsigned incl = warp_inclusive_scan(run, plus_op());
    if (lane == 31) s_scan[warp] = incl;
    digit_off = incl - run;
  }
  __syncthreads();
  if (threadIdx.x < RADIX_BINS) {
    for (int w = 0; w < warp; ++w) digit_off += s_scan[w];
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) warp_hist[w * RADIX_BINS + threadIdx.x] += digit_off;
  }
  __syncthreads();

  // ---- stage keys and values in bucket order; the registers then take the CTA's next tile
  const sweep_stage<UK, UV, HAS_V, PACKED> stage(stage_raw, TILE);
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const unsigned p = (pd[i] & 0xffffu) + my_hist[pd[i] >> 16];
    stage.put(p, r.key[i], r.val[HAS_V ? i : 0]);
  }
  if (TB200_SWEEP_LATE_CLAIM) {
    // claimed as late as the prefetch allows: tiles should start in the order in which they are claimed
    if (threadIdx.x == 0) *s_next = atomicAdd(next_ticket, 1u);
  } else {
    next = *s_next;
    if (next < num_tiles) sweep_load_any<UK, UV, HAS_V, IPT>(r, src, vsrc, n, next);
  }
  __syncwarp();
  // each warp clears its own counters for its next tile (nobody else touches them until the next stacking)
  {
    uint4* z = reinterpret_cast<uint4*>(my_hist);
#pragma unroll
    for (int q = 0; q < RADIX_BINS / 4 / 32; ++q) z[q * 32 + lane] = make_uint4(0, 0, 0, 0);
  }

  // ---- chain to the preceding tiles, one thread per digit.  The preceding tiles had the time of
  // the staging above to publish; their descriptors are fetched LB_BATCH at a time so that the walk
  // back to the nearest inclusive prefix costs one memory round trip per batch, not per tile.
  if (threadIdx.x < RADIX_BINS) {
    LB prefix = 0;
    if (tile != 0) {
      constexpr int LB_BATCH = TB200_SWEEP_LB_BATCH;
      long long t = (long long)tile - 1;   // nearest tile not yet accounted for
      unsigned iter = 0;
      bool done = false;
      while (!done) {
        LB w[LB_BATCH];
#pragma unroll
        for (int j = 0; j < LB_BATCH; ++j) {
          const long long tj = t - j > 0 ? t - j : 0;
          w[j] = *reinterpret_cast<const volatile LB*>(lookback + (size_t)tj * RADIX_BINS + threadIdx.x);
        }
        bool open = true;
        int taken = 0;
#pragma unroll
        for (int j = 0; j < LB_BATCH; ++j) {
          const bool take = open && (w[j] & F_VALID) != 0;
          if (take) { prefix += w[j] & LB_MASK; ++taken; }
          if (take && (w[j] & F_INC) != 0) done = true;
          open = take && (w[j] & F_INC) == 0;
        }
        t -= taken;
        if (taken == 0) {
          if (++iter > SPIN_LIMIT) { record_error(err, ERR_LOOKBACK_TIMEOUT); break; }
          backoff(iter);
        } else {
          iter = 0;
        }
      }
      *reinterpret_cast<volatile LB*>(slot) = F_VALID | F_INC | (prefix + (LB)my_count);
    }
    s_goff[threadIdx.x] = my_bin_base + (unsigned)prefix - digit_off;   // bucket's global offset minus its staged offset
  }
  __syncthreads();
  if (TB200_SWEEP_LATE_CLAIM) {
    next = *s_next;
    if (next < num_tiles) sweep_load_any<UK, UV, HAS_V, IPT>(r, src, vsrc, n, next);
  }
  // consecutive threads take consecutive staged slots, so each bucket's run is written contiguously
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const unsigned j = threadIdx.x + i * ONESWEEP_BLOCK;
    if (FULL || j < tile_n) {
      UK k; UV v;
      stage.get(j, k, v);
      const unsigned d = policy.digit(k);
      const unsigned at = s_goff[d] + j;
      policy.keys_of(d)[at] = k;
      if constexpr (HAS_V) policy.vals_of(d)[at] = v;
    }
  }
  // the next tile's staging, s_goff and s_scan writes all sit behind that tile's own barriers,
  // which every warp reaches only after it has finished the stores above
}

// The persistent loop shared by the digit pass and the bucket scatter: tiles are handed out by an
// atomic ticket in increasing order (which is what lets a tile wait for its predecessors), every CTA
// keeps the tile after its current one in flight in registers.
template <class UK, class UV, bool HAS_V, class Policy, class LB, int IPT>
__device__ __forceinline__ void sweep_tiles(const UK* __restrict__ src, const UV* __restrict__ vsrc, unsigned n, unsigned* ticket, const Policy policy,
                                            unsigned my_bin_base, LB* lookback, unsigned* err, unsigned char* smem_raw) {
  constexpr int NWARPS = ONESWEEP_BLOCK / 32;
  constexpr int TILE = ONESWEEP_BLOCK * IPT;
  unsigned* warp_hist = reinterpret_cast<unsigned*>(smem_raw);   // [NWARPS][256]
  unsigned* s_goff = warp_hist + NWARPS * RADIX_BINS;            // [256]
  unsigned* s_scan = s_goff + RADIX_BINS;                        // [16]
  unsigned char* stage_raw = reinterpret_cast<unsigned char*>(s_scan + 16);
  __shared__ unsigned s_next;
  const unsigned num_tiles = (unsigned)(((unsigned long long)n + TILE - 1) / TILE);

  if (threadIdx.x == 0) s_next = atomicAdd(ticket, 1u);
  for (int i = threadIdx.x; i < NWARPS * RADIX_BINS; i += ONESWEEP_BLOCK) warp_hist[i] = 0;
  __syncthreads();
  unsigned tile = s_next;
  sweep_regs<UK, UV, HAS_V, IPT> r;
  if (tile < num_tiles) sweep_load_any<UK, UV, HAS_V, IPT>(r, src, vsrc, n, tile);
  while (tile < num_tiles) {
    unsigned next;
    if ((unsigned long long)(tile + 1) * TILE <= n)
      onesweep_tile<UK, UV, HAS_V, Policy, LB, IPT, true>(r, src, vsrc, n, tile, num_tiles, ticket, next, policy, my_bin_base, lookback, err, warp_hist,
                                                          s_goff, s_scan, &s_next, stage_raw);
    else
      onesweep_tile<UK, UV, HAS_V, Policy, LB, IPT, false>(r, src, vsrc, n, tile, num_tiles, ticket, next, policy, my_bin_base, lookback, err, warp_hist,
                                                           s_goff, s_scan, &s_next, stage_raw);
    tile = next;
  }
}

template <class UK, class UV, bool HAS_V, bool IS_FLOAT, class LB, int IPT>
__global__ void __launch_bounds__(ONESWEEP_BLOCK, ONESWEEP_CTAS_PER_SM)
onesweep_kernel(UK* buf_a, UK* buf_b, UV* val_a, UV* val_b, unsigned n, key_coding coding, int pass, int first_pass,
                radix_ctrl* ctrl, LB* lookback, ws_header* hdr) {
  if (ctrl->skip[pass]) return;
  int flips = 0;
  for (int q = first_pass; q < pass; ++q) flips += ctrl->skip[q] ? 0 : 1;
  const UK* src = (flips & 1) ? buf_b : buf_a;
  UK* dst = (flips & 1) ? buf_a : buf_b;
  const UV* vsrc = (flips & 1) ? val_b : val_a;
  UV* vdst = (flips & 1) ? val_a : val_b;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int shift = pass * RADIX_BITS;
  using Policy = radix_pass_policy<UK, UV, IS_FLOAT>;
  const Policy policy{dst, vdst, shift, digit_mask<UK>(coding, shift)};
  const unsigned my_bin_base = threadIdx.x < RADIX_BINS ? (unsigned)ctrl->hist[pass][threadIdx.x] : 0u;
  sweep_tiles<UK, UV, HAS_V, Policy, LB, IPT>(src, vsrc, n, &ctrl->tickets[pass], policy, my_bin_base, lookback, &hdr->error, smem_raw);
}

// ---------------------------------------------------------------- multi-GPU: bucket count and scatter
// Destination table handed to the scatter kernel by value.
template <class UK, class UV> struct bucket_table {
  UK* dst_k[MAX_BUCKETS]; UV* dst_v[MAX_BUCKETS]; unsigned long long base[MAX_BUCKETS];
};

// counts[b] = number of keys whose code falls into bucket b (b = number of splitters <= code).
// Lane-private copies of the 16 bins in shared memory keep the atomics conflict-free.
template <class UK>
__global__ void __launch_bounds__(256)
bucket_count_kernel(const UK* keys, size_t n, key_coding coding, const UK* splitters, int buckets, unsigned long long* counts) {
  __shared__ UK code[MAX_BUCKETS];
  __shared__ unsigned local[MAX_BUCKETS * 32];
  for (int i = threadIdx.x; i < MAX_BUCKETS * 32; i += 256) local[i] = 0;
  if ((int)threadIdx.x < buckets - 1) code[threadIdx.x] = key_code(splitters[threadIdx.x], coding);
  __syncthreads();
  const int lane = lane_id();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const UK c = key_code(__ldcs(keys + i), coding);
    unsigned d = 0;
    for (int s = 0; s < buckets - 1; ++s) d += (c >= code[s]) ? 1u : 0u;
    atomicAdd(&local[d * 32 + lane], 1u);
  }
  __syncthreads();
  if ((int)threadIdx.x < buckets) {
    unsigned total = 0;
    for (int q = 0; q < 32; ++q) total += local[threadIdx.x * 32 + ((q + threadIdx.x) & 31)];
    if (total) atomicAdd(&counts[threadIdx.x], (unsigned long long)total);
  }
}

// Stable scatter of (key, value) pairs into per-bucket destinations: item order inside a bucket
// is input order, bucket b's items land at dst[b][base[b] ...].  Same tile machinery as a radix
// pass (ballot ranking, per-bin look-back, staging so that each bin's run is stored contiguously);
// only the bin function and the destinations differ.
template <class UK, class UV, bool HAS_V, class LB, int IPT>
__global__ void __launch_bounds__(ONESWEEP_BLOCK, ONESWEEP_CTAS_PER_SM)
bucket_scatter_kernel(const UK* src, const UV* vsrc, unsigned n, key_coding coding, const UK* splitters, int buckets, bucket_table<UK, UV> table,
                      LB* lookback, ws_header* hdr) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ UK s_code[MAX_BUCKETS];
  __shared__ UK* s_dst_k[MAX_BUCKETS];
  __shared__ UV* s_dst_v[MAX_BUCKETS];
  if (threadIdx.x < MAX_BUCKETS) {
    s_dst_k[threadIdx.x] = table.dst_k[threadIdx.x];
    s_dst_v[threadIdx.x] = table.dst_v[threadIdx.x];
    if ((int)threadIdx.x < buckets - 1) s_code[threadIdx.x] = key_code(splitters[threadIdx.x], coding);
  }
  __syncthreads();
  using Policy = bucket_policy<UK, UV>;
  const Policy policy{coding, buckets, s_code, s_dst_k, s_dst_v};
  const unsigned my_bin_base = threadIdx.x < MAX_BUCKETS ? (unsigned)table.base[threadIdx.x] : 0u;
  sweep_tiles<UK, UV, HAS_V, Policy, LB, IPT>(src, vsrc, n, &hdr->ticket, policy, my_bin_base, lookback, &hdr->error, smem_raw);
}

// ---------------------------------------------------------------- multi-GPU: splitters from a digit histogram
// The exchange of the multi-GPU sort without sampling: every GPU histograms a 12-bit field of its
// keys' order-preserving codes (one read of the keys), the histograms are all-gathered (ONE
// collective), and every GPU derives the same plan from them: which bins go to which GPU (contiguous
// bin ranges, balanced to one bin's size), where its own items start in each destination's receive
// buffer (source-rank-major, which keeps the exchange stable) and how much every GPU receives.
// 32-bit keys use their top 12 bits; 64-bit keys offer their four top 12-bit fields and the plan
// takes the highest one in which the keys differ (all fields above it are then equal in every key,
// so that field alone orders the bins).  Heavily skewed keys make unequal shares; the caller reads
// the shares and may fall back to sampled splitters.
constexpr int EXCH_BITS = 12;
constexpr int EXCH_BINS = 1 << EXCH_BITS;
constexpr int EXCH_MAX_FIELDS = 4;
constexpr int EXCH_ROW_TAIL = 4;   // words behind a rank's histograms: a caller's tag (2 words), its item count (2 words)
template <class UK> constexpr int exch_fields() { return sizeof(UK) == 8 ? 4 : 1; }
template <class UK> __host__ __device__ constexpr int exch_shift(int field) { return 8 * (int)sizeof(UK) - EXCH_BITS * (field + 1); }
inline size_t exch_row_words(int fields) { return (size_t)fields * EXCH_BINS + EXCH_ROW_TAIL; }

struct exchange_plan {
  unsigned field;                                  // which 12-bit field partitions the keys
  unsigned ranks;
  unsigned long long send_offset[MAX_BUCKETS];     // where this rank's items start in destination d's receive buffer
  unsigned long long recv_total[MAX_BUCKETS];      // items destination d receives in all
  unsigned long long tag[MAX_BUCKETS];             // the tag each rank handed to its histogram call
  unsigned char lut[EXCH_BINS];                    // bin -> destination
};

template <class UK>
__global__ void __launch_bounds__(1024)
exchange_hist_kernel(const UK* keys, size_t n, key_coding coding, unsigned long long tag, unsigned* row) {
  constexpr int F = exch_fields<UK>();
  extern __shared__ __align__(16) unsigned exch_bins[];   // [F][4096]
  for (int i = threadIdx.x; i < F * EXCH_BINS; i += 1024) exch_bins[i] = 0;
  __syncthreads();
  const size_t stride = (size_t)gridDim.x * 1024;
  constexpr int U = 4;
  size_t i = (size_t)blockIdx.x * 1024 + threadIdx.x;
  auto account = [&](UK k) {
    const UK c = key_code(k, coding);
#pragma unroll
    for (int f = 0; f < F; ++f) atomicAdd(&exch_bins[f * EXCH_BINS + ((unsigned)(c >> exch_shift<UK>(f)) & (EXCH_BINS - 1))], 1u);
  };
  for (; i + (U - 1) * stride < n; i += U * stride) {
    UK k[U];
#pragma unroll
    for (int u = 0; u < U; ++u) k[u] = __ldcs(keys + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) account(k[u]);
  }
  for (; i < n; i += stride) account(__ldcs(keys + i));
  __syncthreads();
  for (int j = threadIdx.x; j < F * EXCH_BINS; j += 1024) {
    const unsigned c = exch_bins[j];
    if (c) atomicAdd(&row[j], c);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned* tail = row + F * EXCH_BINS;
    tail[0] = (unsigned)tag; tail[1] = (unsigned)(tag >> 32);
    tail[2] = (unsigned)n; tail[3] = (unsigned)((unsigned long long)n >> 32);
  }
}

// One CTA.  rows: [ranks][fields * 4096 + EXCH_ROW_TAIL] words, the all-gathered histograms.
template <int UNUSED = 0>
__global__ void __launch_bounds__(1024)
exchange_plan_kernel(const unsigned* rows, int ranks, int rank, int fields, exchange_plan* plan) {
  __shared__ unsigned long long s_total[EXCH_BINS];
  __shared__ unsigned long long s_cnt[MAX_BUCKETS][MAX_BUCKETS];   // [source][destination]
  __shared__ unsigned long long s_warp[32];
  __shared__ unsigned char s_dest[EXCH_BINS];
  const size_t row_words = (size_t)fields * EXCH_BINS + EXCH_ROW_TAIL;
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  // the highest field in which the keys differ (a field whose every key shares one bin is skipped)
  int field = 0;
  for (; field < fields; ++field) {
    int nonzero = 0;
    for (int b = threadIdx.x; b < EXCH_BINS; b += 1024) {
      unsigned long long t = 0;
      for (int g = 0; g < ranks; ++g) t += rows[(size_t)g * row_words + (size_t)field * EXCH_BINS + b];
      s_total[b] = t;
      nonzero += t != 0;
    }
    int used = nonzero;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) used += __shfl_xor_sync(FULL_MASK, used, d);
    if (lane == 0) s_warp[warp] = (unsigned long long)used;
    __syncthreads();
    unsigned long long all_used = 0;
    for (int w = 0; w < 32; ++w) all_used += s_warp[w];
    __syncthreads();
    if (all_used > 1 || field == fields - 1) break;
  }
  // exclusive prefix of the bins: thread t owns bins 4t .. 4t+3
  unsigned long long mine[4], sum = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) { mine[j] = sum; sum += s_total[threadIdx.x * 4 + j]; }
  unsigned long long incl = warp_inclusive_scan(sum, plus_op());
  if (lane == 31) s_warp[warp] = incl;
  for (int i = threadIdx.x; i < MAX_BUCKETS * MAX_BUCKETS; i += 1024) (&s_cnt[0][0])[i] = 0;
  __syncthreads();
  unsigned long long before = incl - sum, n_all = 0;
  for (int w = 0; w < 32; ++w) { if (w < warp) before += s_warp[w]; n_all += s_warp[w]; }
  unsigned dest[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int b = threadIdx.x * 4 + j;
    unsigned long long d = n_all ? (before + mine[j]) * (unsigned long long)ranks / n_all : 0;   // the share in which the bin starts
    if (d > (unsigned long long)(ranks - 1)) d = ranks - 1;
    dest[j] = (unsigned)d;
    s_dest[b] = (unsigned char)d;
    plan->lut[b] = (unsigned char)d;
  }
  // [source][destination] counts.  Destinations grow with the bin, so nearly every warp's 128 bins
  // go to one destination: such a warp adds its bins up with a shuffle reduction and issues one
  // atomic per source; only the few warps that straddle a boundary add bin by bin.
  const unsigned first_dest = __shfl_sync(FULL_MASK, dest[0], 0);           // every lane takes part: not inside a short-circuit
  const bool warp_uniform = __all_sync(FULL_MASK, (dest[0] == dest[3]) & (dest[0] == first_dest));
  for (int g = 0; g < ranks; ++g) {
    const uint4 c = *reinterpret_cast<const uint4*>(rows + (size_t)g * row_words + (size_t)field * EXCH_BINS + threadIdx.x * 4);
    if (warp_uniform) {
      unsigned long long t = (unsigned long long)c.x + c.y + c.z + c.w;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(FULL_MASK, t, d);
      if (lane == 0 && t) atomicAdd(&s_cnt[g][dest[0]], t);
    } else {
      if (c.x) atomicAdd(&s_cnt[g][dest[0]], (unsigned long long)c.x);
      if (c.y) atomicAdd(&s_cnt[g][dest[1]], (unsigned long long)c.y);
      if (c.z) atomicAdd(&s_cnt[g][dest[2]], (unsigned long long)c.z);
      if (c.w) atomicAdd(&s_cnt[g][dest[3]], (unsigned long long)c.w);
    }
  }
  __syncthreads();
  if ((int)threadIdx.x < ranks) {
    const int d = threadIdx.x;
    unsigned long long off = 0, total = 0;
    for (int g = 0; g < ranks; ++g) { if (g < rank) off += s_cnt[g][d]; total += s_cnt[g][d]; }
    plan->send_offset[d] = off;
    plan->recv_total[d] = total;
    const unsigned* tail = rows + (size_t)d * row_words + (size_t)fields * EXCH_BINS;
    plan->tag[d] = (unsigned long long)tail[0] | ((unsigned long long)tail[1] << 32);
  }
  if (threadIdx.x == 0) { plan->field = (unsigned)field; plan->ranks = (unsigned)ranks; }
}

// bin of a key = plan->lut[its field]; bin b goes to destination b, possibly a buffer in another
// GPU's memory (ordinary stores over NVLink)
template <class UK, class UV> struct exchange_policy {
  static constexpr int BITS = 4;
  static constexpr int MATCH_EVERY = 0;
  key_coding coding; int shift;
  const unsigned char* lut;              // shared memory, 4096 entries
  UK* const* dst_k; UV* const* dst_v;    // shared memory tables of destination pointers
  __device__ __forceinline__ unsigned digit(UK k) const { return lut[(unsigned)(key_code(k, coding) >> shift) & (EXCH_BINS - 1)]; }
  __device__ __forceinline__ UK* keys_of(unsigned d) const { return dst_k[d]; }
  __device__ __forceinline__ UV* vals_of(unsigned d) const { return dst_v[d]; }
};

template <class UK, class UV, bool HAS_V, class LB, int IPT>
__global__ void __launch_bounds__(ONESWEEP_BLOCK, ONESWEEP_CTAS_PER_SM)
exchange_scatter_kernel(const UK* src, const UV* vsrc, unsigned n, key_coding coding, const exchange_plan* plan, bucket_table<UK, UV> table,
                        LB* lookback, ws_header* hdr) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ unsigned char s_lut[EXCH_BINS];
  __shared__ UK* s_dst_k[MAX_BUCKETS];
  __shared__ UV* s_dst_v[MAX_BUCKETS];
  for (int i = threadIdx.x; i < EXCH_BINS / 4; i += ONESWEEP_BLOCK) reinterpret_cast<unsigned*>(s_lut)[i] = reinterpret_cast<const unsigned*>(plan->lut)[i];
  if (threadIdx.x < MAX_BUCKETS) {
    s_dst_k[threadIdx.x] = table.dst_k[threadIdx.x];
    s_dst_v[threadIdx.x] = table.dst_v[threadIdx.x];
  }
  __syncthreads();
  using Policy = exchange_policy<UK, UV>;
  const Policy policy{coding, exch_shift<UK>((int)plan->field), s_lut, s_dst_k, s_dst_v};
  const unsigned my_bin_base = threadIdx.x < MAX_BUCKETS ? (unsigned)plan->send_offset[threadIdx.x] : 0u;
  sweep_tiles<UK, UV, HAS_V, Policy, LB, IPT>(src, vsrc, n, &hdr->ticket, policy, my_bin_base, lookback, &hdr->error, smem_raw);
}

// ---------------------------------------------------------------- 4. copy back after an odd number of passes
template <class UK, class UV, bool HAS_V>
__global__ void __launch_bounds__(256)
radix_copy_back_kernel(UK* buf_a, const UK* buf_b, UV* val_a, const UV* val_b, size_t n, int first_pass, int num_passes,
                       const radix_ctrl* ctrl) {
  int active = 0;
  for (int q = first_pass; q < first_pass + num_passes; ++q) active += ctrl->skip[q] ? 0 : 1;
  if (!(active & 1)) return;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    buf_a[i] = __ldcs(buf_b + i);
    if constexpr (HAS_V) val_a[i] = __ldcs(val_b + i);
  }
}

// ---------------------------------------------------------------- host side
template <int KB, int VB> constexpr int onesweep_tile_items() { return ONESWEEP_BLOCK * onesweep_tuning<KB, VB>::IPT; }

// per-warp counters, bucket offsets, digit scan, tile counts, look-back window, staged items
template <int KB, int VB> size_t onesweep_smem_bytes() {
  return (size_t)(ONESWEEP_BLOCK / 32) * RADIX_BINS * 4 + RADIX_BINS * 4 + 16 * 4 + (size_t)onesweep_tile_items<KB, VB>() * (KB + VB);
}

// scratch (not counting the alternate key/value buffers, which the caller provides)
template <int KB, int VB> size_t sweep_tiles_of(size_t n) { return (n + onesweep_tile_items<KB, VB>() - 1) / onesweep_tile_items<KB, VB>(); }
template <int KB, int VB> size_t radix_workspace_bytes(size_t n) {
  size_t lb_word = n < (1ull << 30) ? 4 : 8;
  return sizeof(ws_header) + sizeof(radix_ctrl) + align_up(sweep_tiles_of<KB, VB>(n) * RADIX_BINS * lb_word, 256) * KB;
}

// Sorts keys (and values) held in keys_a / vals_a, in place from the caller's point of view:
// keys_b / vals_b are same-sized alternate buffers.  Only bits [begin_bit, end_bit) of the key
// code take part; both must be multiples of 8.  n < 2^31.  No sync.
template <class UK, class UV, bool HAS_V>
cudaError_t radix_sort_async(UK* keys_a, UK* keys_b, UV* vals_a, UV* vals_b, size_t n, key_coding coding, int begin_bit,
                             int end_bit, void* ws, cudaStream_t stream) {
  constexpr int KB = sizeof(UK);
  constexpr int VB = HAS_V ? sizeof(UV) : 0;
  constexpr int IPT = onesweep_tuning<KB, VB>::IPT;
  if (n >= (1ull << 31) || begin_bit % RADIX_BITS || end_bit % RADIX_BITS || end_bit > 8 * KB || begin_bit > end_bit) return cudaErrorInvalidValue;
  if (n <= 1 || begin_bit == end_bit) return cudaMemsetAsync(ws, 0, sizeof(ws_header), stream);
  const int first_pass = begin_bit / RADIX_BITS, num_passes = (end_bit - begin_bit) / RADIX_BITS;
  const size_t tiles = (n + onesweep_tile_items<KB, VB>() - 1) / onesweep_tile_items<KB, VB>();
  const bool lb32 = n < (1ull << 30);
  const size_t lb_bytes = align_up(sweep_tiles_of<KB, VB>(n) * RADIX_BINS * (lb32 ? 4 : 8), 256);
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  radix_ctrl* ctrl = reinterpret_cast<radix_ctrl*>(base + sizeof(ws_header));
  char* lb0 = base + sizeof(ws_header) + sizeof(radix_ctrl);
  cudaError_t e = cudaMemsetAsync(base, 0, (size_t)(lb0 - base) + lb_bytes * num_passes, stream);
  if (e != cudaSuccess) return e;

  const device_info& di = current_device_info();
  size_t hist_grid = (n + HIST_BLOCK * 16 - 1) / (HIST_BLOCK * 16);
  if (hist_grid > (size_t)di.sm_count) hist_grid = (size_t)di.sm_count;
  const size_t hist_smem = (size_t)KB * RADIX_BINS * hist_tuning<UK>::COPIES * 4;
  auto hk = coding.kind == KEY_FLOAT ? radix_hist_kernel<UK, true> : radix_hist_kernel<UK, false>;
  if ((e = cudaFuncSetAttribute(hk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist_smem)) != cudaSuccess) return e;
  { timed_launch tl(KID_RADIX_HIST, stream);
  hk<<<(unsigned)hist_grid, HIST_BLOCK, hist_smem, stream>>>(keys_a, n, coding, first_pass, num_passes, ctrl); }
  log_launch("radix_hist_kernel", hist_grid, HIST_BLOCK, hist_smem, n, stream);
  radix_scan_hist_kernel<><<<num_passes, RADIX_BINS, 0, stream>>>(ctrl, n, first_pass);

  const size_t smem = onesweep_smem_bytes<KB, VB>();
  const bool isf = coding.kind == KEY_FLOAT;
  auto k32 = isf ? onesweep_kernel<UK, UV, HAS_V, true, uint32_t, IPT> : onesweep_kernel<UK, UV, HAS_V, false, uint32_t, IPT>;
  auto k64 = isf ? onesweep_kernel<UK, UV, HAS_V, true, unsigned long long, IPT> : onesweep_kernel<UK, UV, HAS_V, false, unsigned long long, IPT>;
  // opting in to large dynamic shared memory is per kernel and per device; it is cheap, so do it every call
  if ((e = cudaFuncSetAttribute(lb32 ? (const void*)k32 : (const void*)k64, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
  // persistent CTAs, two resident per SM; tiles are handed out by ticket
  const size_t tiles_all = sweep_tiles_of<KB, VB>(n);
  const unsigned grid = (unsigned)(tiles_all < (size_t)di.sm_count * ONESWEEP_CTAS_PER_SM ? tiles_all : (size_t)di.sm_count * ONESWEEP_CTAS_PER_SM);
  for (int p = 0; p < num_passes; ++p) {
    char* lb = lb0 + lb_bytes * p;
    timed_launch tl(KID_ONESWEEP, stream);
    if (lb32)
      k32<<<grid, ONESWEEP_BLOCK, smem, stream>>>(keys_a, keys_b, vals_a, vals_b, (unsigned)n, coding, first_pass + p, first_pass, ctrl,
                                                  reinterpret_cast<uint32_t*>(lb), hdr);
    else
      k64<<<grid, ONESWEEP_BLOCK, smem, stream>>>(keys_a, keys_b, vals_a, vals_b, (unsigned)n, coding, first_pass + p, first_pass, ctrl,
                                                  reinterpret_cast<unsigned long long*>(lb), hdr);
    log_launch("onesweep_kernel", grid, ONESWEEP_BLOCK, smem, n, stream);
  }
  size_t cb_grid = (n + 256 * 8 - 1) / (256 * 8);
  if (cb_grid > (size_t)di.sm_count * 8) cb_grid = (size_t)di.sm_count * 8;
  radix_copy_back_kernel<UK, UV, HAS_V><<<(unsigned)cb_grid, 256, 0, stream>>>(keys_a, keys_b, vals_a, vals_b, n, first_pass, num_passes, ctrl);
  return cudaGetLastError();
}

// counts[0..buckets) += histogram of bucket ids (the caller zeroes counts); no sync
template <class UK>
cudaError_t bucket_count_async(const UK* keys, size_t n, key_coding coding, const UK* d_splitters, int buckets, unsigned long long* d_counts,
                               cudaStream_t stream) {
  if (buckets < 1 || buckets > MAX_BUCKETS) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  const device_info& di = current_device_info();
  size_t grid = (n + 256 * 16 - 1) / (256 * 16);
  if (grid > (size_t)di.sm_count * 8) grid = (size_t)di.sm_count * 8;
  bucket_count_kernel<UK><<<(unsigned)grid, 256, 0, stream>>>(keys, n, coding, d_splitters, buckets, d_counts);
  return cudaGetLastError();
}

template <int KB, int VB> size_t bucket_scatter_workspace_bytes(size_t n) {
  return sizeof(ws_header) + align_up(sweep_tiles_of<KB, VB>(n) * RADIX_BINS * 4, 256);
}

// Stable scatter into up to MAX_BUCKETS destinations (see bucket_scatter_kernel); n < 2^30.  No sync.
template <class UK, class UV, bool HAS_V>
cudaError_t bucket_scatter_async(const UK* keys, const UV* vals, size_t n, key_coding coding, const UK* d_splitters, int buckets,
                                 const bucket_table<UK, UV>& table, void* ws, cudaStream_t stream) {
  constexpr int KB = sizeof(UK);
  constexpr int VB = HAS_V ? sizeof(UV) : 0;
  constexpr int IPT = onesweep_tuning<KB, VB>::IPT;
  if (buckets < 1 || buckets > MAX_BUCKETS || n >= (1ull << 30)) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(ws, 0, bucket_scatter_workspace_bytes<KB, VB>(n), stream);
  if (e != cudaSuccess || n == 0) return e;
  const size_t tiles = (n + onesweep_tile_items<KB, VB>() - 1) / onesweep_tile_items<KB, VB>();
  char* base = static_cast<char*>(ws);
  auto kern = bucket_scatter_kernel<UK, UV, HAS_V, uint32_t, IPT>;
  const size_t smem = onesweep_smem_bytes<KB, VB>();
  if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
  const device_info& di = current_device_info();
  const size_t tiles_all = sweep_tiles_of<KB, VB>(n);
  const unsigned grid = (unsigned)(tiles_all < (size_t)di.sm_count * ONESWEEP_CTAS_PER_SM ? tiles_all : (size_t)di.sm_count * ONESWEEP_CTAS_PER_SM);
  kern<<<grid, ONESWEEP_BLOCK, smem, stream>>>(keys, vals, (unsigned)n, coding, d_splitters, buckets, table,
                                               reinterpret_cast<uint32_t*>(base + sizeof(ws_header)), reinterpret_cast<ws_header*>(base));
  return cudaGetLastError();
}

// row[0, fields * 4096 + EXCH_ROW_TAIL) = this GPU's histograms, the tag and n; no sync
template <class UK>
cudaError_t exchange_hist_async(const UK* keys, size_t n, key_coding coding, unsigned long long tag, unsigned* d_row, cudaStream_t stream) {
  constexpr int F = exch_fields<UK>();
  cudaError_t e = cudaMemsetAsync(d_row, 0, exch_row_words(F) * sizeof(unsigned), stream);
  if (e != cudaSuccess) return e;
  const device_info& di = current_device_info();
  size_t grid = (n + 1024 * 8 - 1) / (1024 * 8);
  if (grid > (size_t)di.sm_count) grid = (size_t)di.sm_count;
  if (grid < 1) grid = 1;
  const size_t smem = (size_t)F * EXCH_BINS * sizeof(unsigned);
  auto kern = exchange_hist_kernel<UK>;
  if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
  kern<<<(unsigned)grid, 1024, smem, stream>>>(keys, n, coding, tag, d_row);
  return cudaGetLastError();
}

inline cudaError_t exchange_plan_async(const unsigned* d_rows, int ranks, int rank, int fields, exchange_plan* d_plan, cudaStream_t stream) {
  if (ranks < 1 || ranks > MAX_BUCKETS || rank < 0 || rank >= ranks || fields < 1 || fields > EXCH_MAX_FIELDS) return cudaErrorInvalidValue;
  exchange_plan_kernel<><<<1, 1024, 0, stream>>>(d_rows, ranks, rank, fields, d_plan);
  return cudaGetLastError();
}

// Stable scatter by the plan's bins (see exchange_scatter_kernel); n < 2^30; workspace as bucket_scatter.  No sync.
template <class UK, class UV, bool HAS_V>
cudaError_t exchange_scatter_async(const UK* keys, const UV* vals, size_t n, key_coding coding, const exchange_plan* d_plan,
                                   const bucket_table<UK, UV>& table, void* ws, cudaStream_t stream) {
  constexpr int KB = sizeof(UK);
  constexpr int VB = HAS_V ? sizeof(UV) : 0;
  constexpr int IPT = onesweep_tuning<KB, VB>::IPT;
  if (n >= (1ull << 30)) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(ws, 0, bucket_scatter_workspace_bytes<KB, VB>(n), stream);
  if (e != cudaSuccess || n == 0) return e;
  char* base = static_cast<char*>(ws);
  auto kern = exchange_scatter_kernel<UK, UV, HAS_V, uint32_t, IPT>;
  const size_t smem = onesweep_smem_bytes<KB, VB>();
  if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
  const device_info& di = current_device_info();
  const size_t tiles_all = sweep_tiles_of<KB, VB>(n);
  const unsigned grid = (unsigned)(tiles_all < (size_t)di.sm_count * ONESWEEP_CTAS_PER_SM ? tiles_all : (size_t)di.sm_count * ONESWEEP_CTAS_PER_SM);
  kern<<<grid, ONESWEEP_BLOCK, smem, stream>>>(keys, vals, (unsigned)n, coding, d_plan, table, reinterpret_cast<uint32_t*>(base + sizeof(ws_header)),
                                               reinterpret_cast<ws_header*>(base));
  return cudaGetLastError();
}

}  // namespace tb200
