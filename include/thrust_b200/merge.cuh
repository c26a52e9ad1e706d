// Merge-path merge and merge sort for sm_100a.
//
// merge / merge_by_key (replaces PartitionAgent + MergeAgent of
// thrust/system/cuda/detail/merge.h:152-660): merge_partition_kernel finds, for every output
// tile boundary, how many items of range A precede it (binary search along the merge-path
// diagonal); merge_kernel then loads a tile's slice of A and of B into shared memory with
// coalesced loads, every thread finds its own start with a second merge-path search in shared
// memory and merges ITEMS outputs serially, and keys (then payloads, gathered by source index)
// go back through shared memory so that the stores are coalesced.  Ties take from A first, so
// the merge is stable.
//
// merge sort (replaces BlockSortAgent + PartitionAgent + MergeAgent of
// thrust/system/cuda/detail/sort.h:235-1138): block_sort_kernel sorts each tile (per-thread
// odd-even transposition network, then log2(BLOCK) rounds of pairwise merge-path merges in
// shared memory, all stable), and the same two merge kernels run in "pairwise" mode over runs of
// doubling length, ping-ponging between the data and a scratch copy.
#pragma once
#include "common.cuh"

namespace tb200 {

constexpr int MERGE_BLOCK = 256;
// Tunables: items per thread and resident CTAs per SM asked of the compiler (a register cap) for
// items of up to 8 and up to 12 bytes (key + payload).  The merge kernels are bound by the latency
// of their barrier-separated phases, not by issue slots or memory, so small tiles and many resident
// CTAs pay: measured on B200, 11 items per thread at 8 CTAs per SM (32 registers) for 8-byte items
// and 7 items at 7 CTAs (36 registers) for 12-byte items took a merge pass over 2^26 (u32, f32)
// pairs from 0.545 to 0.32 ms and merge_by_key of 2 x 2^27 (u64, u32) from 2.16 to 1.79 ms against
// 15 / 11 items at the compiler's own 58 registers (4 CTAs).  The block sort gains little (5 CTAs).
#ifndef TB200_MERGE_IPT8
#define TB200_MERGE_IPT8 11
#endif
#ifndef TB200_MERGE_IPT12
#define TB200_MERGE_IPT12 7
#endif
#ifndef TB200_MERGE_CTAS8
#define TB200_MERGE_CTAS8 8
#endif
#ifndef TB200_MERGE_CTAS12
#define TB200_MERGE_CTAS12 7
#endif
#ifndef TB200_BSORT_IPT8
#define TB200_BSORT_IPT8 16
#endif
#ifndef TB200_BSORT_CTAS8
#define TB200_BSORT_CTAS8 5
#endif

// Items per thread: tuned for the small types, then whatever keeps the staged tile (keys and
// payloads of 256 * IPT items) inside 44 KB of static shared memory, as the reference sizes its
// tiles by sizeof(T) (thrust/system/cuda/detail/merge.h:301-360).
constexpr int MERGE_SMEM_BUDGET = 44 * 1024;
template <int KB, int VB> struct merge_tuning {
  static constexpr int TUNED = (KB + VB) <= 8 ? TB200_MERGE_IPT8 : ((KB + VB) <= 12 ? TB200_MERGE_IPT12 : 9);
  static constexpr int MIN_CTAS = (KB + VB) <= 8 ? TB200_MERGE_CTAS8 : ((KB + VB) <= 12 ? TB200_MERGE_CTAS12 : 1);
  static constexpr int FIT = MERGE_SMEM_BUDGET / (MERGE_BLOCK * (KB + VB));
  static constexpr int IPT = TUNED < FIT ? TUNED : (FIT < 1 ? 1 : FIT);
  static_assert(MERGE_BLOCK * IPT * (KB + VB) + KB <= 48 * 1024, "key + payload too large for the merge tile (more than 160 bytes per item)");
};

// Number of items taken from A among the first `diag` outputs of merge(A[0,na), B[0,nb)).
template <class KeyItA, class KeyItB, class Comp>
__host__ __device__ __forceinline__ size_t merge_path(KeyItA a, size_t na, KeyItB b, size_t nb, size_t diag, Comp comp) {
  size_t lo = diag > nb ? diag - nb : 0;
  size_t hi = diag < na ? diag : na;
  while (lo < hi) {
    size_t mid = (lo + hi) >> 1;
    if (!comp(b[diag - 1 - mid], a[mid])) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Which slices a tile merges.  The output is cut into "pairs": in single mode one pair, A = [0, na)
// of one array and B = [0, nb) of another; in pairwise mode (merge sort) one array of n items in
// sorted runs of length `run`, pair p merging runs 2p and 2p+1.  Tiles never straddle a pair:
// each pair is covered by tiles_per_pair tiles of TILE outputs.
struct merge_geometry {
  size_t na, nb;          // single mode
  size_t n, run;          // pairwise mode (run == 0 selects single mode)
  size_t tiles_per_pair;
  template <int TILE> __host__ __device__ static merge_geometry single(size_t na, size_t nb) {
    merge_geometry g; g.na = na; g.nb = nb; g.n = na + nb; g.run = 0;
    g.tiles_per_pair = (na + nb + TILE - 1) / TILE; if (g.tiles_per_pair == 0) g.tiles_per_pair = 1;
    return g;
  }
  template <int TILE> __host__ __device__ static merge_geometry pairwise(size_t n, size_t run) {
    merge_geometry g; g.na = g.nb = 0; g.n = n; g.run = run; g.tiles_per_pair = (2 * run + TILE - 1) / TILE;
    return g;
  }
  __host__ __device__ size_t num_tiles() const {
    if (run == 0) return tiles_per_pair;
    return (n + 2 * run - 1) / (2 * run) * tiles_per_pair;
  }
  // tile t -> its pair's slices (offsets into the A / B arrays), the pair's first output position
  // and the tile's first output position relative to that
  template <int TILE>
  __host__ __device__ void locate(size_t t, size_t& a0, size_t& alen, size_t& b0, size_t& blen, size_t& pair_out, size_t& local) const {
    const size_t p = t / tiles_per_pair;
    local = (t % tiles_per_pair) * (size_t)TILE;
    if (run == 0) { a0 = 0; alen = na; b0 = 0; blen = nb; pair_out = 0; return; }
    pair_out = p * 2 * run;
    a0 = pair_out;
    alen = n - a0 < run ? n - a0 : run;
    b0 = a0 + alen;
    blen = n - b0 < run ? n - b0 : run;
  }
};

// One thread per tile: where in A the tile's outputs start and end.
template <class KeyItA, class KeyItB, class Comp, int TILE>
__global__ void __launch_bounds__(256)
merge_partition_kernel(KeyItA ka, KeyItB kb, merge_geometry g, size_t num_tiles, Comp comp, size_t* a_split) {
  size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= num_tiles) return;
  size_t a0, alen, b0, blen, pair_out, local;
  g.locate<TILE>(t, a0, alen, b0, blen, pair_out, local);
  const size_t pair_total = alen + blen;
  size_t d0 = local < pair_total ? local : pair_total;
  size_t d1 = local + TILE < pair_total ? local + TILE : pair_total;
  a_split[2 * t] = a0 + merge_path(ka + a0, alen, kb + b0, blen, d0, comp);
  a_split[2 * t + 1] = a0 + merge_path(ka + a0, alen, kb + b0, blen, d1, comp);
}

template <class KeyItA, class KeyItB, class ValItA, class ValItB, class KeyOutIt, class ValOutIt, class K, class V, bool HAS_V, class Comp, int IPT>
__global__ void __launch_bounds__(MERGE_BLOCK, merge_tuning<sizeof(K), HAS_V ? sizeof(V) : 0>::MIN_CTAS)
merge_kernel(KeyItA ka, KeyItB kb, ValItA va, ValItB vb, KeyOutIt ko, ValOutIt vo, merge_geometry g, Comp comp, const size_t* a_split) {
  constexpr int TILE = MERGE_BLOCK * IPT;
  TB200_SHARED_ARRAY(K, s_key, TILE + 1);
  TB200_SHARED_ARRAY(V, s_val, HAS_V ? TILE : 1);
  const size_t t = blockIdx.x;
  size_t a0p, alen, b0p, blen, pair_out, local;
  g.locate<TILE>(t, a0p, alen, b0p, blen, pair_out, local);
  const size_t pair_total = alen + blen;
  if (local >= pair_total) return;                       // a short last pair leaves its later tiles empty
  const size_t out0 = pair_out + local;
  const unsigned tile_n = pair_total - local < TILE ? (unsigned)(pair_total - local) : (unsigned)TILE;
  const size_t a_begin = a_split[2 * t], a_end = a_split[2 * t + 1];
  const size_t b_begin = b0p + local - (a_begin - a0p);
  const unsigned na = (unsigned)(a_end - a_begin), nb = tile_n - na;

  // ---- stage both key slices: A at [0, na), B at [na, na + nb)
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    unsigned c = threadIdx.x + i * MERGE_BLOCK;
    if (c < tile_n) stash(&s_key[c], c < na ? (K)ka[a_begin + c] : (K)kb[b_begin + (c - na)]);
  }
  __syncthreads();

  // ---- per-thread merge path + serial merge of IPT outputs
  unsigned d0 = threadIdx.x * IPT; if (d0 > tile_n) d0 = tile_n;
  unsigned ai = (unsigned)merge_path(s_key, (size_t)na, s_key + na, (size_t)nb, (size_t)d0, comp);
  unsigned bi = d0 - ai;
  K out_k[IPT]; unsigned short src[IPT];
  K keyA = ai < na ? s_key[ai] : K();
  K keyB = bi < nb ? s_key[na + bi] : K();
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    bool take_b = (bi < nb) && (ai >= na || comp(keyB, keyA));
    out_k[i] = take_b ? keyB : keyA;
    src[i] = (unsigned short)(take_b ? na + bi : ai);
    if (take_b) { ++bi; keyB = bi < nb ? s_key[na + bi] : keyB; }
    else { ++ai; keyA = ai < na ? s_key[ai] : keyA; }
  }
  __syncthreads();
  // ---- keys out through shared memory (thread's outputs are consecutive; stores become coalesced)
#pragma unroll
  for (int i = 0; i < IPT; ++i) { unsigned j = threadIdx.x * IPT + i; if (j < tile_n) stash(&s_key[j], out_k[i]); }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < IPT; ++i) { unsigned c = threadIdx.x + i * MERGE_BLOCK; if (c < tile_n) ko[out0 + c] = s_key[c]; }

  if constexpr (HAS_V) {
    V v_in[IPT];
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      unsigned c = threadIdx.x + i * MERGE_BLOCK;
      if (c < tile_n) v_in[i] = c < na ? (V)va[a_begin + c] : (V)vb[b_begin + (c - na)];
    }
#pragma unroll
    for (int i = 0; i < IPT; ++i) { unsigned c = threadIdx.x + i * MERGE_BLOCK; if (c < tile_n) stash(&s_val[c], v_in[i]); }
    __syncthreads();
    V out_v[IPT];
#pragma unroll
    for (int i = 0; i < IPT; ++i) { unsigned j = threadIdx.x * IPT + i; if (j < tile_n) out_v[i] = s_val[src[i]]; }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < IPT; ++i) { unsigned j = threadIdx.x * IPT + i; if (j < tile_n) stash(&s_val[j], out_v[i]); }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < IPT; ++i) { unsigned c = threadIdx.x + i * MERGE_BLOCK; if (c < tile_n) vo[out0 + c] = s_val[c]; }
  }
}

template <class K, class V, bool HAS_V> constexpr int merge_tile_items() { return MERGE_BLOCK * merge_tuning<sizeof(K), HAS_V ? sizeof(V) : 0>::IPT; }

template <class K, class V, bool HAS_V> size_t merge_workspace_bytes(size_t total) {
  // pairwise passes round every pair up to whole tiles: at most one extra tile per pair, and a pair
  // is never smaller than a block-sort tile, so 2x the single-mode tile count is a safe bound
  size_t tiles = (total + merge_tile_items<K, V, HAS_V>() - 1) / merge_tile_items<K, V, HAS_V>();
  return sizeof(ws_header) + align_up((4 * tiles + 8) * sizeof(size_t), 256);
}

// One merge pass (single or pairwise geometry); no sync.
template <class K, class V, bool HAS_V, class KeyItA, class KeyItB, class ValItA, class ValItB, class KeyOutIt, class ValOutIt, class Comp>
cudaError_t merge_pass_async(KeyItA ka, KeyItB kb, ValItA va, ValItB vb, KeyOutIt ko, ValOutIt vo, merge_geometry g, Comp comp, void* ws,
                             cudaStream_t stream) {
  constexpr int IPT = merge_tuning<sizeof(K), HAS_V ? sizeof(V) : 0>::IPT;
  constexpr int TILE = MERGE_BLOCK * IPT;
  if (g.n == 0) return cudaSuccess;
  const size_t tiles = g.num_tiles();
  size_t* a_split = reinterpret_cast<size_t*>(static_cast<char*>(ws) + sizeof(ws_header));
  merge_partition_kernel<KeyItA, KeyItB, Comp, TILE><<<(unsigned)((tiles + 255) / 256), 256, 0, stream>>>(ka, kb, g, tiles, comp, a_split);
  timed_launch tl(KID_MERGE, stream);
  merge_kernel<KeyItA, KeyItB, ValItA, ValItB, KeyOutIt, ValOutIt, K, V, HAS_V, Comp, IPT>
      <<<(unsigned)tiles, MERGE_BLOCK, 0, stream>>>(ka, kb, va, vb, ko, vo, g, comp, a_split);
  return cudaGetLastError();
}

// thrust::merge / merge_by_key: A[0,na) and B[0,nb) sorted by comp -> out[0, na+nb).
template <class K, class V, bool HAS_V, class KeyItA, class KeyItB, class ValItA, class ValItB, class KeyOutIt, class ValOutIt, class Comp>
cudaError_t merge_async(KeyItA ka, size_t na, KeyItB kb, size_t nb, ValItA va, ValItB vb, KeyOutIt ko, ValOutIt vo, Comp comp, void* ws,
                        cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(ws, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess) return e;
  constexpr int TILE = merge_tile_items<K, V, HAS_V>();
  return merge_pass_async<K, V, HAS_V>(ka, kb, va, vb, ko, vo, merge_geometry::single<TILE>(na, nb), comp, ws, stream);
}

// ---------------------------------------------------------------- merge sort
template <int KB, int VB> struct block_sort_tuning {
  // power-of-two friendly tile of 256 * IPT items whose keys (+ a 2-byte index each) fit 44 KB of shared memory
  static constexpr int FIT = MERGE_SMEM_BUDGET / (MERGE_BLOCK * (KB + 2));
  static constexpr int IPT = (KB + VB) <= 8 ? TB200_BSORT_IPT8 : (FIT >= 8 ? 8 : FIT >= 4 ? 4 : FIT >= 2 ? 2 : 1);
  static_assert(MERGE_BLOCK * IPT * (KB + 2) + KB + 2 <= 48 * 1024, "key too large for the block sort tile (more than 170 bytes)");
};

template <class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, class K, class V, bool HAS_V, class Comp, int IPT>
__global__ void __launch_bounds__(MERGE_BLOCK, sizeof(K) <= 4 ? TB200_BSORT_CTAS8 : 1)
block_sort_kernel(KeyIt keys, ValIt vals, KeyOutIt keys_out, ValOutIt vals_out, size_t n, Comp comp) {
  constexpr int TILE = MERGE_BLOCK * IPT;
  TB200_SHARED_ARRAY(K, s_key, TILE + 1);
  __shared__ unsigned short s_idx[TILE + 1];
  const size_t base = (size_t)blockIdx.x * TILE;
  const unsigned tile_n = n - base < TILE ? (unsigned)(n - base) : (unsigned)TILE;

  // ---- coalesced load, then each thread takes IPT consecutive items
#pragma unroll
  for (int i = 0; i < IPT; ++i) { unsigned c = threadIdx.x + i * MERGE_BLOCK; if (c < tile_n) stash(&s_key[c], (K)keys[base + c]); }
  __syncthreads();
  K k[IPT]; unsigned short idx[IPT];
  const unsigned first = threadIdx.x * IPT;
  // items past the end are "infinite": they carry the flag in idx and never move ahead of a real item
  const unsigned mine = first >= tile_n ? 0u : (tile_n - first < (unsigned)IPT ? tile_n - first : (unsigned)IPT);
#pragma unroll
  for (int i = 0; i < IPT; ++i) { idx[i] = (unsigned short)(first + i); if ((unsigned)i < mine) k[i] = s_key[first + i]; else k[i] = K(); }
  auto before = [&](const K& x, unsigned short xi, const K& y, unsigned short yi) {
    // strict "x must come before y" honouring padding: real < pad; pad never before anything
    const bool xp = xi >= tile_n, yp = yi >= tile_n;
    if (xp) return false;
    if (yp) return true;
    return (bool)comp(x, y);
  };
  // ---- odd-even transposition sort of the thread's items (stable: only swaps when strictly out of order)
#pragma unroll
  for (int r = 0; r < IPT; ++r) {
#pragma unroll
    for (int i = r & 1; i + 1 < IPT; i += 2) {
      if (before(k[i + 1], idx[i + 1], k[i], idx[i])) {
        K tk = k[i]; k[i] = k[i + 1]; k[i + 1] = tk;
        unsigned short ti = idx[i]; idx[i] = idx[i + 1]; idx[i + 1] = ti;
      }
    }
  }
  // ---- log2(BLOCK) rounds: runs of `len` items merge pairwise in shared memory
  for (unsigned len = IPT; len < (unsigned)TILE; len <<= 1) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < IPT; ++i) { stash(&s_key[first + i], k[i]); s_idx[first + i] = idx[i]; }
    __syncthreads();
    const unsigned pair0 = first / (2 * len) * (2 * len);
    const unsigned a0 = pair0, b0 = pair0 + len;
    const unsigned d = first - pair0;
    // merge path over the two runs (padding compares as +infinity, ties take from the left run)
    unsigned lo = d > len ? d - len : 0, hi = d < len ? d : len;
    while (lo < hi) {
      unsigned mid = (lo + hi) >> 1;
      if (!before(s_key[b0 + d - 1 - mid], s_idx[b0 + d - 1 - mid], s_key[a0 + mid], s_idx[a0 + mid])) lo = mid + 1; else hi = mid;
    }
    unsigned ai = lo, bi = d - lo;
    // the two candidates stay in registers; only the side that was taken is read again
    K cand_a = K(), cand_b = K();
    unsigned short cand_ai = 0, cand_bi = 0;
    if (ai < len) { cand_a = s_key[a0 + ai]; cand_ai = s_idx[a0 + ai]; }
    if (bi < len) { cand_b = s_key[b0 + bi]; cand_bi = s_idx[b0 + bi]; }
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      bool take_b;
      if (bi >= len) take_b = false;
      else if (ai >= len) take_b = true;
      else take_b = before(cand_b, cand_bi, cand_a, cand_ai);
      if (take_b) {
        k[i] = cand_b; idx[i] = cand_bi;
        ++bi;
        if (bi < len) { cand_b = s_key[b0 + bi]; cand_bi = s_idx[b0 + bi]; }
      } else {
        k[i] = cand_a; idx[i] = cand_ai;
        ++ai;
        if (ai < len) { cand_a = s_key[a0 + ai]; cand_ai = s_idx[a0 + ai]; }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < IPT; ++i) { stash(&s_key[first + i], k[i]); s_idx[first + i] = idx[i]; }
  __syncthreads();
  // gather the payloads by source index before anything is written: the output may be the input
  V v_out[HAS_V ? IPT : 1];
  if constexpr (HAS_V) {
#pragma unroll
    for (int i = 0; i < IPT; ++i) { unsigned c = threadIdx.x + i * MERGE_BLOCK; if (c < tile_n) v_out[i] = vals[base + s_idx[c]]; }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    unsigned c = threadIdx.x + i * MERGE_BLOCK;
    if (c < tile_n) {
      keys_out[base + c] = s_key[c];
      if constexpr (HAS_V) vals_out[base + c] = v_out[i];
    }
  }
}

template <class K, class V, bool HAS_V> constexpr int block_sort_tile_items() { return MERGE_BLOCK * block_sort_tuning<sizeof(K), HAS_V ? sizeof(V) : 0>::IPT; }

template <class K, class V, bool HAS_V> size_t merge_sort_workspace_bytes(size_t n) { return merge_workspace_bytes<K, V, HAS_V>(n); }

// Stable merge sort of keys (and values) in place; keys_alt / vals_alt are same-sized scratch.
template <class K, class V, bool HAS_V, class Comp>
cudaError_t merge_sort_async(K* keys, K* keys_alt, V* vals, V* vals_alt, size_t n, Comp comp, void* ws, cudaStream_t stream) {
  constexpr int BS_IPT = block_sort_tuning<sizeof(K), HAS_V ? sizeof(V) : 0>::IPT;
  constexpr size_t BS_TILE = (size_t)MERGE_BLOCK * BS_IPT;
  cudaError_t e = cudaMemsetAsync(ws, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess || n <= 1) return e;
  const size_t tiles = (n + BS_TILE - 1) / BS_TILE;
  int passes = 0;
  for (size_t run = BS_TILE; run < n; run <<= 1) ++passes;
  // the block sort writes to whichever buffer makes the last merge pass land in `keys`
  K* cur_k = (passes & 1) ? keys_alt : keys;
  V* cur_v = (passes & 1) ? vals_alt : vals;
  K* oth_k = (passes & 1) ? keys : keys_alt;
  V* oth_v = (passes & 1) ? vals : vals_alt;
  { timed_launch tl(KID_BLOCK_SORT, stream);
  block_sort_kernel<const K*, const V*, K*, V*, K, V, HAS_V, Comp, BS_IPT><<<(unsigned)tiles, MERGE_BLOCK, 0, stream>>>(keys, vals, cur_k, cur_v, n, comp); }
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  for (size_t run = BS_TILE; run < n; run <<= 1) {
    constexpr int TILE = merge_tile_items<K, V, HAS_V>();
    e = merge_pass_async<K, V, HAS_V>((const K*)cur_k, (const K*)cur_k, (const V*)cur_v, (const V*)cur_v, oth_k, oth_v,
                                      merge_geometry::pairwise<TILE>(n, run), comp, ws, stream);
    if (e != cudaSuccess) return e;
    K* tk = cur_k; cur_k = oth_k; oth_k = tk;
    V* tv = cur_v; cur_v = oth_v; oth_v = tv;
  }
  return cudaSuccess;
}

}  // namespace tb200
