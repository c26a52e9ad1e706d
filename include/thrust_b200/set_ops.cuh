// Set operations on sorted ranges (set_union, set_intersection, set_difference,
// set_symmetric_difference, with or without values "by key") for sm_100a.
//
// Replaces the balanced-path agents of thrust/system/cuda/detail/set_operations.h:318-890.
// Multiset semantics as in the reference: an element that occurs m times in A and n times in B
// appears max(m, n) times in the union (A's copies first), min(m, n) times in the intersection (A's),
// max(m - n, 0) times in the difference (A's last copies) and |m - n| times in the symmetric
// difference (the surplus side's last copies).  In every case the result is the stable merge of A
// and B (A first among equivalent elements) with some elements dropped, and whether an element is
// dropped depends only on its rank r inside its own run of equivalent elements and on whether the
// other side has more than r such elements.  So the merge is cut into tiles of 2048 consecutive
// merged positions along its merge path (any cut works: nothing is decided from tile-local
// information alone), and two stream-ordered launches with no host round trip do the rest:
//   1. set_partition_kernel  one thread per tile boundary: a binary search along the diagonal;
//   2. set_tile_kernel       every thread takes eight consecutive positions of the tile's merge: one
//                            binary search along its diagonal finds where they start in A and in B,
//                            one galloping search backwards per side gives the ranks of the two
//                            current elements inside their runs; then it merges serially, keeping
//                            the ranks up to date with one comparison per step, and decides each
//                            element with one probe of the other side's element number r.  The
//                            tile's number of kept elements is published, a decoupled look-back
//                            over the earlier tiles' counts (tiles by atomic ticket, bounded waits)
//                            gives the tile's place in the output, and every thread writes its
//                            kept elements (and their values) in order: one pass over the inputs.
// The workspace is 24 bytes per tile; sizes are 64-bit throughout.
#pragma once
#include "common.cuh"

namespace tb200 {

enum set_op : int { SET_UNION = 0, SET_INTERSECTION = 1, SET_DIFFERENCE = 2, SET_SYMMETRIC_DIFFERENCE = 3 };
constexpr int SETOP_BLOCK = 256;
constexpr int SETOP_IPT = 8;
constexpr int SETOP_TILE = SETOP_BLOCK * SETOP_IPT;

// first index in [0, n) whose element does not order before x
template <class It, class T, class Comp> __device__ __forceinline__ size_t set_lower_bound(It a, size_t n, const T& x, Comp comp) {
  size_t lo = 0, hi = n;
  while (lo < hi) { const size_t mid = (lo + hi) >> 1; if (comp(a[mid], x)) lo = mid + 1; else hi = mid; }
  return lo;
}
// first index in [0, n) whose element orders after x
template <class It, class T, class Comp> __device__ __forceinline__ size_t set_upper_bound(It a, size_t n, const T& x, Comp comp) {
  size_t lo = 0, hi = n;
  while (lo < hi) { const size_t mid = (lo + hi) >> 1; if (!comp(x, a[mid])) lo = mid + 1; else hi = mid; }
  return lo;
}
// how many elements directly before s[i] are equivalent to x = s[i]: doubling steps backwards, then a
// binary search inside the last step
template <class It, class T, class Comp> __device__ __forceinline__ size_t set_run_rank(It s, size_t i, const T& x, Comp comp) {
  if (i == 0 || comp(s[i - 1], x)) return 0;
  size_t step = 1;                                             // s[i - step] is equivalent to x
  while (step * 2 <= i && !comp(s[i - step * 2], x)) step *= 2;
  size_t lo = i > step * 2 ? i - step * 2 : 0, hi = i - step;
  while (lo < hi) { const size_t mid = (lo + hi) >> 1; if (comp(s[mid], x)) lo = mid + 1; else hi = mid; }
  return i - lo;
}
// number of A's elements among the first d of the stable merge of A and B
template <class ItA, class ItB, class Comp> __device__ __forceinline__ size_t set_merge_split(ItA a, size_t na, ItB b, size_t nb, size_t d, Comp comp) {
  size_t lo = d > nb ? d - nb : 0, hi = d < na ? d : na;
  while (lo < hi) {
    const size_t mid = (lo + hi) >> 1;
    if (!comp(b[d - 1 - mid], a[mid])) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// split[t] = A's share of the first t * SETOP_TILE merged elements, t in [0, tiles]
template <class ItA, class ItB, class Comp>
__global__ void __launch_bounds__(256) set_partition_kernel(ItA a, size_t na, ItB b, size_t nb, size_t tiles, Comp comp, unsigned long long* split) {
  const size_t t = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (t > tiles) return;
  const size_t d = t * SETOP_TILE < na + nb ? t * SETOP_TILE : na + nb;
  split[t] = set_merge_split(a, na, b, nb, d, comp);
}

template <bool HAS_V, class T, class ItA, class ItB, class VItA, class VItB, class KeyOutIt, class ValOutIt, class Comp>
__global__ void __launch_bounds__(SETOP_BLOCK)
set_tile_kernel(ItA a, size_t na, ItB b, size_t nb, VItA va, VItB vb, KeyOutIt out, ValOutIt vout, int op, Comp comp, const unsigned long long* split,
                tile_state<unsigned long long> ts, size_t tiles, ws_header* hdr, unsigned long long* d_count) {
  __shared__ unsigned s_warp[SETOP_BLOCK / 32];
  __shared__ unsigned s_ticket;
  __shared__ unsigned long long s_base;
  // tiles are taken in the order in which CTAs start, so a tile only ever waits for tiles whose CTAs run
  if (threadIdx.x == 0) s_ticket = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const size_t tile = s_ticket;
  const size_t d0 = tile * SETOP_TILE;
  const size_t a0 = split[tile], a1 = split[tile + 1];
  const size_t d1 = d0 + SETOP_TILE < na + nb ? d0 + SETOP_TILE : na + nb;
  const size_t b0 = d0 - a0, b1 = d1 - a1;
  const unsigned count = (unsigned)(d1 - d0);
  // this thread's SETOP_IPT consecutive positions of the merge: where they start in A and in B
  unsigned t0 = threadIdx.x * SETOP_IPT; if (t0 > count) t0 = count;
  unsigned t1 = t0 + SETOP_IPT; if (t1 > count) t1 = count;
  size_t ai = a0 + set_merge_split(a + a0, a1 - a0, b + b0, b1 - b0, (size_t)t0, comp);
  size_t bi = b0 + (t0 - (ai - a0));
  // ranks of the two current elements inside their runs of equivalent elements
  size_t ra = 0, rb = 0;
  T ka = T(), kb = T();
  if (t0 < t1) {
    if (ai < na) { ka = a[ai]; ra = set_run_rank(a, ai, ka, comp); }
    if (bi < nb) { kb = b[bi]; rb = set_run_rank(b, bi, kb, comp); }
  }
  unsigned keep_bits = 0, from_b = 0, kept = 0;
  unsigned src[SETOP_IPT];                                      // offset of every position's element inside its slice
#pragma unroll
  for (int i = 0; i < SETOP_IPT; ++i) {
    src[i] = 0;
    if (t0 + i >= t1) continue;
    const bool take_a = ai < a1 && (bi >= b1 || !comp(kb, ka));   // A first among equivalent elements
    bool keep;
    if (take_a) {
      // B's elements ahead of this one in the merge are exactly those that order before it: bi of them
      if (op == SET_UNION) keep = true;
      else {
        const bool other_has = bi + ra < nb && !comp(ka, b[bi + ra]);         // B holds more than ra elements equivalent to it
        keep = op == SET_INTERSECTION ? other_has : !other_has;
      }
      src[i] = (unsigned)(ai - a0);
      ++ai;
      if (ai < na) { const T next = a[ai]; ra = comp(ka, next) ? 0 : ra + 1; ka = next; }
    } else {
      // A's elements ahead of this one are those that order before it or are equivalent: ai of them
      if (op == SET_UNION || op == SET_SYMMETRIC_DIFFERENCE) {
        const bool other_has = ai > rb && !comp(a[ai - 1 - rb], kb);          // A holds more than rb elements equivalent to it
        keep = !other_has;
      } else keep = false;
      src[i] = (unsigned)(bi - b0);
      from_b |= 1u << i;
      ++bi;
      if (bi < nb) { const T next = b[bi]; rb = comp(kb, next) ? 0 : rb + 1; kb = next; }
    }
    if (keep) { keep_bits |= 1u << i; ++kept; }
  }
  // where the tile's output starts: its count is published, the counts of the tiles before it are
  // folded by a decoupled look-back (bounded waits), the running total is published for the tiles behind
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned incl = warp_inclusive_scan(kept, plus_op());
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  unsigned before = 0, tile_total = 0;
  for (unsigned w = 0; w < SETOP_BLOCK / 32; ++w) { if (w < warp) before += s_warp[w]; tile_total += s_warp[w]; }
  if (warp == 0) {
    unsigned long long prefix = 0;
    if (tile == 0) {
      if (lane == 0) ts.publish(0, TILE_INCLUSIVE, (unsigned long long)tile_total);
    } else {
      if (lane == 0) ts.publish(tile, TILE_AGGREGATE, (unsigned long long)tile_total);
      prefix = lookback_prefix<unsigned long long>(ts, tile, plus_op(), &hdr->error);
      if (lane == 0) ts.publish(tile, TILE_INCLUSIVE, prefix + tile_total);
    }
    if (lane == 0) s_base = prefix;
  }
  __syncthreads();
  const unsigned long long base = s_base;
  size_t at = (size_t)base + before + (incl - kept);
#pragma unroll
  for (int i = 0; i < SETOP_IPT; ++i) {
    if ((keep_bits >> i) & 1) {
      if ((from_b >> i) & 1) {
        out[at] = b[b0 + src[i]];
        if constexpr (HAS_V) vout[at] = vb[b0 + src[i]];
      } else {
        out[at] = a[a0 + src[i]];
        if constexpr (HAS_V) vout[at] = va[a0 + src[i]];
      }
      ++at;
    }
  }
  if (tile + 1 == tiles && threadIdx.x == 0) {
    const unsigned long long total = base + tile_total;
    hdr->count = total;
    if (d_count) *d_count = total;
  }
}

inline size_t set_op_tiles(size_t na, size_t nb) { return (na + nb + SETOP_TILE - 1) / SETOP_TILE; }
// header | split [tiles + 1] | one look-back descriptor per tile
inline size_t set_op_workspace_bytes(size_t na, size_t nb) {
  const size_t tiles = set_op_tiles(na, nb);
  return sizeof(ws_header) + align_up((tiles + 1) * 8, 256) + tile_state<unsigned long long>::bytes(tiles + 1);
}

// A[0, na) and B[0, nb) sorted by comp; keys (and, HAS_V, the values that travel with the kept keys:
// va[i] with A[i], vb[j] with B[j] -- B's elements are kept only by the union and the symmetric
// difference, so vb is not read otherwise) go to out / vout, whose capacity must be na + nb (union,
// symmetric difference), na (difference) or min(na, nb) (intersection).  The number of items written
// lands in the workspace header and *d_count.  No sync.
template <class T, bool HAS_V, class ItA, class ItB, class VItA, class VItB, class KeyOutIt, class ValOutIt, class Comp>
cudaError_t set_operation_async(int op, ItA a, size_t na, ItB b, size_t nb, VItA va, VItB vb, KeyOutIt out, ValOutIt vout, Comp comp,
                                unsigned long long* d_count, void* ws, cudaStream_t stream) {
  const size_t tiles = set_op_tiles(na, nb);
  if (op < SET_UNION || op > SET_SYMMETRIC_DIFFERENCE || tiles >= 0x7fffffffull) return cudaErrorInvalidValue;
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  unsigned long long* split = reinterpret_cast<unsigned long long*>(base + sizeof(ws_header));
  char* desc = base + sizeof(ws_header) + align_up((tiles + 1) * 8, 256);
  if (tiles == 0) {
    cudaError_t e0 = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream);
    if (e0 != cudaSuccess) return e0;
    return d_count ? cudaMemsetAsync(d_count, 0, sizeof(unsigned long long), stream) : cudaSuccess;
  }
  // header (ticket, status, count) and descriptors start out zero; the split array is written in full
  cudaError_t e = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess) return e;
  if ((e = cudaMemsetAsync(desc, 0, tile_state<unsigned long long>::bytes(tiles + 1), stream)) != cudaSuccess) return e;
  tile_state<unsigned long long> ts;
  ts.bind(desc, tiles + 1);
  set_partition_kernel<<<(unsigned)((tiles + 1 + 255) / 256), 256, 0, stream>>>(a, na, b, nb, tiles, comp, split);
  set_tile_kernel<HAS_V, T><<<(unsigned)tiles, SETOP_BLOCK, 0, stream>>>(a, na, b, nb, va, vb, out, vout, op, comp, split, ts, tiles, hdr, d_count);
  log_launch("set_partition_kernel + set_tile_kernel", tiles, SETOP_BLOCK, 0, na + nb, stream);
  return cudaGetLastError();
}

}  // namespace tb200
