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
// information alone), and three stream-ordered steps with no host round trip do the rest:
//   1. set_partition_kernel  one thread per tile boundary: a binary search along the diagonal;
//   2. set_tile_kernel<COUNT> every element finds its merged position (a binary search inside the
//                            tile's slice of the other side), its rank r (a galloping search
//                            backwards, one probe when keys are unique) and probes the other side's
//                            element number r; the tile's number of kept elements goes to an array
//                            that scan.cuh scans;
//   3. set_tile_kernel<EMIT>  the same, then a block scan over the kept flags in merged order and
//                            the kept elements (and their values) are written out in order.
// The workspace is 24 bytes per tile; sizes are 64-bit throughout.
#pragma once
#include "common.cuh"
#include "scan.cuh"

namespace tb200 {

enum set_op : int { SET_UNION = 0, SET_INTERSECTION = 1, SET_DIFFERENCE = 2, SET_SYMMETRIC_DIFFERENCE = 3 };
constexpr int SETOP_BLOCK = 512;
constexpr int SETOP_IPT = 4;
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

template <bool EMIT, bool HAS_V, class T, class ItA, class ItB, class VItA, class VItB, class KeyOutIt, class ValOutIt, class Comp>
__global__ void __launch_bounds__(SETOP_BLOCK)
set_tile_kernel(ItA a, size_t na, ItB b, size_t nb, VItA va, VItB vb, KeyOutIt out, ValOutIt vout, int op, Comp comp, const unsigned long long* split,
                unsigned long long* totals, const unsigned long long* bases, size_t tiles, ws_header* hdr, const ws_header* scan_hdr,
                unsigned long long* d_count) {
  __shared__ unsigned s_src[EMIT ? SETOP_TILE : 1];            // by merged position: item number | kept << 31
  __shared__ unsigned s_warp[SETOP_BLOCK / 32];
  const size_t tile = blockIdx.x;
  const size_t d0 = tile * SETOP_TILE;
  const size_t a0 = split[tile], a1 = split[tile + 1];
  const size_t d1 = d0 + SETOP_TILE < na + nb ? d0 + SETOP_TILE : na + nb;
  const size_t b0 = d0 - a0, b1 = d1 - a1;
  const unsigned ca = (unsigned)(a1 - a0), count = (unsigned)(d1 - d0);
  if constexpr (EMIT) {
    if (count < SETOP_TILE) {
      for (unsigned p = threadIdx.x; p < SETOP_TILE; p += SETOP_BLOCK) s_src[p] = 0;
      __syncthreads();
    }
  }
  unsigned kept = 0;
#pragma unroll
  for (int it = 0; it < SETOP_IPT; ++it) {
    const unsigned k = threadIdx.x + it * SETOP_BLOCK;
    if (k >= count) break;
    bool keep;
    unsigned pos;
    if (k < ca) {
      const size_t i = a0 + k;
      const T x = a[i];
      const size_t lb = b0 + set_lower_bound(b + b0, b1 - b0, x, comp);        // B's elements that order before x
      pos = k + (unsigned)(lb - b0);
      if (op == SET_UNION) keep = true;
      else {
        const size_t r = set_run_rank(a, i, x, comp);
        const bool other_has = lb + r < nb && !comp(x, b[lb + r]);            // B holds more than r elements equivalent to x
        keep = op == SET_INTERSECTION ? other_has : !other_has;
      }
    } else {
      const size_t j = b0 + (k - ca);
      const T y = b[j];
      const size_t ub = a0 + set_upper_bound(a + a0, a1 - a0, y, comp);        // A's elements that order before y or are equivalent
      pos = (k - ca) + (unsigned)(ub - a0);
      if (op == SET_UNION || op == SET_SYMMETRIC_DIFFERENCE) {
        const size_t r = set_run_rank(b, j, y, comp);
        const bool other_has = ub > r && !comp(a[ub - 1 - r], y);             // A holds more than r elements equivalent to y
        keep = !other_has;
      } else keep = false;
    }
    kept += keep ? 1u : 0u;
    if constexpr (EMIT) s_src[pos] = k | (keep ? 0x80000000u : 0u);
  }
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if constexpr (!EMIT) {
    kept = __reduce_add_sync(0xffffffffu, kept);
    if (lane == 0) s_warp[warp] = kept;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned total = 0;
      for (int w = 0; w < SETOP_BLOCK / 32; ++w) total += s_warp[w];
      totals[tile] = total;
    }
  } else {
    __syncthreads();
    unsigned mine[SETOP_IPT];
    unsigned c = 0;
#pragma unroll
    for (int q = 0; q < SETOP_IPT; ++q) { mine[q] = s_src[threadIdx.x * SETOP_IPT + q]; c += mine[q] >> 31; }
    const unsigned incl = warp_inclusive_scan(c, plus_op());
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    unsigned before = 0;
    for (unsigned w = 0; w < warp; ++w) before += s_warp[w];
    const unsigned long long base = bases[tile];
    size_t at = (size_t)base + before + (incl - c);
#pragma unroll
    for (int q = 0; q < SETOP_IPT; ++q) {
      if (mine[q] >> 31) {
        const unsigned k = mine[q] & 0x7fffffffu;
        if (k < ca) {
          out[at] = a[a0 + k];
          if constexpr (HAS_V) vout[at] = va[a0 + k];
        } else {
          out[at] = b[b0 + (k - ca)];
          if constexpr (HAS_V) vout[at] = vb[b0 + (k - ca)];
        }
        ++at;
      }
    }
    if (tile + 1 == tiles && threadIdx.x == SETOP_BLOCK - 1) {
      const unsigned long long total = base + before + incl;
      hdr->count = total;
      hdr->error = scan_hdr->error;
      if (d_count) *d_count = total;
    }
  }
}

inline size_t set_op_tiles(size_t na, size_t nb) { return (na + nb + SETOP_TILE - 1) / SETOP_TILE; }
// header | split [tiles + 1] | totals [tiles] | bases [tiles] | the scan's workspace
inline size_t set_op_workspace_bytes(size_t na, size_t nb) {
  const size_t tiles = set_op_tiles(na, nb);
  return sizeof(ws_header) + align_up((tiles + 1) * 8, 256) + 2 * align_up(tiles * 8 + 8, 256) + scan_workspace_bytes<unsigned long long>(tiles + 1);
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
  char* p = base + sizeof(ws_header);
  unsigned long long* split = reinterpret_cast<unsigned long long*>(p); p += align_up((tiles + 1) * 8, 256);
  unsigned long long* totals = reinterpret_cast<unsigned long long*>(p); p += align_up(tiles * 8 + 8, 256);
  unsigned long long* bases = reinterpret_cast<unsigned long long*>(p); p += align_up(tiles * 8 + 8, 256);
  void* scan_ws = p;
  cudaError_t e = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess) return e;
  if (tiles == 0) return d_count ? cudaMemsetAsync(d_count, 0, sizeof(unsigned long long), stream) : cudaSuccess;
  set_partition_kernel<<<(unsigned)((tiles + 1 + 255) / 256), 256, 0, stream>>>(a, na, b, nb, tiles, comp, split);
  set_tile_kernel<false, HAS_V, T><<<(unsigned)tiles, SETOP_BLOCK, 0, stream>>>(a, na, b, nb, va, vb, out, vout, op, comp, split, totals, bases, tiles, hdr,
                                                                                 static_cast<const ws_header*>(scan_ws), d_count);
  if ((e = scan_async<false>((const unsigned long long*)totals, bases, tiles, 0ull, true, plus_op(), scan_ws, stream)) != cudaSuccess) return e;
  set_tile_kernel<true, HAS_V, T><<<(unsigned)tiles, SETOP_BLOCK, 0, stream>>>(a, na, b, nb, va, vb, out, vout, op, comp, split, totals, bases, tiles, hdr,
                                                                                static_cast<const ws_header*>(scan_ws), d_count);
  log_launch("set_partition_kernel + set_tile_kernel x2 + scan", tiles, SETOP_BLOCK, 0, na + nb, stream);
  return cudaGetLastError();
}

}  // namespace tb200
