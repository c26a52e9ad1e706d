// Single-pass reduce_by_key for sm_100a.
//
// A run starts at item 0 and wherever !key_eq(key[i-1], key[i]).  One CTA per tile (dynamic
// ticket).  The tile's keys and values are loaded with coalesced 16-byte loads into shared memory;
// every thread then takes ITEMS *consecutive* items (an odd count, so the strided shared-memory
// reads are conflict-free) and walks them once to get its summary pair
//     (number of run heads in my items, reduction of my still-open last run).
// Summaries combine as (c1, v1) (+) (c2, v2) = (c1 + c2, c2 ? v2 : op(v1, v2)); ONE scan of these
// pairs over the CTA's threads (warp shuffles) plus the decoupled look-back over the preceding
// tiles gives each thread the number of heads before it and the value carried into its first
// item.  A second walk over the registers then emits, at every head, the key of the new run and
// the finished total of the run before it; heads are compacted through shared memory so that
// keys_out / values_out are written with consecutive threads on consecutive addresses.  Values
// inside a run are combined left to right.  Replaces InitAgent + ReduceByKeyAgent of
// thrust/system/cuda/detail/reduce_by_key.h:197-860.
#pragma once
#include "common.cuh"
#include "reduce_by_key_stream.cuh"

namespace tb200 {

constexpr int RBK_BLOCK = 256;

template <class Off, class V> struct rbk_pair { Off count; V value; };

template <class Off, class V, class Op> struct rbk_combine {
  Op op;
  __device__ __forceinline__ rbk_pair<Off, V> operator()(const rbk_pair<Off, V>& a, const rbk_pair<Off, V>& b) const {
    rbk_pair<Off, V> r;
    r.count = a.count + b.count;
    r.value = b.count ? b.value : op(a.value, b.value);
    return r;
  }
};

template <class K, class V> struct rbk_tuning {
  static constexpr int BYTES = sizeof(K) > sizeof(V) ? sizeof(K) : sizeof(V);
#ifndef TB200_RBK_IPT4
#define TB200_RBK_IPT4 17   /* 25 measured slower; the head mask limits it to 31 */
#endif
  static constexpr int IPT = BYTES <= 4 ? TB200_RBK_IPT4 : (BYTES <= 8 ? (TB200_RBK_IPT4 / 2) | 1 : 5);   // odd: thread t reads shared words t*IPT + j
};

template <class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, class K, class V, class Eq, class Op, class Off, bool VEC_LOAD, int IPT>
__global__ void __launch_bounds__(RBK_BLOCK)
reduce_by_key_kernel(KeyIt keys, ValIt vals, KeyOutIt keys_out, ValOutIt vals_out, size_t n, Eq key_eq, Op op,
                     tile_state<rbk_pair<Off, V>> ts, ws_header* hdr, unsigned long long* d_count) {
  using P = rbk_pair<Off, V>;
  using Comb = rbk_combine<Off, V, Op>;
  constexpr int NWARPS = RBK_BLOCK / 32;
  constexpr int TILE = RBK_BLOCK * IPT;
  static_assert((TILE * sizeof(K)) % 16 == 0 && (TILE * sizeof(V)) % 16 == 0, "tile must be whole 16-byte vectors");
  __shared__ unsigned s_tile;
  using prefix_smem_t = tile_prefix_smem<P, NWARPS>;
  TB200_SHARED_OBJECT(prefix_smem_t, sm);
  extern __shared__ __align__(16) unsigned char rbk_smem[];          // keys of the tile, then its values
  K* s_key = reinterpret_cast<K*>(rbk_smem);
  V* s_val = reinterpret_cast<V*>(rbk_smem + (TILE * sizeof(K) + 15) / 16 * 16);
  TB200_SHARED_OBJECT(K, s_prev);

  if (threadIdx.x == 0) s_tile = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const size_t tile = s_tile;
  const size_t tile_base = tile * (size_t)TILE;
  const bool full = tile_base + TILE <= n;
  const unsigned tile_n = full ? (unsigned)TILE : (unsigned)(n - tile_base);
  Comb comb; comb.op = op;

  // ---- coalesced load of the tile into shared memory
  bool vec_done = false;
  if constexpr (VEC_LOAD) {
    if (full) {
      const char* gk = reinterpret_cast<const char*>(keys) + tile_base * sizeof(K);
      const char* gv = reinterpret_cast<const char*>(vals) + tile_base * sizeof(V);
      for (unsigned v = threadIdx.x; v < TILE * sizeof(K) / 16; v += RBK_BLOCK) reinterpret_cast<vec16*>(s_key)[v] = load_stream16(gk + (size_t)v * 16);
      for (unsigned v = threadIdx.x; v < TILE * sizeof(V) / 16; v += RBK_BLOCK) reinterpret_cast<vec16*>(s_val)[v] = load_stream16(gv + (size_t)v * 16);
      vec_done = true;
    }
  }
  if (!vec_done) {
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      const unsigned c = threadIdx.x + i * RBK_BLOCK;
      if (c < tile_n) { stash(&s_key[c], (K)keys[tile_base + c]); stash(&s_val[c], (V)vals[tile_base + c]); }
    }
  }
  if (threadIdx.x == 0 && tile_base > 0) s_prev = keys[tile_base - 1];
  __syncthreads();

  // ---- my ITEMS consecutive items; walk 1: head flags and summary
  const unsigned first = threadIdx.x * IPT;
  const unsigned mine = first >= tile_n ? 0u : (tile_n - first < (unsigned)IPT ? tile_n - first : (unsigned)IPT);
  K k[IPT]; V x[IPT];
#pragma unroll
  for (int j = 0; j < IPT; ++j) if ((unsigned)j < mine) { k[j] = s_key[first + j]; x[j] = s_val[first + j]; }
  unsigned heads = 0;
  P summary; summary.count = 0; summary.value = V();
  if (mine) {
    const bool has_prev = first > 0 || tile_base > 0;
    K prev = k[0];
    if (has_prev) prev = first > 0 ? s_key[first - 1] : s_prev;
    V acc = x[0];
#pragma unroll
    for (int j = 0; j < IPT; ++j) {
      if ((unsigned)j < mine) {
        const bool h = (j == 0) ? (!has_prev || !key_eq(prev, k[0])) : !key_eq(k[j - 1], k[j]);
        if (h) { heads |= 1u << j; ++summary.count; acc = x[j]; }
        else if (j > 0) acc = op(acc, x[j]);
      }
    }
    summary.value = acc;
  }

  // ---- one pair scan over the threads of the tile, chained to the preceding tiles
  P vec_total[1] = {summary};
  opt<P> pre[1];
  P none; none.count = 0; none.value = V();
  tile_exclusive_prefix<P, Comb, 1, NWARPS>(vec_total, pre, tile, none, false, comb, ts, &hdr->error, sm);
  const Off head_off = sm.has_prefix ? sm.prefix.count : (Off)0;   // run heads in all preceding tiles
  __syncthreads();                                                  // everyone has its items in registers: reuse the tile buffers

  // ---- walk 2: every head opens a run (its key) and closes the one before it (its total)
  if (mine) {
    Off run = pre[0].has ? pre[0].v.count : (Off)0;                // heads before my first item, globally
    V acc = pre[0].has ? pre[0].v.value : x[0];                    // value carried into my first item
    const size_t g0 = tile_base + first;
#pragma unroll
    for (int j = 0; j < IPT; ++j) {
      if ((unsigned)j < mine) {
        if ((heads >> j) & 1) {
          const unsigned r = (unsigned)(run - head_off);
          stash(&s_key[r], k[j]);
          stash(&s_val[r], acc);                                           // total of the run that ends before this head (unused for run 0)
          ++run;
          acc = x[j];
        } else if (j > 0 || pre[0].has) {
          acc = op(acc, x[j]);
        }
        if (g0 + j == n - 1) {
          vals_out[(size_t)run - 1] = acc;
          hdr->count = (unsigned long long)run;
          if (d_count) *d_count = (unsigned long long)run;
        }
      }
    }
  }
  __syncthreads();
  // heads of this tile: the inclusive count of its last real thread minus the tile's prefix; padding threads add none
  const unsigned tile_heads = (unsigned)(sm.inclusive.count - head_off);
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const unsigned j = threadIdx.x + i * RBK_BLOCK;
    if (j < tile_heads) {
      const size_t g = (size_t)head_off + j;
      keys_out[g] = s_key[j];
      if (g > 0) vals_out[g - 1] = s_val[j];
    }
  }
}

template <class K, class V> constexpr size_t rbk_tile_items() { return (size_t)RBK_BLOCK * rbk_tuning<K, V>::IPT; }
template <class K, class V> size_t rbk_workspace_bytes(size_t n) {
  size_t tiles = (n + rbk_tile_items<K, V>() - 1) / rbk_tile_items<K, V>();
  const size_t single = sizeof(ws_header) + tile_state<rbk_pair<unsigned long long, V>>::bytes(tiles + 1);
  if constexpr (sizeof(K) == sizeof(V) && (sizeof(K) == 4 || sizeof(K) == 8)) {
    const size_t stream = rbk_stream_workspace_bytes<K, V>(n);
    return single > stream ? single : stream;
  }
  return single;
}

// Launches reduce_by_key; no sync.  The number of runs goes to the workspace header and, if
// d_count != nullptr, to *d_count.  keys_out / vals_out need room for one entry per run.
template <bool ALLOW_BIG = true, class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, class K, class V, class Eq, class Op>
cudaError_t reduce_by_key_async(KeyIt keys, ValIt vals, KeyOutIt keys_out, ValOutIt vals_out, size_t n, K, V, Eq eq, Op op,
                                unsigned long long* d_count, void* ws, cudaStream_t stream) {
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  constexpr int IPT = rbk_tuning<K, V>::IPT;
  const size_t tiles = (n + rbk_tile_items<K, V>() - 1) / rbk_tile_items<K, V>();
  // large contiguous inputs with keys and values of one size and outputs elsewhere: the two-pass
  // streaming kernels (reduce_by_key_stream.cuh)
  if constexpr (std::is_pointer<KeyIt>::value && std::is_pointer<ValIt>::value && std::is_pointer<KeyOutIt>::value && std::is_pointer<ValOutIt>::value &&
                sizeof(K) == sizeof(V) && (sizeof(K) == 4 || sizeof(K) == 8) && std::is_trivially_copyable<K>::value && std::is_trivially_copyable<V>::value) {
    using KIn = typename std::remove_cv<typename std::remove_pointer<KeyIt>::type>::type;
    using VIn = typename std::remove_cv<typename std::remove_pointer<ValIt>::type>::type;
    using KOut = typename std::remove_pointer<KeyOutIt>::type;
    using VOut = typename std::remove_pointer<ValOutIt>::type;
    if constexpr (std::is_same<KIn, K>::value && std::is_same<VIn, V>::value && std::is_same<KOut, K>::value && std::is_same<VOut, V>::value) {
      if (rbk_stream_eligible(keys, vals, keys_out, vals_out, n, sizeof(K)))
        return reduce_by_key_stream_async<K, V, Eq, Op>(keys, vals, keys_out, vals_out, n, eq, op, d_count, ws, stream);
    }
  }
  cudaError_t e = cudaMemsetAsync(base, 0, sizeof(ws_header) + tile_state<rbk_pair<unsigned long long, V>>::bytes(tiles + 1), stream);
  if (e != cudaSuccess) return e;
  if (n == 0) { if (d_count) return cudaMemsetAsync(d_count, 0, sizeof(unsigned long long), stream); return cudaSuccess; }
  const bool small = n < (1ull << 31);
  if (!ALLOW_BIG && !small) return cudaErrorInvalidValue;
  auto launch = [&](auto off_tag, auto vec_tag) {
    using Off = decltype(off_tag);
    constexpr bool VEC = decltype(vec_tag)::value;
    tile_state<rbk_pair<Off, V>> ts;
    ts.bind(base + sizeof(ws_header), tiles + 1);
    auto kern = reduce_by_key_kernel<KeyIt, ValIt, KeyOutIt, ValOutIt, K, V, Eq, Op, Off, VEC, IPT>;
    const size_t smem = (rbk_tile_items<K, V>() * sizeof(K) + 15) / 16 * 16 + rbk_tile_items<K, V>() * sizeof(V);
    if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return;
    timed_launch tl(KID_REDUCE_BY_KEY, stream);
    kern<<<(unsigned)tiles, RBK_BLOCK, smem, stream>>>(keys, vals, keys_out, vals_out, n, eq, op, ts, hdr, d_count);
  };
  constexpr bool ptrs = std::is_pointer<KeyIt>::value && std::is_pointer<ValIt>::value;
  bool use_vec = false;
  if constexpr (ptrs) {
    using KIn = typename std::remove_cv<typename std::remove_pointer<KeyIt>::type>::type;
    using VIn = typename std::remove_cv<typename std::remove_pointer<ValIt>::type>::type;
    if constexpr (std::is_same<KIn, K>::value && std::is_same<VIn, V>::value && std::is_trivially_copyable<K>::value && std::is_trivially_copyable<V>::value) {
      use_vec = is_aligned16((const void*)keys) && is_aligned16((const void*)vals);
      if (use_vec) {
        if (small) launch((unsigned)0, std::true_type()); else if constexpr (ALLOW_BIG) launch((unsigned long long)0, std::true_type());
        return e != cudaSuccess ? e : cudaGetLastError();
      }
    }
  }
  if (small) launch((unsigned)0, std::false_type()); else if constexpr (ALLOW_BIG) launch((unsigned long long)0, std::false_type());
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace tb200
