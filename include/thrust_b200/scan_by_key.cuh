// Single-pass inclusive / exclusive scan_by_key (segmented scan) for sm_100a.
//
// A run starts at item 0 and wherever !key_eq(key[i-1], key[i]); the scan restarts at every run
// head.  Same skeleton as reduce_by_key: the tile's keys and values are staged in shared memory
// with coalesced 16-byte loads, every thread walks ITEMS consecutive items to get its summary
// (does a run start inside my items?  reduction of my still-open last run), one scan of those
// summaries over the CTA plus the decoupled look-back over preceding tiles yields the value
// carried into each thread's first item, and a second walk writes the results back into shared
// memory, from where they leave with coalesced stores.  Replaces InitAgent + ScanByKeyAgent of
// thrust/system/cuda/detail/scan_by_key.h:172-588.
#pragma once
#include "common.cuh"
#include "reduce_by_key.cuh"

namespace tb200 {

template <class KeyIt, class ValIt, class OutIt, class K, class V, class Eq, class Op, bool INCLUSIVE, bool VEC_LOAD, int IPT>
__global__ void __launch_bounds__(RBK_BLOCK)
scan_by_key_kernel(KeyIt keys, ValIt vals, OutIt out, size_t n, V init, Eq key_eq, Op op, tile_state<rbk_pair<unsigned, V>> ts, ws_header* hdr) {
  using P = rbk_pair<unsigned, V>;
  using Comb = rbk_combine<unsigned, V, Op>;
  constexpr int NWARPS = RBK_BLOCK / 32;
  constexpr int TILE = RBK_BLOCK * IPT;
  static_assert((TILE * sizeof(K)) % 16 == 0 && (TILE * sizeof(V)) % 16 == 0, "tile must be whole 16-byte vectors");
  __shared__ unsigned s_tile;
  using prefix_smem_t = tile_prefix_smem<P, NWARPS>;
  TB200_SHARED_OBJECT(prefix_smem_t, sm);
  extern __shared__ __align__(16) unsigned char sbk_smem[];          // keys of the tile, then its values (later: its results)
  K* s_key = reinterpret_cast<K*>(sbk_smem);
  V* s_val = reinterpret_cast<V*>(sbk_smem + (TILE * sizeof(K) + 15) / 16 * 16);
  TB200_SHARED_OBJECT(K, s_prev);

  if (threadIdx.x == 0) s_tile = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const size_t tile = s_tile;
  const size_t tile_base = tile * (size_t)TILE;
  const bool full = tile_base + TILE <= n;
  const unsigned tile_n = full ? (unsigned)TILE : (unsigned)(n - tile_base);
  Comb comb; comb.op = op;

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
  P vec_total[1] = {summary};
  opt<P> pre[1];
  P none; none.count = 0; none.value = V();
  tile_exclusive_prefix<P, Comb, 1, NWARPS>(vec_total, pre, tile, none, false, comb, ts, &hdr->error, sm);
  __syncthreads();                                                  // all items are in registers: results may overwrite the value buffer

  if (mine) {
    // acc = reduction of the items of the current run before item j (inclusive: through item j)
    V acc = pre[0].has ? pre[0].v.value : x[0];
    if (!INCLUSIVE && pre[0].has) acc = op(init, acc);
#pragma unroll
    for (int j = 0; j < IPT; ++j) {
      if ((unsigned)j < mine) {
        const bool h = (heads >> j) & 1;
        if (INCLUSIVE) {
          if (h) acc = x[j]; else if (j > 0 || pre[0].has) acc = op(acc, x[j]);
          s_val[first + j] = acc;
        } else {
          if (h) { s_val[first + j] = init; acc = op(init, x[j]); }
          else { s_val[first + j] = acc; acc = op(acc, x[j]); }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const unsigned c = threadIdx.x + i * RBK_BLOCK;
    if (c < tile_n) out[tile_base + c] = s_val[c];
  }
}

template <class K, class V> size_t scan_by_key_workspace_bytes(size_t n) {
  size_t tiles = (n + rbk_tile_items<K, V>() - 1) / rbk_tile_items<K, V>();
  const size_t single = sizeof(ws_header) + tile_state<rbk_pair<unsigned, V>>::bytes(tiles + 1);
  if constexpr (sizeof(K) == sizeof(V) && (sizeof(K) == 4 || sizeof(K) == 8)) {
    const size_t stream = rbk_stream_workspace_bytes<K, V>(n);
    return single > stream ? single : stream;
  }
  return single;
}

// Launches the segmented scan; no sync.  out may be vals (in place).  n < 2^32 * tile size.
template <bool INCLUSIVE, class KeyIt, class ValIt, class OutIt, class K, class V, class Eq, class Op>
cudaError_t scan_by_key_async(KeyIt keys, ValIt vals, OutIt out, size_t n, K, V init, Eq eq, Op op, void* ws, cudaStream_t stream) {
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  constexpr int IPT = rbk_tuning<K, V>::IPT;
  const size_t tiles = (n + rbk_tile_items<K, V>() - 1) / rbk_tile_items<K, V>();
  // large contiguous inputs with keys and values of one size: the two-pass streaming kernels
  // (reduce_by_key_stream.cuh)
  if constexpr (std::is_pointer<KeyIt>::value && std::is_pointer<ValIt>::value && std::is_pointer<OutIt>::value && sizeof(K) == sizeof(V) &&
                (sizeof(K) == 4 || sizeof(K) == 8) && std::is_trivially_copyable<K>::value && std::is_trivially_copyable<V>::value) {
    using KIn = typename std::remove_cv<typename std::remove_pointer<KeyIt>::type>::type;
    using VIn = typename std::remove_cv<typename std::remove_pointer<ValIt>::type>::type;
    using VOut = typename std::remove_pointer<OutIt>::type;
    if constexpr (std::is_same<KIn, K>::value && std::is_same<VIn, V>::value && std::is_same<VOut, V>::value) {
      if (scan_by_key_stream_eligible(keys, vals, out, n, sizeof(K)))
        return scan_by_key_stream_async<INCLUSIVE, K, V, Eq, Op>(keys, vals, out, n, init, eq, op, ws, stream);
    }
  }
  cudaError_t e = cudaMemsetAsync(base, 0, n ? sizeof(ws_header) + tile_state<rbk_pair<unsigned, V>>::bytes(tiles + 1) : sizeof(ws_header), stream);
  if (e != cudaSuccess || n == 0) return e;
  tile_state<rbk_pair<unsigned, V>> ts;
  ts.bind(base + sizeof(ws_header), tiles + 1);
  const size_t smem = (rbk_tile_items<K, V>() * sizeof(K) + 15) / 16 * 16 + rbk_tile_items<K, V>() * sizeof(V);
  auto launch = [&](auto vec_tag) {
    constexpr bool VEC = decltype(vec_tag)::value;
    auto kern = scan_by_key_kernel<KeyIt, ValIt, OutIt, K, V, Eq, Op, INCLUSIVE, VEC, IPT>;
    if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return;
    kern<<<(unsigned)tiles, RBK_BLOCK, smem, stream>>>(keys, vals, out, n, init, eq, op, ts, hdr);
  };
  constexpr bool ptrs = std::is_pointer<KeyIt>::value && std::is_pointer<ValIt>::value;
  if constexpr (ptrs) {
    using KIn = typename std::remove_cv<typename std::remove_pointer<KeyIt>::type>::type;
    using VIn = typename std::remove_cv<typename std::remove_pointer<ValIt>::type>::type;
    if constexpr (std::is_same<KIn, K>::value && std::is_same<VIn, V>::value && std::is_trivially_copyable<K>::value && std::is_trivially_copyable<V>::value) {
      if (is_aligned16((const void*)keys) && is_aligned16((const void*)vals)) {
        launch(std::true_type());
        return e != cudaSuccess ? e : cudaGetLastError();
      }
    }
  }
  launch(std::false_type());
  return e != cudaSuccess ? e : cudaGetLastError();
}

struct first_op { template <class T> __host__ __device__ T operator()(const T& a, const T&) const { return a; } };

}  // namespace tb200
