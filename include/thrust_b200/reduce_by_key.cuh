// Single-pass reduce_by_key for sm_100a.
//
// A run starts at item 0 and wherever !key_eq(key[i-1], key[i]).  Each item contributes the pair
// (is_head, value); pairs combine as  (c1, v1) (+) (c2, v2) = (c1 + c2, c2 ? v2 : op(v1, v2)),
// i.e. a running count of run heads and the reduction of the still-open run.  One CTA per tile
// scans these pairs (registers, warp shuffles, decoupled look-back across tiles) and every run
// head i > 0 emits the finished total of the run before it -- the exclusive scan value at i --
// while the owner of the last item emits the final run.  Heads are compacted through shared
// memory so keys_out / values_out are written with consecutive threads on consecutive addresses.
// Values inside a run are combined left to right.  Replaces InitAgent + ReduceByKeyAgent of
// thrust/system/cuda/detail/reduce_by_key.h:197-860.
#pragma once
#include "common.cuh"

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
  static constexpr int IPT = BYTES >= 16 ? 4 : (BYTES >= 4 ? 64 / BYTES : 16);
};

template <class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, class K, class V, class Eq, class Op, class Off, int VEC, int IPT>
__global__ void __launch_bounds__(RBK_BLOCK, 3)
reduce_by_key_kernel(KeyIt keys, ValIt vals, KeyOutIt keys_out, ValOutIt vals_out, size_t n, Eq key_eq, Op op,
                     tile_state<rbk_pair<Off, V>> ts, ws_header* hdr, unsigned long long* d_count) {
  using P = rbk_pair<Off, V>;
  using Comb = rbk_combine<Off, V, Op>;
  constexpr int VPT = IPT / VEC;
  constexpr int NWARPS = RBK_BLOCK / 32;
  constexpr int WCHUNK = 32 * IPT;
  constexpr int TILE = RBK_BLOCK * IPT;
  __shared__ unsigned s_tile;
  using prefix_smem_t = tile_prefix_smem<P, NWARPS>;
  TB200_SHARED_OBJECT(prefix_smem_t, sm);
  TB200_SHARED_ARRAY(K, stage_k, TILE);
  TB200_SHARED_ARRAY(V, stage_v, TILE);

  if (threadIdx.x == 0) s_tile = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const size_t tile = s_tile;
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const size_t tile_base = tile * (size_t)TILE;
  const size_t wbase = tile_base + (size_t)warp * WCHUNK;
  const bool full = tile_base + TILE <= n;
  Comb comb; comb.op = op;

  // ---- load keys and values
  K k[VPT][VEC]; V x[VPT][VEC];
  if constexpr (VEC > 1) {
    if (full) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const size_t i0 = wbase + (size_t)(v * 32 + lane) * VEC;
        vec16 rk = load_stream16(reinterpret_cast<const char*>(keys) + i0 * sizeof(K));
        vec16 rv = load_stream16(reinterpret_cast<const char*>(vals) + i0 * sizeof(V));
        const K* ek = reinterpret_cast<const K*>(&rk); const V* ev = reinterpret_cast<const V*>(&rv);
#pragma unroll
        for (int j = 0; j < VEC; ++j) { k[v][j] = ek[j]; x[v][j] = ev[j]; }
      }
    } else {
#pragma unroll
      for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          size_t i = wbase + (size_t)(v * 32 + lane) * VEC + j;
          if (i < n) { k[v][j] = keys[i]; x[v][j] = (V)vals[i]; } else { k[v][j] = K(); x[v][j] = V(); }
        }
    }
  } else {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      size_t i = wbase + (size_t)(v * 32 + lane);
      if (full || i < n) { k[v][0] = keys[i]; x[v][0] = (V)vals[i]; } else { k[v][0] = K(); x[v][0] = V(); }
    }
  }

  // ---- head flags, scan inside each vector
  unsigned head[VPT];
  P vec_total[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const size_t i0 = wbase + (size_t)(v * 32 + lane) * VEC;
    K prev = shfl_up(k[v][VEC - 1], 1);
    if (v > 0) { K wrap = shfl_idx(k[v - 1][VEC - 1], 31); if (lane == 0) prev = wrap; }
    bool has_prev = true;
    if (v == 0 && lane == 0) { has_prev = i0 > 0 && i0 < n; if (has_prev) prev = keys[i0 - 1]; }
    unsigned bits = 0;
    Off cnt = 0;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      // items past the end count as heads so that they never extend a real run
      bool h = (j == 0 && !has_prev) ? true : !key_eq(j == 0 ? prev : k[v][j - 1], k[v][j]);
      if (!(full || i0 + j < n)) h = true;
      if (h) { bits |= 1u << j; ++cnt; }
      if (j > 0 && !h) x[v][j] = op(x[v][j - 1], x[v][j]);   // x becomes the in-vector inclusive run sum
    }
    head[v] = bits;
    vec_total[v].count = cnt;
    vec_total[v].value = x[v][VEC - 1];
  }

  opt<P> pre[VPT];
  P none; none.count = 0; none.value = V();
  tile_exclusive_prefix<P, Comb, VPT, NWARPS>(vec_total, pre, tile, none, false, comb, ts, &hdr->error, sm);
  const Off head_off = sm.has_prefix ? sm.prefix.count : (Off)0;   // run heads in all preceding tiles

  // ---- every head closes the run before it; compact heads through shared memory
  const size_t last = n - 1;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const size_t i0 = wbase + (size_t)(v * 32 + lane) * VEC;
    Off cnt_before = pre[v].has ? pre[v].v.count : (Off)0;      // heads before this vector (global)
    V open = pre[v].has ? pre[v].v.value : V();                  // total so far of the run open at this vector's start
    bool open_valid = pre[v].has;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const bool valid = full || i0 + j < n;
      const bool h = (head[v] >> j) & 1;
      // does the run open at the vector's start still run on at item j (no head in items 0..j)?
      const bool from_before = open_valid && (head[v] & ((2u << j) - 1)) == 0;
      if (valid && h) {
        // total of the run that ends just before item j = exclusive scan value at j
        const unsigned r = (unsigned)(cnt_before - head_off);
        stage_k[r] = k[v][j];
        if (j == 0) { if (open_valid) stage_v[r] = open; }
        else stage_v[r] = (open_valid && (head[v] & ((1u << j) - 1)) == 0) ? op(open, x[v][j - 1]) : x[v][j - 1];
      }
      if (h) ++cnt_before;
      if (valid && i0 + j == last) {
        vals_out[(size_t)cnt_before - 1] = from_before ? op(open, x[v][j]) : x[v][j];
        hdr->count = (unsigned long long)cnt_before;
        if (d_count) *d_count = (unsigned long long)cnt_before;
      }
    }
  }
  __syncthreads();
  const unsigned tile_heads_all = (unsigned)(sm.inclusive.count - head_off);
  // heads contributed by padding items of a partial tile come last; drop them
  const unsigned pad = full ? 0u : (unsigned)(tile_base + TILE - n);
  const unsigned tile_heads = tile_heads_all - pad;
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const unsigned j = threadIdx.x + i * RBK_BLOCK;
    if (j < tile_heads) {
      const size_t g = (size_t)head_off + j;
      keys_out[g] = stage_k[j];
      if (g > 0) vals_out[g - 1] = stage_v[j];
    }
  }
}

template <class K, class V> constexpr size_t rbk_tile_items() { return (size_t)RBK_BLOCK * rbk_tuning<K, V>::IPT; }
template <class K, class V> size_t rbk_workspace_bytes(size_t n) {
  size_t tiles = (n + rbk_tile_items<K, V>() - 1) / rbk_tile_items<K, V>();
  return sizeof(ws_header) + tile_state<rbk_pair<unsigned long long, V>>::bytes(tiles + 1);
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
  cudaError_t e = cudaMemsetAsync(base, 0, rbk_workspace_bytes<K, V>(n), stream);
  if (e != cudaSuccess) return e;
  if (n == 0) { if (d_count) return cudaMemsetAsync(d_count, 0, sizeof(unsigned long long), stream); return cudaSuccess; }
  auto launch = [&](auto off_tag, auto vec_tag) {
    using Off = decltype(off_tag);
    constexpr int VEC = decltype(vec_tag)::value;
    tile_state<rbk_pair<Off, V>> ts;
    ts.bind(base + sizeof(ws_header), tiles + 1);
    timed_launch tl(KID_REDUCE_BY_KEY, stream);
    reduce_by_key_kernel<KeyIt, ValIt, KeyOutIt, ValOutIt, K, V, Eq, Op, Off, VEC, IPT>
        <<<(unsigned)tiles, RBK_BLOCK, 0, stream>>>(keys, vals, keys_out, vals_out, n, eq, op, ts, hdr, d_count);
  };
  const bool small = n < (1ull << 31);
  if (!ALLOW_BIG && !small) return cudaErrorInvalidValue;
  constexpr bool vec_ok = std::is_pointer<KeyIt>::value && std::is_pointer<ValIt>::value && std::is_arithmetic<K>::value &&
                          std::is_arithmetic<V>::value && sizeof(K) == sizeof(V) && (sizeof(K) == 4 || sizeof(K) == 8);
  if constexpr (vec_ok) {
    using VIn = typename std::remove_cv<typename std::remove_pointer<ValIt>::type>::type;
    if constexpr (std::is_same<VIn, V>::value) {
      if (is_aligned16((const void*)keys) && is_aligned16((const void*)vals)) {
        constexpr int VV = 16 / sizeof(K);
        if (small) launch((unsigned)0, std::integral_constant<int, VV>()); else if constexpr (ALLOW_BIG) launch((unsigned long long)0, std::integral_constant<int, VV>());
        return cudaGetLastError();
      }
    }
  }
  if (small) launch((unsigned)0, std::integral_constant<int, 1>()); else if constexpr (ALLOW_BIG) launch((unsigned long long)0, std::integral_constant<int, 1>());
  return cudaGetLastError();
}

}  // namespace tb200
