// Inclusive / exclusive scan for sm_100a: a single-pass kernel with decoupled look-back (any operator,
// any iterator, small and medium inputs) and a two-pass "reduce, then scan" route for large inputs
// (further down).
//
// Single pass:
// One CTA per tile; tiles are handed out by an atomic ticket so that a tile's predecessors have
// always started.  Each lane of a warp loads 16-byte vectors lane-interleaved (a warp instruction
// touches 512 contiguous bytes), scans its vectors in registers, the warp scans each row of
// vector totals with shuffles, and warp 0 resolves the tile's prefix by looking back over the
// preceding tiles' published aggregates.  The output is written with the same 16-byte pattern,
// so every element is read once and written once: 2 * sizeof(T) bytes of HBM traffic per element.
// Replaces the cub::DispatchScan call of thrust/system/cuda/detail/scan.h:61-114 and :139-192.
#pragma once
#include "common.cuh"
#include "reduce.cuh"

namespace tb200 {

constexpr int SCAN_BLOCK = 256;
// Bytes of input per thread.  Measured on B200 at 2^28 int32: 64 B -> 0.75 ms, 128 B -> 0.62 ms; the
// kernel is bound by the wait for the preceding tiles' prefixes, which shrinks with the number of
// tiles in flight, so fewer and larger tiles win.
constexpr int SCAN_BYTES_PER_THREAD = 128;

template <class T> struct scan_tuning {
  static constexpr int IPT = sizeof(T) >= 32 ? 4 : (int)(SCAN_BYTES_PER_THREAD / sizeof(T));
};

template <class InIt, class OutIt, class T, class Op, bool INCLUSIVE, int VEC, int IPT>
__global__ void __launch_bounds__(SCAN_BLOCK, 4)
scan_kernel(InIt in, OutIt out, size_t n, T init, bool has_init, Op op, tile_state<T> ts, ws_header* hdr) {
  constexpr int VPT = IPT / VEC;
  constexpr int NWARPS = SCAN_BLOCK / 32;
  constexpr int WCHUNK = 32 * IPT;
  constexpr size_t TILE = (size_t)SCAN_BLOCK * IPT;
  static_assert(IPT % VEC == 0, "items per thread must be whole vectors");

  __shared__ unsigned s_tile;
  using prefix_smem_t = tile_prefix_smem<T, NWARPS>;
  TB200_SHARED_OBJECT(prefix_smem_t, sm);

  if (threadIdx.x == 0) s_tile = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const size_t tile = s_tile;
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const size_t wbase = tile * TILE + (size_t)warp * WCHUNK;
  const bool full = tile * TILE + TILE <= n;

  T x[VPT][VEC];
  // ---- load: vector v of this lane covers items wbase + (v*32 + lane)*VEC ... +VEC
  if constexpr (VEC > 1) {
    if (full) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        vec16 r = load_stream16(reinterpret_cast<const char*>(in) + (wbase + (size_t)(v * 32 + lane) * VEC) * sizeof(T));
        const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
        for (int k = 0; k < VEC; ++k) x[v][k] = e[k];
      }
    } else {
#pragma unroll
      for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          size_t i = wbase + (size_t)(v * 32 + lane) * VEC + k;
          x[v][k] = i < n ? (T)in[i] : T();
        }
    }
  } else {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      size_t i = wbase + (size_t)(v * 32 + lane);
      if (full || i < n) x[v][0] = (T)in[i]; else x[v][0] = T();
    }
  }

  // ---- scan inside each vector, then chain vector totals: warp rows, warps, preceding tiles
  T vec_total[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
#pragma unroll
    for (int k = 1; k < VEC; ++k) x[v][k] = op(x[v][k - 1], x[v][k]);
    vec_total[v] = x[v][VEC - 1];
  }
  opt<T> pre[VPT];   // everything before vector v of this lane, across tiles, including init
  tile_exclusive_prefix<T, Op, VPT, NWARPS>(vec_total, pre, tile, init, has_init, op, ts, &hdr->error, sm);

  // ---- apply and store
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const opt<T> E = pre[v];
    T y[VEC];
    if (INCLUSIVE) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) y[k] = E.has ? op(E.v, x[v][k]) : x[v][k];
    } else {
      y[0] = E.v;
#pragma unroll
      for (int k = 1; k < VEC; ++k) y[k] = op(E.v, x[v][k - 1]);
    }
    const size_t i0 = wbase + (size_t)(v * 32 + lane) * VEC;
    if constexpr (VEC > 1) {
      if (full) {
        vec16 r;
        T* e = reinterpret_cast<T*>(&r);
#pragma unroll
        for (int k = 0; k < VEC; ++k) e[k] = y[k];
        store_stream16(reinterpret_cast<char*>(out) + i0 * sizeof(T), r);
      } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) if (i0 + k < n) out[i0 + k] = y[k];
      }
    } else {
      if (full || i0 < n) out[i0] = y[0];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Two-pass route ("reduce, then scan") for large inputs and commutative operators on arithmetic types.
//
// The single-pass kernel above moves the minimum number of bytes, but on this GPU its tiles spend
// most of their life waiting for the slowest of the few hundred tiles ahead of them (measured: 7 of
// the 10 microseconds a tile lives).  Here the
// input is cut into one contiguous chunk per resident CTA and nothing waits for anything:
//   scan_chunk_reduce_kernel  every CTA reduces its chunk, walking it from the back so that the
//                             chunk's head is what stays in L2;
//   scan_chunk_kernel         every CTA folds the totals of the chunks before its own (a few
//                             hundred values) into a carry and scans its chunk front to back, the
//                             carry passing from tile to tile in registers.
// 3 * sizeof(T) bytes of traffic per element instead of 2, both passes at streaming speed.
// Measured on B200, 2^28 int32: 64 bytes per thread and tile with four CTAs per SM 0.514 ms (128 bytes:
// 0.530; three CTAs: 0.519; five to eight CTAs: 0.53-0.57) against 0.63 ms for the single-pass kernel;
// the first pass runs at 99 % and the second at 94 % of the measured copy bandwidth.
constexpr int SCAN2_CTAS_PER_SM = 4;
template <class T> struct scan2_tuning { static constexpr int IPT = (int)(64 / sizeof(T)); };
constexpr int SCAN2_MAX_CHUNKS = 2048;
constexpr size_t SCAN2_MIN_TILES_PER_CHUNK = 2;   // shorter chunks (n below ~5 M four-byte items) take the single-pass kernel

// plain (not evict-first) load: what the first pass reads last should still be in L2 for the second
template <class T> __device__ __forceinline__ vec16 load_keep16(const void* p) {
  vec16 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <class T, class Op, int VEC, int IPT>
__global__ void __launch_bounds__(SCAN_BLOCK, SCAN2_CTAS_PER_SM)
scan_chunk_reduce_kernel(const T* in, size_t n, size_t tiles, size_t tiles_per_chunk, Op op, T* partials) {
  constexpr int VPT = IPT / VEC;
  constexpr size_t TILE = (size_t)SCAN_BLOCK * IPT;
  TB200_SHARED_ARRAY(opt<T>, smem, 32);
  const size_t first = blockIdx.x * tiles_per_chunk;
  size_t last = first + tiles_per_chunk;
  if (last > tiles) last = tiles;
  opt<T> acc; acc.has = false;
  for (size_t tile = last; tile-- > first;) {
    const size_t base = tile * TILE;
    if (base + TILE <= n) {
      vec16 r[VPT];
#pragma unroll
      for (int v = 0; v < VPT; ++v) r[v] = load_keep16<T>(reinterpret_cast<const char*>(in) + (base + ((size_t)v * SCAN_BLOCK + threadIdx.x) * VEC) * sizeof(T));
      T t = reinterpret_cast<const T*>(&r[0])[0];
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const T* e = reinterpret_cast<const T*>(&r[v]);
#pragma unroll
        for (int k = (v == 0 ? 1 : 0); k < VEC; ++k) t = op(t, e[k]);
      }
      acc.append(t, op);
    } else {
      for (size_t i = base + threadIdx.x; i < n; i += SCAN_BLOCK) acc.append(in[i], op);
    }
  }
  opt<T> total = block_reduce_opt(acc, op, smem);
  if (threadIdx.x == 0) partials[blockIdx.x] = total.v;   // every chunk holds at least one element
}

template <class T, class Op, bool INCLUSIVE, int VEC, int IPT>
__global__ void __launch_bounds__(SCAN_BLOCK, SCAN2_CTAS_PER_SM)
scan_chunk_kernel(const T* in, T* out, size_t n, size_t tiles, size_t tiles_per_chunk, T init, bool has_init, Op op, const T* partials) {
  constexpr int VPT = IPT / VEC;
  constexpr int NWARPS = SCAN_BLOCK / 32;
  constexpr int WCHUNK = 32 * IPT;
  constexpr size_t TILE = (size_t)SCAN_BLOCK * IPT;
  TB200_SHARED_ARRAY(opt<T>, smem, 32);
  __shared__ T s_warp_total[2][NWARPS];
  __shared__ opt<T> s_carry;
  const int lane = lane_id(), warp = threadIdx.x >> 5;

  // carry = init (+) totals of the chunks before this one
  {
    opt<T> acc; acc.has = false;
    for (unsigned c = threadIdx.x; c < blockIdx.x; c += SCAN_BLOCK) acc.append(partials[c], op);
    opt<T> before = block_reduce_opt(acc, op, smem);
    if (threadIdx.x == 0) {
      opt<T> c0; c0.v = init; c0.has = has_init;
      before.prepend(c0, op);
      s_carry = before;
    }
    __syncthreads();
  }
  opt<T> carry = s_carry;

  const size_t first = blockIdx.x * tiles_per_chunk;
  size_t last = first + tiles_per_chunk;
  if (last > tiles) last = tiles;
  for (size_t tile = first; tile < last; ++tile) {
    const size_t wbase = tile * TILE + (size_t)warp * WCHUNK;
    const bool full = tile * TILE + TILE <= n;
    T x[VPT][VEC];
    if (full) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        vec16 r = load_stream16(reinterpret_cast<const char*>(in) + (wbase + (size_t)(v * 32 + lane) * VEC) * sizeof(T));
        const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
        for (int k = 0; k < VEC; ++k) x[v][k] = e[k];
      }
    } else {
#pragma unroll
      for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          size_t i = wbase + (size_t)(v * 32 + lane) * VEC + k;
          x[v][k] = i < n ? in[i] : T();
        }
    }
    T vec_total[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
#pragma unroll
      for (int k = 1; k < VEC; ++k) x[v][k] = op(x[v][k - 1], x[v][k]);
      vec_total[v] = x[v][VEC - 1];
    }
    // rows of the warp, then the warps of the tile, then the carry
    opt<T> pre[VPT];
    T rowacc = vec_total[0];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      T incl = warp_inclusive_scan(vec_total[v], op);
      T rowtotal = shfl_idx(incl, 31);
      T lanepref = shfl_up(incl, 1);
      pre[v].has = false;
      if (v > 0) { pre[v].v = rowacc; pre[v].has = true; }
      if (lane > 0) pre[v].append(lanepref, op);
      rowacc = v > 0 ? op(rowacc, rowtotal) : rowtotal;
    }
    T* wt = s_warp_total[(tile - first) & 1];   // two copies: one barrier per tile is enough
    if (lane == 0) wt[warp] = rowacc;
    __syncthreads();
    opt<T> wp = carry;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const T t = wt[w];
      if (w < warp) wp.append(t, op);
      carry.append(t, op);
    }
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      opt<T> E = pre[v];
      E.prepend(wp, op);
      T y[VEC];
      if (INCLUSIVE) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) y[k] = E.has ? op(E.v, x[v][k]) : x[v][k];
      } else {
        y[0] = E.v;
#pragma unroll
        for (int k = 1; k < VEC; ++k) y[k] = op(E.v, x[v][k - 1]);
      }
      const size_t i0 = wbase + (size_t)(v * 32 + lane) * VEC;
      if (full) {
        vec16 r;
        T* e = reinterpret_cast<T*>(&r);
#pragma unroll
        for (int k = 0; k < VEC; ++k) e[k] = y[k];
        store_stream16(reinterpret_cast<char*>(out) + i0 * sizeof(T), r);
      } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) if (i0 + k < n) out[i0 + k] = y[k];
      }
    }
  }
}

template <class Op> struct is_commutative_op : std::false_type {};
template <> struct is_commutative_op<plus_op> : std::true_type {};
template <> struct is_commutative_op<min_op> : std::true_type {};
template <> struct is_commutative_op<max_op> : std::true_type {};

template <class T> size_t scan_tile_items() { return (size_t)SCAN_BLOCK * scan_tuning<T>::IPT; }
template <class T> size_t scan_workspace_bytes(size_t n) {
  size_t tiles = (n + scan_tile_items<T>() - 1) / scan_tile_items<T>();
  const size_t single = tile_state<T>::bytes(tiles + 1), chunked = align_up(SCAN2_MAX_CHUNKS * sizeof(T), 256);
  return sizeof(ws_header) + (single > chunked ? single : chunked);   // either route fits
}

// Launches the scan on `stream`; no sync.  in == out is allowed.
template <bool INCLUSIVE, class InIt, class OutIt, class T, class Op>
cudaError_t scan_async(InIt in, OutIt out, size_t n, T init, bool has_init, Op op, void* ws, cudaStream_t stream) {
  if (n == 0) return cudaMemsetAsync(ws, 0, sizeof(ws_header), stream);
  constexpr int IPT = scan_tuning<T>::IPT;
  const size_t tiles = (n + scan_tile_items<T>() - 1) / scan_tile_items<T>();
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  constexpr bool ptrs = std::is_pointer<InIt>::value && std::is_pointer<OutIt>::value;
  bool vectors = false;
  if constexpr (ptrs) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    using Out = typename std::remove_pointer<OutIt>::type;
    constexpr bool vec_ok = std::is_same<In, T>::value && std::is_same<Out, T>::value && std::is_arithmetic<T>::value &&
                            (sizeof(T) == 4 || sizeof(T) == 8);
    if constexpr (vec_ok) {
      vectors = is_aligned16(in) && is_aligned16(out);
      if constexpr (is_commutative_op<Op>::value) {
        size_t chunks = (size_t)current_device_info().sm_count * SCAN2_CTAS_PER_SM;
        if (chunks > SCAN2_MAX_CHUNKS) chunks = SCAN2_MAX_CHUNKS;
        constexpr int IPT2 = scan2_tuning<T>::IPT;
        const size_t tiles2 = (n + (size_t)SCAN_BLOCK * IPT2 - 1) / ((size_t)SCAN_BLOCK * IPT2);
        if (vectors && tiles2 >= SCAN2_MIN_TILES_PER_CHUNK * chunks) {
          constexpr int VEC = 16 / sizeof(T);
          const size_t tiles_per_chunk = (tiles2 + chunks - 1) / chunks;
          chunks = (tiles2 + tiles_per_chunk - 1) / tiles_per_chunk;
          T* partials = reinterpret_cast<T*>(base + sizeof(ws_header));
          cudaError_t e2 = cudaMemsetAsync(base, 0, sizeof(ws_header), stream);
          if (e2 != cudaSuccess) return e2;
          timed_launch tl(KID_SCAN, stream);
          scan_chunk_reduce_kernel<T, Op, VEC, IPT2><<<(unsigned)chunks, SCAN_BLOCK, 0, stream>>>(in, n, tiles2, tiles_per_chunk, op, partials);
          scan_chunk_kernel<T, Op, INCLUSIVE, VEC, IPT2><<<(unsigned)chunks, SCAN_BLOCK, 0, stream>>>(in, out, n, tiles2, tiles_per_chunk, init, has_init, op, partials);
          return cudaGetLastError();
        }
      }
    }
  }
  tile_state<T> ts;
  ts.bind(base + sizeof(ws_header), tiles + 1);
  cudaError_t e = cudaMemsetAsync(base, 0, scan_workspace_bytes<T>(n), stream);
  if (e != cudaSuccess) return e;
  timed_launch tl(KID_SCAN, stream);
  if constexpr (ptrs) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    using Out = typename std::remove_pointer<OutIt>::type;
    constexpr bool vec_ok = std::is_same<In, T>::value && std::is_same<Out, T>::value && std::is_arithmetic<T>::value &&
                            (sizeof(T) == 4 || sizeof(T) == 8);
    if constexpr (vec_ok) {
      if (vectors) {
        constexpr int VEC = 16 / sizeof(T);
        scan_kernel<InIt, OutIt, T, Op, INCLUSIVE, VEC, IPT><<<(unsigned)tiles, SCAN_BLOCK, 0, stream>>>(in, out, n, init, has_init, op, ts, hdr);
        return cudaGetLastError();
      }
    }
  }
  scan_kernel<InIt, OutIt, T, Op, INCLUSIVE, 1, IPT><<<(unsigned)tiles, SCAN_BLOCK, 0, stream>>>(in, out, n, init, has_init, op, ts, hdr);
  return cudaGetLastError();
}

}  // namespace tb200
