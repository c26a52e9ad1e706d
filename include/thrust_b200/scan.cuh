// Single-pass inclusive / exclusive scan with decoupled look-back for sm_100a.
//
// One CTA per tile; tiles are handed out by an atomic ticket so that a tile's predecessors have
// always started.  Each lane of a warp loads 16-byte vectors lane-interleaved (a warp instruction
// touches 512 contiguous bytes), scans its vectors in registers, the warp scans each row of
// vector totals with shuffles, and warp 0 resolves the tile's prefix by looking back over the
// preceding tiles' published aggregates.  The output is written with the same 16-byte pattern,
// so every element is read once and written once: 2 * sizeof(T) bytes of HBM traffic per element.
// Replaces the cub::DispatchScan call of thrust/system/cuda/detail/scan.h:61-114 and :139-192.
#pragma once
#include "common.cuh"

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

template <class T> size_t scan_tile_items() { return (size_t)SCAN_BLOCK * scan_tuning<T>::IPT; }
template <class T> size_t scan_workspace_bytes(size_t n) {
  size_t tiles = (n + scan_tile_items<T>() - 1) / scan_tile_items<T>();
  return sizeof(ws_header) + tile_state<T>::bytes(tiles + 1);
}

// Launches the scan on `stream`; no sync.  in == out is allowed.
template <bool INCLUSIVE, class InIt, class OutIt, class T, class Op>
cudaError_t scan_async(InIt in, OutIt out, size_t n, T init, bool has_init, Op op, void* ws, cudaStream_t stream) {
  if (n == 0) return cudaMemsetAsync(ws, 0, sizeof(ws_header), stream);
  constexpr int IPT = scan_tuning<T>::IPT;
  const size_t tiles = (n + scan_tile_items<T>() - 1) / scan_tile_items<T>();
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  tile_state<T> ts;
  ts.bind(base + sizeof(ws_header), tiles + 1);
  cudaError_t e = cudaMemsetAsync(base, 0, scan_workspace_bytes<T>(n), stream);
  if (e != cudaSuccess) return e;
  timed_launch tl(KID_SCAN, stream);
  constexpr bool ptrs = std::is_pointer<InIt>::value && std::is_pointer<OutIt>::value;
  if constexpr (ptrs) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    using Out = typename std::remove_pointer<OutIt>::type;
    constexpr bool vec_ok = std::is_same<In, T>::value && std::is_same<Out, T>::value && std::is_arithmetic<T>::value &&
                            (sizeof(T) == 4 || sizeof(T) == 8);
    if constexpr (vec_ok) {
      if (is_aligned16(in) && is_aligned16(out)) {
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
