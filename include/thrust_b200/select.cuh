// Stream compaction for sm_100a: copy_if (with or without a stencil), partition, partition_copy and
// unique / unique_copy.  This file holds the single-pass kernel that serves every case (any iterator,
// stencils, in-place forms, small and medium inputs) and the dispatch; large contiguous inputs whose
// outputs do not overlap them go to the two-pass streaming kernels of select_stream.cuh.
//
// Single pass:
// One CTA per tile (dynamic ticket).  A tile loads its items with the same lane-interleaved
// 16-byte pattern as the scan, evaluates a keep/drop flag per item, runs the tile-wide exclusive
// prefix (warp shuffles + decoupled look-back over preceding tiles) on the per-vector keep counts,
// compacts kept items -- and, for partition, dropped items behind them -- through shared memory
// and streams the result out with consecutive threads on consecutive addresses.  Every item is
// read once and written at most once.  Replaces the InitAgent + CopyIfAgent / PartitionAgent /
// UniqueAgent pairs of thrust/system/cuda/detail/copy_if.h:160-593, partition.h:134-602 and
// unique.h:183-541.
//
// Order guarantees: kept items keep their input order (stable).  Dropped items are written in
// input order too, either to a second output (partition_copy) or -- for the in-place partition --
// mirrored from the end of a scratch copy that partition_finish_kernel reads back reversed, which
// restores input order; so partition here is always the stable one.
#pragma once
#include "common.cuh"
#include "select_stream.cuh"

namespace tb200 {

constexpr int SELECT_BLOCK = 256;
enum select_mode : int { SEL_PRED = 0, SEL_STENCIL = 1, SEL_UNIQUE = 2 };

template <class T> struct select_tuning {
  // 128 bytes of input per thread for 4- and 8-byte items (measured: unique_copy 2^28 int32 0.97 ms
  // at 64 bytes, 0.60 ms at 128); the staging buffer is then 32 KB of shared memory
  static constexpr int IPT = sizeof(T) >= 32 ? 4 : (sizeof(T) >= 4 ? (int)(128 / sizeof(T)) : 16);
};

// MODE SEL_PRED:    keep item i iff pred(in[i])
// MODE SEL_STENCIL: keep item i iff pred(stencil[i])
// MODE SEL_UNIQUE:  keep item i iff i == 0 or !pred(in[i-1], in[i])      (pred = equality)
// KEEP_REJECTS: also write dropped items: mirrored == false -> out_rej[r], r = rank among dropped;
//               mirrored == true -> out_sel[n - 1 - r].
template <int MODE, bool KEEP_REJECTS, class InIt, class StIt, class SelIt, class RejIt, class T, class Pred, class Off, int VEC, int IPT>
__global__ void __launch_bounds__(SELECT_BLOCK, 4)
select_kernel(InIt in, StIt stencil, SelIt out_sel, RejIt out_rej, size_t n, Pred pred, tile_state<Off> ts, ws_header* hdr,
              unsigned long long* d_count, bool mirrored) {
  constexpr int VPT = IPT / VEC;
  constexpr int NWARPS = SELECT_BLOCK / 32;
  constexpr int WCHUNK = 32 * IPT;
  constexpr int TILE = SELECT_BLOCK * IPT;
  __shared__ unsigned s_tile;
  __shared__ tile_prefix_smem<Off, NWARPS> sm;
  TB200_SHARED_ARRAY(T, stage, TILE);

  if (threadIdx.x == 0) s_tile = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const size_t tile = s_tile;
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const size_t tile_base = tile * (size_t)TILE;
  const size_t wbase = tile_base + (size_t)warp * WCHUNK;
  const bool full = tile_base + TILE <= n;
  const unsigned tile_n = full ? (unsigned)TILE : (unsigned)(n - tile_base);

  // ---- load
  T x[VPT][VEC];
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
          if (i < n) x[v][k] = in[i]; else x[v][k] = T();
        }
    }
  } else {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      size_t i = wbase + (size_t)(v * 32 + lane);
      if (full || i < n) x[v][0] = in[i]; else x[v][0] = T();
    }
  }

  // ---- keep flags (bit k of keep[v] = item k of vector v)
  unsigned keep[VPT];
  Off vec_total[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    unsigned bits = 0;
    const size_t i0 = wbase + (size_t)(v * 32 + lane) * VEC;
    if constexpr (MODE == SEL_UNIQUE) {
      // predecessor of the vector's first item: previous lane's last item, or the previous row's
      // last item (lane 31), or for the warp chunk's very first item a plain load of in[i0 - 1]
      T prev = shfl_up(x[v][VEC - 1], 1);
      if (v > 0) { T wrap = shfl_idx(x[v - 1][VEC - 1], 31); if (lane == 0) prev = wrap; }
      bool has_prev = true;
      if (v == 0 && lane == 0) { has_prev = i0 > 0 && i0 < n; if (has_prev) prev = in[i0 - 1]; }
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        bool head = (k == 0 && !has_prev) ? true : !pred(k == 0 ? prev : x[v][k - 1], x[v][k]);
        if ((full || i0 + k < n) && head) bits |= 1u << k;
      }
    } else if constexpr (MODE == SEL_STENCIL) {
#pragma unroll
      for (int k = 0; k < VEC; ++k)
        if (full || i0 + k < n) { if (pred(stencil[i0 + k])) bits |= 1u << k; }
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k)
        if ((full || i0 + k < n) && pred(x[v][k])) bits |= 1u << k;
    }
    keep[v] = bits;
    vec_total[v] = (Off)__popc(bits);
  }

  // ---- number of kept items before each vector, across tiles
  opt<Off> pre[VPT];
  tile_exclusive_prefix<Off, plus_op, VPT, NWARPS>(vec_total, pre, tile, (Off)0, true, plus_op(), ts, &hdr->error, sm);
  const Off sel_off = sm.prefix;                       // kept items in all preceding tiles
  const unsigned tile_nsel = (unsigned)(sm.inclusive - sm.prefix);

  // ---- compact through shared memory: kept items first, dropped items behind them
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    unsigned sel_rank = (unsigned)(pre[v].v - sel_off);
    const unsigned local0 = warp * WCHUNK + (v * 32 + lane) * VEC;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      if ((keep[v] >> k) & 1) stash(&stage[sel_rank++], x[v][k]);
      else if (KEEP_REJECTS && local0 + k < tile_n) stash(&stage[tile_nsel + (local0 + k - sel_rank)], x[v][k]);
    }
  }
  __syncthreads();
  const size_t rej_off = tile_base - (size_t)sel_off;  // dropped items in all preceding tiles
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const unsigned j = threadIdx.x + i * SELECT_BLOCK;
    if (j < tile_nsel) out_sel[(size_t)sel_off + j] = stage[j];
    else if (KEEP_REJECTS && j < tile_n) {
      const size_t r = rej_off + (j - tile_nsel);
      if (mirrored) out_sel[n - 1 - r] = stage[j]; else out_rej[r] = stage[j];
    }
  }
  if (threadIdx.x == 0 && tile_base + TILE >= n) {
    hdr->count = (unsigned long long)sm.inclusive;
    if (d_count) *d_count = (unsigned long long)sm.inclusive;
  }
}

// Second half of the in-place partition: scratch holds kept items at the front and dropped items
// mirrored from the back; write them back to `data` with the dropped half un-mirrored.
template <class OutIt, class T>   // OutIt: a pointer or any random-access iterator (a zip_iterator, ...)
__global__ void __launch_bounds__(256)
partition_finish_kernel(OutIt data, const T* scratch, size_t n, const ws_header* hdr) {
  const size_t nsel = (size_t)hdr->count;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) data[i] = i < nsel ? scratch[i] : scratch[n - 1 - (i - nsel)];
}

template <class T> constexpr size_t select_tile_items() { return (size_t)SELECT_BLOCK * select_tuning<T>::IPT; }
template <class T> size_t select_workspace_bytes(size_t n) {
  size_t tiles = (n + select_tile_items<T>() - 1) / select_tile_items<T>();
  const size_t single = sizeof(ws_header) + tile_state<unsigned long long>::bytes(tiles + 1);   // large enough for either offset width
  const size_t stream = select_stream_workspace_bytes<T>(n);
  return single > stream ? single : stream;
}

// Launches the compaction; no sync.  The number of kept items goes to the workspace header and,
// if d_count != nullptr, to *d_count.
// ALLOW_STREAM = false keeps a caller that has already tried select_stream_async itself from
// instantiating those kernels a second time.
template <int MODE, bool KEEP_REJECTS, bool ALLOW_STREAM = true, class InIt, class StIt, class SelIt, class RejIt, class T, class Pred>
cudaError_t select_async(InIt in, StIt stencil, SelIt out_sel, RejIt out_rej, size_t n, T /*type tag*/, Pred pred, bool mirrored,
                         unsigned long long* d_count, void* ws, cudaStream_t stream) {
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  constexpr int IPT = select_tuning<T>::IPT;
  const size_t tiles = (n + select_tile_items<T>() - 1) / select_tile_items<T>();
  // large contiguous inputs whose outputs are plain arrays that do not overlap the input: the
  // two-pass streaming kernels (select_stream.cuh)
  if constexpr (ALLOW_STREAM && MODE != SEL_STENCIL && std::is_pointer<InIt>::value && std::is_pointer<SelIt>::value && std::is_arithmetic<T>::value &&
                (sizeof(T) == 4 || sizeof(T) == 8) && (!KEEP_REJECTS || std::is_pointer<RejIt>::value)) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    using Sel = typename std::remove_pointer<SelIt>::type;
    if constexpr (std::is_same<In, T>::value && std::is_same<Sel, T>::value) {
      bool ok = true;
      T* rej = nullptr;
      if constexpr (KEEP_REJECTS) {
        using Rej = typename std::remove_pointer<RejIt>::type;
        if constexpr (std::is_same<Rej, T>::value) rej = out_rej; else ok = false;
      }
      if (ok && select_stream_eligible(in, out_sel, rej, KEEP_REJECTS && !mirrored, n, sizeof(T)))
        return select_stream_async<MODE == SEL_UNIQUE, KEEP_REJECTS, T, Pred>(in, out_sel, rej, n, pred, mirrored ? SELECT_REJ_MIRRORED : SELECT_REJ_SECOND_ARRAY, d_count, ws,
                                                                              stream);
    }
  }
  cudaError_t e = cudaMemsetAsync(base, 0, sizeof(ws_header) + tile_state<unsigned long long>::bytes(tiles + 1), stream);
  if (e != cudaSuccess) return e;
  if (n == 0) { if (d_count) return cudaMemsetAsync(d_count, 0, sizeof(unsigned long long), stream); return cudaSuccess; }
  auto launch = [&](auto off_tag, auto vec_tag) {
    using Off = decltype(off_tag);
    constexpr int VEC = decltype(vec_tag)::value;
    tile_state<Off> ts;
    ts.bind(base + sizeof(ws_header), tiles + 1);
    timed_launch tl(KID_SELECT, stream);
    select_kernel<MODE, KEEP_REJECTS, InIt, StIt, SelIt, RejIt, T, Pred, Off, VEC, IPT>
        <<<(unsigned)tiles, SELECT_BLOCK, 0, stream>>>(in, stencil, out_sel, out_rej, n, pred, ts, hdr, d_count, mirrored);
  };
  constexpr bool vec_ok = std::is_pointer<InIt>::value && std::is_arithmetic<T>::value && (sizeof(T) == 4 || sizeof(T) == 8) && MODE != SEL_STENCIL;
  bool use_vec = false;
  if constexpr (vec_ok) use_vec = is_aligned16((const void*)in);
  const bool small = n < (1ull << 31);
  if constexpr (vec_ok) {
    constexpr int V = 16 / sizeof(T);
    if (use_vec) {
      if (small) launch((unsigned)0, std::integral_constant<int, V>()); else launch((unsigned long long)0, std::integral_constant<int, V>());
      return cudaGetLastError();
    }
  }
  if (small) launch((unsigned)0, std::integral_constant<int, 1>()); else launch((unsigned long long)0, std::integral_constant<int, 1>());
  return cudaGetLastError();
}

template <class T>
cudaError_t partition_finish_async(T* data, const T* scratch, size_t n, const void* ws, cudaStream_t stream) {
  const device_info& di = current_device_info();
  size_t grid = (n + 256 * 8 - 1) / (256 * 8);
  if (grid > (size_t)di.sm_count * 8) grid = (size_t)di.sm_count * 8;
  partition_finish_kernel<<<(unsigned)grid, 256, 0, stream>>>(data, scratch, n, reinterpret_cast<const ws_header*>(ws));
  return cudaGetLastError();
}

// The in-place partition through the streaming kernels only (the caller has checked
// select_stream_eligible()): they know the number of kept items before they scatter, so the dropped
// items land behind the kept ones in input order and the way back is a plain copy.
template <class T, class Pred>
cudaError_t partition_inplace_stream_async(T* data, T* scratch, size_t n, Pred pred, unsigned long long* d_count, void* ws, cudaStream_t stream) {
cudaError_t e = select_stream_async<false, true, T, Pred>((const T*)data, scratch, (T*)nullptr, n, pred, SELECT_REJ_BEHIND_SELECTED, d_count, ws, stream);
  if (e != cudaSuccess) return e;
  return cudaMemcpyAsync(data, scratch, n * sizeof(T), cudaMemcpyDeviceToDevice, stream);
}

// In-place stable partition of data[0, n): `scratch` holds n items.
template <bool ALLOW_STREAM = true, class T, class Pred>
cudaError_t partition_inplace_async(T* data, T* scratch, size_t n, Pred pred, unsigned long long* d_count, void* ws, cudaStream_t stream) {
  if constexpr (ALLOW_STREAM && std::is_arithmetic<T>::value && (sizeof(T) == 4 || sizeof(T) == 8)) {
    if (select_stream_eligible(data, scratch, nullptr, false, n, sizeof(T))) return partition_inplace_stream_async(data, scratch, n, pred, d_count, ws, stream);
  }
  cudaError_t e = select_async<SEL_PRED, true, false>((const T*)data, (const T*)nullptr, scratch, (T*)nullptr, n, T(), pred, true, d_count, ws, stream);
  if (e != cudaSuccess || n == 0) return e;
  return partition_finish_async(data, scratch, n, ws, stream);
}

}  // namespace tb200
