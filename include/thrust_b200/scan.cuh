// Inclusive / exclusive scan for sm_100a: a single-pass kernel with decoupled look-back (any operator,
// any iterator, small and medium inputs) and, for large inputs with a commutative operator and a
// contiguous output, one persistent kernel that walks the input in L2-sized windows -- reduce, fold,
// scan per window, the second read served from L2 (scan_window_kernel, further down; the two-launch
// "reduce, then scan" route it grew out of remains for -DTB200_SCAN_NO_WINDOW).
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
scan_kernel(InIt in, OutIt out, size_t n, T init, bool has_init, const T* init_ptr, Op op, tile_state<T> ts, ws_header* hdr) {
  if (init_ptr) { init = *init_ptr; has_init = true; }   // an initial value that lives on the device (the carry of a sharded scan)
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
#ifndef TB200_SCAN2_TILE_BYTES_PER_THREAD
#define TB200_SCAN2_TILE_BYTES_PER_THREAD 64
#endif
template <class T> struct scan2_tuning { static constexpr int IPT = (int)(TB200_SCAN2_TILE_BYTES_PER_THREAD / sizeof(T)); };
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
scan_chunk_kernel(const T* in, T* out, size_t n, size_t tiles, size_t tiles_per_chunk, T init, bool has_init, const T* init_ptr, Op op, const T* partials) {
  if (init_ptr) { init = *init_ptr; has_init = true; }
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

// ------------------------------------------------------------------------------------------------
// Windowed route: the two passes above, but over one window of the input at a time, so that the
// second pass finds its window in the 126 MB L2 and HBM sees every element once on the way in and
// once on the way out (2 * sizeof(T) bytes per element again, without the single-pass convoy).
//
// One persistent kernel, one CTA per resident slot (`gridDim.x` CTAs, all resident: the host sizes the
// grid from the occupancy query).  Window w is the tiles [w * G * TPC, (w + 1) * G * TPC); CTA c owns the
// chunk of TPC consecutive tiles number c in every window.  Per window a CTA
//   A: reduces its chunk (plain loads: the lines stay in L2) and publishes the total in a
//      descriptor (value and status in one word);
//   F: folds the descriptors of the whole window -- the totals of the chunks before its own give
//      its carry, all of them the running total for the next window; the wait for a descriptor is
//      bounded, and since A of window w + 1 is issued BEFORE F of window w, the other CTAs' totals
//      have normally arrived long before they are asked for;
//   B: scans its chunk front to back (evict-first loads that hit L2, streaming stores), the carry
//      passing from tile to tile in registers.
// Every CTA publishes A(w) before it waits for anything of window w, so the waits cannot deadlock
// as long as all CTAs are resident; CTAs are never more than one window apart, so about two windows
// of input and two of output are live in L2 at a time.
#ifndef TB200_SCANW_CTAS
#define TB200_SCANW_CTAS 4
#endif
constexpr int SCANW_CTAS_PER_SM = TB200_SCANW_CTAS;
constexpr size_t SCANW_MAX_GRID = 2048;   // CTAs at most (the fold gives every thread GRID / 256 descriptors)
#ifndef TB200_SCANW_TPC
#define TB200_SCANW_TPC 3        // tiles per chunk: window = resident CTAs * TPC * 16 KB (28 MB on a B200; 2 and 3 measured alike, 1 and 4+ slower)
#endif

// The operators of this route have an identity, so nothing here needs the "value may be absent"
// bookkeeping of the generic kernels: plus starts from -0.0 for floating point (x + -0.0 == x for
// every x, signed zeros included) and 0 otherwise, min from the largest and max from the smallest value.
template <class Op, class T> struct op_identity;
template <class T> struct op_identity<plus_op, T> {
  __host__ __device__ static T value() { return std::is_floating_point<T>::value ? (T)-0.0 : (T)0; }
};
template <class T> struct op_identity<min_op, T> {
  __host__ __device__ static T value() {
    if constexpr (std::is_floating_point<T>::value) return (T)INFINITY;
    else if constexpr (std::is_signed<T>::value) return (T)(((unsigned long long)1 << (8 * sizeof(T) - 1)) - 1);
    else return (T)~(T)0;
  }
};
template <class T> struct op_identity<max_op, T> {
  __host__ __device__ static T value() {
    if constexpr (std::is_floating_point<T>::value) return (T)-INFINITY;
    else if constexpr (std::is_signed<T>::value) return (T)((unsigned long long)1 << (8 * sizeof(T) - 1));
    else return (T)0;
  }
};

template <class T, class Op> __device__ __forceinline__ T warp_reduce_id(T x, Op op) {
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) x = op(x, shfl_generic(x, 0, 3, d));   // butterfly: the operators here commute
  return x;
}

// 16-byte load that asks L2 to keep the line (it is read again shortly) / policy for it
__device__ __forceinline__ unsigned long long l2_keep_policy() {
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ vec16 load_l2_keep16(const void* p, unsigned long long pol) {
  vec16 v;
  asm volatile("ld.global.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
  return v;
}

// InIt: `const T*` (16-byte aligned: vector loads) or any random-access iterator whose values convert
// to T (one element per load; a transform_iterator over a pointer, say).
template <class InIt, class T, class Op, bool INCLUSIVE, int VEC, int IPT>
__global__ void __launch_bounds__(SCAN_BLOCK, SCANW_CTAS_PER_SM)
scan_window_kernel(InIt in, T* out, size_t n, size_t tiles, unsigned tiles_per_chunk, T init, bool has_init, const T* init_ptr, Op op,
                   tile_state<T> ts, ws_header* hdr) {
  constexpr bool VECTOR_IN = std::is_same<InIt, const T*>::value;
  if (init_ptr) { init = *init_ptr; has_init = true; }
  constexpr int VPT = IPT / VEC;
  constexpr int NWARPS = SCAN_BLOCK / 32;
  constexpr size_t WT = 32 * IPT;           // a warp's tile: each lane holds VPT 16-byte vectors, lane-interleaved
  const T ID = op_identity<Op, T>::value();
#ifdef TB200_SCANW_EVICT_LAST
  const unsigned long long keep = l2_keep_policy();
#endif
  __shared__ T s_part[2][NWARPS];          // each warp's total of its part of the chunk, by window parity
  __shared__ T s_fold[2][NWARPS];          // per warp: fold of the chunks before this CTA's, of all chunks
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const size_t G = gridDim.x, c = blockIdx.x;
  const size_t wtiles = (n + WT - 1) / WT;
  const size_t chunk_wtiles = (size_t)tiles_per_chunk * NWARPS;   // a CTA's chunk; warp w owns the w-th run of tiles_per_chunk warp tiles
  const size_t windows = (wtiles + G * chunk_wtiles - 1) / (G * chunk_wtiles);
  (void)tiles;

  auto chunk_first = [&](size_t w, size_t chunk) { return (w * G + chunk) * chunk_wtiles; };
  auto load_tile = [&](vec16 (&r)[VPT], size_t wt, bool keep_in_l2) {
    const size_t base = wt * WT;
    const bool full = base + WT <= n;
    if constexpr (VECTOR_IN) {
      if (full) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
          const char* p = reinterpret_cast<const char*>(in) + (base + (size_t)(v * 32 + lane) * VEC) * sizeof(T);
#ifdef TB200_SCANW_EVICT_LAST
          r[v] = keep_in_l2 ? load_l2_keep16(p, keep) : load_stream16(p);
#else
          r[v] = keep_in_l2 ? load_keep16<T>(p) : load_stream16(p);
#endif
        }
        return;
      }
    }
    (void)keep_in_l2;
    if (full) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        T* e = reinterpret_cast<T*>(&r[v]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) e[k] = (T)in[base + (size_t)(v * 32 + lane) * VEC + k];
      }
    } else {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        T* e = reinterpret_cast<T*>(&r[v]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const size_t i = base + (size_t)(v * 32 + lane) * VEC + k;
          e[k] = i < n ? (T)in[i] : ID;
        }
      }
    }
  };
  // A: every warp reduces its part of the CTA's chunk of window w; the CTA's total is published
  auto phase_a = [&](size_t w) {
    const size_t first = chunk_first(w, c);
    if (first >= wtiles) return;
    const size_t mine = first + (size_t)warp * tiles_per_chunk;
    T acc = ID;
    for (unsigned t = 0; t < tiles_per_chunk; ++t) {
      if (mine + t >= wtiles) break;
      vec16 r[VPT];
      load_tile(r, mine + t, true);
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const T* e = reinterpret_cast<const T*>(&r[v]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc = op(acc, e[k]);
      }
    }
    acc = warp_reduce_id(acc, op);
    T* part = s_part[w & 1];
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (warp == 0) {
      T t = lane < NWARPS ? part[lane] : ID;
      t = warp_reduce_id(t, op);
      if (lane == 0) ts.publish(w * G + c, TILE_AGGREGATE, t);
    }
  };

  T running = has_init ? init : ID;   // init (+) everything before the current window
  phase_a(0);
  for (size_t w = 0; w < windows; ++w) {
    if (w + 1 < windows) phase_a(w + 1);
    const size_t first = chunk_first(w, c);
    if (first >= wtiles) break;   // only in the last window: no chunk of this CTA, and nobody waits for it
    // ---- F: fold the window's descriptors: every thread polls a few (all loads in flight at once),
    // each warp leaves its partial fold in shared memory
    {
      constexpr int SLOTS = (int)(SCANW_MAX_GRID / SCAN_BLOCK);
      T v[SLOTS];
      unsigned st[SLOTS];
#pragma unroll
      for (int j = 0; j < SLOTS; ++j) {
        const size_t k = threadIdx.x + (size_t)j * SCAN_BLOCK;
        st[j] = TILE_AGGREGATE; v[j] = ID;
        if (k < G && chunk_first(w, k) < wtiles) st[j] = ts.poll(w * G + k, v[j]);
      }
      T before = ID, total = ID;
#pragma unroll
      for (int j = 0; j < SLOTS; ++j) {
        const size_t k = threadIdx.x + (size_t)j * SCAN_BLOCK;
        unsigned iter = 0;
        while (st[j] == TILE_INVALID) {
          if (++iter > SPIN_LIMIT) { record_error(&hdr->error, ERR_LOOKBACK_TIMEOUT); v[j] = ID; break; }
          backoff(iter);
          st[j] = ts.poll(w * G + k, v[j]);
        }
        if (k < c) before = op(before, v[j]);
        total = op(total, v[j]);
      }
      before = warp_reduce_id(before, op);
      total = warp_reduce_id(total, op);
      if (lane == 0) { s_fold[0][warp] = before; s_fold[1][warp] = total; }
    }
    __syncthreads();
    // this warp's carry: init and the windows before, the chunks before this CTA's, the warps before this one
    T carry;
    {
      T before = ID, total = ID;
#pragma unroll
      for (int w2 = 0; w2 < NWARPS; ++w2) { before = op(before, s_fold[0][w2]); total = op(total, s_fold[1][w2]); }
      carry = op(running, before);
      running = op(running, total);
      const T* part = s_part[w & 1];
#pragma unroll
      for (int w2 = 0; w2 < NWARPS; ++w2) if (w2 < warp) carry = op(carry, part[w2]);
    }
    // ---- B: the warp scans its part of the chunk, tile after tile, no barrier
    const size_t mine = first + (size_t)warp * tiles_per_chunk;
#ifdef TB200_SCANW_PREFETCH
    vec16 rn[VPT];
    if (mine < wtiles) load_tile(rn, mine, false);
#endif
    for (unsigned t = 0; t < tiles_per_chunk; ++t) {
      const size_t wt = mine + t;
      if (wt >= wtiles) break;
      vec16 r[VPT];
#ifdef TB200_SCANW_PREFETCH
#pragma unroll
      for (int v = 0; v < VPT; ++v) r[v] = rn[v];
      if (t + 1 < tiles_per_chunk && wt + 1 < wtiles) load_tile(rn, wt + 1, false);   // in flight while this tile is scanned
#else
      load_tile(r, wt, false);
#endif
      T x[VPT][VEC];
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const T* e = reinterpret_cast<const T*>(&r[v]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) x[v][k] = e[k];
      }
      T pre[VPT];   // carry (+) everything of this tile before vector v of this lane
      T rowacc = carry;
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
#pragma unroll
        for (int k = 1; k < VEC; ++k) x[v][k] = op(x[v][k - 1], x[v][k]);
        const T incl = warp_inclusive_scan(x[v][VEC - 1], op);
        T lanepref = shfl_up(incl, 1);
        if (lane == 0) lanepref = ID;
        pre[v] = op(rowacc, lanepref);
        rowacc = op(rowacc, shfl_idx(incl, 31));
      }
      carry = rowacc;
      const size_t base = wt * WT;
      const bool full = base + WT <= n;
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const T E = pre[v];
        T y[VEC];
        if (INCLUSIVE) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) y[k] = op(E, x[v][k]);
        } else {
          y[0] = E;
#pragma unroll
          for (int k = 1; k < VEC; ++k) y[k] = op(E, x[v][k - 1]);
        }
        const size_t i0 = base + (size_t)(v * 32 + lane) * VEC;
        if (full) {
          vec16 o;
          T* e = reinterpret_cast<T*>(&o);
#pragma unroll
          for (int k = 0; k < VEC; ++k) e[k] = y[k];
          store_stream16(reinterpret_cast<char*>(out) + i0 * sizeof(T), o);
        } else {
#pragma unroll
          for (int k = 0; k < VEC; ++k) if (i0 + k < n) out[i0 + k] = y[k];
        }
      }
    }
    __syncthreads();   // s_fold is rewritten in the next window
  }
}

// Resident CTAs of the windowed kernel on the current device (cached per kernel and device).
template <class Kernel> int resident_ctas(Kernel kernel, int block, size_t smem) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, smem) != cudaSuccess || per_sm < 1) return 0;
  return per_sm * current_device_info().sm_count;
}

template <class Op> struct is_commutative_op : std::false_type {};
template <> struct is_commutative_op<plus_op> : std::true_type {};
template <> struct is_commutative_op<min_op> : std::true_type {};
template <> struct is_commutative_op<max_op> : std::true_type {};

template <class T> size_t scan_tile_items() { return (size_t)SCAN_BLOCK * scan_tuning<T>::IPT; }
// descriptors of the windowed route: one per chunk, the last window padded to a whole grid
template <class T> size_t scanw_descriptor_bound(size_t n) {
  const size_t tile = (size_t)SCAN_BLOCK * scan2_tuning<T>::IPT;
  return ((n + tile - 1) / tile + TB200_SCANW_TPC - 1) / TB200_SCANW_TPC + SCANW_MAX_GRID;
}
template <class T> size_t scan_workspace_bytes(size_t n) {
  size_t tiles = (n + scan_tile_items<T>() - 1) / scan_tile_items<T>();
  const size_t single = tile_state<T>::bytes(tiles + 1), chunked = align_up(SCAN2_MAX_CHUNKS * sizeof(T), 256);
  size_t need = single > chunked ? single : chunked;
  if (tile_state_mode<T>::value != 0 && tile_state<T>::bytes(scanw_descriptor_bound<T>(n)) > need) need = tile_state<T>::bytes(scanw_descriptor_bound<T>(n));
  return sizeof(ws_header) + need;   // every route fits
}

// The windowed route: launches it if the input is large enough for windows to pay (launched = true).
template <bool INCLUSIVE, class InIt, class T, class Op>
cudaError_t scan_window_launch(InIt in, T* out, size_t n, T init, bool has_init, const T* d_init, Op op, char* base, ws_header* hdr,
                               cudaStream_t stream, bool& launched) {
  launched = false;
#ifndef TB200_SCAN_NO_WINDOW
  constexpr int VEC = 16 / sizeof(T);
  constexpr int IPT2 = scan2_tuning<T>::IPT;
  const size_t tiles2 = (n + (size_t)SCAN_BLOCK * IPT2 - 1) / ((size_t)SCAN_BLOCK * IPT2);
  auto kern = scan_window_kernel<InIt, T, Op, INCLUSIVE, VEC, IPT2>;
  static thread_local int resident[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && resident[dev] == 0) resident[dev] = resident_ctas(kern, SCAN_BLOCK, 0);
  size_t grid = (dev >= 0 && dev < 64) ? (size_t)resident[dev] : 0;
  if (grid > SCANW_MAX_GRID) grid = SCANW_MAX_GRID;
  const unsigned tpc = TB200_SCANW_TPC;
  if (grid == 0 || tiles2 < 2 * grid * tpc) return cudaSuccess;
  const size_t windows = (tiles2 + grid * tpc - 1) / (grid * tpc);
  tile_state<T> tsw;
  tsw.bind(base + sizeof(ws_header), windows * grid);
  cudaError_t e3 = cudaMemsetAsync(base, 0, sizeof(ws_header) + tile_state<T>::bytes(windows * grid), stream);
  if (e3 != cudaSuccess) return e3;
  launched = true;
  timed_launch tl(KID_SCAN, stream);
  kern<<<(unsigned)grid, SCAN_BLOCK, 0, stream>>>(in, out, n, tiles2, tpc, init, has_init, d_init, op, tsw, hdr);
  log_launch(std::is_pointer<InIt>::value ? "scan_window_kernel" : "scan_window_kernel (generic input)", grid, SCAN_BLOCK, 0, n, stream);
  return cudaGetLastError();
#else
  return cudaSuccess;
#endif
}

// Launches the scan on `stream`; no sync.  in == out is allowed.  d_init, if not null, points at an
// initial value in device memory that replaces (init, has_init); it is read when the kernels run.
template <bool INCLUSIVE, class InIt, class OutIt, class T, class Op>
cudaError_t scan_async(InIt in, OutIt out, size_t n, T init, bool has_init, Op op, void* ws, cudaStream_t stream, const T* d_init = nullptr) {
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
#ifndef TB200_SCAN_NO_WINDOW
          {
            bool launched = false;
            cudaError_t e3 = scan_window_launch<INCLUSIVE>((const T*)in, out, n, init, has_init, d_init, op, base, hdr, stream, launched);
            if (launched || e3 != cudaSuccess) return e3;
          }
#endif
          const size_t tiles_per_chunk = (tiles2 + chunks - 1) / chunks;
          chunks = (tiles2 + tiles_per_chunk - 1) / tiles_per_chunk;
          T* partials = reinterpret_cast<T*>(base + sizeof(ws_header));
          cudaError_t e2 = cudaMemsetAsync(base, 0, sizeof(ws_header), stream);
          if (e2 != cudaSuccess) return e2;
          timed_launch tl(KID_SCAN, stream);
          scan_chunk_reduce_kernel<T, Op, VEC, IPT2><<<(unsigned)chunks, SCAN_BLOCK, 0, stream>>>(in, n, tiles2, tiles_per_chunk, op, partials);
          scan_chunk_kernel<T, Op, INCLUSIVE, VEC, IPT2><<<(unsigned)chunks, SCAN_BLOCK, 0, stream>>>(in, out, n, tiles2, tiles_per_chunk, init, has_init, d_init, op, partials);
          log_launch("scan_chunk_reduce_kernel + scan_chunk_kernel", chunks, SCAN_BLOCK, 0, n, stream);
          return cudaGetLastError();
        }
      }
    }
  }
  // any other input iterator with a contiguous, aligned output of T: the windowed kernel with one
  // element per load (transform_inclusive_scan / transform_exclusive_scan over a device range)
  if constexpr (!std::is_pointer<InIt>::value && std::is_pointer<OutIt>::value && is_commutative_op<Op>::value) {
    using Out = typename std::remove_pointer<OutIt>::type;
    if constexpr (std::is_same<Out, T>::value && std::is_arithmetic<T>::value && (sizeof(T) == 4 || sizeof(T) == 8)) {
      size_t chunks = (size_t)current_device_info().sm_count * SCAN2_CTAS_PER_SM;
      if (chunks > SCAN2_MAX_CHUNKS) chunks = SCAN2_MAX_CHUNKS;
      const size_t tiles2 = (n + (size_t)SCAN_BLOCK * scan2_tuning<T>::IPT - 1) / ((size_t)SCAN_BLOCK * scan2_tuning<T>::IPT);
      if (is_aligned16(out) && tiles2 >= SCAN2_MIN_TILES_PER_CHUNK * chunks) {
        bool launched = false;
        cudaError_t e3 = scan_window_launch<INCLUSIVE>(in, out, n, init, has_init, d_init, op, base, hdr, stream, launched);
        if (launched || e3 != cudaSuccess) return e3;
      }
    }
  }
  tile_state<T> ts;
  ts.bind(base + sizeof(ws_header), tiles + 1);
  cudaError_t e = cudaMemsetAsync(base, 0, scan_workspace_bytes<T>(n), stream);
  if (e != cudaSuccess) return e;
#ifdef TB200_TEST_HOOKS
  if (test_hook_flags() & 1u) { if ((e = cudaMemsetAsync(&hdr->flags, 1, 1, stream)) != cudaSuccess) return e; }
#endif
  timed_launch tl(KID_SCAN, stream);
  if constexpr (ptrs) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    using Out = typename std::remove_pointer<OutIt>::type;
    constexpr bool vec_ok = std::is_same<In, T>::value && std::is_same<Out, T>::value && std::is_arithmetic<T>::value &&
                            (sizeof(T) == 4 || sizeof(T) == 8);
    if constexpr (vec_ok) {
      if (vectors) {
        constexpr int VEC = 16 / sizeof(T);
        scan_kernel<InIt, OutIt, T, Op, INCLUSIVE, VEC, IPT><<<(unsigned)tiles, SCAN_BLOCK, 0, stream>>>(in, out, n, init, has_init, d_init, op, ts, hdr);
        log_launch("scan_kernel (16-byte loads)", tiles, SCAN_BLOCK, 0, n, stream);
        return cudaGetLastError();
      }
    }
  }
  scan_kernel<InIt, OutIt, T, Op, INCLUSIVE, 1, IPT><<<(unsigned)tiles, SCAN_BLOCK, 0, stream>>>(in, out, n, init, has_init, d_init, op, ts, hdr);
  log_launch("scan_kernel (generic iterator)", tiles, SCAN_BLOCK, 0, n, stream);
  return cudaGetLastError();
}

}  // namespace tb200
