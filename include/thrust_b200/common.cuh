// Shared device/host helpers for the B200 (sm_100a) parallel-algorithm kernels.
//
// Everything here is header-only so that the same kernel templates serve two callers: the
// precompiled C-ABI library (fixed element types and functors) and the Thrust header overlay
// (the user's iterator and functor types).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include <type_traits>
#include <mutex>
#include <new>
#include <string.h>
#include <stdio.h>
#include <stdlib.h>

namespace tb200 {

constexpr int WARP_THREADS = 32;

// Shared-memory storage for element types that are not trivially constructible (tuples, user
// structs): raw bytes viewed as T, never constructed.
#define TB200_SHARED_ARRAY(T, name, count) \
  __shared__ __align__(16) unsigned char name##_raw[sizeof(T) * (count)]; \
  T* name = reinterpret_cast<T*>(name##_raw)
#define TB200_SHARED_OBJECT(T, name) \
  __shared__ __align__(16) unsigned char name##_raw[sizeof(T)]; \
  T& name = *reinterpret_cast<T*>(name##_raw)

constexpr unsigned FULL_MASK = 0xffffffffu;

// Stores a value into a slot of such raw storage: plain assignment for trivially copyable types, copy
// construction in place otherwise -- assigning to memory in which no object was ever constructed is
// wrong for a type with a non-trivial assignment operator (the reference guards this case:
// testing/copy.cu:470-520).
template <class T> __device__ __forceinline__ void stash(T* slot, const T& v) {
  if constexpr (std::is_trivially_copyable<T>::value) *slot = v;
  else ::new (static_cast<void*>(slot)) T(v);
}

// Error codes a kernel may leave in the workspace status word (see ws_header).
enum : unsigned { ERR_NONE = 0, ERR_LOOKBACK_TIMEOUT = 1 };

// Number of polls of a predecessor's status word before a look-back gives up, records
// ERR_LOOKBACK_TIMEOUT and carries on with whatever it has.  Polls past the first few sleep
// ~100 ns, so the bound is of the order of a second: far beyond any legitimate wait, short
// enough that a broken launch returns instead of hanging the device.
#ifndef TB200_SPIN_LIMIT
#define TB200_SPIN_LIMIT (1u << 23)
#endif
constexpr unsigned SPIN_LIMIT = TB200_SPIN_LIMIT;   // a test build of the library shortens it to make a wait run out

// First 256 bytes of every workspace.
struct ws_header {
  unsigned error;          // ERR_* (sticky until the next call clears it)
  unsigned ticket;         // dynamic tile counter / last-block counter
  unsigned long long count;  // number of selected items / runs / ... written by the kernel
  unsigned ticket2;
  unsigned flags;
  unsigned long long aux[29];
};
static_assert(sizeof(ws_header) == 256, "workspace header is 256 bytes");

#ifdef TB200_TEST_HOOKS
// Test build of the library only: a process-wide switch that the single-pass scan copies into the
// workspace header's flags (bit 0: tile 0 does not publish).
inline unsigned& test_hook_flags() { static unsigned f = 0; return f; }
#endif

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Properties of the current device, looked up once per host thread and device.  If the runtime
// cannot answer (no device, a failed context) the fallback describes a B200 and is NOT cached: the
// launch that follows reports the real error.
struct device_info { int sm_count; int max_smem_optin; };
inline const device_info& current_device_info() {
  static thread_local device_info cache[64];
  static thread_local bool have[64] = {false};
  static const device_info fallback = {148, 232448};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fallback;
  if (!have[dev]) {
    device_info di;
    if (cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&di.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || di.sm_count < 1)
      return fallback;
    cache[dev] = di;
    have[dev] = true;
  }
  return cache[dev];
}

// ---------------------------------------------------------------- optional per-kernel timing
// When switched on, launchers bracket their dominant kernel with CUDA events on the launching
// stream so that a caller can read each launch's device time afterwards (the library's analogue of
// the reference's THRUST_DEBUG_SYNC launch log, thrust/system/cuda/detail/core/agent_launcher.h:
// 518-590).  Off by default: no events are created or recorded.
enum kernel_id : int {
  KID_REDUCE = 1, KID_SCAN = 2, KID_ONESWEEP = 3, KID_RADIX_HIST = 4, KID_SELECT = 5, KID_REDUCE_BY_KEY = 6,
  KID_MERGE = 7, KID_BLOCK_SORT = 8
};
struct kernel_timer {
  static constexpr int CAP = 256;
  bool enabled = false;
  int used = 0;
  int ids[CAP];
  cudaEvent_t start[CAP], stop[CAP];
  bool created[CAP] = {false};
  std::mutex lock;                       // slots are handed out under it; calls may come from several host threads
  int begin(int id, cudaStream_t s) {
    if (!enabled) return -1;
    std::lock_guard<std::mutex> guard(lock);
    if (used >= CAP) return -1;
    int i = used++;
    if (!created[i]) { cudaEventCreate(&start[i]); cudaEventCreate(&stop[i]); created[i] = true; }
    ids[i] = id;
    cudaEventRecord(start[i], s);
    return i;
  }
  void end(int i, cudaStream_t s) { if (i >= 0) cudaEventRecord(stop[i], s); }
};
inline kernel_timer& global_kernel_timer() { static kernel_timer t; return t; }
struct timed_launch {
  int slot; cudaStream_t s;
  timed_launch(int id, cudaStream_t stream) : slot(global_kernel_timer().begin(id, stream)), s(stream) {}
  ~timed_launch() { global_kernel_timer().end(slot, s); }
};

// Launch log, the analogue of the reference's THRUST_DEBUG_SYNC trace
// (thrust/system/cuda/detail/core/agent_launcher.h:518-590): with THRUST_B200_LOG=1 in the
// environment every dominant kernel launch prints one line to stderr -- kernel, grid, block, dynamic
// shared memory, items -- and, like the reference's debug mode, waits for the stream and reports the
// launch's status.  Off (one cached flag test) otherwise.
inline bool launch_log_enabled() {
  static const bool on = [] { const char* e = getenv("THRUST_B200_LOG"); return e && e[0] && e[0] != '0'; }();
  return on;
}
inline void log_launch(const char* kernel, size_t grid, int block, size_t smem, size_t items, cudaStream_t stream) {
  if (!launch_log_enabled()) return;
  const cudaError_t e = cudaStreamSynchronize(stream);
  fprintf(stderr, "thrust_b200: %s<<<%zu, %d, %zu>>> items=%zu status=%s\n", kernel, grid, block, smem, items, cudaGetErrorName(e));
}

// ---------------------------------------------------------------- functors
struct plus_op { template <class T> __host__ __device__ T operator()(const T& a, const T& b) const { return a + b; } };
struct min_op { template <class T> __host__ __device__ T operator()(const T& a, const T& b) const { return b < a ? b : a; } };
struct max_op { template <class T> __host__ __device__ T operator()(const T& a, const T& b) const { return a < b ? b : a; } };
struct equal_op { template <class T> __host__ __device__ bool operator()(const T& a, const T& b) const { return a == b; } };
struct less_op { template <class T> __host__ __device__ bool operator()(const T& a, const T& b) const { return a < b; } };
struct greater_op { template <class T> __host__ __device__ bool operator()(const T& a, const T& b) const { return b < a; } };

// Predicates of the C ABI.  kind 0: x % a == b, 1: x < a, 2: x >= a, 3: x != a; make() adds cheaper
// forms of the modulo test where they give the same answer: kind 4, a mask, when a is a power of two
// and b is 0 (true for negative x too in two's complement; kind 6 when the mask fits 31 bits),
// kind 5, 32-bit division, when the operands fit; the 64-bit division remains the general case.
//
// abi_pred itself decides per element (a switch on `kind`: about 20 instructions per element, which
// is what a streaming kernel can afford in total); visit() hands a caller the same predicate as a
// type whose operator() is the one comparison, so that the hot kernels are compiled per kind.
struct pred_mod64 { long long a, b; template <class T> __host__ __device__ bool operator()(const T& x) const { return (long long)x % a == b; } };
struct pred_lt { long long a; template <class T> __host__ __device__ bool operator()(const T& x) const { return x < (T)a; } };
struct pred_ge { long long a; template <class T> __host__ __device__ bool operator()(const T& x) const { return x >= (T)a; } };
struct pred_ne { long long a; template <class T> __host__ __device__ bool operator()(const T& x) const { return x != (T)a; } };
struct pred_mask { long long a; template <class T> __host__ __device__ bool operator()(const T& x) const { return ((long long)x & a) == 0; } };
struct pred_mask32 {   // the mask fits 31 bits: only the low word of x matters
  long long a;
  template <class T> __host__ __device__ bool operator()(const T& x) const {
    if (std::is_integral<T>::value) return ((unsigned)x & (unsigned)a) == 0;
    return ((long long)x & a) == 0;
  }
};
struct pred_mod32 {
  long long a, b;
  template <class T> __host__ __device__ bool operator()(const T& x) const {
    if (sizeof(T) <= 4 && std::is_integral<T>::value) {
      if (std::is_signed<T>::value) return (int)x % (int)a == (int)b;
      return (unsigned)x % (unsigned)a == (unsigned)b;
    }
    return (long long)x % a == b;
  }
};
struct abi_pred {
  int kind; long long a, b;
  static abi_pred make(int kind, long long a, long long b) {
    abi_pred p; p.kind = kind; p.a = a; p.b = b;
    if (kind == 0) {
      if (b == 0 && a > 0 && (a & (a - 1)) == 0) { p.kind = a - 1 <= 0x7fffffffll ? 6 : 4; p.a = a - 1; }
      else if (a > 0 && a <= 0x7fffffffll && b >= 0 && b <= 0x7fffffffll) p.kind = 5;
    }
    return p;
  }
  template <class T> __host__ __device__ bool operator()(const T& x) const {
    switch (kind) {
      case 0: return pred_mod64{a, b}(x);
      case 1: return pred_lt{a}(x);
      case 2: return pred_ge{a}(x);
      case 3: return pred_ne{a}(x);
      case 4: return pred_mask{a}(x);
      case 6: return pred_mask32{a}(x);
      default: return pred_mod32{a, b}(x);
    }
  }
  // f(typed predicate): host side
  template <class F> auto visit(F f) const -> decltype(f(pred_lt{0})) {
    switch (kind) {
      case 0: return f(pred_mod64{a, b});
      case 1: return f(pred_lt{a});
      case 2: return f(pred_ge{a});
      case 3: return f(pred_ne{a});
      case 4: return f(pred_mask{a});
      case 6: return f(pred_mask32{a});
      default: return f(pred_mod32{a, b});
    }
  }
};

// A value that may be absent: lets scans and reductions run on operators without an identity.
template <class T> struct opt {
  T v; bool has;
  template <class Op> __device__ __forceinline__ void append(const T& x, Op op) {  // this = this (+) x
    v = has ? op(v, x) : x; has = true;
  }
  template <class Op> __device__ __forceinline__ void append_opt(const opt<T>& right, Op op) {  // this = this (+) right
    if (right.has) append(right.v, op);
  }
  template <class Op> __device__ __forceinline__ void prepend(const opt<T>& left, Op op) {  // this = left (+) this
    if (left.has) { v = has ? op(left.v, v) : left.v; has = true; }
  }
};

// ---------------------------------------------------------------- shuffles of any small POD
template <class T> __device__ __forceinline__ T shfl_generic(const T& x, int src_lane, int mode, int arg) {
  // mode 0: idx, 1: up, 2: down, 3: xor
  constexpr int W = (sizeof(T) + 3) / 4;
  unsigned in[W], out[W];
  in[W - 1] = 0;
  memcpy(in, &x, sizeof(T));
#pragma unroll
  for (int i = 0; i < W; ++i) {
    if (mode == 0) out[i] = __shfl_sync(FULL_MASK, in[i], src_lane);
    else if (mode == 1) out[i] = __shfl_up_sync(FULL_MASK, in[i], arg);
    else if (mode == 2) out[i] = __shfl_down_sync(FULL_MASK, in[i], arg);
    else out[i] = __shfl_xor_sync(FULL_MASK, in[i], arg);
  }
  T r;
  memcpy(&r, out, sizeof(T));
  return r;
}
template <class T> __device__ __forceinline__ T shfl_idx(const T& x, int lane) { return shfl_generic(x, lane, 0, 0); }
template <class T> __device__ __forceinline__ T shfl_up(const T& x, int d) { return shfl_generic(x, 0, 1, d); }
template <class T> __device__ __forceinline__ T shfl_down(const T& x, int d) { return shfl_generic(x, 0, 2, d); }

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// Inclusive scan across the lanes of a warp; lane 0 keeps its own value.
template <class T, class Op> __device__ __forceinline__ T warp_inclusive_scan(T x, Op op) {
  const int lane = lane_id();
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    T y = shfl_up(x, d);
    if (lane >= d) x = op(y, x);
  }
  return x;
}

// The same where a lane may hold nothing (`has` false): such a lane ends up with what precedes it.
template <class T, class Op> __device__ __forceinline__ T warp_inclusive_scan_if(T x, bool has, Op op) {
  const int lane = lane_id();
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    T y = shfl_up(x, d);
    const bool yh = __shfl_up_sync(FULL_MASK, (int)has, d) != 0;
    if (lane >= d && yh) { x = has ? op(y, x) : y; has = true; }
  }
  return x;
}

// Reduction across a warp of values that may be absent; operands keep lane order (lower lane on
// the left), so the operator need not commute.  Result valid in lane 0.
template <class T, class Op> __device__ __forceinline__ opt<T> warp_reduce_opt(opt<T> x, Op op) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    T y = shfl_down(x.v, d);
    int yh = __shfl_down_sync(FULL_MASK, (int)x.has, d);
    if (lane_id() + d < 32 && yh) { x.v = x.has ? op(x.v, y) : y; x.has = true; }
  }
  return x;
}

// ---------------------------------------------------------------- memory access
// Streaming (evict-first) 16-byte load/store: the data is touched once.
struct __align__(16) vec16 { unsigned x, y, z, w; };
__device__ __forceinline__ vec16 load_stream16(const void* p) {
  vec16 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void store_stream16(void* p, const vec16& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u32(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// L2-coherent load of any trivially copyable value (what another CTA of the same grid has just
// written, after a __threadfence on both sides): built-in 4- and 8-byte words where the size allows,
// bytes otherwise, so that structs and tuples work like scalars.
template <class T> __device__ __forceinline__ T load_cg_any(const T* p) {
  T v;
  if constexpr (sizeof(T) % 8 == 0 && alignof(T) >= 8) {
    unsigned long long w[sizeof(T) / 8];
#pragma unroll
    for (int q = 0; q < (int)(sizeof(T) / 8); ++q) w[q] = __ldcg(reinterpret_cast<const unsigned long long*>(p) + q);
    memcpy(&v, w, sizeof(T));
  } else if constexpr (sizeof(T) % 4 == 0 && alignof(T) >= 4) {
    unsigned w[sizeof(T) / 4];
#pragma unroll
    for (int q = 0; q < (int)(sizeof(T) / 4); ++q) w[q] = __ldcg(reinterpret_cast<const unsigned*>(p) + q);
    memcpy(&v, w, sizeof(T));
  } else {
    unsigned char w[sizeof(T)];
#pragma unroll
    for (int q = 0; q < (int)sizeof(T); ++q) w[q] = __ldcg(reinterpret_cast<const unsigned char*>(p) + q);
    memcpy(&v, w, sizeof(T));
  }
  return v;
}

__device__ __forceinline__ void record_error(unsigned* err, unsigned code) { atomicCAS(err, ERR_NONE, code); }

__device__ __forceinline__ void backoff(unsigned iter) { if (iter > 8) __nanosleep(iter > 64 ? 200 : 40); }

inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------- decoupled look-back state
// One descriptor per tile.  status: 0 = nothing yet, 1 = tile aggregate available,
// 2 = inclusive prefix (everything up to and including this tile) available.
enum : unsigned { TILE_INVALID = 0, TILE_AGGREGATE = 1, TILE_INCLUSIVE = 2 };

// 4-byte values travel with their status in one 64-bit word and 8-byte values in one 128-bit word
// (a single relaxed store / load each, no fence); anything else is written first and published by
// a release store of the status.
__device__ __forceinline__ void st_relaxed_b128(void* p, unsigned long long lo, unsigned long long hi) {
  asm volatile("{\n\t.reg .b128 t;\n\tmov.b128 t, {%1, %2};\n\tst.relaxed.gpu.global.b128 [%0], t;\n\t}" ::"l"(p), "l"(lo), "l"(hi) : "memory");
}
__device__ __forceinline__ void ld_relaxed_b128(const void* p, unsigned long long& lo, unsigned long long& hi) {
  asm volatile("{\n\t.reg .b128 t;\n\tld.relaxed.gpu.global.b128 t, [%2];\n\tmov.b128 {%0, %1}, t;\n\t}" : "=l"(lo), "=l"(hi) : "l"(p) : "memory");
}

template <class T> struct tile_state_mode {
  static constexpr int value = (sizeof(T) == 4 && std::is_trivially_copyable<T>::value) ? 1
                             : (sizeof(T) == 8 && std::is_trivially_copyable<T>::value) ? 2 : 0;
};
template <class T, int MODE = tile_state_mode<T>::value> struct tile_state;

template <class T> struct tile_state<T, 1> {
  unsigned long long* words;
  static size_t bytes(size_t tiles) { return align_up(tiles * 8, 256); }
  void bind(void* p, size_t) { words = static_cast<unsigned long long*>(p); }
  __device__ __forceinline__ void publish(size_t tile, unsigned status, const T& v) const {
    unsigned u;
    memcpy(&u, &v, 4);
    st_relaxed_u64(words + tile, ((unsigned long long)status << 32) | u);
  }
  __device__ __forceinline__ unsigned poll(size_t tile, T& v) const {
    unsigned long long w = ld_relaxed_u64(words + tile);
    unsigned u = (unsigned)w;
    memcpy(&v, &u, 4);
    return (unsigned)(w >> 32);
  }
};

template <class T> struct tile_state<T, 2> {
  unsigned long long* words;   // [tile][2]: value bits, status
  static size_t bytes(size_t tiles) { return align_up(tiles * 16, 256); }
  void bind(void* p, size_t) { words = static_cast<unsigned long long*>(p); }
  __device__ __forceinline__ void publish(size_t tile, unsigned status, const T& v) const {
    unsigned long long u;
    memcpy(&u, &v, 8);
    st_relaxed_b128(words + 2 * tile, u, (unsigned long long)status);
  }
  __device__ __forceinline__ unsigned poll(size_t tile, T& v) const {
    unsigned long long u, st;
    ld_relaxed_b128(words + 2 * tile, u, st);
    memcpy(&v, &u, 8);
    return (unsigned)st;
  }
};

template <class T> struct tile_state<T, 0> {
  unsigned* status; T* agg; T* inc;
  static size_t slot() { return (sizeof(T) + 15) / 16 * 16; }
  static size_t bytes(size_t tiles) { return align_up(tiles * 4, 256) + 2 * align_up(tiles * sizeof(T), 256); }
  void bind(void* p, size_t tiles) {
    char* c = static_cast<char*>(p);
    status = reinterpret_cast<unsigned*>(c); c += align_up(tiles * 4, 256);
    agg = reinterpret_cast<T*>(c); c += align_up(tiles * sizeof(T), 256);
    inc = reinterpret_cast<T*>(c);
  }
  __device__ __forceinline__ void publish(size_t tile, unsigned st, const T& v) const {
    (st == TILE_AGGREGATE ? agg : inc)[tile] = v;
    st_release_u32(status + tile, st);
  }
  __device__ __forceinline__ unsigned poll(size_t tile, T& v) const {
    unsigned st = ld_acquire_u32(status + tile);
    if (st == TILE_AGGREGATE) v = agg[tile];
    else if (st == TILE_INCLUSIVE) v = inc[tile];
    return st;
  }
};

// Warp-wide decoupled look-back.  Called by all 32 lanes of one warp of tile `tile` (> 0) after
// that tile's own aggregate has been published.  Returns (in every lane) the combination of all
// preceding tiles, oldest on the left.  Tile 0 always publishes TILE_INCLUSIVE, so the walk ends
// there at the latest.  Waits are bounded by SPIN_LIMIT.
template <class T, class Op, class State>
__device__ __forceinline__ T lookback_prefix(const State& ts, size_t tile, Op op, unsigned* err) {
  const int lane = lane_id();
  opt<T> running; running.has = false;
  long long window_end = (long long)tile - 1;
  while (true) {
    long long idx = window_end - lane;
    opt<T> mine; mine.has = false;
    unsigned st = TILE_INCLUSIVE;  // lanes before tile 0 read as "stop", contributing nothing
    if (idx >= 0) {
      unsigned iter = 0;
      while ((st = ts.poll((size_t)idx, mine.v)) == TILE_INVALID) {
        if (++iter > SPIN_LIMIT) { record_error(err, ERR_LOOKBACK_TIMEOUT); st = TILE_INCLUSIVE; mine.has = false; break; }
        backoff(iter);
      }
      if (iter <= SPIN_LIMIT) mine.has = true;
    }
    unsigned stop_mask = __ballot_sync(FULL_MASK, st == TILE_INCLUSIVE);
    int first_stop = stop_mask ? (__ffs(stop_mask) - 1) : 32;
    if (lane > first_stop) mine.has = false;
    // combine lanes: higher lane = older tile = left operand
    opt<T> w = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      T y = shfl_down(w.v, d);
      int yh = __shfl_down_sync(FULL_MASK, (int)w.has, d);
      if (lane + d < 32 && yh) { w.v = w.has ? op(y, w.v) : y; w.has = true; }
    }
    w.v = shfl_idx(w.v, 0);
    w.has = __shfl_sync(FULL_MASK, (int)w.has, 0);
    running.prepend(w, op);
    if (stop_mask) break;
    window_end -= 32;
  }
  return running.v;
}

// ---------------------------------------------------------------- tile-wide exclusive prefix
// The common core of scan, stream compaction and reduce-by-key.  A tile is BLOCK threads; every
// thread holds VPT "vectors" laid out lane-interleaved inside its warp's chunk: tile order is
// (warp, v, lane).  Given each vector's total, computes for each vector the combination of
// everything that precedes it -- earlier lanes of the row, earlier rows, earlier warps, earlier
// tiles (decoupled look-back) and the optional initial value -- without needing an identity.
template <class T, int NWARPS> struct tile_prefix_smem {
  T warp_total[NWARPS];
  T prefix;          // combination of all preceding tiles (and init)
  T inclusive;       // prefix (+) this tile's aggregate
  bool has_prefix;
};

template <class T, class Op, int VPT, int NWARPS, class State>
__device__ __forceinline__ void tile_exclusive_prefix(const T (&vec_total)[VPT], opt<T> (&pre)[VPT], size_t tile, const T& init,
                                                      bool has_init, Op op, const State& ts, unsigned* err,
                                                      tile_prefix_smem<T, NWARPS>& sm) {
  const int lane = lane_id(), warp = threadIdx.x >> 5;
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
  if (lane == 0) sm.warp_total[warp] = rowacc;
  __syncthreads();
  opt<T> wp; wp.has = false;
  for (int w = 0; w < warp; ++w) wp.append(sm.warp_total[w], op);
  if (warp == 0) {
    T agg = sm.warp_total[0];
#pragma unroll
    for (int w = 1; w < NWARPS; ++w) agg = op(agg, sm.warp_total[w]);
    if (tile == 0) {
      T inc = has_init ? op(init, agg) : agg;
      if (lane == 0) {
#ifdef TB200_TEST_HOOKS
        // test build only: with bit 0 of the header's flags set, tile 0 never publishes, so that its
        // successors' bounded waits run out (err points at the header's first word)
        if ((reinterpret_cast<const ws_header*>(err)->flags & 1u) == 0)
#endif
        ts.publish(0, TILE_INCLUSIVE, inc);
        sm.prefix = init; sm.has_prefix = has_init; sm.inclusive = inc;
      }
    } else {
      if (lane == 0) ts.publish(tile, TILE_AGGREGATE, agg);
      __syncwarp();
      T p = lookback_prefix<T>(ts, tile, op, err);
      if (lane == 0) {
        T inc = op(p, agg);
        ts.publish(tile, TILE_INCLUSIVE, inc);
        sm.prefix = p; sm.has_prefix = true; sm.inclusive = inc;
      }
    }
  }
  __syncthreads();
  opt<T> tp; tp.v = sm.prefix; tp.has = sm.has_prefix;
  wp.prepend(tp, op);
#pragma unroll
  for (int v = 0; v < VPT; ++v) pre[v].prepend(wp, op);
}

}  // namespace tb200
