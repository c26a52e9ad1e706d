// Two-pass stream compaction for large contiguous inputs on sm_100a: copy_if, partition_copy,
// the scratch half of the in-place partition, and unique_copy.
//
// The single-pass kernel of select.cuh spends its time in the barrier-separated phases of a tile
// (flags, block-wide scan, compaction through shared memory, stores).  Here no thread ever waits for
// another warp: the input is cut into batches of SELECT_STREAM_ROWS rows of 512 bytes, consecutive
// warps of the grid take consecutive batches (so the grid reads one contiguous window at a time), and
//   select_count_kernel    counts the items each batch will keep;
//   an exclusive scan      (scan.cuh) turns the batches' counts into output offsets;
//   select_scatter_kernel  every warp reads its batches again: one 16-byte load per lane and row, the keep
//                          flags, a shuffle scan of the per-lane counts, compaction of the row in
//                          512 bytes of shared memory private to the warp, coalesced stores.
// No __syncthreads, no descriptors.  The input is read twice and every flag is
// evaluated twice; in exchange both passes stream.  Same results as the single-pass kernel (stable
// order).  Used by select_async for inputs of at least SELECT_STREAM_MIN_ITEMS when the outputs do
// not overlap the input.  The predicate is evaluated ~2^29 times per 2^28-item call, so it has to be
// cheap: the C ABI hands these kernels its predicates as types (abi_pred::visit), not as a switch.
// Every batch but the last lies wholly inside the input and takes a code path without any bounds
// check (the checks were two thirds of the count kernel's instructions and a third of the scatter
// kernel's); both kernels then run at the speed of their memory traffic.
// Measured on B200, 2^28 int32, x % 2 == 0: copy_if 0.46 ms against 0.71 single-pass, partition_copy
// 0.64 against 0.92, unique_copy 0.43 against 0.60.  (The same two passes run window by window inside
// one persistent kernel, so that the second read comes from L2 -- the scheme that pays for the scan,
// scan.cuh -- measured slower here, 0.53 - 0.59 ms for copy_if, and was not kept.)  Replaces, like select.cuh, the agents of
// thrust/system/cuda/detail/copy_if.h:160-593, partition.h:134-602 and unique.h:183-541.
#pragma once
#include "common.cuh"
#include "scan.cuh"

namespace tb200 {

// where dropped items go (KEEP_REJECTS): a second array in input order; mirrored from the end of
// out_sel; or behind the kept items in out_sel, in input order
enum : int { SELECT_REJ_SECOND_ARRAY = 0, SELECT_REJ_MIRRORED = 1, SELECT_REJ_BEHIND_SELECTED = 2 };

constexpr int SELECT_STREAM_BLOCK = 256;
constexpr int SELECT_STREAM_CTAS_PER_SM = 5;   // 48 registers; 4 and 6 measured 2-4 % slower
// below this the three launches cost more than they save (2^22 items: 0.040 ms against 0.030 single-pass)
constexpr size_t SELECT_STREAM_MIN_ITEMS = (size_t)1 << 24;
constexpr int SELECT_STREAM_ROWS = 4;   // rows (512 bytes each) a warp has in flight; 8 measured slower

// This lane's VEC items of row `row` (32 lanes x VEC items); items past the end read as T().
// FULL: the caller knows that the row lies wholly inside the input (no bounds checks at all).
template <class T, int VEC, bool FULL = false>
__device__ __forceinline__ void select_row_load(const T* in, size_t n, size_t row, int lane, T (&x)[VEC]) {
  const size_t i0 = (row * 32 + lane) * VEC;
  if (FULL || (row + 1) * 32 * VEC <= n) {
    vec16 r = load_stream16(reinterpret_cast<const char*>(in) + i0 * sizeof(T));
    const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int k = 0; k < VEC; ++k) x[k] = e[k];
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) x[k] = i0 + k < n ? in[i0 + k] : T();
  }
}

// Shared by both passes: this lane's keep bits for the items x of row `row`.  `prev_tail` carries
// the last item of the previous row for SEL_UNIQUE-style predicates.
template <bool UNIQUE, class T, class Pred, int VEC, bool FULL = false>
__device__ __forceinline__ unsigned select_row_flags(size_t n, size_t row, int lane, Pred pred, const T (&x)[VEC], T& prev_tail, bool& have_prev) {
  const size_t i0 = (row * 32 + lane) * VEC;
  const bool row_full = FULL || (row + 1) * 32 * VEC <= n;
  unsigned bits = 0;
  if constexpr (UNIQUE) {
    // predecessor of this lane's first item: the previous lane's last item, or the previous row's
    T prev = shfl_up(x[VEC - 1], 1);
    bool has = true;
    if (lane == 0) { prev = prev_tail; has = have_prev; }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      const bool head = (k == 0 && !has) ? true : !pred(k == 0 ? prev : x[k - 1], x[k]);
      if ((row_full || i0 + k < n) && head) bits |= 1u << k;
    }
    prev_tail = shfl_idx(x[VEC - 1], 31);
    have_prev = true;
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      if ((row_full || i0 + k < n) && pred(x[k])) bits |= 1u << k;
  }
  return bits;
}

// predecessor of a batch's first item, for SEL_UNIQUE-style predicates
template <class T> __device__ __forceinline__ void select_batch_start(const T* in, size_t first_row, int vec, T& prev_tail, bool& have_prev) {
  have_prev = first_row > 0;
  prev_tail = have_prev ? in[first_row * 32 * vec - 1] : T();
}

template <bool UNIQUE, class T, class Pred, int VEC>
__global__ void __launch_bounds__(SELECT_STREAM_BLOCK, SELECT_STREAM_CTAS_PER_SM)
select_count_kernel(const T* in, size_t n, size_t rows, size_t batches, Pred pred, unsigned long long* batch_counts) {
  const int lane = lane_id();
  const size_t gwarp = ((size_t)blockIdx.x * SELECT_STREAM_BLOCK + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * SELECT_STREAM_BLOCK) >> 5;
  // consecutive warps take consecutive batches: at any moment the grid reads one contiguous window
  for (size_t batch = gwarp; batch < batches; batch += nwarps) {
    const size_t first = batch * SELECT_STREAM_ROWS;
    T prev_tail = T(); bool have_prev = false;
    if (UNIQUE) select_batch_start(in, first, VEC, prev_tail, have_prev);
    unsigned count = 0;
    // all batches but the last lie wholly inside the input: no bounds checks for them
    auto body = [&](auto full_tag) {
      constexpr bool FULL = decltype(full_tag)::value;
      T x[SELECT_STREAM_ROWS][VEC];
#pragma unroll
      for (int u = 0; u < SELECT_STREAM_ROWS; ++u)
        if (FULL || first + u < rows) select_row_load<T, VEC, FULL>(in, n, first + u, lane, x[u]);
#pragma unroll
      for (int u = 0; u < SELECT_STREAM_ROWS; ++u)
        if (FULL || first + u < rows) count += __popc(select_row_flags<UNIQUE, T, Pred, VEC, FULL>(n, first + u, lane, pred, x[u], prev_tail, have_prev));
    };
    if ((first + SELECT_STREAM_ROWS) * 32 * VEC <= n) body(std::true_type()); else body(std::false_type());
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) count += __shfl_xor_sync(FULL_MASK, count, d);
    if (lane == 0) batch_counts[batch] = count;
  }
}

// the total (exclusive offset of the last batch + its count) goes to the header and to *d_count
template <int UNUSED = 0>   // a template only so that the header can be included in several translation units
__global__ void select_total_kernel(const unsigned long long* batch_counts, const unsigned long long* batch_offsets, size_t batches, ws_header* hdr,
                                    const ws_header* scan_hdr, unsigned long long* d_count) {
  const unsigned long long total = batch_offsets[batches - 1] + batch_counts[batches - 1];
  hdr->error = scan_hdr->error;   // the offsets' scan reports a look-back time-out in its own header
  hdr->count = total;
  if (d_count) *d_count = total;
}

template <bool UNIQUE, bool KEEP_REJECTS, class T, class Pred, int VEC>
__global__ void __launch_bounds__(SELECT_STREAM_BLOCK, SELECT_STREAM_CTAS_PER_SM)
select_scatter_kernel(const T* in, T* out_sel, T* out_rej, size_t n, size_t rows, size_t batches, Pred pred, const unsigned long long* batch_offsets,
                      int rej_mode, const ws_header* hdr) {
  const int lane = lane_id();
  const size_t gwarp = ((size_t)blockIdx.x * SELECT_STREAM_BLOCK + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * SELECT_STREAM_BLOCK) >> 5;
  __shared__ __align__(16) unsigned char s_stage[SELECT_STREAM_BLOCK / 32][512];
  T* buf = reinterpret_cast<T*>(s_stage[threadIdx.x >> 5]);
  for (size_t batch = gwarp; batch < batches; batch += nwarps) {
    const size_t first = batch * SELECT_STREAM_ROWS;
    size_t kept = (size_t)batch_offsets[batch];   // kept items before the current row
    T prev_tail = T(); bool have_prev = false;
    if (UNIQUE) select_batch_start(in, first, VEC, prev_tail, have_prev);
    auto body = [&](auto full_tag) {
      constexpr bool FULL = decltype(full_tag)::value;
      T xs[SELECT_STREAM_ROWS][VEC];
#pragma unroll
      for (int u = 0; u < SELECT_STREAM_ROWS; ++u)
        if (FULL || first + u < rows) select_row_load<T, VEC, FULL>(in, n, first + u, lane, xs[u]);
#pragma unroll
      for (int u = 0; u < SELECT_STREAM_ROWS; ++u) {
        if (!FULL && first + u >= rows) break;
        const size_t row = first + u;
        const T (&x)[VEC] = xs[u];
        const unsigned bits = select_row_flags<UNIQUE, T, Pred, VEC, FULL>(n, row, lane, pred, x, prev_tail, have_prev);
        const unsigned cnt = __popc(bits);
        unsigned incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { unsigned y = __shfl_up_sync(FULL_MASK, incl, d); if (lane >= d) incl += y; }
        const unsigned row_total = __shfl_sync(FULL_MASK, incl, 31);
        unsigned rank = incl - cnt;                                  // kept items of this row before this lane's
        const size_t row_base = row * 32 * VEC;
        const size_t rej_base = row_base - kept;                     // dropped items before this row
        const unsigned local0 = lane * VEC;
        const unsigned row_n = (FULL || (row + 1) * 32 * VEC <= n) ? 32u * VEC : (unsigned)(n - row_base);
        // compact the row in the warp's own 512 bytes of shared memory (kept items first, dropped ones
        // behind them), then store with consecutive lanes on consecutive addresses
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          if ((bits >> k) & 1) buf[rank++] = x[k];
          else if (KEEP_REJECTS && (FULL || local0 + k < row_n)) buf[row_total + (local0 + k - rank)] = x[k];
        }
        __syncwarp();
        T* const sel_out = out_sel + kept + lane;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const unsigned idx = lane + 32 * j;
          if (idx < row_total) sel_out[32 * j] = buf[idx];
          else if (KEEP_REJECTS && idx < row_n) {
            const size_t r = rej_base + (idx - row_total);
            if (rej_mode == SELECT_REJ_SECOND_ARRAY) out_rej[r] = buf[idx];
            else if (rej_mode == SELECT_REJ_MIRRORED) out_sel[n - 1 - r] = buf[idx];
            else out_sel[(size_t)hdr->count + r] = buf[idx];   // the total was published before this kernel started
          }
        }
        __syncwarp();
        kept += row_total;
      }
    };
    if ((first + SELECT_STREAM_ROWS) * 32 * VEC <= n) body(std::true_type()); else body(std::false_type());
  }
}

template <class T> size_t select_stream_batches(size_t n) {
  const size_t per = (size_t)SELECT_STREAM_ROWS * 32 * (sizeof(T) <= 16 ? 16 / sizeof(T) : 1);
  return (n + per - 1) / per;
}
// header, the batches' counts, their offsets, the scan's own workspace
template <class T> size_t select_stream_workspace_bytes(size_t n) {
  const size_t b = select_stream_batches<T>(n);
  return sizeof(ws_header) + 2 * align_up(b * sizeof(unsigned long long), 256) + scan_workspace_bytes<unsigned long long>(b);
}

// Whether the streaming kernels may serve a call: a large, 16-byte aligned input and outputs that do
// not overlap it (their warps write while others still read).  `out_rej` only matters when rejected
// items go to a second array (not mirrored into out_sel).
inline bool select_stream_eligible(const void* in, const void* out_sel, const void* out_rej, bool rejects_to_second_array, size_t n, size_t item_bytes) {
  const char* ib = static_cast<const char*>(in);
  const char* ob = static_cast<const char*>(out_sel);
  const char* rb = static_cast<const char*>(out_rej);
  const size_t bytes = n * item_bytes;
  if (n < SELECT_STREAM_MIN_ITEMS || (reinterpret_cast<uintptr_t>(in) & 15) != 0) return false;
  if (ob < ib + bytes && ib < ob + bytes) return false;
  if (rejects_to_second_array && (rb == nullptr || (rb < ib + bytes && ib < rb + bytes))) return false;
  return true;
}

// The caller has checked select_stream_eligible().
template <bool UNIQUE, bool KEEP_REJECTS, class T, class Pred>
cudaError_t select_stream_async(const T* in, T* out_sel, T* out_rej, size_t n, Pred pred, int rej_mode, unsigned long long* d_count, void* ws,
                                cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(T);
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  const size_t rows = (n + 32 * VEC - 1) / (32 * VEC);
  const size_t batches = select_stream_batches<T>(n);
  const size_t arr = align_up(batches * sizeof(unsigned long long), 256);
  unsigned long long* counts = reinterpret_cast<unsigned long long*>(base + sizeof(ws_header));
  unsigned long long* offsets = reinterpret_cast<unsigned long long*>(base + sizeof(ws_header) + arr);
  void* scan_ws = base + sizeof(ws_header) + 2 * arr;
  size_t ctas = (size_t)current_device_info().sm_count * SELECT_STREAM_CTAS_PER_SM;
  const size_t want = (batches + SELECT_STREAM_BLOCK / 32 - 1) / (SELECT_STREAM_BLOCK / 32);
  if (ctas > want) ctas = want;
  timed_launch tl(KID_SELECT, stream);
  select_count_kernel<UNIQUE, T, Pred, VEC><<<(unsigned)ctas, SELECT_STREAM_BLOCK, 0, stream>>>(in, n, rows, batches, pred, counts);
  cudaError_t e = scan_async<false>((const unsigned long long*)counts, offsets, batches, 0ull, true, plus_op(), scan_ws, stream);
  if (e != cudaSuccess) return e;
  // the scan's status word lives in its own workspace; this call's header carries the count
  if ((e = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream)) != cudaSuccess) return e;
  select_total_kernel<><<<1, 1, 0, stream>>>(counts, offsets, batches, hdr, static_cast<const ws_header*>(scan_ws), d_count);
  select_scatter_kernel<UNIQUE, KEEP_REJECTS, T, Pred, VEC>
      <<<(unsigned)ctas, SELECT_STREAM_BLOCK, 0, stream>>>(in, out_sel, out_rej, n, rows, batches, pred, offsets, rej_mode, hdr);
  return cudaGetLastError();
}

}  // namespace tb200
