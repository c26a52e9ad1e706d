// Two-pass reduce_by_key for large contiguous inputs on sm_100a (keys and values of the same size,
// 4 or 8 bytes), in the manner of select_stream.cuh: no thread waits for another warp.
//
// The input is cut into batches of RBK_STREAM_ROWS rows of 32 lanes x 16 bytes; consecutive warps of
// the grid take consecutive batches.  A batch is summarised by the pair
//     (number of run heads in it, reduction of the values behind its last head -- or of all its
//      values if it has no head)
// and pairs combine as (c1, v1) (+) (c2, v2) = (c1 + c2, c2 ? v2 : op(v1, v2)).
//   rbk_stream_count_kernel    writes every batch's pair;
//   an inclusive scan          (scan.cuh, with that operator) gives each batch what precedes it: how
//                              many runs have started and the value of the run still open;
//   rbk_stream_emit_kernel     reads the batch again and, at every run head, emits the head's key
//                              and the finished total of the run before it, compacted per row in
//                              shared memory private to the warp and stored coalesced; the last
//                              batch also closes the last run.
// Keys and values are read twice, every output is written once.  Same results as the single-pass
// kernel of reduce_by_key.cuh for exact operators; floating-point sums associate differently.
// Replaces, like it, InitAgent + ReduceByKeyAgent of thrust/system/cuda/detail/reduce_by_key.h:197-860.
#pragma once
#include "common.cuh"
#include "scan.cuh"
#include "select_stream.cuh"

namespace tb200 {

constexpr int RBK_STREAM_BLOCK = 256;
// Measured on B200, 2^28 int32 keys + fp32 values, runs of mean length 4: 1.24 ms with two rows per batch
// and four CTAs per SM (three or four rows: 1.27, registers spill; five CTAs: 1.48) against 1.37 ms
// for the single-pass kernel.
#ifndef TB200_RBK_STREAM_CTAS
#define TB200_RBK_STREAM_CTAS 4
#endif
constexpr int RBK_STREAM_CTAS_PER_SM = TB200_RBK_STREAM_CTAS;
constexpr int RBK_STREAM_ROWS = 2;
constexpr size_t RBK_STREAM_MIN_ITEMS = (size_t)1 << 24;

template <class V> struct rbk_stream_pair { unsigned long long count; V value; };

template <class V, class Op> struct rbk_stream_combine {
  Op op;
  __host__ __device__ __forceinline__ rbk_stream_pair<V> operator()(const rbk_stream_pair<V>& a, const rbk_stream_pair<V>& b) const {
    rbk_stream_pair<V> r;
    r.count = a.count + b.count;
    r.value = b.count ? b.value : op(a.value, b.value);
    return r;
  }
};

// One row: the lane's keys and values, its head bits, and the pair of its own items.
// FULL: the caller knows that the row lies wholly inside the input (no bounds checks).
template <class K, class V, class Eq, class Op, int VEC, bool FULL = false>
__device__ __forceinline__ rbk_stream_pair<V> rbk_stream_row(const K* keys, const V* vals, size_t n, size_t row, int lane, Eq eq, Op op, const K (&k)[VEC],
                                                            const V (&v)[VEC], K& prev_tail, bool& have_prev, unsigned& bits, unsigned& valid) {
  bits = select_row_flags<true, K, Eq, VEC, FULL>(n, row, lane, eq, k, prev_tail, have_prev);
  const size_t i0 = (row * 32 + lane) * VEC;
  valid = FULL ? (1u << VEC) - 1 : 0u;
  if (!FULL) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) if (i0 + j < n) valid |= 1u << j;
  }
  rbk_stream_pair<V> p;
  p.count = 0; p.value = v[0];
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    if ((valid >> j) & 1) {
      if ((bits >> j) & 1) { ++p.count; p.value = v[j]; }
      else if (j > 0) p.value = op(p.value, v[j]);
    }
  }
  return p;
}

// What a lane needs to know about the rest of its row.
template <class V> struct rbk_stream_row_info {
  unsigned heads_before;   // run heads in the row's earlier lanes
  unsigned row_heads;      // run heads in the whole row
  V carry_in;              // reduction of the values between the last head ahead of this lane (or the row's start) and this lane
  bool from_row_start;     // no head ahead of this lane in the row: what precedes the row continues into it
  V row_open;              // reduction of the values behind the row's last head (or of the whole row)
};

// Full rows: head counts by an integer scan, values by a segmented scan over lanes whose segment
// boundaries come from one ballot -- a fraction of the instructions of a scan of (count, value) pairs.
// A row with lanes past the end of the input (only the last one) takes the scan of pairs.
template <class V, class Op>
__device__ __forceinline__ rbk_stream_row_info<V> rbk_stream_row_scan(const rbk_stream_pair<V>& mine, bool row_full, bool lane_valid, int lane, Op op) {
  rbk_stream_row_info<V> r;
  if (row_full) {
    const unsigned c = (unsigned)mine.count;
    unsigned ci = c;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const unsigned y = __shfl_up_sync(FULL_MASK, ci, d); if (lane >= d) ci += y; }
    r.heads_before = ci - c;
    r.row_heads = __shfl_sync(FULL_MASK, ci, 31);
    const unsigned head_lanes = __ballot_sync(FULL_MASK, c != 0);
    const unsigned at_or_before = head_lanes & (0xffffffffu >> (31 - lane));
    const int seg_start = at_or_before ? 31 - __clz((int)at_or_before) : 0;   // first lane of this lane's segment
    V x = mine.value;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const V y = shfl_up(x, d); if (lane - d >= seg_start) x = op(y, x); }
    r.carry_in = shfl_up(x, 1);
    r.from_row_start = (head_lanes & ((1u << lane) - 1)) == 0;
    r.row_open = shfl_idx(x, 31);
  } else {
    const rbk_stream_combine<V, Op> comb{op};
    const rbk_stream_pair<V> incl = warp_inclusive_scan_if(mine, lane_valid, comb);
    const rbk_stream_pair<V> row_pair = shfl_idx(incl, 31);
    const rbk_stream_pair<V> before = shfl_up(incl, 1);
    r.heads_before = lane == 0 ? 0u : (unsigned)before.count;
    r.row_heads = (unsigned)row_pair.count;
    r.carry_in = before.value;
    r.from_row_start = lane == 0 || before.count == 0;
    r.row_open = row_pair.value;
  }
  return r;
}

template <class K, class V, class Eq, class Op, int VEC>
__global__ void __launch_bounds__(RBK_STREAM_BLOCK, RBK_STREAM_CTAS_PER_SM)
rbk_stream_count_kernel(const K* keys, const V* vals, size_t n, size_t rows, size_t batches, Eq eq, Op op, rbk_stream_pair<V>* batch_pairs) {
  using P = rbk_stream_pair<V>;
  const rbk_stream_combine<V, Op> comb{op};
  const int lane = lane_id();
  const size_t gwarp = ((size_t)blockIdx.x * RBK_STREAM_BLOCK + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * RBK_STREAM_BLOCK) >> 5;
  for (size_t batch = gwarp; batch < batches; batch += nwarps) {
    const size_t first = batch * RBK_STREAM_ROWS;
    K prev_tail = K(); bool have_prev = false;
    select_batch_start(keys, first, VEC, prev_tail, have_prev);
    P acc; acc.count = 0; acc.value = V();
    bool have_acc = false;
    // all batches but the last lie wholly inside the input: no bounds checks for them
    auto body = [&](auto full_tag) {
      constexpr bool FULL = decltype(full_tag)::value;
      K k[RBK_STREAM_ROWS][VEC];
      V v[RBK_STREAM_ROWS][VEC];
#pragma unroll
      for (int u = 0; u < RBK_STREAM_ROWS; ++u)
        if (FULL || first + u < rows) { select_row_load<K, VEC, FULL>(keys, n, first + u, lane, k[u]); select_row_load<V, VEC, FULL>(vals, n, first + u, lane, v[u]); }
#pragma unroll
      for (int u = 0; u < RBK_STREAM_ROWS; ++u) {
        if (!FULL && first + u >= rows) break;
        unsigned bits, valid;
        P mine = rbk_stream_row<K, V, Eq, Op, VEC, FULL>(keys, vals, n, first + u, lane, eq, op, k[u], v[u], prev_tail, have_prev, bits, valid);
        const rbk_stream_row_info<V> info = rbk_stream_row_scan<V, Op>(mine, FULL || (first + u + 1) * 32 * VEC <= n, valid != 0, lane, op);
        P row_pair; row_pair.count = info.row_heads; row_pair.value = info.row_open;
        acc = have_acc ? comb(acc, row_pair) : row_pair;
        have_acc = true;
      }
    };
    if ((first + RBK_STREAM_ROWS) * 32 * VEC <= n) body(std::true_type()); else body(std::false_type());
    if (lane == 0) batch_pairs[batch] = acc;
  }
}

template <class K, class V, class Eq, class Op, int VEC>
__global__ void __launch_bounds__(RBK_STREAM_BLOCK, RBK_STREAM_CTAS_PER_SM)
rbk_stream_emit_kernel(const K* keys, const V* vals, K* keys_out, V* vals_out, size_t n, size_t rows, size_t batches, Eq eq, Op op,
                       const rbk_stream_pair<V>* batch_incl, ws_header* hdr, const ws_header* scan_hdr, unsigned long long* d_count) {
  using P = rbk_stream_pair<V>;
  const rbk_stream_combine<V, Op> comb{op};
  const int lane = lane_id();
  const size_t gwarp = ((size_t)blockIdx.x * RBK_STREAM_BLOCK + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * RBK_STREAM_BLOCK) >> 5;
  __shared__ __align__(16) unsigned char s_keys[RBK_STREAM_BLOCK / 32][32 * VEC * sizeof(K)];
  __shared__ __align__(16) unsigned char s_vals[RBK_STREAM_BLOCK / 32][32 * VEC * sizeof(V)];
  K* skey = reinterpret_cast<K*>(s_keys[threadIdx.x >> 5]);
  V* sval = reinterpret_cast<V*>(s_vals[threadIdx.x >> 5]);
  for (size_t batch = gwarp; batch < batches; batch += nwarps) {
    const size_t first = batch * RBK_STREAM_ROWS;
    // what precedes the batch: runs started so far, value of the run still open
    P carry; carry.count = 0; carry.value = V();
    if (batch > 0) carry = batch_incl[batch - 1];
    K prev_tail = K(); bool have_prev = false;
    select_batch_start(keys, first, VEC, prev_tail, have_prev);
    auto body = [&](auto full_tag) {
    constexpr bool FULL = decltype(full_tag)::value;
    K k[RBK_STREAM_ROWS][VEC];
    V v[RBK_STREAM_ROWS][VEC];
#pragma unroll
    for (int u = 0; u < RBK_STREAM_ROWS; ++u)
      if (FULL || first + u < rows) { select_row_load<K, VEC, FULL>(keys, n, first + u, lane, k[u]); select_row_load<V, VEC, FULL>(vals, n, first + u, lane, v[u]); }
#pragma unroll
    for (int u = 0; u < RBK_STREAM_ROWS; ++u) {
      if (!FULL && first + u >= rows) break;
      unsigned bits, valid;
      P mine = rbk_stream_row<K, V, Eq, Op, VEC, FULL>(keys, vals, n, first + u, lane, eq, op, k[u], v[u], prev_tail, have_prev, bits, valid);
      const rbk_stream_row_info<V> info = rbk_stream_row_scan<V, Op>(mine, FULL || (first + u + 1) * 32 * VEC <= n, valid != 0, lane, op);
      P row_pair; row_pair.count = info.row_heads; row_pair.value = info.row_open;
      // second walk: at each head, the run before it is complete
      const unsigned long long row_first = carry.count;        // ordinal of the row's first head
      unsigned long long g = row_first + info.heads_before;
      V running = !info.from_row_start ? info.carry_in : (lane == 0 ? carry.value : op(carry.value, info.carry_in));
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        if ((valid >> j) & 1) {
          if ((bits >> j) & 1) {
            const unsigned local = (unsigned)(g - row_first);
            skey[local] = k[u][j];
            sval[local] = running;      // total of run g - 1 (unused when g == 0: nothing precedes the first item)
            ++g;
            running = v[u][j];
          } else {
            running = op(running, v[u][j]);
          }
        }
      }
      __syncwarp();
      const unsigned row_heads = (unsigned)row_pair.count;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const unsigned idx = lane + 32 * j;
        if (idx < row_heads) {
          const unsigned long long o = row_first + idx;
          keys_out[o] = skey[idx];
          if (o > 0) vals_out[o - 1] = sval[idx];
        }
      }
      __syncwarp();
      carry = comb(carry, row_pair);
    }
    };
    if ((first + RBK_STREAM_ROWS) * 32 * VEC <= n) body(std::true_type()); else body(std::false_type());
    if (batch == batches - 1 && lane == 0) {
      // the last run ends with the input
      vals_out[carry.count - 1] = carry.value;
      hdr->error = scan_hdr->error;
      hdr->count = carry.count;
      if (d_count) *d_count = carry.count;
    }
  }
}

template <class K> size_t rbk_stream_batches(size_t n) {
  const size_t per = (size_t)RBK_STREAM_ROWS * 32 * (sizeof(K) <= 16 ? 16 / sizeof(K) : 1);
  return (n + per - 1) / per;
}
template <class K, class V> size_t rbk_stream_workspace_bytes(size_t n) {
  const size_t b = rbk_stream_batches<K>(n);
  return sizeof(ws_header) + 2 * align_up(b * sizeof(rbk_stream_pair<V>), 256) + scan_workspace_bytes<rbk_stream_pair<V>>(b);
}

// Whether the streaming kernels may serve a call: large, 16-byte aligned inputs and outputs that
// overlap neither input.
inline bool rbk_stream_eligible(const void* keys, const void* vals, const void* keys_out, const void* vals_out, size_t n, size_t item_bytes) {
  if (n < RBK_STREAM_MIN_ITEMS) return false;
  if (((reinterpret_cast<uintptr_t>(keys) | reinterpret_cast<uintptr_t>(vals)) & 15) != 0) return false;
  const size_t bytes = n * item_bytes;
  const char* in[2] = {static_cast<const char*>(keys), static_cast<const char*>(vals)};
  const char* out[2] = {static_cast<const char*>(keys_out), static_cast<const char*>(vals_out)};
  for (int i = 0; i < 2; ++i)
    for (int o = 0; o < 2; ++o)
      if (out[o] < in[i] + bytes && in[i] < out[o] + bytes) return false;
  return true;
}

// The caller has checked rbk_stream_eligible() and sizeof(K) == sizeof(V) in {4, 8}.
template <class K, class V, class Eq, class Op>
cudaError_t reduce_by_key_stream_async(const K* keys, const V* vals, K* keys_out, V* vals_out, size_t n, Eq eq, Op op, unsigned long long* d_count,
                                       void* ws, cudaStream_t stream) {
  static_assert(sizeof(K) == sizeof(V) && (sizeof(K) == 4 || sizeof(K) == 8), "keys and values of the same size, 4 or 8 bytes");
  constexpr int VEC = 16 / sizeof(K);
  using P = rbk_stream_pair<V>;
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  const size_t rows = (n + 32 * VEC - 1) / (32 * VEC);
  const size_t batches = rbk_stream_batches<K>(n);
  const size_t arr = align_up(batches * sizeof(P), 256);
  P* pairs = reinterpret_cast<P*>(base + sizeof(ws_header));
  P* incl = reinterpret_cast<P*>(base + sizeof(ws_header) + arr);
  void* scan_ws = base + sizeof(ws_header) + 2 * arr;
  size_t ctas = (size_t)current_device_info().sm_count * RBK_STREAM_CTAS_PER_SM;
  const size_t want = (batches + RBK_STREAM_BLOCK / 32 - 1) / (RBK_STREAM_BLOCK / 32);
  if (ctas > want) ctas = want;
  cudaError_t e = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess) return e;
  timed_launch tl(KID_REDUCE_BY_KEY, stream);
  rbk_stream_count_kernel<K, V, Eq, Op, VEC><<<(unsigned)ctas, RBK_STREAM_BLOCK, 0, stream>>>(keys, vals, n, rows, batches, eq, op, pairs);
  P none; none.count = 0; none.value = V();
  e = scan_async<true>((const P*)pairs, incl, batches, none, false, rbk_stream_combine<V, Op>{op}, scan_ws, stream);
  if (e != cudaSuccess) return e;
  rbk_stream_emit_kernel<K, V, Eq, Op, VEC><<<(unsigned)ctas, RBK_STREAM_BLOCK, 0, stream>>>(keys, vals, keys_out, vals_out, n, rows, batches, eq, op, incl, hdr,
                                                                                             static_cast<const ws_header*>(scan_ws), d_count);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// inclusive / exclusive scan_by_key on the same plan: the batches' pairs and their scan are those of
// reduce_by_key; the second pass writes, for every item, the reduction of its run so far (16-byte
// stores at the items' own positions: nothing is compacted).  out may be vals exactly (in place).
// Replaces the ScanByKeyAgent of thrust/system/cuda/detail/scan_by_key.h:172-588 for such inputs.
template <bool INCLUSIVE, class K, class V, class Eq, class Op, int VEC>
__global__ void __launch_bounds__(RBK_STREAM_BLOCK, RBK_STREAM_CTAS_PER_SM)
scan_by_key_stream_kernel(const K* keys, const V* vals, V* out, size_t n, size_t rows, size_t batches, V init, Eq eq, Op op,
                          const rbk_stream_pair<V>* batch_incl, ws_header* hdr, const ws_header* scan_hdr) {
  using P = rbk_stream_pair<V>;
  const rbk_stream_combine<V, Op> comb{op};
  const int lane = lane_id();
  const size_t gwarp = ((size_t)blockIdx.x * RBK_STREAM_BLOCK + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * RBK_STREAM_BLOCK) >> 5;
  for (size_t batch = gwarp; batch < batches; batch += nwarps) {
    const size_t first = batch * RBK_STREAM_ROWS;
    P carry; carry.count = 0; carry.value = V();
    if (batch > 0) carry = batch_incl[batch - 1];
    K prev_tail = K(); bool have_prev = false;
    select_batch_start(keys, first, VEC, prev_tail, have_prev);
    auto body = [&](auto full_tag) {
    constexpr bool FULL = decltype(full_tag)::value;
    K k[RBK_STREAM_ROWS][VEC];
    V v[RBK_STREAM_ROWS][VEC];
#pragma unroll
    for (int u = 0; u < RBK_STREAM_ROWS; ++u)
      if (FULL || first + u < rows) { select_row_load<K, VEC, FULL>(keys, n, first + u, lane, k[u]); select_row_load<V, VEC, FULL>(vals, n, first + u, lane, v[u]); }
#pragma unroll
    for (int u = 0; u < RBK_STREAM_ROWS; ++u) {
      if (!FULL && first + u >= rows) break;
      const size_t row = first + u;
      const bool row_full = FULL || (row + 1) * 32 * VEC <= n;
      unsigned bits, valid;
      P mine = rbk_stream_row<K, V, Eq, Op, VEC, FULL>(keys, vals, n, row, lane, eq, op, k[u], v[u], prev_tail, have_prev, bits, valid);
      const rbk_stream_row_info<V> info = rbk_stream_row_scan<V, Op>(mine, row_full, valid != 0, lane, op);
      P row_pair; row_pair.count = info.row_heads; row_pair.value = info.row_open;
      // reduction of the run's items ahead of this lane's first item (meaningless if that item is a head)
      V prev = !info.from_row_start ? info.carry_in : (lane == 0 ? carry.value : op(carry.value, info.carry_in));
      V y[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        if ((bits >> j) & 1) {
          y[j] = INCLUSIVE ? v[u][j] : init;
          prev = v[u][j];
        } else {
          const V cur = op(prev, v[u][j]);
          y[j] = INCLUSIVE ? cur : op(init, prev);
          prev = cur;
        }
      }
      const size_t i0 = (row * 32 + lane) * VEC;
      if (row_full) {
        vec16 r;
        V* e = reinterpret_cast<V*>(&r);
#pragma unroll
        for (int j = 0; j < VEC; ++j) e[j] = y[j];
        store_stream16(reinterpret_cast<char*>(out) + i0 * sizeof(V), r);
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) if (i0 + j < n) out[i0 + j] = y[j];
      }
      carry = comb(carry, row_pair);
    }
    };
    if ((first + RBK_STREAM_ROWS) * 32 * VEC <= n) body(std::true_type()); else body(std::false_type());
    if (batch == batches - 1 && lane == 0) hdr->error = scan_hdr->error;
  }
}

// Whether the streaming kernels may serve a scan_by_key: large, 16-byte aligned arrays; out is vals
// itself or overlaps neither input.
inline bool scan_by_key_stream_eligible(const void* keys, const void* vals, const void* out, size_t n, size_t item_bytes) {
  if (n < RBK_STREAM_MIN_ITEMS) return false;
  if (((reinterpret_cast<uintptr_t>(keys) | reinterpret_cast<uintptr_t>(vals) | reinterpret_cast<uintptr_t>(out)) & 15) != 0) return false;
  const size_t bytes = n * item_bytes;
  const char* kb = static_cast<const char*>(keys);
  const char* vb = static_cast<const char*>(vals);
  const char* ob = static_cast<const char*>(out);
  if (ob < kb + bytes && kb < ob + bytes) return false;
  if (ob != vb && ob < vb + bytes && vb < ob + bytes) return false;
  return true;
}

// The caller has checked scan_by_key_stream_eligible() and sizeof(K) == sizeof(V) in {4, 8}.
template <bool INCLUSIVE, class K, class V, class Eq, class Op>
cudaError_t scan_by_key_stream_async(const K* keys, const V* vals, V* out, size_t n, V init, Eq eq, Op op, void* ws, cudaStream_t stream) {
  static_assert(sizeof(K) == sizeof(V) && (sizeof(K) == 4 || sizeof(K) == 8), "keys and values of the same size, 4 or 8 bytes");
  constexpr int VEC = 16 / sizeof(K);
  using P = rbk_stream_pair<V>;
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  const size_t rows = (n + 32 * VEC - 1) / (32 * VEC);
  const size_t batches = rbk_stream_batches<K>(n);
  const size_t arr = align_up(batches * sizeof(P), 256);
  P* pairs = reinterpret_cast<P*>(base + sizeof(ws_header));
  P* incl = reinterpret_cast<P*>(base + sizeof(ws_header) + arr);
  void* scan_ws = base + sizeof(ws_header) + 2 * arr;
  size_t ctas = (size_t)current_device_info().sm_count * RBK_STREAM_CTAS_PER_SM;
  const size_t want = (batches + RBK_STREAM_BLOCK / 32 - 1) / (RBK_STREAM_BLOCK / 32);
  if (ctas > want) ctas = want;
  cudaError_t e = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess) return e;
  rbk_stream_count_kernel<K, V, Eq, Op, VEC><<<(unsigned)ctas, RBK_STREAM_BLOCK, 0, stream>>>(keys, vals, n, rows, batches, eq, op, pairs);
  P none; none.count = 0; none.value = V();
  e = scan_async<true>((const P*)pairs, incl, batches, none, false, rbk_stream_combine<V, Op>{op}, scan_ws, stream);
  if (e != cudaSuccess) return e;
  scan_by_key_stream_kernel<INCLUSIVE, K, V, Eq, Op, VEC><<<(unsigned)ctas, RBK_STREAM_BLOCK, 0, stream>>>(keys, vals, out, n, rows, batches, init, eq, op, incl, hdr,
                                                                                                          static_cast<const ws_header*>(scan_ws));
  return cudaGetLastError();
}

}  // namespace tb200
