// Onesweep-style least-significant-digit radix sort (keys or key/value pairs) for sm_100a.
//
// Replaces the cub::DeviceRadixSort::SortKeys / SortPairs call of
// thrust/system/cuda/detail/sort.h:1343-1427.  Structure:
//   1. radix_hist_kernel      one read of the keys builds the 256-bin histogram of EVERY 8-bit
//                             digit place at once (shared-memory bins, then global atomics);
//   2. radix_scan_hist_kernel exclusive-scans each histogram into bucket bases and marks a digit
//                             place as skippable when one bucket holds every key;
//   3. onesweep_kernel        once per non-skipped digit place: a tile of keys is ranked inside
//                             the CTA (warp match + per-warp counters), the tile's per-digit
//                             counts are chained to the preceding tiles by decoupled look-back
//                             (one thread per digit), and keys then values are staged through
//                             shared memory so that each bucket's run is written contiguously;
//   4. radix_copy_back_kernel only if an odd number of places ran: moves the result from the
//                             alternate buffer to the caller's.
// A pass therefore reads and writes each key (and value) exactly once.  The sort is stable.
// Key order is defined on an unsigned code of the key: unsigned keys unchanged, signed keys
// with the sign bit flipped, IEEE floats with all bits flipped when negative and the sign bit
// flipped otherwise (the encoders of thrust/system/detail/sequential/stable_radix_sort.inl:54-138);
// descending order complements the code.
#pragma once
#include "common.cuh"

namespace tb200 {

constexpr int RADIX_BITS = 8;
constexpr int RADIX_BINS = 256;
constexpr int RADIX_MAX_PASSES = 8;
constexpr int ONESWEEP_BLOCK = 512;
constexpr int HIST_BLOCK = 512;

enum key_kind : int { KEY_UNSIGNED = 0, KEY_SIGNED = 1, KEY_FLOAT = 2 };

struct key_coding {
  int kind; int descending;
};

template <class UK> __device__ __forceinline__ UK encode_key(UK k, key_coding c) {
  constexpr int B = 8 * sizeof(UK);
  const UK sign = (UK)1 << (B - 1);
  UK mask = 0;
  if (c.kind == KEY_SIGNED) mask = sign;
  else if (c.kind == KEY_FLOAT) mask = (k & sign) ? (UK)~(UK)0 : sign;
  k ^= mask;
  return c.descending ? (UK)~k : k;
}

// Control block in the workspace, after ws_header.
struct radix_ctrl {
  unsigned long long hist[RADIX_MAX_PASSES][RADIX_BINS];   // counts, then exclusive bases
  unsigned skip[RADIX_MAX_PASSES];                         // 1: every key shares this digit
  unsigned tickets[RADIX_MAX_PASSES];
  unsigned pad[48];
};

// ---------------------------------------------------------------- 1. histograms of all digit places
template <class UK>
__global__ void __launch_bounds__(HIST_BLOCK)
radix_hist_kernel(const UK* keys, size_t n, key_coding coding, int first_pass, int num_passes, radix_ctrl* ctrl) {
  constexpr int NP = sizeof(UK);
  __shared__ unsigned bins[NP][RADIX_BINS];
  for (int i = threadIdx.x; i < NP * RADIX_BINS; i += HIST_BLOCK) (&bins[0][0])[i] = 0;
  __syncthreads();
  // thread-local run compression: a digit place where consecutive keys agree (for example the
  // all-zero high bytes of narrow keys) costs one shared-memory atomic per run, not per key
  unsigned last[NP]; unsigned run[NP];
#pragma unroll
  for (int p = 0; p < NP; ++p) { last[p] = 0; run[p] = 0; }
  const size_t stride = (size_t)gridDim.x * HIST_BLOCK;
  constexpr int U = 4;
  size_t i = (size_t)blockIdx.x * HIST_BLOCK + threadIdx.x;
  auto account = [&](UK k) {
    UK e = encode_key(k, coding);
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      unsigned d = (unsigned)(e >> (p * RADIX_BITS)) & (RADIX_BINS - 1);
      if (d == last[p]) ++run[p];
      else { if (run[p]) atomicAdd(&bins[p][last[p]], run[p]); last[p] = d; run[p] = 1; }
    }
  };
  for (; i + (U - 1) * stride < n; i += U * stride) {
    UK k[U];
#pragma unroll
    for (int u = 0; u < U; ++u) k[u] = __ldcs(keys + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) account(k[u]);
  }
  for (; i < n; i += stride) account(__ldcs(keys + i));
#pragma unroll
  for (int p = 0; p < NP; ++p) if (run[p]) atomicAdd(&bins[p][last[p]], run[p]);
  __syncthreads();
  for (int j = threadIdx.x; j < NP * RADIX_BINS; j += HIST_BLOCK) {
    int p = j / RADIX_BINS;
    unsigned c = (&bins[0][0])[j];
    if (c && p >= first_pass && p < first_pass + num_passes) atomicAdd(&ctrl->hist[p][j % RADIX_BINS], (unsigned long long)c);
  }
}

// ---------------------------------------------------------------- 2. bucket bases + skip flags
__global__ void __launch_bounds__(RADIX_BINS)
radix_scan_hist_kernel(radix_ctrl* ctrl, size_t n, int first_pass) {
  const int p = first_pass + blockIdx.x;
  __shared__ unsigned long long warp_tot[RADIX_BINS / 32];
  __shared__ unsigned degenerate;
  if (threadIdx.x == 0) degenerate = 0;
  __syncthreads();
  unsigned long long c = ctrl->hist[p][threadIdx.x];
  if (c == n) degenerate = 1;
  unsigned long long incl = warp_inclusive_scan(c, plus_op());
  if (lane_id() == 31) warp_tot[threadIdx.x >> 5] = incl;
  __syncthreads();
  unsigned long long base = 0;
  for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) base += warp_tot[w];
  ctrl->hist[p][threadIdx.x] = base + incl - c;
  if (threadIdx.x == 0) ctrl->skip[p] = degenerate;
}

// ---------------------------------------------------------------- 3. one digit place
template <int KB, int VB> struct onesweep_tuning {
  // items per thread so that one tile's staging (keys + values) stays near 80 KB
  static constexpr int IPT = (KB + VB) <= 4 ? 22 : (KB + VB) <= 8 ? 18 : (KB + VB) <= 12 ? 13 : 10;
};

template <class UK, class UV, bool HAS_V, class LB, int IPT>
__global__ void __launch_bounds__(ONESWEEP_BLOCK)
onesweep_kernel(UK* buf_a, UK* buf_b, UV* val_a, UV* val_b, unsigned n, key_coding coding, int pass, int first_pass,
                radix_ctrl* ctrl, LB* lookback, ws_header* hdr) {
  constexpr int NWARPS = ONESWEEP_BLOCK / 32;
  constexpr int TILE = ONESWEEP_BLOCK * IPT;
  constexpr int WCHUNK = 32 * IPT;
  constexpr int LB_BITS = 8 * sizeof(LB) - 2;
  constexpr LB LB_MASK = ((LB)1 << LB_BITS) - 1;

  if (ctrl->skip[pass]) return;
  int flips = 0;
  for (int q = first_pass; q < pass; ++q) flips += ctrl->skip[q] ? 0 : 1;
  const UK* src = (flips & 1) ? buf_b : buf_a;
  UK* dst = (flips & 1) ? buf_a : buf_b;
  const UV* vsrc = (flips & 1) ? val_b : val_a;
  UV* vdst = (flips & 1) ? val_a : val_b;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned* warp_hist = reinterpret_cast<unsigned*>(smem_raw);                    // [NWARPS][256]
  unsigned* s_goff = warp_hist + NWARPS * RADIX_BINS;                              // [256] global offset - staged position
  unsigned* s_scan = s_goff + RADIX_BINS;                                          // [8] warp totals for the digit scan
  UK* stage_k = reinterpret_cast<UK*>(s_scan + 16);
  UV* stage_v = reinterpret_cast<UV*>(stage_k + TILE);
  __shared__ unsigned s_tile;

  if (threadIdx.x == 0) s_tile = atomicAdd(&ctrl->tickets[pass], 1u);
  for (int i = threadIdx.x; i < NWARPS * RADIX_BINS; i += ONESWEEP_BLOCK) warp_hist[i] = 0;
  __syncthreads();
  const unsigned tile = s_tile;
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const unsigned tile_base = tile * (unsigned)TILE;
  const unsigned tile_n = min((unsigned)TILE, n - tile_base);
  const unsigned wbase = tile_base + warp * WCHUNK;
  const int shift = pass * RADIX_BITS;

  // ---- load keys (and values: issued now so their latency hides behind the ranking)
  UK key[IPT]; UV val[IPT];
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    unsigned g = wbase + i * 32 + lane;
    key[i] = g < n ? __ldcs(src + g) : (UK)0;
  }
  if constexpr (HAS_V) {
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      unsigned g = wbase + i * 32 + lane;
      val[i] = g < n ? __ldcs(vsrc + g) : (UV)0;
    }
  }

  // ---- rank inside the warp: keys of equal digit find each other with match.any; the lowest
  // lane of each group bumps the warp's private counter for that digit
  unsigned short pos[IPT];
  unsigned* my_hist = warp_hist + warp * RADIX_BINS;
  const unsigned lanemask_lt = (1u << lane) - 1;
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    unsigned g = wbase + i * 32 + lane;
    unsigned d = g < n ? ((unsigned)(encode_key(key[i], coding) >> shift) & (RADIX_BINS - 1)) : (RADIX_BINS - 1);
    unsigned peers = __match_any_sync(FULL_MASK, d);
    int leader = __ffs(peers) - 1;
    unsigned before = 0;
    if (lane == leader) { before = my_hist[d]; my_hist[d] = before + __popc(peers); }
    before = __shfl_sync(FULL_MASK, before, leader);
    pos[i] = (unsigned short)(before + __popc(peers & lanemask_lt));
    __syncwarp();
  }
  __syncthreads();

  // ---- per digit: stack the warps' counts, scan digits, chain to preceding tiles
  unsigned my_count = 0, digit_off = 0;
  if (threadIdx.x < RADIX_BINS) {
    unsigned run = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) { unsigned c = warp_hist[w * RADIX_BINS + threadIdx.x]; warp_hist[w * RADIX_BINS + threadIdx.x] = run; run += c; }
    my_count = run;
    unsigned incl = warp_inclusive_scan(my_count, plus_op());
    if (lane == 31) s_scan[warp] = incl;
    digit_off = incl - my_count;
  }
  __syncthreads();
  if (threadIdx.x < RADIX_BINS) {
    for (int w = 0; w < warp; ++w) digit_off += s_scan[w];
    // a partial tile pads with pseudo-keys of digit 255, ranked after every real key
    unsigned real_count = my_count;
    if (threadIdx.x == RADIX_BINS - 1) real_count -= (unsigned)TILE - tile_n;
    LB* slot = lookback + (size_t)tile * RADIX_BINS + threadIdx.x;
    LB prefix = 0;
    if (tile == 0) {
      *reinterpret_cast<volatile LB*>(slot) = ((LB)TILE_INCLUSIVE << LB_BITS) | (LB)real_count;
    } else {
      *reinterpret_cast<volatile LB*>(slot) = ((LB)TILE_AGGREGATE << LB_BITS) | (LB)real_count;
      long long t = (long long)tile - 1;
      unsigned iter = 0;
      while (true) {
        LB w = *reinterpret_cast<volatile LB*>(lookback + (size_t)t * RADIX_BINS + threadIdx.x);
        unsigned st = (unsigned)(w >> LB_BITS);
        if (st == TILE_INVALID) {
          if (++iter > SPIN_LIMIT) { record_error(&hdr->error, ERR_LOOKBACK_TIMEOUT); break; }
          backoff(iter);
          continue;
        }
        prefix += w & LB_MASK;
        if (st == TILE_INCLUSIVE) break;
        --t; iter = 0;
      }
      *reinterpret_cast<volatile LB*>(slot) = ((LB)TILE_INCLUSIVE << LB_BITS) | (LB)(prefix + real_count);
    }
    s_goff[threadIdx.x] = (unsigned)ctrl->hist[pass][threadIdx.x] + (unsigned)prefix - digit_off;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) warp_hist[w * RADIX_BINS + threadIdx.x] += digit_off;
  }
  __syncthreads();

  // ---- stage keys in bucket order, then stream each bucket's run out contiguously
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    unsigned g = wbase + i * 32 + lane;
    unsigned d = g < n ? ((unsigned)(encode_key(key[i], coding) >> shift) & (RADIX_BINS - 1)) : (RADIX_BINS - 1);
    pos[i] = (unsigned short)(pos[i] + my_hist[d]);
    stage_k[pos[i]] = key[i];
  }
  __syncthreads();
  unsigned char dig[IPT];
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    unsigned j = threadIdx.x + i * ONESWEEP_BLOCK;
    if (j < tile_n) {
      UK k = stage_k[j];
      unsigned d = (unsigned)(encode_key(k, coding) >> shift) & (RADIX_BINS - 1);
      dig[i] = (unsigned char)d;
      dst[s_goff[d] + j] = k;
    }
  }
  if constexpr (HAS_V) {
#pragma unroll
    for (int i = 0; i < IPT; ++i) stage_v[pos[i]] = val[i];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      unsigned j = threadIdx.x + i * ONESWEEP_BLOCK;
      if (j < tile_n) vdst[s_goff[dig[i]] + j] = stage_v[j];
    }
  }
}

// ---------------------------------------------------------------- 4. copy back after an odd number of passes
template <class UK, class UV, bool HAS_V>
__global__ void __launch_bounds__(256)
radix_copy_back_kernel(UK* buf_a, const UK* buf_b, UV* val_a, const UV* val_b, size_t n, int first_pass, int num_passes,
                       const radix_ctrl* ctrl) {
  int active = 0;
  for (int q = first_pass; q < first_pass + num_passes; ++q) active += ctrl->skip[q] ? 0 : 1;
  if (!(active & 1)) return;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    buf_a[i] = __ldcs(buf_b + i);
    if constexpr (HAS_V) val_a[i] = __ldcs(val_b + i);
  }
}

// ---------------------------------------------------------------- host side
template <int KB, int VB> constexpr int onesweep_tile_items() { return ONESWEEP_BLOCK * onesweep_tuning<KB, VB>::IPT; }

template <int KB, int VB> size_t onesweep_smem_bytes() {
  return (size_t)(ONESWEEP_BLOCK / 32) * RADIX_BINS * 4 + RADIX_BINS * 4 + 16 * 4 + (size_t)onesweep_tile_items<KB, VB>() * (KB + VB);
}

// scratch (not counting the alternate key/value buffers, which the caller provides)
template <int KB, int VB> size_t radix_workspace_bytes(size_t n) {
  size_t tiles = (n + onesweep_tile_items<KB, VB>() - 1) / onesweep_tile_items<KB, VB>();
  size_t lb_word = n < (1ull << 30) ? 4 : 8;
  return sizeof(ws_header) + sizeof(radix_ctrl) + align_up(tiles * RADIX_BINS * lb_word, 256) * KB;
}

// Sorts keys (and values) held in keys_a / vals_a, in place from the caller's point of view:
// keys_b / vals_b are same-sized alternate buffers.  Only bits [begin_bit, end_bit) of the key
// code take part; both must be multiples of 8.  n < 2^31.  No sync.
template <class UK, class UV, bool HAS_V>
cudaError_t radix_sort_async(UK* keys_a, UK* keys_b, UV* vals_a, UV* vals_b, size_t n, key_coding coding, int begin_bit,
                             int end_bit, void* ws, cudaStream_t stream) {
  constexpr int KB = sizeof(UK);
  constexpr int VB = HAS_V ? sizeof(UV) : 0;
  constexpr int IPT = onesweep_tuning<KB, VB>::IPT;
  if (n >= (1ull << 31) || begin_bit % RADIX_BITS || end_bit % RADIX_BITS || end_bit > 8 * KB || begin_bit > end_bit) return cudaErrorInvalidValue;
  if (n <= 1 || begin_bit == end_bit) return cudaMemsetAsync(ws, 0, sizeof(ws_header), stream);
  const int first_pass = begin_bit / RADIX_BITS, num_passes = (end_bit - begin_bit) / RADIX_BITS;
  const size_t tiles = (n + onesweep_tile_items<KB, VB>() - 1) / onesweep_tile_items<KB, VB>();
  const bool lb32 = n < (1ull << 30);
  const size_t lb_bytes = align_up(tiles * RADIX_BINS * (lb32 ? 4 : 8), 256);
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  radix_ctrl* ctrl = reinterpret_cast<radix_ctrl*>(base + sizeof(ws_header));
  char* lb0 = base + sizeof(ws_header) + sizeof(radix_ctrl);
  cudaError_t e = cudaMemsetAsync(base, 0, sizeof(ws_header) + sizeof(radix_ctrl) + lb_bytes * num_passes, stream);
  if (e != cudaSuccess) return e;

  const device_info& di = current_device_info();
  size_t hist_grid = (n + HIST_BLOCK * 4 - 1) / (HIST_BLOCK * 4);
  if (hist_grid > (size_t)di.sm_count * 4) hist_grid = (size_t)di.sm_count * 4;
  radix_hist_kernel<UK><<<(unsigned)hist_grid, HIST_BLOCK, 0, stream>>>(keys_a, n, coding, first_pass, num_passes, ctrl);
  radix_scan_hist_kernel<<<num_passes, RADIX_BINS, 0, stream>>>(ctrl, n, first_pass);

  const size_t smem = onesweep_smem_bytes<KB, VB>();
  auto k32 = onesweep_kernel<UK, UV, HAS_V, uint32_t, IPT>;
  auto k64 = onesweep_kernel<UK, UV, HAS_V, unsigned long long, IPT>;
  static thread_local bool attr_done[64] = {false};
  int dev = 0; cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    if ((e = cudaFuncSetAttribute(k32, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(k64, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  for (int p = 0; p < num_passes; ++p) {
    char* lb = lb0 + lb_bytes * p;
    if (lb32)
      k32<<<(unsigned)tiles, ONESWEEP_BLOCK, smem, stream>>>(keys_a, keys_b, vals_a, vals_b, (unsigned)n, coding, first_pass + p, first_pass, ctrl,
                                                            reinterpret_cast<uint32_t*>(lb), hdr);
    else
      k64<<<(unsigned)tiles, ONESWEEP_BLOCK, smem, stream>>>(keys_a, keys_b, vals_a, vals_b, (unsigned)n, coding, first_pass + p, first_pass, ctrl,
                                                            reinterpret_cast<unsigned long long*>(lb), hdr);
  }
  size_t cb_grid = (n + 256 * 8 - 1) / (256 * 8);
  if (cb_grid > (size_t)di.sm_count * 8) cb_grid = (size_t)di.sm_count * 8;
  radix_copy_back_kernel<UK, UV, HAS_V><<<(unsigned)cb_grid, 256, 0, stream>>>(keys_a, keys_b, vals_a, vals_b, n, first_pass, num_passes, ctrl);
  return cudaGetLastError();
}

}  // namespace tb200
