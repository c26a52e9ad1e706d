// C ABI: tb200_sequence_u32 and tb200_gather, the two helpers of the host-buffer sort_by_key, which
// sorts (key, position) pairs while the values are still on their way to the device and then permutes
// the values by the sorted positions.
#include "abi_common.cuh"

using namespace tb200_abi;

namespace {
constexpr int GATHER_BLOCK = 256;
constexpr int GATHER_IPT = 8;

__global__ void __launch_bounds__(GATHER_BLOCK) sequence_kernel(unsigned* out, size_t n) {
  const size_t stride = (size_t)gridDim.x * GATHER_BLOCK * 4;
  for (size_t i = ((size_t)blockIdx.x * GATHER_BLOCK + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      *reinterpret_cast<uint4*>(out + i) = make_uint4((unsigned)i, (unsigned)i + 1, (unsigned)i + 2, (unsigned)i + 3);
    } else {
      for (size_t j = i; j < n; ++j) out[j] = (unsigned)j;
    }
  }
}

// out[i] = src[idx[i]]: GATHER_IPT independent random reads in flight per thread, streaming index
// loads and result stores (both are touched once), plain loads for src (what reuse there is sits in L2)
template <class V>
__global__ void __launch_bounds__(GATHER_BLOCK) gather_kernel(const V* __restrict__ src, const unsigned* __restrict__ idx, V* __restrict__ out, size_t n) {
  const size_t tile = (size_t)GATHER_BLOCK * GATHER_IPT;
  for (size_t base = (size_t)blockIdx.x * tile; base < n; base += (size_t)gridDim.x * tile) {
    unsigned at[GATHER_IPT];
    V v[GATHER_IPT];
#pragma unroll
    for (int j = 0; j < GATHER_IPT; ++j) {
      const size_t i = base + threadIdx.x + (size_t)j * GATHER_BLOCK;
      at[j] = i < n ? __ldcs(idx + i) : 0u;
    }
#pragma unroll
    for (int j = 0; j < GATHER_IPT; ++j) {
      const size_t i = base + threadIdx.x + (size_t)j * GATHER_BLOCK;
      if (i < n) v[j] = src[at[j]];
    }
#pragma unroll
    for (int j = 0; j < GATHER_IPT; ++j) {
      const size_t i = base + threadIdx.x + (size_t)j * GATHER_BLOCK;
      if (i < n) __stcs(out + i, v[j]);
    }
  }
}

unsigned capped_grid(size_t want) {
  const size_t cap = (size_t)tb200::current_device_info().sm_count * 32;
  return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}
}  // namespace

TB200_API int tb200_sequence_u32(void* d_out, size_t n, tb200_stream_t stream) {
  if (n == 0) return 0;
  if (!d_out || n > 0xffffffffull || (reinterpret_cast<uintptr_t>(d_out) & 15)) return ERR_INVALID;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  sequence_kernel<<<capped_grid((n / 4 + GATHER_BLOCK) / GATHER_BLOCK), GATHER_BLOCK, 0, s>>>(static_cast<unsigned*>(d_out), n);
  return (int)cudaGetLastError();
}

TB200_API int tb200_gather(const void* d_src, const void* d_index_u32, void* d_out, size_t n, int val_bytes, tb200_stream_t stream) {
  if (n == 0) return 0;
  if (!d_src || !d_index_u32 || !d_out) return ERR_INVALID;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = capped_grid((n + GATHER_BLOCK * GATHER_IPT - 1) / (GATHER_BLOCK * GATHER_IPT));
  const unsigned* idx = static_cast<const unsigned*>(d_index_u32);
  switch (val_bytes) {
    case 4: gather_kernel<unsigned><<<grid, GATHER_BLOCK, 0, s>>>(static_cast<const unsigned*>(d_src), idx, static_cast<unsigned*>(d_out), n); break;
    case 8: gather_kernel<unsigned long long><<<grid, GATHER_BLOCK, 0, s>>>(static_cast<const unsigned long long*>(d_src), idx, static_cast<unsigned long long*>(d_out), n); break;
    default: return ERR_UNSUPPORTED;
  }
  return (int)cudaGetLastError();
}
