// C ABI: kernel timing switch and read-out, tb200_lower_bound.
#include "abi_common.cuh"

using namespace tb200_abi;

TB200_API int tb200_kernel_timing(int enable) {
  tb200::kernel_timer& t = tb200::global_kernel_timer();
  std::lock_guard<std::mutex> guard(t.lock);
  t.enabled = enable != 0;
  t.used = 0;
  return 0;
}

TB200_API int tb200_kernel_timing_read(int capacity, int* h_kernel_ids, float* h_ms, int* h_count) {
  if (!h_kernel_ids || !h_ms || !h_count || capacity < 0) return ERR_INVALID;
  tb200::kernel_timer& t = tb200::global_kernel_timer();
  std::lock_guard<std::mutex> guard(t.lock);
  int n = t.used < capacity ? t.used : capacity;
  for (int i = 0; i < n; ++i) {
    cudaError_t e = cudaEventSynchronize(t.stop[i]);
    if (e != cudaSuccess) return (int)e;
    float ms = 0.f;
    e = cudaEventElapsedTime(&ms, t.start[i], t.stop[i]);
    if (e != cudaSuccess) return (int)e;
    h_kernel_ids[i] = t.ids[i];
    h_ms[i] = ms;
  }
  *h_count = n;
  t.used = 0;
  return 0;
}

namespace {
// out[j] = number of elements of sorted[0, n) that order strictly before needle[j]
template <class K, class Comp>
__global__ void lower_bound_kernel(const K* sorted, size_t n, const K* needles, size_t m, unsigned long long* out, Comp comp) {
  size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= m) return;
  const K x = needles[j];
  size_t lo = 0, hi = n;
  while (lo < hi) { size_t mid = (lo + hi) >> 1; if (comp(sorted[mid], x)) lo = mid + 1; else hi = mid; }
  out[j] = lo;
}
}  // namespace

TB200_API int tb200_lower_bound(const void* d_sorted, size_t n, const void* d_needles, size_t m, unsigned long long* d_out, int key_t,
                                int descending, tb200_stream_t stream) {
  if (m == 0) return 0;
  if (!d_needles || !d_out || (n && !d_sorted)) return ERR_INVALID;
  return by_wide_dtype(key_t, [&](auto kv) -> int {
    using K = decltype(kv);
    const unsigned grid = (unsigned)((m + 127) / 128);
    if (descending)
      lower_bound_kernel<K><<<grid, 128, 0, stream>>>(static_cast<const K*>(d_sorted), n, static_cast<const K*>(d_needles), m, d_out, tb200::greater_op());
    else
      lower_bound_kernel<K><<<grid, 128, 0, stream>>>(static_cast<const K*>(d_sorted), n, static_cast<const K*>(d_needles), m, d_out, tb200::less_op());
    return (int)cudaGetLastError();
  });
}

#ifdef TB200_TEST_HOOKS
// Exported by the test build only (thrust_b200.build.build_shortwait): see test_hook_flags().
TB200_API int tb200_test_hooks(unsigned flags) { tb200::test_hook_flags() = flags; return 0; }
#endif
