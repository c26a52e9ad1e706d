// C ABI: tb200_inclusive_scan_static -- the inclusive scan for callers that cannot allocate.
//
// Every other entry point takes its scratch memory from the caller, which presumes the caller
// can obtain device memory.  Some cannot: code running inside a memory-pool callback or a
// real-time loop where cudaMalloc's implicit device synchronisation is forbidden, a plug-in
// sandbox that is handed input and output buffers but no allocator, a host whose device memory
// is fully committed to its own data.  For them this one entry point carries its own scratch: a
// fixed array in the library's device data segment, present on every GPU that loads the library
// from the moment it is loaded until the process exits.
#include <atomic>

#include "abi_common.cuh"
#include "thrust_b200/scan.cuh"

using namespace tb200_abi;

namespace {

// 512 KiB: the descriptors of up to 536,600,576 four-byte or 134,148,096 eight-byte elements (the
// exact figure follows the kernels' tile sizes; tb200_inclusive_scan_static_limit reports it).
constexpr size_t STATIC_SCRATCH_BYTES = 512 * 1024;
static __device__ __align__(256) unsigned char g_scan_scratch[STATIC_SCRATCH_BYTES];

// In host code the name g_scan_scratch is only a handle for the runtime, not a device address, so
// the address is looked up once per device (with that device current) and remembered.
// (Threads that race on a device's first call each look the address up and store the same value.)
void* scratch_address(cudaError_t& err) {
  static std::atomic<void*> per_device[64];
  int dev = 0;
  err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) { err = cudaErrorInvalidDevice; return nullptr; }
  void* p = per_device[dev].load(std::memory_order_acquire);
  if (!p) {
    err = cudaGetSymbolAddress(&p, g_scan_scratch);
    if (err != cudaSuccess) return nullptr;
    per_device[dev].store(p, std::memory_order_release);
  }
  return p;
}

template <class T> size_t largest_n() {
  size_t lo = 0, hi = (size_t)1 << 40;   // scan_workspace_bytes grows with n
  while (lo < hi) {
    const size_t mid = lo + (hi - lo + 1) / 2;
    if (tb200::scan_workspace_bytes<T>(mid) <= STATIC_SCRATCH_BYTES) lo = mid; else hi = mid - 1;
  }
  return lo;
}

}  // namespace

TB200_API int tb200_inclusive_scan_static(const void* d_in, void* d_out, size_t n, int t, int op, const void* h_init, tb200_stream_t stream) {
  return by_wide_dtype(t, [&](auto tv) -> int {
    using T = decltype(tv);
    if (tb200::scan_workspace_bytes<T>(n) > STATIC_SCRATCH_BYTES) return TB200_ERR_EXCEEDS_STATIC_SCRATCH;
    if (n && (!d_in || !d_out)) return ERR_INVALID;
    cudaError_t err = cudaSuccess;
    void* ws = scratch_address(err);
    if (!ws) return (int)err;
    T init = T();
    const bool has_init = h_init != nullptr;
    if (has_init) memcpy(&init, h_init, sizeof(T));
    // scan_async clears the part of the scratch it is about to use, so what an earlier call left
    // behind is never read
    return by_op(op, [&](auto o) {
      return (int)tb200::scan_async<true>(static_cast<const T*>(d_in), static_cast<T*>(d_out), n, init, has_init, o, ws, stream);
    });
  });
}

TB200_API int tb200_inclusive_scan_static_limit(int t, size_t* h_max_n) {
  if (!h_max_n) return ERR_INVALID;
  return by_wide_dtype(t, [&](auto tv) -> int {
    *h_max_n = largest_n<decltype(tv)>();
    return 0;
  });
}

TB200_API int tb200_inclusive_scan_static_status(tb200_stream_t stream, unsigned* h_status) {
  if (!h_status) return ERR_INVALID;
  cudaError_t err = cudaSuccess;
  void* ws = scratch_address(err);
  if (!ws) return (int)err;
  // the array begins with the same header as a caller's workspace: its first word is the status
  err = cudaMemcpyAsync(h_status, ws, sizeof(unsigned), cudaMemcpyDeviceToHost, stream);
  if (err != cudaSuccess) return (int)err;
  return (int)cudaStreamSynchronize(stream);
}
