// C ABI: sharing device buffers between the one-process-per-GPU ranks of a multi-GPU job, so that a
// kernel on one GPU can read another GPU's buffer directly over NVLink (plain loads; no TMA).
#include "abi_common.cuh"

#include <cuda.h>
#include <map>
#include <mutex>
#include <string>

using namespace tb200_abi;

namespace {

struct opened { void* base; };
std::mutex g_lock;
std::map<std::string, opened> g_open;   // IPC handle bytes -> mapping in this process

// base address of the allocation that contains p (driver entry point fetched at run time, so the
// library carries no link-time dependency on libcuda)
cudaError_t allocation_base(const void* p, void** base) {
  using fn_t = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static fn_t fn = nullptr;
  if (!fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q);
    if (e != cudaSuccess) return e;
    if (!f || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
    fn = reinterpret_cast<fn_t>(f);
  }
  CUdeviceptr b = 0;
  size_t size = 0;
  if (fn(&b, &size, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS) return cudaErrorInvalidValue;
  *base = reinterpret_cast<void*>(b);
  return cudaSuccess;
}

}  // namespace

TB200_API int tb200_ipc_export(const void* d_ptr, void* h_handle64, size_t* h_offset) {
  if (!d_ptr || !h_handle64 || !h_offset) return ERR_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  void* base = nullptr;
  cudaError_t e = allocation_base(d_ptr, &base);
  if (e != cudaSuccess) return (int)e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, base);
  if (e != cudaSuccess) return (int)e;
  memcpy(h_handle64, &h, 64);
  *h_offset = (size_t)(static_cast<const char*>(d_ptr) - static_cast<const char*>(base));
  return 0;
}

TB200_API int tb200_ipc_open(const void* h_handle64, size_t offset, void** d_ptr_out) {
  if (!h_handle64 || !d_ptr_out) return ERR_INVALID;
  std::string key(static_cast<const char*>(h_handle64), 64);
  std::lock_guard<std::mutex> guard(g_lock);
  auto it = g_open.find(key);
  if (it == g_open.end()) {
    cudaIpcMemHandle_t h;
    memcpy(&h, h_handle64, 64);
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    it = g_open.emplace(key, opened{base}).first;
  }
  *d_ptr_out = static_cast<char*>(it->second.base) + offset;
  return 0;
}

TB200_API int tb200_ipc_close(const void* h_handle64) {
  if (!h_handle64) return ERR_INVALID;
  std::string key(static_cast<const char*>(h_handle64), 64);
  std::lock_guard<std::mutex> guard(g_lock);
  auto it = g_open.find(key);
  if (it == g_open.end()) return 0;                       // never opened here, or closed already
  cudaError_t e = cudaIpcCloseMemHandle(it->second.base);
  g_open.erase(it);
  return (int)e;
}

TB200_API int tb200_ipc_close_all(void) {
  std::lock_guard<std::mutex> guard(g_lock);
  int rc = 0;
  for (auto& kv : g_open) {
    cudaError_t e = cudaIpcCloseMemHandle(kv.second.base);
    if (e != cudaSuccess) rc = (int)e;
  }
  g_open.clear();
  return rc;
}
