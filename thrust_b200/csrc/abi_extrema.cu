// C ABI: tb200_min_element, tb200_max_element, tb200_minmax_element.
#include "abi_common.cuh"
#include "thrust_b200/extrema.cuh"

using namespace tb200_abi;

namespace {

// which: bit 0 = the minimum is wanted, bit 1 = the maximum; d_index receives them in that order
int extrema_entry(const void* d_in, size_t n, int t, int which, unsigned long long* d_index, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  return by_dtype(t, [&](auto tv) -> int {
    using T = decltype(tv);
    int rc;
    // the pair of positions is produced in the workspace and the wanted ones copied out
    const size_t need = tb200::extrema_workspace_bytes<T>() + 256;
    if (workspace_gate(d_ws, ws_bytes, need, rc)) return rc;
    if ((n && !d_in) || !d_index) return ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long* both = reinterpret_cast<unsigned long long*>(static_cast<char*>(d_ws) + tb200::extrema_workspace_bytes<T>());
    cudaError_t e = tb200::extrema_async(static_cast<const T*>(d_in), n, T(), tb200::less_op(), both, d_ws, s);
    if (e != cudaSuccess) return (int)e;
    if (which == 3) return (int)cudaMemcpyAsync(d_index, both, 16, cudaMemcpyDeviceToDevice, s);
    return (int)cudaMemcpyAsync(d_index, both + (which == 2 ? 1 : 0), 8, cudaMemcpyDeviceToDevice, s);
  });
}

}  // namespace

TB200_API int tb200_min_element(const void* d_in, size_t n, int t, unsigned long long* d_index, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  return extrema_entry(d_in, n, t, 1, d_index, d_ws, ws_bytes, stream);
}

TB200_API int tb200_max_element(const void* d_in, size_t n, int t, unsigned long long* d_index, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  return extrema_entry(d_in, n, t, 2, d_index, d_ws, ws_bytes, stream);
}

TB200_API int tb200_minmax_element(const void* d_in, size_t n, int t, unsigned long long* d_index, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  return extrema_entry(d_in, n, t, 3, d_index, d_ws, ws_bytes, stream);
}
