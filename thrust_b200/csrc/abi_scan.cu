// C ABI: tb200_inclusive_scan, tb200_exclusive_scan.
#include "abi_common.cuh"
#include "thrust_b200/scan.cuh"

using namespace tb200_abi;

namespace {
template <bool INCLUSIVE>
int scan_entry(const void* d_in, void* d_out, size_t n, int t, int op, const void* h_init, const void* d_init, void* d_ws, size_t* ws_bytes,
               cudaStream_t stream) {
  return by_wide_dtype(t, [&](auto tv) -> int {
    using T = decltype(tv);
    int rc;
    if (workspace_gate(d_ws, ws_bytes, tb200::scan_workspace_bytes<T>(n), rc)) return rc;
    if (n && (!d_in || !d_out)) return ERR_INVALID;
    T init = T();
    if (!INCLUSIVE && !h_init && !d_init) return ERR_INVALID;
    const bool has_init = h_init != nullptr;
    if (has_init) memcpy(&init, h_init, sizeof(T));
    return by_op(op, [&](auto o) {
      return (int)tb200::scan_async<INCLUSIVE>(static_cast<const T*>(d_in), static_cast<T*>(d_out), n, init, has_init, o, d_ws, stream,
                                               static_cast<const T*>(d_init));
    });
  });
}
}  // namespace

TB200_API int tb200_inclusive_scan(const void* d_in, void* d_out, size_t n, int t, int op, const void* h_init, void* d_ws, size_t* ws_bytes,
                                   tb200_stream_t stream) {
  return scan_entry<true>(d_in, d_out, n, t, op, h_init, nullptr, d_ws, ws_bytes, stream);
}
TB200_API int tb200_exclusive_scan(const void* d_in, void* d_out, size_t n, int t, int op, const void* h_init, void* d_ws, size_t* ws_bytes,
                                   tb200_stream_t stream) {
  return scan_entry<false>(d_in, d_out, n, t, op, h_init, nullptr, d_ws, ws_bytes, stream);
}
// the same with the initial value in device memory (read when the kernels run): the carry of a
// sharded scan never visits the host
TB200_API int tb200_inclusive_scan_dinit(const void* d_in, void* d_out, size_t n, int t, int op, const void* d_init, void* d_ws, size_t* ws_bytes,
                                         tb200_stream_t stream) {
  return scan_entry<true>(d_in, d_out, n, t, op, nullptr, d_init, d_ws, ws_bytes, stream);
}
TB200_API int tb200_exclusive_scan_dinit(const void* d_in, void* d_out, size_t n, int t, int op, const void* d_init, void* d_ws, size_t* ws_bytes,
                                         tb200_stream_t stream) {
  if (!d_init && d_ws) return ERR_INVALID;
  return scan_entry<false>(d_in, d_out, n, t, op, nullptr, d_init, d_ws, ws_bytes, stream);
}
