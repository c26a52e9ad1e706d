// C ABI: tb200_partition (in place, stable), tb200_unique_copy.
#include "abi_common.cuh"
#include "thrust_b200/select.cuh"

using namespace tb200_abi;
using tb200::abi_pred;

TB200_API int tb200_partition(void* d_data, size_t n, int t, int pred, long long a, long long b, unsigned long long* d_count, void* d_ws,
                              size_t* ws_bytes, tb200_stream_t stream) {
  if (pred < 0 || pred > 3) return ERR_UNSUPPORTED;
  if (pred == TB200_PRED_MOD_EQ && a == 0) return ERR_INVALID;
  return by_dtype(t, [&](auto tv) -> int {
    using T = decltype(tv);
    const size_t sel = tb200::align_up(tb200::select_workspace_bytes<T>(n), 256);
    int rc;
    if (workspace_gate(d_ws, ws_bytes, sel + tb200::align_up(n * sizeof(T), 256), rc)) return rc;
    if (n && !d_data) return ERR_INVALID;
    T* scratch = reinterpret_cast<T*>(static_cast<char*>(d_ws) + sel);
    abi_pred p = abi_pred::make(pred, a, b);
    // large inputs: the streaming kernels, compiled per predicate kind
    if constexpr (sizeof(T) == 4 || sizeof(T) == 8) {
      if (tb200::select_stream_eligible(d_data, scratch, nullptr, false, n, sizeof(T)))
        return p.visit([&](auto typed) { return (int)tb200::partition_inplace_stream_async(static_cast<T*>(d_data), scratch, n, typed, d_count, d_ws, stream); });
    }
    return (int)tb200::partition_inplace_async<false>(static_cast<T*>(d_data), scratch, n, p, d_count, d_ws, stream);
  });
}

TB200_API int tb200_unique_copy(const void* d_in, void* d_out, size_t n, int t, unsigned long long* d_count, void* d_ws, size_t* ws_bytes,
                                tb200_stream_t stream) {
  return by_dtype(t, [&](auto tv) -> int {
    using T = decltype(tv);
    int rc;
    if (workspace_gate(d_ws, ws_bytes, tb200::select_workspace_bytes<T>(n), rc)) return rc;
    if (n && (!d_in || !d_out)) return ERR_INVALID;
    return (int)tb200::select_async<tb200::SEL_UNIQUE, false>(static_cast<const T*>(d_in), (const T*)nullptr, static_cast<T*>(d_out), (T*)nullptr, n,
                                                              T(), tb200::equal_op(), false, d_count, d_ws, stream);
  });
}
