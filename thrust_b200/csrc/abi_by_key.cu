// C ABI: tb200_scan_by_key, tb200_unique_by_key_copy.
#include "abi_rbk.cuh"
#include "thrust_b200/scan_by_key.cuh"

using namespace tb200_abi;

TB200_API int tb200_scan_by_key(const void* d_keys, const void* d_vals, void* d_out, size_t n, int key_t, int val_t, int op, int exclusive,
                                const void* h_init, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  return by_key_class(key_t, [&](auto kv) -> int {
    using K = decltype(kv);
    return by_wide_dtype(val_t, [&](auto vv) -> int {
      using V = decltype(vv);
      int rc;
      if (workspace_gate(d_ws, ws_bytes, tb200::scan_by_key_workspace_bytes<K, V>(n), rc)) return rc;
      if (n && (!d_keys || !d_vals || !d_out)) return ERR_INVALID;
      if (exclusive && !h_init) return ERR_INVALID;
      V init = V();
      if (exclusive) memcpy(&init, h_init, sizeof(V));
      return by_op(op, [&](auto o) {
        if (exclusive)
          return (int)tb200::scan_by_key_async<false>(static_cast<const K*>(d_keys), static_cast<const V*>(d_vals), static_cast<V*>(d_out), n, K(), init,
                                                      tb200::equal_op(), o, d_ws, stream);
        return (int)tb200::scan_by_key_async<true>(static_cast<const K*>(d_keys), static_cast<const V*>(d_vals), static_cast<V*>(d_out), n, K(), init,
                                                   tb200::equal_op(), o, d_ws, stream);
      });
    });
  });
}

// unique_by_key_copy = reduce_by_key whose reduction keeps the first value of every run
TB200_API int tb200_unique_by_key_copy(const void* d_keys, const void* d_vals, void* d_keys_out, void* d_vals_out, size_t n, int key_t, int val_bytes,
                                       unsigned long long* d_count, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  return by_key_class(key_t, [&](auto kv) -> int {
    using K = decltype(kv);
    auto run = [&](auto vv) -> int {
      using V = decltype(vv);
      int rc;
      if (workspace_gate(d_ws, ws_bytes, tb200::rbk_workspace_bytes<K, V>(n), rc)) return rc;
      if (n && (!d_keys || !d_vals || !d_keys_out || !d_vals_out)) return ERR_INVALID;
      return (int)tb200::reduce_by_key_async<false>(static_cast<const K*>(d_keys), static_cast<const V*>(d_vals), static_cast<K*>(d_keys_out),
                                                    static_cast<V*>(d_vals_out), n, K(), V(), tb200::equal_op(), tb200::first_op(), d_count, d_ws, stream);
    };
    switch (val_bytes) {
      case 4: return run((uint32_t)0);
      case 8: return run((unsigned long long)0);
    }
    return ERR_UNSUPPORTED;
  });
}
