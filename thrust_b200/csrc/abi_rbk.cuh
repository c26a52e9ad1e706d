// reduce_by_key C-ABI plumbing, split by value type so the translation units compile in parallel.
#pragma once
#include "abi_common.cuh"
#include "thrust_b200/reduce_by_key.cuh"

namespace tb200_abi {

// Integer keys are compared by their bits, so one instantiation per key width serves both
// signednesses; floating-point keys keep IEEE equality (-0.0 == +0.0, NaN != NaN).
template <class F> int by_key_class(int t, F f) {
  switch (t) {
    case TB200_I8: case TB200_U8: return f((uint8_t)0);
    case TB200_I16: case TB200_U16: return f((uint16_t)0);
    case TB200_I32: case TB200_U32: return f((uint32_t)0);
    case TB200_I64: case TB200_U64: return f((unsigned long long)0);
    case TB200_F32: return f((float)0);
    case TB200_F64: return f((double)0);
  }
  return ERR_UNSUPPORTED;
}

template <class V>
int rbk_for_value(const void* d_keys, const void* d_vals, void* d_keys_out, void* d_vals_out, size_t n, int key_t, int op,
                  unsigned long long* d_count, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  return by_key_class(key_t, [&](auto kv) -> int {
    using K = decltype(kv);
    int rc;
    if (workspace_gate(d_ws, ws_bytes, tb200::rbk_workspace_bytes<K, V>(n), rc)) return rc;
    if (n && (!d_keys || !d_vals || !d_keys_out || !d_vals_out)) return ERR_INVALID;
    return by_op(op, [&](auto o) {
      return (int)tb200::reduce_by_key_async<false>(static_cast<const K*>(d_keys), static_cast<const V*>(d_vals), static_cast<K*>(d_keys_out),
                                                    static_cast<V*>(d_vals_out), n, K(), V(), tb200::equal_op(), o, d_count, d_ws, stream);
    });
  });
}

#define TB200_RBK_DECL(V) \
  extern template int rbk_for_value<V>(const void*, const void*, void*, void*, size_t, int, int, unsigned long long*, void*, size_t*, cudaStream_t);
#define TB200_RBK_INST(V) \
  template int rbk_for_value<V>(const void*, const void*, void*, void*, size_t, int, int, unsigned long long*, void*, size_t*, cudaStream_t);

}  // namespace tb200_abi
