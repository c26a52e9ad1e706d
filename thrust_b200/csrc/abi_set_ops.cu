// C ABI: tb200_set_operation (set_union, set_intersection, set_difference, set_symmetric_difference, ± values).
#include "abi_common.cuh"
#include "thrust_b200/set_ops.cuh"

using namespace tb200_abi;

namespace {
template <class K, class V, bool HAS_V>
int set_typed(int op, const void* ka, size_t na, const void* kb, size_t nb, const void* va, const void* vb, void* ko, void* vo, int descending,
              unsigned long long* d_count, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::set_op_workspace_bytes(na, nb), rc)) return rc;
  const size_t cap = op == tb200::SET_INTERSECTION ? (na < nb ? na : nb) : (op == tb200::SET_DIFFERENCE ? na : na + nb);   // the result's largest size
  if ((na && !ka) || (nb && !kb) || (cap && !ko) || (HAS_V && cap && (!vo || (na && !va)))) return ERR_INVALID;
  const K* a = static_cast<const K*>(ka); const K* b = static_cast<const K*>(kb);
  const V* x = static_cast<const V*>(va); const V* y = static_cast<const V*>(vb ? vb : va);
  if (descending)
    return (int)tb200::set_operation_async<K, HAS_V>(op, a, na, b, nb, x, y, static_cast<K*>(ko), static_cast<V*>(vo), tb200::greater_op(), d_count, d_ws, stream);
  return (int)tb200::set_operation_async<K, HAS_V>(op, a, na, b, nb, x, y, static_cast<K*>(ko), static_cast<V*>(vo), tb200::less_op(), d_count, d_ws, stream);
}
}  // namespace

TB200_API int tb200_set_operation(int op, const void* d_keys_a, size_t na, const void* d_keys_b, size_t nb, const void* d_vals_a, const void* d_vals_b,
                                  void* d_keys_out, void* d_vals_out, int key_t, int val_bytes, int descending, unsigned long long* d_count,
                                  void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  if (op < 0 || op > 3) return ERR_INVALID;
  return by_wide_dtype(key_t, [&](auto kv) -> int {
    using K = decltype(kv);
    switch (val_bytes) {
      case 0: return set_typed<K, uint32_t, false>(op, d_keys_a, na, d_keys_b, nb, nullptr, nullptr, d_keys_out, nullptr, descending, d_count, d_ws, ws_bytes, stream);
      case 4: return set_typed<K, uint32_t, true>(op, d_keys_a, na, d_keys_b, nb, d_vals_a, d_vals_b, d_keys_out, d_vals_out, descending, d_count, d_ws, ws_bytes, stream);
      case 8: return set_typed<K, unsigned long long, true>(op, d_keys_a, na, d_keys_b, nb, d_vals_a, d_vals_b, d_keys_out, d_vals_out, descending, d_count, d_ws, ws_bytes, stream);
    }
    return ERR_UNSUPPORTED;
  });
}
