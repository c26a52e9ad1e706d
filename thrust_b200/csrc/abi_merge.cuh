// merge / merge sort C-ABI plumbing, split by key type so the translation units compile in parallel.
#pragma once
#include "abi_common.cuh"
#include "thrust_b200/merge.cuh"

namespace tb200_abi {

template <class K, class V, bool HAS_V>
int merge_typed(const void* ka, const void* va, size_t na, const void* kb, const void* vb, size_t nb, void* ko, void* vo, int descending,
                void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::merge_workspace_bytes<K, V, HAS_V>(na + nb), rc)) return rc;
  if ((na && !ka) || (nb && !kb) || ((na + nb) && !ko)) return ERR_INVALID;
  if (HAS_V && (((na && !va) || (nb && !vb)) || ((na + nb) && !vo))) return ERR_INVALID;
  const K* a = static_cast<const K*>(ka); const K* b = static_cast<const K*>(kb);
  const V* pa = static_cast<const V*>(va); const V* pb = static_cast<const V*>(vb);
  if (descending)
    return (int)tb200::merge_async<K, V, HAS_V>(a, na, b, nb, pa, pb, static_cast<K*>(ko), static_cast<V*>(vo), tb200::greater_op(), d_ws, stream);
  return (int)tb200::merge_async<K, V, HAS_V>(a, na, b, nb, pa, pb, static_cast<K*>(ko), static_cast<V*>(vo), tb200::less_op(), d_ws, stream);
}

template <class K>
int merge_for_key(const void* ka, const void* va, size_t na, const void* kb, const void* vb, size_t nb, void* ko, void* vo, int val_bytes,
                  int descending, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  switch (val_bytes) {
    case 0: return merge_typed<K, uint32_t, false>(ka, va, na, kb, vb, nb, ko, vo, descending, d_ws, ws_bytes, stream);
    case 4: return merge_typed<K, uint32_t, true>(ka, va, na, kb, vb, nb, ko, vo, descending, d_ws, ws_bytes, stream);
    case 8: return merge_typed<K, unsigned long long, true>(ka, va, na, kb, vb, nb, ko, vo, descending, d_ws, ws_bytes, stream);
  }
  return ERR_UNSUPPORTED;
}

template <class K, class V, bool HAS_V>
int merge_sort_typed(void* k, void* ka, void* v, void* va, size_t n, int descending, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::merge_sort_workspace_bytes<K, V, HAS_V>(n), rc)) return rc;
  if (n > 1 && (!k || !ka || (HAS_V && (!v || !va)))) return ERR_INVALID;
  if (descending)
    return (int)tb200::merge_sort_async<K, V, HAS_V>(static_cast<K*>(k), static_cast<K*>(ka), static_cast<V*>(v), static_cast<V*>(va), n, tb200::greater_op(), d_ws, stream);
  return (int)tb200::merge_sort_async<K, V, HAS_V>(static_cast<K*>(k), static_cast<K*>(ka), static_cast<V*>(v), static_cast<V*>(va), n, tb200::less_op(), d_ws, stream);
}

template <class K>
int merge_sort_for_key(void* k, void* ka, void* v, void* va, size_t n, int val_bytes, int descending, void* d_ws, size_t* ws_bytes,
                       cudaStream_t stream) {
  switch (val_bytes) {
    case 0: return merge_sort_typed<K, uint32_t, false>(k, ka, v, va, n, descending, d_ws, ws_bytes, stream);
    case 4: return merge_sort_typed<K, uint32_t, true>(k, ka, v, va, n, descending, d_ws, ws_bytes, stream);
    case 8: return merge_sort_typed<K, unsigned long long, true>(k, ka, v, va, n, descending, d_ws, ws_bytes, stream);
  }
  return ERR_UNSUPPORTED;
}

#define TB200_MERGE_DECL(K) \
  extern template int merge_for_key<K>(const void*, const void*, size_t, const void*, const void*, size_t, void*, void*, int, int, void*, size_t*, cudaStream_t); \
  extern template int merge_sort_for_key<K>(void*, void*, void*, void*, size_t, int, int, void*, size_t*, cudaStream_t);
#define TB200_MERGE_INST(K) \
  template int merge_for_key<K>(const void*, const void*, size_t, const void*, const void*, size_t, void*, void*, int, int, void*, size_t*, cudaStream_t); \
  template int merge_sort_for_key<K>(void*, void*, void*, void*, size_t, int, int, void*, size_t*, cudaStream_t);

}  // namespace tb200_abi
