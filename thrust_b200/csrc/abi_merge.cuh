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

// Stable merge of `num_runs` sorted runs (given in order; ties keep the earlier run first) by a
// pairwise tree that ping-pongs between `out` and `tmp`; the result always ends in `out`.
template <class K, class V, bool HAS_V>
int merge_runs_typed(const void* const* run_keys, const void* const* run_vals, const size_t* counts, int num_runs, void* out_k, void* out_v,
                     void* tmp_k, void* tmp_v, int descending, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  size_t total = 0;
  for (int i = 0; i < num_runs; ++i) total += counts[i];
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::merge_workspace_bytes<K, V, HAS_V>(total), rc)) return rc;
  if (num_runs <= 0 || num_runs > 64) return ERR_INVALID;
  if (total && (!out_k || !tmp_k || (HAS_V && (!out_v || !tmp_v)))) return ERR_INVALID;
  int levels = 0;
  for (int r = num_runs; r > 1; r = (r + 1) / 2) ++levels;
  const K* ck[64]; const V* cv[64]; size_t cn[64];
  for (int i = 0; i < num_runs; ++i) { ck[i] = static_cast<const K*>(run_keys[i]); cv[i] = HAS_V ? static_cast<const V*>(run_vals[i]) : nullptr; cn[i] = counts[i]; }
  int cur = num_runs;
  cudaError_t e = cudaMemsetAsync(d_ws, 0, sizeof(tb200::ws_header), stream);
  if (e != cudaSuccess) return (int)e;
  if (levels == 0) {   // a single run: copy it
    if (cn[0]) {
      if ((e = cudaMemcpyAsync(out_k, ck[0], cn[0] * sizeof(K), cudaMemcpyDefault, stream)) != cudaSuccess) return (int)e;
      if (HAS_V && (e = cudaMemcpyAsync(out_v, cv[0], cn[0] * sizeof(V), cudaMemcpyDefault, stream)) != cudaSuccess) return (int)e;
    }
    return 0;
  }
  constexpr int TILE = tb200::merge_tile_items<K, V, HAS_V>();
  for (int level = 1; level <= levels; ++level) {
    K* dk = static_cast<K*>(((levels - level) % 2 == 0) ? out_k : tmp_k);
    V* dv = static_cast<V*>(((levels - level) % 2 == 0) ? out_v : tmp_v);
    size_t off = 0;
    int next = 0;
    for (int i = 0; i < cur; i += 2) {
      if (i + 1 < cur) {
        const size_t na = cn[i], nb = cn[i + 1];
        if (na + nb) {
          if (descending)
            e = tb200::merge_pass_async<K, V, HAS_V>(ck[i], ck[i + 1], cv[i], cv[i + 1], dk + off, dv + (HAS_V ? off : 0), tb200::merge_geometry::single<TILE>(na, nb),
                                                   tb200::greater_op(), d_ws, stream);
          else
            e = tb200::merge_pass_async<K, V, HAS_V>(ck[i], ck[i + 1], cv[i], cv[i + 1], dk + off, dv + (HAS_V ? off : 0), tb200::merge_geometry::single<TILE>(na, nb),
                                                   tb200::less_op(), d_ws, stream);
          if (e != cudaSuccess) return (int)e;
        }
        ck[next] = dk + off; cv[next] = HAS_V ? dv + off : nullptr; cn[next] = na + nb;
        off += na + nb;
      } else {   // odd run out: carry it to this level's buffer so that the next level finds it there
        if (cn[i]) {
          if ((e = cudaMemcpyAsync(dk + off, ck[i], cn[i] * sizeof(K), cudaMemcpyDefault, stream)) != cudaSuccess) return (int)e;
          if (HAS_V && (e = cudaMemcpyAsync(dv + off, cv[i], cn[i] * sizeof(V), cudaMemcpyDefault, stream)) != cudaSuccess) return (int)e;
        }
        ck[next] = dk + off; cv[next] = HAS_V ? dv + off : nullptr; cn[next] = cn[i];
        off += cn[i];
      }
      ++next;
    }
    cur = next;
  }
  return 0;
}

template <class K>
int merge_runs_for_key(const void* const* run_keys, const void* const* run_vals, const size_t* counts, int num_runs, void* out_k, void* out_v, void* tmp_k,
                       void* tmp_v, int val_bytes, int descending, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  switch (val_bytes) {
    case 0: return merge_runs_typed<K, uint32_t, false>(run_keys, run_vals, counts, num_runs, out_k, out_v, tmp_k, tmp_v, descending, d_ws, ws_bytes, stream);
    case 4: return merge_runs_typed<K, uint32_t, true>(run_keys, run_vals, counts, num_runs, out_k, out_v, tmp_k, tmp_v, descending, d_ws, ws_bytes, stream);
    case 8: return merge_runs_typed<K, unsigned long long, true>(run_keys, run_vals, counts, num_runs, out_k, out_v, tmp_k, tmp_v, descending, d_ws, ws_bytes, stream);
  }
  return ERR_UNSUPPORTED;
}

#define TB200_MERGE_DECL(K) \
  extern template int merge_runs_for_key<K>(const void* const*, const void* const*, const size_t*, int, void*, void*, void*, void*, int, int, void*, size_t*, cudaStream_t); \
  extern template int merge_for_key<K>(const void*, const void*, size_t, const void*, const void*, size_t, void*, void*, int, int, void*, size_t*, cudaStream_t); \
  extern template int merge_sort_for_key<K>(void*, void*, void*, void*, size_t, int, int, void*, size_t*, cudaStream_t);
#define TB200_MERGE_INST(K) \
  template int merge_runs_for_key<K>(const void* const*, const void* const*, const size_t*, int, void*, void*, void*, void*, int, int, void*, size_t*, cudaStream_t); \
  template int merge_for_key<K>(const void*, const void*, size_t, const void*, const void*, size_t, void*, void*, int, int, void*, size_t*, cudaStream_t); \
  template int merge_sort_for_key<K>(void*, void*, void*, void*, size_t, int, int, void*, size_t*, cudaStream_t);

}  // namespace tb200_abi
