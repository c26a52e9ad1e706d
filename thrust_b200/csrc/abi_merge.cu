// C ABI: tb200_merge_by_key, tb200_merge_sort_by_key, tb200_stable_sort_pairs_by_first (entry
// points; per-key-type bodies live in abi_merge_*.cu).
#include "abi_merge.cuh"

namespace tb200_abi {
TB200_MERGE_DECL(int32_t) TB200_MERGE_DECL(uint32_t) TB200_MERGE_DECL(long long) TB200_MERGE_DECL(unsigned long long) TB200_MERGE_DECL(float) TB200_MERGE_DECL(double)
}
using namespace tb200_abi;

TB200_API int tb200_merge_by_key(const void* d_keys_a, const void* d_vals_a, size_t na, const void* d_keys_b, const void* d_vals_b, size_t nb,
                                 void* d_keys_out, void* d_vals_out, int key_t, int val_bytes, int descending, void* d_ws, size_t* ws_bytes,
                                 tb200_stream_t stream) {
#define ARGS d_keys_a, d_vals_a, na, d_keys_b, d_vals_b, nb, d_keys_out, d_vals_out, val_bytes, descending, d_ws, ws_bytes, stream
  switch (key_t) {
    case TB200_I32: return merge_for_key<int32_t>(ARGS);
    case TB200_U32: return merge_for_key<uint32_t>(ARGS);
    case TB200_I64: return merge_for_key<long long>(ARGS);
    case TB200_U64: return merge_for_key<unsigned long long>(ARGS);
    case TB200_F32: return merge_for_key<float>(ARGS);
    case TB200_F64: return merge_for_key<double>(ARGS);
  }
#undef ARGS
  return ERR_UNSUPPORTED;
}

TB200_API int tb200_merge_sort_by_key(void* d_keys, void* d_keys_alt, void* d_vals, void* d_vals_alt, size_t n, int key_t, int val_bytes,
                                      int descending, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
#define ARGS d_keys, d_keys_alt, d_vals, d_vals_alt, n, val_bytes, descending, d_ws, ws_bytes, stream
  switch (key_t) {
    case TB200_I32: return merge_sort_for_key<int32_t>(ARGS);
    case TB200_U32: return merge_sort_for_key<uint32_t>(ARGS);
    case TB200_I64: return merge_sort_for_key<long long>(ARGS);
    case TB200_U64: return merge_sort_for_key<unsigned long long>(ARGS);
    case TB200_F32: return merge_sort_for_key<float>(ARGS);
    case TB200_F64: return merge_sort_for_key<double>(ARGS);
  }
#undef ARGS
  return ERR_UNSUPPORTED;
}

TB200_API int tb200_merge_runs(const void* const* h_run_keys, const void* const* h_run_vals, const size_t* h_counts, int num_runs, void* d_keys_out,
                               void* d_vals_out, void* d_keys_tmp, void* d_vals_tmp, int key_t, int val_bytes, int descending, void* d_ws,
                               size_t* ws_bytes, tb200_stream_t stream) {
  if (!h_run_keys || !h_counts || (val_bytes && !h_run_vals)) return ERR_INVALID;
#define ARGS h_run_keys, h_run_vals, h_counts, num_runs, d_keys_out, d_vals_out, d_keys_tmp, d_vals_tmp, val_bytes, descending, d_ws, ws_bytes, stream
  switch (key_t) {
    case TB200_I32: return merge_runs_for_key<int32_t>(ARGS);
    case TB200_U32: return merge_runs_for_key<uint32_t>(ARGS);
    case TB200_I64: return merge_runs_for_key<long long>(ARGS);
    case TB200_U64: return merge_runs_for_key<unsigned long long>(ARGS);
    case TB200_F32: return merge_runs_for_key<float>(ARGS);
    case TB200_F64: return merge_runs_for_key<double>(ARGS);
  }
#undef ARGS
  return ERR_UNSUPPORTED;
}
