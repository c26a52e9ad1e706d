// C ABI: tb200_bucket_count, tb200_bucket_scatter -- the exchange step of the multi-GPU sort.
#include <cstddef>

#include "abi_common.cuh"
#include "thrust_b200/radix_sort.cuh"

using namespace tb200_abi;

namespace {
bool coding_of(int key_t, int descending, tb200::key_coding& c) {
  c.descending = descending ? 1 : 0;
  switch (key_t) {
    case TB200_U32: case TB200_U64: c.kind = tb200::KEY_UNSIGNED; return true;
    case TB200_I32: case TB200_I64: c.kind = tb200::KEY_SIGNED; return true;
    case TB200_F32: case TB200_F64: c.kind = tb200::KEY_FLOAT; return true;
  }
  return false;
}

template <class UK, class UV, bool HAS_V>
int scatter_typed(const void* k, const void* v, size_t n, tb200::key_coding coding, const void* d_splitters, int buckets, void* const* h_dst_k,
                  void* const* h_dst_v, const unsigned long long* h_base, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::bucket_scatter_workspace_bytes<sizeof(UK), HAS_V ? sizeof(UV) : 0>(n), rc)) return rc;
  if (!h_dst_k || !h_base || (HAS_V && !h_dst_v) || (n && (!k || (HAS_V && !v))) || (buckets > 1 && !d_splitters)) return ERR_INVALID;
  tb200::bucket_table<UK, UV> table;
  for (int b = 0; b < tb200::MAX_BUCKETS; ++b) {
    table.dst_k[b] = b < buckets ? static_cast<UK*>(h_dst_k[b]) : nullptr;
    table.dst_v[b] = (HAS_V && b < buckets) ? static_cast<UV*>(h_dst_v[b]) : nullptr;
    table.base[b] = b < buckets ? h_base[b] : 0ull;
  }
  return (int)tb200::bucket_scatter_async<UK, UV, HAS_V>(static_cast<const UK*>(k), static_cast<const UV*>(v), n, coding,
                                                         static_cast<const UK*>(d_splitters), buckets, table, d_ws, stream);
}

template <class UK>
int scatter_by_val(const void* k, const void* v, size_t n, int val_bytes, tb200::key_coding coding, const void* d_splitters, int buckets,
                   void* const* h_dst_k, void* const* h_dst_v, const unsigned long long* h_base, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  switch (val_bytes) {
    case 0: return scatter_typed<UK, uint32_t, false>(k, v, n, coding, d_splitters, buckets, h_dst_k, h_dst_v, h_base, d_ws, ws_bytes, stream);
    case 4: return scatter_typed<UK, uint32_t, true>(k, v, n, coding, d_splitters, buckets, h_dst_k, h_dst_v, h_base, d_ws, ws_bytes, stream);
    case 8: return scatter_typed<UK, unsigned long long, true>(k, v, n, coding, d_splitters, buckets, h_dst_k, h_dst_v, h_base, d_ws, ws_bytes, stream);
  }
  return ERR_UNSUPPORTED;
}
}  // namespace

TB200_API int tb200_bucket_count(const void* d_keys, size_t n, int key_t, int descending, const void* d_splitters, int num_buckets,
                                 unsigned long long* d_counts, tb200_stream_t stream) {
  tb200::key_coding coding;
  if (!coding_of(key_t, descending, coding)) return ERR_UNSUPPORTED;
  if (!d_counts || (n && !d_keys) || (num_buckets > 1 && !d_splitters)) return ERR_INVALID;
  if (dtype_size(key_t) == 4)
    return (int)tb200::bucket_count_async(static_cast<const uint32_t*>(d_keys), n, coding, static_cast<const uint32_t*>(d_splitters), num_buckets, d_counts, stream);
  return (int)tb200::bucket_count_async(static_cast<const unsigned long long*>(d_keys), n, coding, static_cast<const unsigned long long*>(d_splitters),
                                        num_buckets, d_counts, stream);
}

TB200_API int tb200_bucket_scatter(const void* d_keys, const void* d_vals, size_t n, int key_t, int val_bytes, int descending, const void* d_splitters,
                                   int num_buckets, void* const* h_dst_keys, void* const* h_dst_vals, const unsigned long long* h_dst_offsets,
                                   void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  tb200::key_coding coding;
  if (!coding_of(key_t, descending, coding)) return ERR_UNSUPPORTED;
  if (dtype_size(key_t) == 4)
    return scatter_by_val<uint32_t>(d_keys, d_vals, n, val_bytes, coding, d_splitters, num_buckets, h_dst_keys, h_dst_vals, h_dst_offsets, d_ws, ws_bytes, stream);
  return scatter_by_val<unsigned long long>(d_keys, d_vals, n, val_bytes, coding, d_splitters, num_buckets, h_dst_keys, h_dst_vals, h_dst_offsets, d_ws, ws_bytes,
                                            stream);
}

// ---- splitters from a digit histogram (tb200_exchange_*)
namespace {
template <class UK, class UV, bool HAS_V>
int exchange_scatter_typed(const void* k, const void* v, size_t n, tb200::key_coding coding, const void* d_plan, int ranks, void* const* h_dst_k,
                           void* const* h_dst_v, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::bucket_scatter_workspace_bytes<sizeof(UK), HAS_V ? sizeof(UV) : 0>(n), rc)) return rc;
  if (!d_plan || !h_dst_k || (HAS_V && !h_dst_v) || (n && (!k || (HAS_V && !v))) || ranks < 1 || ranks > tb200::MAX_BUCKETS) return ERR_INVALID;
  tb200::bucket_table<UK, UV> table;
  for (int b = 0; b < tb200::MAX_BUCKETS; ++b) {
    table.dst_k[b] = b < ranks ? static_cast<UK*>(h_dst_k[b]) : nullptr;
    table.dst_v[b] = (HAS_V && b < ranks) ? static_cast<UV*>(h_dst_v[b]) : nullptr;
    table.base[b] = 0ull;
  }
  return (int)tb200::exchange_scatter_async<UK, UV, HAS_V>(static_cast<const UK*>(k), static_cast<const UV*>(v), n, coding,
                                                           static_cast<const tb200::exchange_plan*>(d_plan), table, d_ws, stream);
}
template <class UK>
int exchange_scatter_by_val(const void* k, const void* v, size_t n, int val_bytes, tb200::key_coding coding, const void* d_plan, int ranks,
                            void* const* h_dst_k, void* const* h_dst_v, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  switch (val_bytes) {
    case 0: return exchange_scatter_typed<UK, uint32_t, false>(k, v, n, coding, d_plan, ranks, h_dst_k, h_dst_v, d_ws, ws_bytes, stream);
    case 4: return exchange_scatter_typed<UK, uint32_t, true>(k, v, n, coding, d_plan, ranks, h_dst_k, h_dst_v, d_ws, ws_bytes, stream);
    case 8: return exchange_scatter_typed<UK, unsigned long long, true>(k, v, n, coding, d_plan, ranks, h_dst_k, h_dst_v, d_ws, ws_bytes, stream);
  }
  return ERR_UNSUPPORTED;
}
}  // namespace

TB200_API int tb200_exchange_sizes(int key_t, size_t* h_row_words, size_t* h_plan_bytes, size_t* h_plan_head_bytes) {
  if (!h_row_words || !h_plan_bytes || !h_plan_head_bytes) return ERR_INVALID;
  const size_t kb = dtype_size(key_t);
  if (kb != 4 && kb != 8) return ERR_UNSUPPORTED;
  *h_row_words = tb200::exch_row_words(kb == 8 ? tb200::exch_fields<unsigned long long>() : tb200::exch_fields<uint32_t>());
  *h_plan_bytes = sizeof(tb200::exchange_plan);
  *h_plan_head_bytes = offsetof(tb200::exchange_plan, lut);
  return 0;
}

TB200_API int tb200_exchange_hist(const void* d_keys, size_t n, int key_t, int descending, unsigned long long tag, unsigned* d_row,
                                  tb200_stream_t stream) {
  tb200::key_coding coding;
  if (!coding_of(key_t, descending, coding)) return ERR_UNSUPPORTED;
  if (!d_row || (n && !d_keys)) return ERR_INVALID;
  if (dtype_size(key_t) == 4) return (int)tb200::exchange_hist_async(static_cast<const uint32_t*>(d_keys), n, coding, tag, d_row, stream);
  return (int)tb200::exchange_hist_async(static_cast<const unsigned long long*>(d_keys), n, coding, tag, d_row, stream);
}

TB200_API int tb200_exchange_plan(const unsigned* d_rows, int ranks, int rank, int key_t, void* d_plan, tb200_stream_t stream) {
  const size_t kb = dtype_size(key_t);
  if (kb != 4 && kb != 8) return ERR_UNSUPPORTED;
  if (!d_rows || !d_plan) return ERR_INVALID;
  const int fields = kb == 8 ? tb200::exch_fields<unsigned long long>() : tb200::exch_fields<uint32_t>();
  return (int)tb200::exchange_plan_async(d_rows, ranks, rank, fields, static_cast<tb200::exchange_plan*>(d_plan), stream);
}

TB200_API int tb200_exchange_scatter(const void* d_keys, const void* d_vals, size_t n, int key_t, int val_bytes, int descending, const void* d_plan,
                                     int ranks, void* const* h_dst_keys, void* const* h_dst_vals, void* d_ws, size_t* ws_bytes,
                                     tb200_stream_t stream) {
  tb200::key_coding coding;
  if (!coding_of(key_t, descending, coding)) return ERR_UNSUPPORTED;
  if (dtype_size(key_t) == 4)
    return exchange_scatter_by_val<uint32_t>(d_keys, d_vals, n, val_bytes, coding, d_plan, ranks, h_dst_keys, h_dst_vals, d_ws, ws_bytes, stream);
  return exchange_scatter_by_val<unsigned long long>(d_keys, d_vals, n, val_bytes, coding, d_plan, ranks, h_dst_keys, h_dst_vals, d_ws, ws_bytes, stream);
}
