// C ABI: tb200_sort_by_key (radix path).
#include "abi_common.cuh"
#include "thrust_b200/radix_sort.cuh"

using namespace tb200_abi;

namespace {
template <class UK, class UV, bool HAS_V>
int sort_typed(void* k, void* ka, void* v, void* va, size_t n, tb200::key_coding coding, int b0, int b1, void* d_ws, size_t* ws_bytes,
               cudaStream_t stream) {
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::radix_workspace_bytes<sizeof(UK), HAS_V ? sizeof(UV) : 0>(n), rc)) return rc;
  if (n > 1 && (!k || !ka || (HAS_V && (!v || !va)))) return ERR_INVALID;
  return (int)tb200::radix_sort_async<UK, UV, HAS_V>(static_cast<UK*>(k), static_cast<UK*>(ka), static_cast<UV*>(v), static_cast<UV*>(va), n, coding,
                                                     b0, b1, d_ws, stream);
}
template <class UK>
int sort_by_val(void* k, void* ka, void* v, void* va, size_t n, int val_bytes, tb200::key_coding coding, int b0, int b1, void* d_ws,
                size_t* ws_bytes, cudaStream_t stream) {
  switch (val_bytes) {
    case 0: return sort_typed<UK, uint32_t, false>(k, ka, v, va, n, coding, b0, b1, d_ws, ws_bytes, stream);
    case 4: return sort_typed<UK, uint32_t, true>(k, ka, v, va, n, coding, b0, b1, d_ws, ws_bytes, stream);
    case 8: return sort_typed<UK, unsigned long long, true>(k, ka, v, va, n, coding, b0, b1, d_ws, ws_bytes, stream);
  }
  return ERR_UNSUPPORTED;
}
}  // namespace

TB200_API int tb200_sort_by_key(void* d_keys, void* d_keys_alt, void* d_vals, void* d_vals_alt, size_t n, int key_t, int val_bytes,
                                int descending, int begin_bit, int end_bit, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  tb200::key_coding coding;
  coding.descending = descending ? 1 : 0;
  switch (key_t) {
    case TB200_U8: case TB200_U16: case TB200_U32: case TB200_U64: coding.kind = tb200::KEY_UNSIGNED; break;
    case TB200_I8: case TB200_I16: case TB200_I32: case TB200_I64: coding.kind = tb200::KEY_SIGNED; break;
    case TB200_F32: case TB200_F64: coding.kind = tb200::KEY_FLOAT; break;
    default: return ERR_UNSUPPORTED;
  }
  switch (dtype_size(key_t)) {
    case 1: return sort_by_val<uint8_t>(d_keys, d_keys_alt, d_vals, d_vals_alt, n, val_bytes, coding, begin_bit, end_bit, d_ws, ws_bytes, stream);
    case 2: return sort_by_val<uint16_t>(d_keys, d_keys_alt, d_vals, d_vals_alt, n, val_bytes, coding, begin_bit, end_bit, d_ws, ws_bytes, stream);
    case 4: return sort_by_val<uint32_t>(d_keys, d_keys_alt, d_vals, d_vals_alt, n, val_bytes, coding, begin_bit, end_bit, d_ws, ws_bytes, stream);
  }
  return sort_by_val<unsigned long long>(d_keys, d_keys_alt, d_vals, d_vals_alt, n, val_bytes, coding, begin_bit, end_bit, d_ws, ws_bytes, stream);
}
