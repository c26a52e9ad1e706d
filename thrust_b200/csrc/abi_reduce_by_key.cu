// C ABI: tb200_reduce_by_key (entry point; the per-value-type bodies live in abi_rbk_*.cu).
#include "abi_rbk.cuh"

namespace tb200_abi {
TB200_RBK_DECL(int32_t) TB200_RBK_DECL(uint32_t) TB200_RBK_DECL(long long) TB200_RBK_DECL(unsigned long long) TB200_RBK_DECL(float) TB200_RBK_DECL(double)
}
using namespace tb200_abi;

TB200_API int tb200_reduce_by_key(const void* d_keys, const void* d_vals, void* d_keys_out, void* d_vals_out, size_t n, int key_t, int val_t,
                                  int op, unsigned long long* d_count, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  switch (val_t) {
    case TB200_I32: return rbk_for_value<int32_t>(d_keys, d_vals, d_keys_out, d_vals_out, n, key_t, op, d_count, d_ws, ws_bytes, stream);
    case TB200_U32: return rbk_for_value<uint32_t>(d_keys, d_vals, d_keys_out, d_vals_out, n, key_t, op, d_count, d_ws, ws_bytes, stream);
    case TB200_I64: return rbk_for_value<long long>(d_keys, d_vals, d_keys_out, d_vals_out, n, key_t, op, d_count, d_ws, ws_bytes, stream);
    case TB200_U64: return rbk_for_value<unsigned long long>(d_keys, d_vals, d_keys_out, d_vals_out, n, key_t, op, d_count, d_ws, ws_bytes, stream);
    case TB200_F32: return rbk_for_value<float>(d_keys, d_vals, d_keys_out, d_vals_out, n, key_t, op, d_count, d_ws, ws_bytes, stream);
    case TB200_F64: return rbk_for_value<double>(d_keys, d_vals, d_keys_out, d_vals_out, n, key_t, op, d_count, d_ws, ws_bytes, stream);
  }
  return ERR_UNSUPPORTED;
}
