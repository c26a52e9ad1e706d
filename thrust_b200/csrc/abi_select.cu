// C ABI: tb200_copy_if, tb200_partition_copy.
#include "abi_common.cuh"
#include "thrust_b200/select.cuh"

using namespace tb200_abi;
using tb200::abi_pred;

namespace {

template <class T, bool REJ>
int select_pred(const void* in, const void* stencil, int stencil_t, void* out_sel, void* out_rej, size_t n, abi_pred pred,
                unsigned long long* d_count, void* d_ws, cudaStream_t stream) {
  const T* i = static_cast<const T*>(in);
  T* os = static_cast<T*>(out_sel);
  T* orj = static_cast<T*>(out_rej);
  if (!stencil) {
    // large inputs: the streaming kernels, compiled per predicate kind
    if constexpr (sizeof(T) == 4 || sizeof(T) == 8) {
      if (tb200::select_stream_eligible(in, out_sel, out_rej, REJ, n, sizeof(T)))
        return pred.visit([&](auto typed) {
          return (int)tb200::select_stream_async<false, REJ, T, decltype(typed)>(i, os, orj, n, typed, false, d_count, d_ws, stream);
        });
    }
    return (int)tb200::select_async<tb200::SEL_PRED, REJ, false>(i, (const T*)nullptr, os, orj, n, T(), pred, false, d_count, d_ws, stream);
  }
  if (stencil_t == TB200_U8)
    return (int)tb200::select_async<tb200::SEL_STENCIL, REJ>(i, static_cast<const uint8_t*>(stencil), os, orj, n, T(), pred, false, d_count, d_ws, stream);
  if (stencil_t == TB200_I32)
    return (int)tb200::select_async<tb200::SEL_STENCIL, REJ>(i, static_cast<const int32_t*>(stencil), os, orj, n, T(), pred, false, d_count, d_ws, stream);
  return ERR_UNSUPPORTED;
}

template <bool REJ>
int select_entry(const void* in, const void* stencil, void* out_sel, void* out_rej, size_t n, int t, int stencil_t, int pred, long long a,
                 long long b, unsigned long long* d_count, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  if (pred < 0 || pred > 3) return ERR_UNSUPPORTED;
  if (pred == TB200_PRED_MOD_EQ && a == 0) return ERR_INVALID;
  return by_dtype(t, [&](auto tv) -> int {
    using T = decltype(tv);
    int rc;
    if (workspace_gate(d_ws, ws_bytes, tb200::select_workspace_bytes<T>(n), rc)) return rc;
    if (n && (!in || !out_sel || (REJ && !out_rej))) return ERR_INVALID;
    abi_pred p = abi_pred::make(pred, a, b);
    return select_pred<T, REJ>(in, stencil, stencil_t, out_sel, out_rej, n, p, d_count, d_ws, stream);
  });
}

}  // namespace

TB200_API int tb200_copy_if(const void* d_in, const void* d_stencil, void* d_out, size_t n, int t, int stencil_t, int pred, long long a,
                            long long b, unsigned long long* d_count, void* d_ws, size_t* ws_bytes, tb200_stream_t stream) {
  return select_entry<false>(d_in, d_stencil, d_out, nullptr, n, t, stencil_t, pred, a, b, d_count, d_ws, ws_bytes, stream);
}

TB200_API int tb200_partition_copy(const void* d_in, const void* d_stencil, void* d_out_true, void* d_out_false, size_t n, int t,
                                   int stencil_t, int pred, long long a, long long b, unsigned long long* d_count, void* d_ws,
                                   size_t* ws_bytes, tb200_stream_t stream) {
  return select_entry<true>(d_in, d_stencil, d_out_true, d_out_false, n, t, stencil_t, pred, a, b, d_count, d_ws, ws_bytes, stream);
}
