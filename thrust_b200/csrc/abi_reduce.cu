// C ABI: tb200_reduce, tb200_version, tb200_sm_arch, tb200_workspace_status.
#include "abi_common.cuh"
#include "thrust_b200/reduce.cuh"

using namespace tb200_abi;

TB200_API int tb200_version(void) { return 100; }
TB200_API int tb200_sm_arch(void) { return 100; }

TB200_API int tb200_workspace_status(const void* d_ws, tb200_stream_t stream, unsigned* h_status) {
  if (!d_ws || !h_status) return ERR_INVALID;
  cudaError_t e = cudaMemcpyAsync(h_status, d_ws, sizeof(unsigned), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(stream);
}

namespace {

template <class In, class Acc>
int reduce_typed(const void* d_in, size_t n, int op, const void* h_init, void* d_out, void* d_ws, size_t* ws_bytes, cudaStream_t stream) {
  int rc;
  if (workspace_gate(d_ws, ws_bytes, tb200::reduce_workspace_bytes<Acc>(), rc)) return rc;
  if (!h_init || !d_out || (n && !d_in)) return ERR_INVALID;
  Acc init; memcpy(&init, h_init, sizeof(Acc));
  return by_op(op, [&](auto o) {
    return (int)tb200::reduce_async(static_cast<const In*>(d_in), n, init, o, static_cast<Acc*>(d_out), d_ws, stream);
  });
}

}  // namespace

TB200_API int tb200_reduce(const void* d_in, size_t n, int in_t, int acc_t, int op, const void* h_init, void* d_out, void* d_ws,
                           size_t* ws_bytes, tb200_stream_t stream) {
#define CASE(ti, In, ta, Acc) \
  if (in_t == ti && acc_t == ta) return reduce_typed<In, Acc>(d_in, n, op, h_init, d_out, d_ws, ws_bytes, stream);
  CASE(TB200_I8, int8_t, TB200_I32, int32_t) CASE(TB200_I8, int8_t, TB200_I64, long long)
  CASE(TB200_I16, int16_t, TB200_I32, int32_t) CASE(TB200_I16, int16_t, TB200_I64, long long)
  CASE(TB200_I32, int32_t, TB200_I32, int32_t) CASE(TB200_I32, int32_t, TB200_I64, long long)
  CASE(TB200_U8, uint8_t, TB200_U32, uint32_t) CASE(TB200_U8, uint8_t, TB200_U64, unsigned long long)
  CASE(TB200_U16, uint16_t, TB200_U32, uint32_t) CASE(TB200_U16, uint16_t, TB200_U64, unsigned long long)
  CASE(TB200_U32, uint32_t, TB200_U32, uint32_t) CASE(TB200_U32, uint32_t, TB200_U64, unsigned long long)
  CASE(TB200_I64, long long, TB200_I64, long long) CASE(TB200_U64, unsigned long long, TB200_U64, unsigned long long)
  CASE(TB200_F32, float, TB200_F32, float) CASE(TB200_F32, float, TB200_F64, double)
  CASE(TB200_F64, double, TB200_F64, double)
#undef CASE
  return ERR_UNSUPPORTED;
}
