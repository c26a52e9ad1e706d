// Single-pass device-wide reduction for sm_100a.
//
// One launch: a grid sized to the SM count streams the input with 16-byte evict-first loads
// (four in flight per thread), folds it with warp shuffles, and the last CTA to finish (found
// with an atomic ticket) folds the per-CTA partials and `init` into the result.  Replaces the
// two-kernel cub::DispatchReduce call of thrust/system/cuda/detail/reduce.h:946-983.
// Like that path it needs an associative and commutative operator.
#pragma once
#include "common.cuh"

namespace tb200 {

constexpr int REDUCE_BLOCK = 256;
constexpr int REDUCE_UNROLL = 4;
constexpr int REDUCE_UNROLL_GENERIC = 16;
constexpr int REDUCE_CTAS_PER_SM = 4;
constexpr int REDUCE_MAX_GRID = 4096;

template <class AccT, class Op>
__device__ __forceinline__ opt<AccT> block_reduce_opt(opt<AccT> x, Op op, opt<AccT>* smem /*[32]*/) {
  const int lane = lane_id(), warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  x = warp_reduce_opt(x, op);
  if (lane == 0) smem[warp] = x;
  __syncthreads();
  opt<AccT> r; r.has = false;
  if (warp == 0) {
    if (lane < nwarps) r = smem[lane];
    r = warp_reduce_opt(r, op);
  }
  return r;  // valid in thread 0
}

// In = element type read from memory (or an iterator's value), AccT = accumulator.
// VEC = elements per 16-byte load when `in` is a 16-byte-aligned pointer to a 1/2/4/8-byte type,
// 0 for the generic path (any random-access iterator, one element per load).
template <class InIt, class AccT, class Op, int VEC>
__global__ void __launch_bounds__(REDUCE_BLOCK)
reduce_kernel(InIt in, size_t n, AccT init, Op op, AccT* partials, unsigned* partial_has,
              unsigned* ticket, AccT* out) {
  TB200_SHARED_ARRAY(opt<AccT>, smem, 32);
  __shared__ bool is_last;
  const size_t tid = (size_t)blockIdx.x * REDUCE_BLOCK + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * REDUCE_BLOCK;
  opt<AccT> acc; acc.has = false;

  if constexpr (VEC > 0) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    const size_t nvec = n / VEC;
    const vec16* vin = reinterpret_cast<const vec16*>(in);
    size_t v = tid;
    for (; v + (REDUCE_UNROLL - 1) * stride < nvec; v += REDUCE_UNROLL * stride) {
      vec16 r[REDUCE_UNROLL];
#pragma unroll
      for (int u = 0; u < REDUCE_UNROLL; ++u) r[u] = load_stream16(vin + v + u * stride);
#pragma unroll
      for (int u = 0; u < REDUCE_UNROLL; ++u) {
        const In* e = reinterpret_cast<const In*>(&r[u]);
        AccT t = (AccT)e[0];
#pragma unroll
        for (int k = 1; k < VEC; ++k) t = op(t, (AccT)e[k]);
        acc.append(t, op);
      }
    }
    for (; v < nvec; v += stride) {
      vec16 r = load_stream16(vin + v);
      const In* e = reinterpret_cast<const In*>(&r);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc.append((AccT)e[k], op);
    }
    // ragged tail (fewer than VEC elements)
    size_t t = nvec * VEC + tid;
    if (t < n) acc.append((AccT)in[t], op);
  } else {
    // one element per load: sixteen of them in flight per thread keep as many bytes on their way as
    // the four 16-byte loads of the vector path (a transform_iterator over 4-byte items, say)
    constexpr int U = REDUCE_UNROLL_GENERIC;
    size_t i = tid;
    for (; i + (U - 1) * stride < n; i += U * stride) {
      AccT r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) r[u] = (AccT)in[i + u * stride];
      AccT t = r[0];
#pragma unroll
      for (int u = 1; u < U; ++u) t = op(t, r[u]);
      acc.append(t, op);
    }
    for (; i < n; i += stride) acc.append((AccT)in[i], op);
  }

  opt<AccT> blk = block_reduce_opt(acc, op, smem);
  if (threadIdx.x == 0) {
    if (blk.has) partials[blockIdx.x] = blk.v;
    partial_has[blockIdx.x] = blk.has;
    __threadfence();
    unsigned t = atomicAdd(ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  opt<AccT> f; f.has = false;
  for (unsigned b = threadIdx.x; b < gridDim.x; b += REDUCE_BLOCK) {
    if (__ldcg(partial_has + b)) f.append(load_cg_any(partials + b), op);
  }
  __syncthreads();
  f = block_reduce_opt(f, op, smem);
  if (threadIdx.x == 0) {
    *out = f.has ? op(init, f.v) : init;
    *ticket = 0;
  }
}

inline int reduce_grid(size_t work_items /* vectors or elements */) {
  const device_info& di = current_device_info();
  size_t want = (work_items + REDUCE_BLOCK - 1) / REDUCE_BLOCK;
  size_t cap = (size_t)di.sm_count * REDUCE_CTAS_PER_SM;
  if (cap > REDUCE_MAX_GRID) cap = REDUCE_MAX_GRID;
  if (want < 1) want = 1;
  return (int)(want < cap ? want : cap);
}

template <class AccT> size_t reduce_workspace_bytes() {
  return sizeof(ws_header) + align_up(REDUCE_MAX_GRID * sizeof(AccT), 256) + align_up(REDUCE_MAX_GRID * 4, 256) +
         align_up(sizeof(AccT), 256);
}

// Launches the reduction on `stream`; the result lands in *d_out (device memory).  No sync.
// `ws` must hold reduce_workspace_bytes<AccT>().  n == 0 writes init.
template <class InIt, class AccT, class Op>
cudaError_t reduce_async(InIt in, size_t n, AccT init, Op op, AccT* d_out, void* ws, cudaStream_t stream) {
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  AccT* partials = reinterpret_cast<AccT*>(base + sizeof(ws_header));
  unsigned* has = reinterpret_cast<unsigned*>(base + sizeof(ws_header) + align_up(REDUCE_MAX_GRID * sizeof(AccT), 256));
  cudaError_t e = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess) return e;
  constexpr bool is_ptr = std::is_pointer<InIt>::value;
  if constexpr (is_ptr) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    constexpr bool vec_ok = std::is_arithmetic<In>::value && (16 % sizeof(In) == 0);
    if constexpr (vec_ok) {
      if (is_aligned16(in)) {
        constexpr int VEC = 16 / sizeof(In);
        int grid = reduce_grid(n / VEC);
        timed_launch tl(KID_REDUCE, stream);
        reduce_kernel<InIt, AccT, Op, VEC><<<grid, REDUCE_BLOCK, 0, stream>>>(in, n, init, op, partials, has, &hdr->ticket, d_out);
        log_launch("reduce_kernel (16-byte loads)", grid, REDUCE_BLOCK, 0, n, stream);
        return cudaGetLastError();
      }
    }
  }
  int grid = reduce_grid(n);
  timed_launch tl(KID_REDUCE, stream);
  reduce_kernel<InIt, AccT, Op, 0><<<grid, REDUCE_BLOCK, 0, stream>>>(in, n, init, op, partials, has, &hdr->ticket, d_out);
  log_launch("reduce_kernel (generic iterator)", grid, REDUCE_BLOCK, 0, n, stream);
  return cudaGetLastError();
}

}  // namespace tb200
