// min_element / max_element / minmax_element for sm_100a: one launch, every element read once.
//
// Each thread walks its share of the input with 16-byte streaming loads and keeps the smallest and
// the largest value seen together with their positions; strict comparisons and increasing positions
// inside a thread, and "equivalent values: the smaller position wins" wherever two candidates meet
// (warp shuffles, CTA partials, the last CTA's fold of all partials), give the FIRST smallest and
// the FIRST largest element, as the arg_min_f / arg_max_f functors of
// thrust/system/cuda/detail/extrema.h:48-108 define them.  Replaces the ReduceAgent-based
// extrema() of thrust/system/cuda/detail/extrema.h:173-374.
#pragma once
#include "common.cuh"
#include "reduce.cuh"

namespace tb200 {

template <class T> struct extrema_state {
  T min_v; T max_v;
  unsigned long long min_i, max_i;
};

// a (+) b for two candidates pairs; less(x, y) orders the values
template <class T, class Less> struct extrema_merge {
  Less less;
  __device__ __forceinline__ extrema_state<T> operator()(const extrema_state<T>& a, const extrema_state<T>& b) const {
    extrema_state<T> r = a;
    if (less(b.min_v, a.min_v) || (!less(a.min_v, b.min_v) && b.min_i < a.min_i)) { r.min_v = b.min_v; r.min_i = b.min_i; }
    if (less(a.max_v, b.max_v) || (!less(b.max_v, a.max_v) && b.max_i < a.max_i)) { r.max_v = b.max_v; r.max_i = b.max_i; }
    return r;
  }
};

constexpr int EXTREMA_BLOCK = 256;
constexpr int EXTREMA_UNROLL = 4;

// VEC = elements per 16-byte load when `in` is a 16-byte aligned pointer to an arithmetic type, 0 for
// any other random-access iterator.  out_index[0] = position of the minimum, [1] = of the maximum.
template <class InIt, class T, class Less, int VEC>
__global__ void __launch_bounds__(EXTREMA_BLOCK)
extrema_kernel(InIt in, size_t n, Less less, extrema_state<T>* partials, unsigned* ticket, unsigned long long* out_index) {
  using S = extrema_state<T>;
  TB200_SHARED_ARRAY(opt<S>, smem, 32);
  __shared__ bool is_last;
  const size_t tid = (size_t)blockIdx.x * EXTREMA_BLOCK + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * EXTREMA_BLOCK;
  opt<S> acc; acc.has = false;
  auto see = [&](const T& x, size_t i) {
    if (!acc.has) { acc.v.min_v = x; acc.v.max_v = x; acc.v.min_i = i; acc.v.max_i = i; acc.has = true; }
    else {
      if (less(x, acc.v.min_v)) { acc.v.min_v = x; acc.v.min_i = i; }
      if (less(acc.v.max_v, x)) { acc.v.max_v = x; acc.v.max_i = i; }
    }
  };
  if constexpr (VEC > 0) {
    // Per 16-byte vector only its smallest and largest value are compared with the running
    // extremes, and only the VECTOR's position is recorded (strict comparisons: the earliest
    // vector holding the extreme wins); the element inside the two winning vectors is found at
    // the end by reading them once more.
    const size_t nvec = n / VEC;
    const vec16* vin = reinterpret_cast<const vec16*>(in);
    T lo_v = T(), hi_v = T();
    size_t lo_at = 0, hi_at = 0;
    bool any = false;
    auto see_vector = [&](const vec16& r, size_t at) {
      const T* e = reinterpret_cast<const T*>(&r);
      T lo = e[0], hi = e[0];
#pragma unroll
      for (int k = 1; k < VEC; ++k) { if (less(e[k], lo)) lo = e[k]; if (less(hi, e[k])) hi = e[k]; }
      if (!any || less(lo, lo_v)) { lo_v = lo; lo_at = at; }
      if (!any || less(hi_v, hi)) { hi_v = hi; hi_at = at; }
      any = true;
    };
    size_t v = tid;
    for (; v + (EXTREMA_UNROLL - 1) * stride < nvec; v += EXTREMA_UNROLL * stride) {
      vec16 r[EXTREMA_UNROLL];
#pragma unroll
      for (int u = 0; u < EXTREMA_UNROLL; ++u) r[u] = load_stream16(vin + v + u * stride);
#pragma unroll
      for (int u = 0; u < EXTREMA_UNROLL; ++u) see_vector(r[u], v + u * stride);
    }
    for (; v < nvec; v += stride) see_vector(load_stream16(vin + v), v);
    if (any) {
      const T* e = in + lo_at * VEC;
      int k = 0;
      while (k < VEC - 1 && (less(lo_v, e[k]) || less(e[k], lo_v))) ++k;     // first element equivalent to the minimum
      see(e[k], lo_at * VEC + k);
      e = in + hi_at * VEC;
      k = 0;
      while (k < VEC - 1 && (less(hi_v, e[k]) || less(e[k], hi_v))) ++k;
      see(e[k], hi_at * VEC + k);
    }
    const size_t t = nvec * VEC + tid;
    if (t < n) see(in[t], t);
  } else {
    for (size_t i = tid; i < n; i += stride) { const T x = in[i]; see(x, i); }
  }

  const extrema_merge<T, Less> merge{less};
  opt<S> blk = block_reduce_opt(acc, merge, smem);
  if (threadIdx.x == 0) {
    // a CTA without elements (grid larger than the input) publishes a neutral marker: position n
    S p;
    if (blk.has) p = blk.v; else { p.min_v = T(); p.max_v = T(); p.min_i = n; p.max_i = n; }
    partials[blockIdx.x] = p;
    __threadfence();
    is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  opt<S> f; f.has = false;
  for (unsigned b = threadIdx.x; b < gridDim.x; b += EXTREMA_BLOCK) {
    S p;
    const unsigned long long* src = reinterpret_cast<const unsigned long long*>(partials + b);
    static_assert(sizeof(S) % 8 == 0, "extrema_state is read back in 8-byte words");
    unsigned long long w[sizeof(S) / 8];
#pragma unroll
    for (int q = 0; q < (int)(sizeof(S) / 8); ++q) w[q] = __ldcg(src + q);
    memcpy(&p, w, sizeof(S));
    if (p.min_i < n) f.append(p, merge);
  }
  __syncthreads();
  f = block_reduce_opt(f, merge, smem);
  if (threadIdx.x == 0) {
    out_index[0] = f.has ? f.v.min_i : 0;
    out_index[1] = f.has ? f.v.max_i : 0;
    *ticket = 0;
  }
}

template <class T> size_t extrema_workspace_bytes() {
  return sizeof(ws_header) + align_up(REDUCE_MAX_GRID * sizeof(extrema_state<T>), 256);
}

// Positions of the first minimum and the first maximum of in[0, n) under `less`, written to
// d_index[0] and d_index[1] (device memory); n == 0 writes 0 and 0.  No sync.
template <class InIt, class T, class Less>
cudaError_t extrema_async(InIt in, size_t n, T /*value type tag*/, Less less, unsigned long long* d_index, void* ws, cudaStream_t stream) {
  char* base = static_cast<char*>(ws);
  ws_header* hdr = reinterpret_cast<ws_header*>(base);
  extrema_state<T>* partials = reinterpret_cast<extrema_state<T>*>(base + sizeof(ws_header));
  cudaError_t e = cudaMemsetAsync(hdr, 0, sizeof(ws_header), stream);
  if (e != cudaSuccess) return e;
  if (n == 0) return cudaMemsetAsync(d_index, 0, 2 * sizeof(unsigned long long), stream);
  if constexpr (std::is_pointer<InIt>::value) {
    using In = typename std::remove_cv<typename std::remove_pointer<InIt>::type>::type;
    if constexpr (std::is_same<In, T>::value && std::is_arithmetic<T>::value && (16 % sizeof(T) == 0)) {
      if (is_aligned16(in)) {
        constexpr int VEC = 16 / sizeof(T);
        timed_launch tl(KID_REDUCE, stream);
        extrema_kernel<InIt, T, Less, VEC><<<reduce_grid(n / VEC), EXTREMA_BLOCK, 0, stream>>>(in, n, less, partials, &hdr->ticket, d_index);
        return cudaGetLastError();
      }
    }
  }
  timed_launch tl(KID_REDUCE, stream);
  extrema_kernel<InIt, T, Less, 0><<<reduce_grid(n), EXTREMA_BLOCK, 0, stream>>>(in, n, less, partials, &hdr->ticket, d_index);
  return cudaGetLastError();
}

}  // namespace tb200
