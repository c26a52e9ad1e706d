// Times the reduce/scan callers that reach the kernels through a transform_iterator
// (thrust::count, count_if, transform_reduce, inner_product, transform_inclusive_scan) on 2^28 int32,
// compiled as an ordinary Thrust program with the overlay force-included:
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a --extended-lambda -Iinclude \
//        -include thrust_b200/thrust_overlay.cuh tests/cpp/forwarders_bench.cu -o forwarders_bench
// Prints one line per algorithm: milliseconds (median of 9, CUDA events) and input GB/s.
#include <thrust/count.h>
#include <thrust/device_vector.h>
#include <thrust/execution_policy.h>
#include <thrust/functional.h>
#include <thrust/inner_product.h>
#include <thrust/reduce.h>
#include <thrust/sequence.h>
#include <thrust/transform_reduce.h>
#include <thrust/transform_scan.h>

#include <algorithm>
#include <cstdio>
#include <vector>

struct is_odd {
  __host__ __device__ bool operator()(int x) const { return x & 1; }
};
struct square_ll {
  __host__ __device__ long long operator()(int x) const { return (long long)x * x; }
};
struct low_bits {
  __host__ __device__ int operator()(int x) const { return x & 7; }
};

template <class F> static float median_ms(F f) {
  cudaEvent_t a, b;
  cudaEventCreate(&a); cudaEventCreate(&b);
  std::vector<float> t;
  for (int i = 0; i < 12; ++i) {
    cudaEventRecord(a); f(); cudaEventRecord(b); cudaEventSynchronize(b);
    float ms; cudaEventElapsedTime(&ms, a, b);
    if (i >= 3) t.push_back(ms);
  }
  std::sort(t.begin(), t.end());
  return t[t.size() / 2];
}

int main(int argc, char** argv) {
  const size_t n = (size_t)1 << (argc > 1 ? atoi(argv[1]) : 28);
  thrust::device_vector<int> x(n), y(n), out(n);
  thrust::sequence(x.begin(), x.end(), 0);
  thrust::sequence(y.begin(), y.end(), 3);
  long long sink = 0;
  const double gb = n * 4.0 / 1e9;
  float ms;
  ms = median_ms([&] { sink += thrust::reduce(thrust::device, x.begin(), x.end(), 0ll); });
  printf("reduce (pointer input)            %8.3f ms %8.1f GB/s\n", ms, gb / ms * 1e3);
  ms = median_ms([&] { sink += thrust::count(thrust::device, x.begin(), x.end(), 12345); });
  printf("count                             %8.3f ms %8.1f GB/s\n", ms, gb / ms * 1e3);
  ms = median_ms([&] { sink += thrust::count_if(thrust::device, x.begin(), x.end(), is_odd()); });
  printf("count_if                          %8.3f ms %8.1f GB/s\n", ms, gb / ms * 1e3);
  ms = median_ms([&] { sink += thrust::transform_reduce(thrust::device, x.begin(), x.end(), square_ll(), 0ll, thrust::plus<long long>()); });
  printf("transform_reduce                  %8.3f ms %8.1f GB/s\n", ms, gb / ms * 1e3);
  ms = median_ms([&] { sink += thrust::inner_product(thrust::device, x.begin(), x.end(), y.begin(), 0); });
  printf("inner_product (two inputs)        %8.3f ms %8.1f GB/s\n", ms, 2 * gb / ms * 1e3);
  ms = median_ms([&] { thrust::transform_inclusive_scan(thrust::device, x.begin(), x.end(), out.begin(), low_bits(), thrust::plus<int>()); });
  printf("transform_inclusive_scan          %8.3f ms %8.1f GB/s (in + out)\n", ms, 2 * gb / ms * 1e3);
  const long long want_odd = (long long)(n / 2);
  const long long got_odd = thrust::count_if(thrust::device, x.begin(), x.end(), is_odd());
  printf("count_if check: %s; overlay served %llu calls; sink %lld\n", got_odd == want_odd ? "ok" : "WRONG",
         (unsigned long long)thrust::cuda_cub::tb200_overlay::call_count(), sink);
  return got_odd == want_odd ? 0 : 1;
}
