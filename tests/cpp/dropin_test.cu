// Drop-in check: an ordinary Thrust program (device_vector, thrust::device, thrust::cuda::par.on)
// compiled with the overlay header force-included.  Every algorithm on the hot path is called the
// way an existing caller would and compared with a straightforward host computation.  A kernel
// launch counter proves that the overlay, not the stock CUB path, served the calls.
//
//   nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a --extended-lambda -I<repo>/include \
//        -include thrust_b200/thrust_overlay.cuh tests/cpp/dropin_test.cu -o dropin_test
#include <thrust/async/reduce.h>
#include <thrust/async/scan.h>
#include <thrust/async/sort.h>
#include <thrust/copy.h>
#include <thrust/device_vector.h>
#include <thrust/execution_policy.h>
#include <thrust/functional.h>
#include <thrust/host_vector.h>
#include <thrust/iterator/counting_iterator.h>
#include <thrust/iterator/transform_iterator.h>
#include <thrust/iterator/zip_iterator.h>
#include <thrust/merge.h>
#include <thrust/mr/allocator.h>
#include <thrust/mr/disjoint_pool.h>
#include <thrust/mr/new.h>
#include <thrust/system/cuda/memory_resource.h>
#include <thrust/partition.h>
#include <thrust/reduce.h>
#include <thrust/extrema.h>
#include <thrust/scan.h>
#include <thrust/sequence.h>
#include <thrust/sort.h>
#include <thrust/transform_reduce.h>
#include <thrust/transform_scan.h>
#include <thrust/count.h>
#include <thrust/tuple.h>
#include <thrust/unique.h>

#include <algorithm>
#include <cstdio>
#include <numeric>
#include <vector>

#ifndef THRUST_B200_OVERLAY_EXPECTED
#error "compile with -include thrust_b200/thrust_overlay.cuh -DTHRUST_B200_OVERLAY_EXPECTED"
#endif

static int failures = 0;
#define CHECK(cond) do { if (!(cond)) { std::printf("FAILED line %d: %s\n", __LINE__, #cond); ++failures; } } while (0)

static unsigned long long mix(unsigned long long i) {
  unsigned long long z = i + 0x9E3779B97F4A7C15ull * 7;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31);
}
struct is_even { __host__ __device__ bool operator()(int x) const { return (x & 1) == 0; } };
struct square { __host__ __device__ long long operator()(int x) const { return (long long)x * x; } };
// a struct accumulator (examples/minmax.cu in the reference) and a 32-byte key with its own comparator
struct lohi { int lo, hi; };
struct to_lohi { __host__ __device__ lohi operator()(int x) const { lohi r; r.lo = x; r.hi = x; return r; } };
struct lohi_merge { __host__ __device__ lohi operator()(const lohi& a, const lohi& b) const { lohi r; r.lo = a.lo < b.lo ? a.lo : b.lo; r.hi = a.hi > b.hi ? a.hi : b.hi; return r; } };
struct wide { unsigned long long k; unsigned long long pad[3]; };
struct wide_less { __host__ __device__ bool operator()(const wide& a, const wide& b) const { return a.k < b.k; } };
// an allocator of the caller's own, as handed to thrust::cuda::par(alloc): counts what it serves
struct counting_allocator {
  typedef char value_type;
  int* served;
  char* allocate(std::ptrdiff_t bytes) { ++*served; char* p = nullptr; if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) throw std::bad_alloc(); return p; }
  void deallocate(char* p, size_t) { cudaFree(p); }
};
// a device memory resource that counts what reaches it: the upstream of a thrust::mr pool
struct counting_resource final : thrust::mr::memory_resource<thrust::cuda::memory_resource::pointer> {
  thrust::cuda::memory_resource upstream;
  int allocations = 0;
  pointer do_allocate(std::size_t bytes, std::size_t alignment) override { ++allocations; return upstream.do_allocate(bytes, alignment); }
  void do_deallocate(pointer p, std::size_t bytes, std::size_t alignment) override { upstream.do_deallocate(p, bytes, alignment); }
};
struct by_first { template <class A, class B> __host__ __device__ bool operator()(const A& a, const B& b) const { return thrust::get<0>(a) < thrust::get<0>(b); } };

struct low3 { __host__ __device__ int operator()(int x) const { return x & 7; } };
struct is_odd_int { __host__ __device__ bool operator()(int x) const { return x & 1; } };

int main() {
  const int n = 1000003;
  std::vector<int> h(n);
  for (int i = 0; i < n; ++i) h[i] = (int)(mix(i) % 2000001) - 1000000;
  thrust::device_vector<int> d(h.begin(), h.end());

  // reduce: explicit policy, accumulator type from init; and tag dispatch on device_vector iterators
  long long want = std::accumulate(h.begin(), h.end(), 0LL);
  CHECK(thrust::reduce(thrust::device, d.begin(), d.end(), 0LL, thrust::plus<long long>()) == want);
  CHECK(thrust::reduce(d.begin(), d.end(), 0LL) == want);
  CHECK(thrust::reduce(thrust::device, d.begin(), d.end(), -2000000, thrust::maximum<int>()) == *std::max_element(h.begin(), h.end()));
  // a transform_iterator input goes through the generic-iterator kernel
  long long want_sq = 0; for (int x : h) want_sq += (long long)x * x;
  CHECK(thrust::reduce(thrust::device, thrust::make_transform_iterator(d.begin(), square()), thrust::make_transform_iterator(d.end(), square()), 0LL) == want_sq);
  CHECK(thrust::reduce(thrust::device, thrust::counting_iterator<long long>(0), thrust::counting_iterator<long long>(1 << 20), 0LL) == (1LL << 19) * ((1 << 20) - 1));

  // scans, in place and on a user stream
  cudaStream_t s; cudaStreamCreate(&s);
  std::vector<int> small(n); for (int i = 0; i < n; ++i) small[i] = (int)(mix(i + n) % 16);
  thrust::device_vector<int> ds(small.begin(), small.end()), dout(n);
  std::vector<int> hs(n); std::partial_sum(small.begin(), small.end(), hs.begin());
  thrust::inclusive_scan(thrust::cuda::par.on(s), ds.begin(), ds.end(), dout.begin());
  thrust::host_vector<int> got = dout;
  CHECK(std::equal(hs.begin(), hs.end(), got.begin()));
  thrust::exclusive_scan(thrust::device, ds.begin(), ds.end(), dout.begin(), 7);
  got = dout;
  bool ok = got[0] == 7; for (int i = 1; i < n && ok; ++i) ok = got[i] == hs[i - 1] + 7;
  CHECK(ok);
  thrust::inclusive_scan(ds.begin(), ds.end(), ds.begin());                               // in place, tag dispatch
  got = ds;
  CHECK(std::equal(hs.begin(), hs.end(), got.begin()));
  thrust::device_vector<int> dm(small.begin(), small.end());
  thrust::inclusive_scan(thrust::device, dm.begin(), dm.end(), dm.begin(), thrust::maximum<int>());
  got = dm; { int m = small[0]; ok = true; for (int i = 0; i < n && ok; ++i) { m = std::max(m, small[i]); ok = got[i] == m; } } CHECK(ok);

  // sort_by_key (radix path) with stability check, descending sort, float keys
  std::vector<unsigned> hk(n), hv(n); for (int i = 0; i < n; ++i) { hk[i] = (unsigned)(mix(i) >> 44); hv[i] = i; }
  thrust::device_vector<unsigned> dk(hk.begin(), hk.end()), dv(hv.begin(), hv.end());
  thrust::sort_by_key(thrust::device, dk.begin(), dk.end(), dv.begin());
  std::vector<unsigned> idx(n); std::iota(idx.begin(), idx.end(), 0u);
  std::stable_sort(idx.begin(), idx.end(), [&](unsigned a, unsigned b) { return hk[a] < hk[b]; });
  thrust::host_vector<unsigned> gk = dk, gv = dv;
  ok = true; for (int i = 0; i < n && ok; ++i) ok = gv[i] == idx[i] && gk[i] == hk[idx[i]];
  CHECK(ok);
  thrust::device_vector<float> df(n); { std::vector<float> hf(n); for (int i = 0; i < n; ++i) hf[i] = (float)((long long)(mix(i) % 20001) - 10000) / 7.0f;
    df = hf; thrust::sort(thrust::device, df.begin(), df.end(), thrust::greater<float>()); std::sort(hf.begin(), hf.end(), std::greater<float>());
    thrust::host_vector<float> gf = df; CHECK(std::equal(hf.begin(), hf.end(), gf.begin())); }
  // stable_sort on a zip iterator with a user comparator: merge-sort route, keys not contiguous
  { std::vector<unsigned> zk(n); std::vector<float> zv(n); for (int i = 0; i < n; ++i) { zk[i] = (unsigned)(mix(i + 5) >> 50); zv[i] = (float)i; }
    thrust::device_vector<unsigned> dzk(zk.begin(), zk.end()); thrust::device_vector<float> dzv(zv.begin(), zv.end());
    auto z = thrust::make_zip_iterator(thrust::make_tuple(dzk.begin(), dzv.begin()));
    thrust::stable_sort(thrust::device, z, z + n, by_first());
    std::vector<unsigned> id2(n); std::iota(id2.begin(), id2.end(), 0u);
    std::stable_sort(id2.begin(), id2.end(), [&](unsigned a, unsigned b) { return zk[a] < zk[b]; });
    thrust::host_vector<unsigned> g1 = dzk; thrust::host_vector<float> g2 = dzv;
    ok = true; for (int i = 0; i < n && ok; ++i) ok = g1[i] == zk[id2[i]] && g2[i] == (float)id2[i];
    CHECK(ok); }

  // copy_if with a user predicate, partition family, unique, reduce_by_key
  thrust::device_vector<int> dsel(n);
  auto end = thrust::copy_if(thrust::device, d.begin(), d.end(), dsel.begin(), is_even());
  std::vector<int> hsel; for (int x : h) if ((x & 1) == 0) hsel.push_back(x);
  CHECK((size_t)(end - dsel.begin()) == hsel.size());
  got = dsel; CHECK(std::equal(hsel.begin(), hsel.end(), got.begin()));
  thrust::device_vector<int> dp(h.begin(), h.end());
  auto mid = thrust::stable_partition(thrust::device, dp.begin(), dp.end(), is_even());
  std::vector<int> hp(h); auto hmid = std::stable_partition(hp.begin(), hp.end(), [](int x) { return (x & 1) == 0; });
  CHECK((mid - dp.begin()) == (hmid - hp.begin())); got = dp; CHECK(std::equal(hp.begin(), hp.end(), got.begin()));
  thrust::device_vector<int> dt(n), dfalse(n);
  auto pr = thrust::partition_copy(thrust::device, d.begin(), d.end(), dt.begin(), dfalse.begin(), is_even());
  CHECK((size_t)(pr.first - dt.begin()) == hsel.size() && (size_t)(pr.second - dfalse.begin()) == n - hsel.size());
  std::vector<int> runs(n); { int k = 0; for (int i = 0; i < n; ++i) { if (i && mix(i + 99) % 4 == 0) ++k; runs[i] = k; } }
  thrust::device_vector<int> dr(runs.begin(), runs.end()), du(n);
  auto uend = thrust::unique_copy(thrust::device, dr.begin(), dr.end(), du.begin());
  CHECK((uend - du.begin()) == runs.back() + 1);
  thrust::device_vector<int> ones(n, 1), rk(n), rv(n);
  auto re = thrust::reduce_by_key(thrust::device, dr.begin(), dr.end(), ones.begin(), rk.begin(), rv.begin());
  CHECK((re.first - rk.begin()) == runs.back() + 1);
  CHECK(thrust::reduce(thrust::device, rv.begin(), re.second, 0) == n);
  auto uin = thrust::unique(thrust::device, dr.begin(), dr.end());                          // in place
  CHECK((uin - dr.begin()) == runs.back() + 1);

  // the first "next" components: scan_by_key and unique_by_key
  { thrust::device_vector<int> dkeys(runs.begin(), runs.end()), dones(n, 1), dsk(n);
    thrust::inclusive_scan_by_key(thrust::device, dkeys.begin(), dkeys.end(), dones.begin(), dsk.begin());
    got = dsk; ok = true; { int c = 0; for (int i = 0; i < n && ok; ++i) { c = (i && runs[i] == runs[i - 1]) ? c + 1 : 1; ok = got[i] == c; } } CHECK(ok);
    thrust::exclusive_scan_by_key(thrust::device, dkeys.begin(), dkeys.end(), dones.begin(), dsk.begin(), 10);
    got = dsk; ok = true; { int c = 0; for (int i = 0; i < n && ok; ++i) { c = (i && runs[i] == runs[i - 1]) ? c + 1 : 0; ok = got[i] == 10 + c; } } CHECK(ok);
    thrust::device_vector<int> dpos(n); thrust::sequence(dpos.begin(), dpos.end());
    auto ue = thrust::unique_by_key(thrust::device, dkeys.begin(), dkeys.end(), dpos.begin());
    CHECK((ue.first - dkeys.begin()) == runs.back() + 1);
    got = dpos; ok = true; { int r = 0; for (int i = 0; i < n && ok; ++i) if (i == 0 || runs[i] != runs[i - 1]) { ok = got[r] == i; ++r; } } CHECK(ok); }

  // extrema: first smallest / first largest (testing/minmax_element.cu:8-20)
  { int raw[6] = {3, 5, 1, 2, 5, 1};
    thrust::device_vector<int> dx(raw, raw + 6);
    CHECK(thrust::min_element(thrust::device, dx.begin(), dx.end()) - dx.begin() == 2);
    CHECK(thrust::max_element(thrust::device, dx.begin(), dx.end()) - dx.begin() == 1);
    auto mm = thrust::minmax_element(thrust::device, dx.begin(), dx.end());
    CHECK(mm.first - dx.begin() == 2 && mm.second - dx.begin() == 1);
    auto big = thrust::max_element(thrust::device, d.begin(), d.end(), thrust::greater<int>());   // = the first minimum
    CHECK(big - d.begin() == std::min_element(h.begin(), h.end()) - h.begin()); }

  // merge_by_key: ties take from the first range
  { int na = 300007, nb = 200003; std::vector<unsigned long long> a(na), b(nb); for (int i = 0; i < na; ++i) a[i] = mix(i) >> 52; for (int i = 0; i < nb; ++i) b[i] = mix(i + na) >> 52;
    std::sort(a.begin(), a.end()); std::sort(b.begin(), b.end());
    thrust::device_vector<unsigned long long> da(a.begin(), a.end()), db(b.begin(), b.end()), dko(na + nb);
    thrust::device_vector<unsigned> va(na, 0u), vb(nb, 1u), dvo(na + nb);
    thrust::merge_by_key(thrust::device, da.begin(), da.end(), db.begin(), db.end(), va.begin(), vb.begin(), dko.begin(), dvo.begin());
    std::vector<unsigned long long> hm(na + nb); std::merge(a.begin(), a.end(), b.begin(), b.end(), hm.begin());
    thrust::host_vector<unsigned long long> gm = dko; thrust::host_vector<unsigned> gmv = dvo;
    CHECK(std::equal(hm.begin(), hm.end(), gm.begin()));
    ok = true; for (int i = 1; i < na + nb && ok; ++i) if (gm[i] == gm[i - 1]) ok = gmv[i - 1] <= gmv[i];
    CHECK(ok);
    thrust::device_vector<unsigned long long> dmo(na + nb);
    thrust::merge(da.begin(), da.end(), db.begin(), db.end(), dmo.begin());
    gm = dmo; CHECK(std::equal(hm.begin(), hm.end(), gm.begin())); }

  // a struct accumulator through transform_reduce / reduce
  { lohi init; init.lo = h[0]; init.hi = h[0];
    lohi r = thrust::reduce(thrust::device, thrust::make_transform_iterator(d.begin(), to_lohi()), thrust::make_transform_iterator(d.end(), to_lohi()), init, lohi_merge());
    CHECK(r.lo == *std::min_element(h.begin(), h.end()) && r.hi == *std::max_element(h.begin(), h.end())); }

  // 32-byte keys with a user comparator: comparison sort, sort_by_key and merge size their tiles by sizeof
  { const int nw = 100003; std::vector<wide> hw(nw); for (int i = 0; i < nw; ++i) { hw[i].k = mix(i) >> 44; hw[i].pad[0] = i; hw[i].pad[1] = hw[i].pad[2] = 0; }
    thrust::device_vector<wide> dw(hw.begin(), hw.end());
    thrust::stable_sort(thrust::device, dw.begin(), dw.end(), wide_less());
    std::stable_sort(hw.begin(), hw.end(), [](const wide& a, const wide& b) { return a.k < b.k; });
    thrust::host_vector<wide> gw = dw; ok = true; for (int i = 0; i < nw && ok; ++i) ok = gw[i].k == hw[i].k && gw[i].pad[0] == hw[i].pad[0];
    CHECK(ok);
    thrust::device_vector<wide> dk2(hw.rbegin(), hw.rend()); thrust::device_vector<int> dv2(nw); thrust::sequence(dv2.begin(), dv2.end());
    thrust::stable_sort_by_key(thrust::device, dk2.begin(), dk2.end(), dv2.begin(), wide_less());
    gw = dk2; ok = true; for (int i = 1; i < nw && ok; ++i) ok = gw[i - 1].k <= gw[i].k;
    CHECK(ok);
    thrust::device_vector<wide> dm2(2 * nw);
    thrust::merge(thrust::device, dw.begin(), dw.end(), dk2.begin(), dk2.end(), dm2.begin(), wide_less());
    gw = dm2; ok = true; for (int i = 1; i < 2 * nw && ok; ++i) ok = gw[i - 1].k <= gw[i].k;
    CHECK(ok && gw.size() == (size_t)(2 * nw)); }

  // thrust::cuda::par(alloc): the same kernels, temporary storage from the caller's allocator
  { int served = 0; counting_allocator alloc; alloc.served = &served;
    const unsigned long long before = thrust::cuda_cub::tb200_overlay::call_count();
    CHECK(thrust::reduce(thrust::cuda::par(alloc), d.begin(), d.end(), 0LL, thrust::plus<long long>()) == want);
    thrust::device_vector<int> ds(d.begin(), d.end());
    thrust::sort(thrust::cuda::par(alloc).on(s), ds.begin(), ds.end());
    std::vector<int> hsorted(h.begin(), h.end()); std::sort(hsorted.begin(), hsorted.end());
    got = ds; CHECK(std::equal(hsorted.begin(), hsorted.end(), got.begin()));
    CHECK(served >= 2 && thrust::cuda_cub::tb200_overlay::call_count() == before + 2); }

  // thrust::async: the same kernels without the final wait
  { const unsigned long long before = thrust::cuda_cub::tb200_overlay::call_count();
    auto fut = thrust::async::reduce(thrust::device, d.begin(), d.end(), 0LL, thrust::plus<long long>());
    thrust::device_vector<int> din(small.begin(), small.end()), dout(n), dex(n);
    auto e1 = thrust::async::inclusive_scan(thrust::device, din.begin(), din.end(), dout.begin());
    auto e2 = thrust::async::exclusive_scan(thrust::device, din.begin(), din.end(), dex.begin(), 7);
    thrust::device_vector<int> da2(d.begin(), d.end());
    auto e3 = thrust::async::sort(thrust::device, da2.begin(), da2.end());
    CHECK(fut.get() == want);
    e1.wait(); e2.wait(); e3.wait();
    std::vector<int> hi(n); std::partial_sum(small.begin(), small.end(), hi.begin());
    got = dout; CHECK(std::equal(hi.begin(), hi.end(), got.begin()));
    got = dex; ok = got[0] == 7; for (int i = 1; i < n && ok; ++i) ok = got[i] == hi[i - 1] + 7; CHECK(ok);
    std::vector<int> hsorted(h.begin(), h.end()); std::sort(hsorted.begin(), hsorted.end());
    got = da2; CHECK(std::equal(hsorted.begin(), hsorted.end(), got.begin()));
    CHECK(thrust::cuda_cub::tb200_overlay::call_count() == before + 4); }

  // thrust::mr: a pool resource behind thrust::mr::allocator handed to par(alloc) -- the temporary
  // storage of the kernels comes out of the pool, and the second call is served from what the first
  // one returned to it (nothing new reaches the upstream resource)
  { counting_resource upstream;
    thrust::mr::new_delete_resource bookkeeper;
    typedef thrust::mr::disjoint_unsynchronized_pool_resource<counting_resource, thrust::mr::new_delete_resource> pool_t;
    pool_t pool(&upstream, &bookkeeper);
    thrust::mr::allocator<char, pool_t> alloc(&pool);
    const unsigned long long before = thrust::cuda_cub::tb200_overlay::call_count();
    thrust::device_vector<int> ds(d.begin(), d.end());
    thrust::sort(thrust::cuda::par(alloc), ds.begin(), ds.end());
    const int after_first = upstream.allocations;
    thrust::device_vector<int> ds2(d.begin(), d.end());
    thrust::sort(thrust::cuda::par(alloc), ds2.begin(), ds2.end());
    std::vector<int> hsorted(h.begin(), h.end()); std::sort(hsorted.begin(), hsorted.end());
    got = ds; CHECK(std::equal(hsorted.begin(), hsorted.end(), got.begin()));
    got = ds2; CHECK(std::equal(hsorted.begin(), hsorted.end(), got.begin()));
    CHECK(after_first >= 1 && upstream.allocations == after_first);
    CHECK(thrust::cuda_cub::tb200_overlay::call_count() == before + 2); }

  // callers that arrive through a transform_iterator, on an input large enough for the routes that
  // large inputs take (the windowed scan with one element per load, the reduce with sixteen loads in flight)
  { const int big = (1 << 25) + 7;
    thrust::device_vector<int> bx(big), by(big), bz(big);
    thrust::sequence(bx.begin(), bx.end(), 5);
    thrust::transform_inclusive_scan(thrust::device, bx.begin(), bx.end(), by.begin(), low3(), thrust::plus<int>());
    thrust::transform_exclusive_scan(thrust::device, bx.begin(), bx.end(), bz.begin(), low3(), 11, thrust::plus<int>());
    thrust::host_vector<int> gy = by, gz = bz;
    ok = true; { int run = 0; for (int i = 0; i < big && ok; ++i) { ok = gz[i] == 11 + run; run += (i + 5) & 7; ok = ok && gy[i] == run; } }
    CHECK(ok);
    const long long odd = thrust::count_if(thrust::device, bx.begin(), bx.end(), is_odd_int());
    CHECK(odd == (long long)((big + 1) / 2));      // the values run from 5 to big + 4, both odd
    const long long sq = thrust::transform_reduce(thrust::device, bx.begin(), bx.begin() + 100000, square(), 0LL, thrust::plus<long long>());
    long long want_sq2 = 0; for (long long i = 0; i < 100000; ++i) want_sq2 += (i + 5) * (i + 5);
    CHECK(sq == want_sq2); }

  // the overlay, not the stock CUB path, served these calls
  std::printf("overlay served %llu calls\n", thrust::cuda_cub::tb200_overlay::call_count());
  CHECK(thrust::cuda_cub::tb200_overlay::call_count() == 44);
  cudaStreamDestroy(s);
  if (cudaDeviceSynchronize() != cudaSuccess) { std::printf("FAILED: sticky CUDA error\n"); ++failures; }
  std::printf(failures ? "dropin_test: %d FAILURES\n" : "dropin_test: all checks passed\n", failures);
  return failures ? 1 : 0;
}
