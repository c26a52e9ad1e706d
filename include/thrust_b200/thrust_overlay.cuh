// Drop-in for existing Thrust callers: makes thrust::reduce, inclusive_scan / exclusive_scan,
// sort / stable_sort / sort_by_key / stable_sort_by_key, copy_if, partition / stable_partition /
// partition_copy / stable_partition_copy, unique / unique_copy, reduce_by_key, merge and
// merge_by_key under thrust::device, thrust::cuda::par, thrust::cuda::par.on(stream),
// thrust::cuda::par_nosync(.on(stream)) and device_vector iterators run on the sm_100a kernels of
// this library instead of the CUB-based implementations of thrust/system/cuda/detail/{reduce,scan,
// sort,copy_if,partition,unique,reduce_by_key,merge}.h.
//
// How: Thrust dispatches every algorithm by an unqualified call on the concrete policy object
// (thrust/detail/reduce.inl:57-76 and its siblings), which argument-dependent lookup resolves in
// namespace thrust::cuda_cub (thrust/system/cuda/detail/reduce.h:1031-1043).  This header adds, to
// that namespace, overloads whose first parameter is the concrete policy type itself.  For the
// policy types listed in is_overlaid_policy they are an exact match where the stock overloads need
// a derived-to-base conversion to execution_policy<Derived>&, so overload resolution picks them; for
// any other policy (a user-derived one, par(allocator)) the stock code still runs.  Include this
// header after the Thrust headers (or force-include it with `nvcc -include`); no file of the Thrust
// installation is shadowed or modified.
//
// Inside, contiguous iterators over arithmetic types are unwrapped to raw pointers and take the
// vectorised kernels; any other iterator or functor instantiates the same kernel templates on the
// caller's types (stream compaction with a user predicate, reduce of a transform_iterator, merge
// sort with a user comparator on zip keys, ...).  Temporary storage comes from the policy through
// thrust::detail::temporary_array, as in the reference (reduce.h:959); work runs on
// cuda_cub::stream(policy); every call returns synchronised, like the reference (scan.h:117,
// sort.h:1609); errors surface as thrust::system_error via cuda_cub::throw_on_error
// (detail/util.h:180-243).  Device-side (CDP) invocation is not supported.
#pragma once

#include <thrust/detail/config.h>
#include <thrust/detail/execute_with_allocator.h>
#include <thrust/detail/raw_pointer_cast.h>
#include <thrust/detail/temporary_array.h>
#include <thrust/distance.h>
#include <thrust/execution_policy.h>
#include <thrust/functional.h>
#include <thrust/iterator/iterator_traits.h>
#include <thrust/iterator/transform_iterator.h>
#include <thrust/iterator/zip_iterator.h>
#include <thrust/zip_function.h>
#include <thrust/detail/internal_functional.h>
#include <thrust/pair.h>
#include <thrust/system/cuda/detail/par.h>
#include <thrust/system/cuda/detail/util.h>
#include <thrust/system/cuda/execution_policy.h>
#include <thrust/type_traits/is_contiguous_iterator.h>

#include <cstdint>
#include <type_traits>
#include <vector>

#include "extrema.cuh"
#include "merge.cuh"
#include "radix_sort.cuh"
#include "reduce.cuh"
#include "reduce_by_key.cuh"
#include "scan.cuh"
#include "scan_by_key.cuh"
#include "select.cuh"
#include "set_ops.cuh"

THRUST_NAMESPACE_BEGIN
namespace cuda_cub {

namespace tb200_overlay {

template <class P> struct is_overlaid_policy : std::false_type {};
template <> struct is_overlaid_policy<par_t> : std::true_type {};
template <> struct is_overlaid_policy<par_nosync_t> : std::true_type {};
template <> struct is_overlaid_policy<execute_on_stream> : std::true_type {};
template <> struct is_overlaid_policy<execute_on_stream_nosync> : std::true_type {};
template <> struct is_overlaid_policy<tag> : std::true_type {};
// thrust::cuda::par(alloc), par.on(stream)(alloc), par_nosync(alloc): the same kernels, with
// temporary storage drawn from the caller's allocator (thrust/system/cuda/detail/par.h:86-108,
// thrust/detail/allocator_aware_execution_policy.h)
template <template <class> class Base> struct is_cuda_policy_base : std::false_type {};
template <> struct is_cuda_policy_base<execute_on_stream_base> : std::true_type {};
template <> struct is_cuda_policy_base<execute_on_stream_nosync_base> : std::true_type {};
template <class Alloc, template <class> class Base>
struct is_overlaid_policy<thrust::detail::execute_with_allocator<Alloc, Base>> : is_cuda_policy_base<Base> {};
template <class P> using enable_for = typename std::enable_if<is_overlaid_policy<P>::value, int>::type;

template <class It> using value_t = typename thrust::iterator_traits<It>::value_type;

// contiguous iterator -> raw pointer; anything else unchanged
template <class It, typename std::enable_if<thrust::is_contiguous_iterator<It>::value, int>::type = 0>
auto unwrap(It it) -> decltype(thrust::raw_pointer_cast(&*it)) { return thrust::raw_pointer_cast(&*it); }
template <class It, typename std::enable_if<!thrust::is_contiguous_iterator<It>::value, int>::type = 0>
It unwrap(It it) { return it; }

// Thrust functors -> this library's (so that the arithmetic fast paths are recognised), but only
// where they mean the same: thrust::plus<Acc> or the transparent thrust::plus<> on an accumulator of
// type Acc.  thrust::plus<int> on floats truncates its operands (testing/scan.cu:258-264 relies on
// it), so it stays the caller's functor, like every user functor.
template <class F, class Acc> struct map_op { using type = F; static type get(const F& f) { return f; } };
template <class Acc> struct map_op<thrust::plus<Acc>, Acc> { using type = ::tb200::plus_op; static type get(const thrust::plus<Acc>&) { return {}; } };
template <class Acc> struct map_op<thrust::plus<void>, Acc> { using type = ::tb200::plus_op; static type get(const thrust::plus<void>&) { return {}; } };
template <class Acc> struct map_op<thrust::minimum<Acc>, Acc> { using type = ::tb200::min_op; static type get(const thrust::minimum<Acc>&) { return {}; } };
template <class Acc> struct map_op<thrust::minimum<void>, Acc> { using type = ::tb200::min_op; static type get(const thrust::minimum<void>&) { return {}; } };
template <class Acc> struct map_op<thrust::maximum<Acc>, Acc> { using type = ::tb200::max_op; static type get(const thrust::maximum<Acc>&) { return {}; } };
template <class Acc> struct map_op<thrust::maximum<void>, Acc> { using type = ::tb200::max_op; static type get(const thrust::maximum<void>&) { return {}; } };

template <class Comp, class K> struct radix_order { static constexpr int value = -1; };                       // -1: not a radix order
template <class K> struct radix_order<thrust::less<K>, K> { static constexpr int value = 0; };
template <class K> struct radix_order<thrust::less<void>, K> { static constexpr int value = 0; };
template <class K> struct radix_order<thrust::greater<K>, K> { static constexpr int value = 1; };
template <class K> struct radix_order<thrust::greater<void>, K> { static constexpr int value = 1; };

template <class K> struct radix_key {
  static constexpr bool ok = std::is_arithmetic<K>::value && !std::is_same<K, bool>::value && sizeof(K) <= 8;
  using bits = typename std::conditional<sizeof(K) == 1, std::uint8_t,
               typename std::conditional<sizeof(K) == 2, std::uint16_t,
               typename std::conditional<sizeof(K) == 4, std::uint32_t, unsigned long long>::type>::type>::type;
  static constexpr int kind = std::is_floating_point<K>::value ? ::tb200::KEY_FLOAT : (std::is_signed<K>::value ? ::tb200::KEY_SIGNED : ::tb200::KEY_UNSIGNED);
};

// number of algorithm calls this overlay has served in this process (lets a caller verify that it is active)
inline unsigned long long& call_count() { static unsigned long long c = 0; return c; }

// Temporary storage.  A policy that carries an allocator takes it from that allocator, through
// thrust::detail::temporary_array, as in the reference (thrust/system/cuda/detail/par.h:86-108).
// The other policies would pay a cudaMalloc and a cudaFree per call there (reduce.h:959), several
// times the cost of reducing a gigabyte; for them each host thread keeps one buffer per (device,
// stream), grown on demand and released when the thread ends.  Calls of one thread on one stream
// are ordered on that stream, so they can share it.  -DTHRUST_B200_NO_SCRATCH_CACHE restores the
// allocation per call.
template <class P> struct has_allocator : std::false_type {};
template <class Alloc, template <class> class Base> struct has_allocator<thrust::detail::execute_with_allocator<Alloc, Base>> : std::true_type {};

struct scratch_cache {
  struct entry { int device; cudaStream_t stream; void* p; std::size_t bytes; bool busy; };
  std::vector<entry> entries;
  ~scratch_cache() { for (entry& e : entries) if (e.p) cudaFree(e.p); }            // errors at process exit are not reported
  // the (device, stream) buffer of at least `bytes`, marked busy; nullptr if a call further up the
  // stack of this thread is using it (the caller then allocates for itself)
  void* acquire(cudaStream_t stream, std::size_t bytes, std::size_t& slot) {
    int device = 0;
    cuda_cub::throw_on_error(cudaGetDevice(&device), "temporary storage: no current device");
    entry* hit = nullptr;
    for (entry& e : entries) if (e.device == device && e.stream == stream) { hit = &e; break; }
    if (!hit) { entries.push_back(entry{device, stream, nullptr, 0, false}); hit = &entries.back(); }
    if (hit->busy) return nullptr;
    slot = (std::size_t)(hit - entries.data());
    if (hit->bytes < bytes) {
      if (hit->p) {                                                                  // earlier work on the stream may still use it
        cuda_cub::throw_on_error(cudaStreamSynchronize(stream), "temporary storage: failed to synchronize");
        cuda_cub::throw_on_error(cudaFree(hit->p), "temporary storage: free failed");
        hit->p = nullptr; hit->bytes = 0;
      }
      const std::size_t want = bytes + bytes / 4;
      cuda_cub::throw_on_error(cudaMalloc(&hit->p, want), "temporary storage: allocation failed");
      hit->bytes = want;
    }
    hit->busy = true;
    return hit->p;
  }
  void release(std::size_t slot) { entries[slot].busy = false; }
};
inline scratch_cache& thread_scratch_cache() { static thread_local scratch_cache c; return c; }

#ifdef THRUST_B200_NO_SCRATCH_CACHE
template <class Policy, bool FROM_POLICY = true> struct scratch;
#else
template <class Policy, bool FROM_POLICY = has_allocator<Policy>::value> struct scratch;
#endif
// workspace + result read-back shared by all wrappers
template <class Policy> struct scratch<Policy, true> {
  thrust::detail::temporary_array<std::uint8_t, Policy> storage;
  scratch(Policy& policy, std::size_t bytes) : storage(policy, bytes + 256) { ++call_count(); }
  std::uint8_t* at(std::size_t offset = 0) {
    std::uint8_t* p = thrust::raw_pointer_cast(storage.data());
    std::uintptr_t a = (reinterpret_cast<std::uintptr_t>(p) + 255) & ~std::uintptr_t(255);
    return reinterpret_cast<std::uint8_t*>(a) + offset;
  }
};
template <class Policy> struct scratch<Policy, false> {
  std::uint8_t* base;
  std::size_t slot = 0;
  bool own = false;                                    // a nested call: allocated here, freed here
  scratch(Policy& policy, std::size_t bytes) {
    ++call_count();
    // requests above 256 MiB (the alternate buffers of a large sort) are not worth keeping: the
    // allocation is small beside the work, and the memory would stay with the thread
    base = bytes > (std::size_t(256) << 20) ? nullptr
                                            : static_cast<std::uint8_t*>(thread_scratch_cache().acquire(cuda_cub::stream(policy), bytes + 256, slot));
    if (!base) {
      void* p = nullptr;
      cuda_cub::throw_on_error(cudaMalloc(&p, bytes + 256), "temporary storage: allocation failed");
      base = static_cast<std::uint8_t*>(p);
      own = true;
    }
  }
  scratch(const scratch&) = delete;
  scratch& operator=(const scratch&) = delete;
  ~scratch() {
    if (own) cudaFree(base);                           // synchronises with the work that used it
    else thread_scratch_cache().release(slot);
  }
  std::uint8_t* at(std::size_t offset = 0) {
    std::uintptr_t a = (reinterpret_cast<std::uintptr_t>(base) + 255) & ~std::uintptr_t(255);
    return reinterpret_cast<std::uint8_t*>(a) + offset;
  }
};

// synchronise, surface CUDA errors and the kernels' own status word, return the header's count
template <class Policy>
unsigned long long finish(Policy& policy, cudaError_t launch_status, const void* ws, const char* what) {
  cuda_cub::throw_on_error(launch_status, what);
  ::tb200::ws_header h;
  cuda_cub::throw_on_error(cudaMemcpyAsync(&h, ws, 16, cudaMemcpyDeviceToHost, cuda_cub::stream(policy)), what);
  cuda_cub::throw_on_error(cudaStreamSynchronize(cuda_cub::stream(policy)), what);
  if (h.error != ::tb200::ERR_NONE) cuda_cub::throw_on_error(cudaErrorLaunchTimeout, "thrust_b200: an inter-CTA wait ran out");
  return h.count;
}

constexpr std::size_t up256(std::size_t x) { return (x + 255) / 256 * 256; }

}  // namespace tb200_overlay

// ------------------------------------------------------------------------------------- reduce
// replaces cuda_cub::reduce_n / reduce (thrust/system/cuda/detail/reduce.h:1015-1067)
template <class Policy, class InputIt, class Size, class T, class BinaryOp, tb200_overlay::enable_for<Policy> = 0>
T reduce_n(Policy& policy, InputIt first, Size num_items, T init, BinaryOp binary_op) {
  namespace ov = tb200_overlay;
  if (num_items <= 0) return init;                                                    // reduce.h:863-864
  ov::scratch<Policy> tmp(policy, ::tb200::reduce_workspace_bytes<T>() + 256);
  T* d_out = reinterpret_cast<T*>(tmp.at(ov::up256(::tb200::reduce_workspace_bytes<T>())));
  cudaError_t e = ::tb200::reduce_async(ov::unwrap(first), (std::size_t)num_items, init, ov::map_op<BinaryOp, T>::get(binary_op), d_out, tmp.at(),
                                        cuda_cub::stream(policy));
  cuda_cub::throw_on_error(e, "reduce: launch failed");
  T result;
  cuda_cub::throw_on_error(cudaMemcpyAsync(&result, d_out, sizeof(T), cudaMemcpyDeviceToHost, cuda_cub::stream(policy)), "reduce: read-back failed");
  cuda_cub::throw_on_error(cudaStreamSynchronize(cuda_cub::stream(policy)), "reduce: failed to synchronize");
  return result;
}
template <class Policy, class InputIt, class T, class BinaryOp, tb200_overlay::enable_for<Policy> = 0>
T reduce(Policy& policy, InputIt first, InputIt last, T init, BinaryOp binary_op) {
  return cuda_cub::reduce_n(policy, first, thrust::distance(first, last), init, binary_op);
}
template <class Policy, class InputIt, class T, tb200_overlay::enable_for<Policy> = 0>
T reduce(Policy& policy, InputIt first, InputIt last, T init) {
  return cuda_cub::reduce(policy, first, last, init, thrust::plus<T>());
}
template <class Policy, class InputIt, tb200_overlay::enable_for<Policy> = 0>
tb200_overlay::value_t<InputIt> reduce(Policy& policy, InputIt first, InputIt last) {
  using T = tb200_overlay::value_t<InputIt>;
  return cuda_cub::reduce(policy, first, last, T(0));                                  // reduce.h:1057-1067
}

// ------------------------------------------------------------------------------------- scan
// replaces cuda_cub::inclusive_scan(_n) / exclusive_scan(_n) (thrust/system/cuda/detail/scan.h:215-361)
namespace tb200_overlay {
template <bool INCLUSIVE, class Policy, class InputIt, class OutputIt, class T, class ScanOp>
OutputIt scan_n(Policy& policy, InputIt first, std::size_t n, OutputIt result, T init, bool has_init, ScanOp op) {
  if (n == 0) return result;
  scratch<Policy> tmp(policy, ::tb200::scan_workspace_bytes<T>(n));
  cudaError_t e = ::tb200::scan_async<INCLUSIVE>(unwrap(first), unwrap(result), n, init, has_init, map_op<ScanOp, T>::get(op), tmp.at(), cuda_cub::stream(policy));
  finish(policy, e, tmp.at(), INCLUSIVE ? "inclusive_scan failed" : "exclusive_scan failed");
  return result + n;
}
}  // namespace tb200_overlay

template <class Policy, class InputIt, class Size, class OutputIt, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutputIt inclusive_scan_n(Policy& policy, InputIt first, Size num_items, OutputIt result, ScanOp scan_op) {
  using T = tb200_overlay::value_t<InputIt>;                                          // accumulates in the input value type (P0571)
  return tb200_overlay::scan_n<true>(policy, first, (std::size_t)num_items, result, T(), false, scan_op);
}
template <class Policy, class InputIt, class OutputIt, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutputIt inclusive_scan(Policy& policy, InputIt first, InputIt last, OutputIt result, ScanOp scan_op) {
  return cuda_cub::inclusive_scan_n(policy, first, thrust::distance(first, last), result, scan_op);
}
template <class Policy, class InputIt, class OutputIt, tb200_overlay::enable_for<Policy> = 0>
OutputIt inclusive_scan(Policy& policy, InputIt first, InputIt last, OutputIt result) {
  return cuda_cub::inclusive_scan(policy, first, last, result, thrust::plus<>());
}
template <class Policy, class InputIt, class Size, class OutputIt, class T, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutputIt exclusive_scan_n(Policy& policy, InputIt first, Size num_items, OutputIt result, T init, ScanOp scan_op) {
  return tb200_overlay::scan_n<false>(policy, first, (std::size_t)num_items, result, init, true, scan_op);   // accumulates in the init type
}
template <class Policy, class InputIt, class OutputIt, class T, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutputIt exclusive_scan(Policy& policy, InputIt first, InputIt last, OutputIt result, T init, ScanOp scan_op) {
  return cuda_cub::exclusive_scan_n(policy, first, thrust::distance(first, last), result, init, scan_op);
}
template <class Policy, class InputIt, class OutputIt, class T, tb200_overlay::enable_for<Policy> = 0>
OutputIt exclusive_scan(Policy& policy, InputIt first, InputIt last, OutputIt result, T init) {
  return cuda_cub::exclusive_scan(policy, first, last, result, init, thrust::plus<>());
}
template <class Policy, class InputIt, class OutputIt, tb200_overlay::enable_for<Policy> = 0>
OutputIt exclusive_scan(Policy& policy, InputIt first, InputIt last, OutputIt result) {
  using T = tb200_overlay::value_t<InputIt>;
  return cuda_cub::exclusive_scan(policy, first, last, result, T{});                   // scan.h:359-360
}

// ------------------------------------------------------------------------------------- sort
// replaces cuda_cub::sort / stable_sort / sort_by_key / stable_sort_by_key (thrust/system/cuda/detail/sort.h:1621-1754)
namespace tb200_overlay {
struct no_items {};

// keys (and items) are contiguous raw pointers here
template <class Policy, class K, class V, bool HAS_V, class Comp>
void sort_raw(Policy& policy, K* keys, V* items, std::size_t n, Comp comp) {
  if (n <= 1) return;
  constexpr int order = radix_order<Comp, K>::value;
  const std::size_t kb = up256(n * sizeof(K)), vb = HAS_V ? up256(n * sizeof(V)) : 0;
  if constexpr (radix_key<K>::ok && order >= 0 && (!HAS_V || sizeof(V) == 4 || sizeof(V) == 8) && (!HAS_V || std::is_trivially_copyable<V>::value)) {
    // primitive key with less / greater: radix path (sort.h:1517-1523)
    using UK = typename radix_key<K>::bits;
    using UV = typename std::conditional<(HAS_V && sizeof(V) == 8), unsigned long long, std::uint32_t>::type;
    const std::size_t wsb = up256(::tb200::radix_workspace_bytes<sizeof(UK), HAS_V ? sizeof(UV) : 0>(n));
    scratch<Policy> tmp(policy, wsb + kb + vb);
    ::tb200::key_coding coding{radix_key<K>::kind, order};
    cudaError_t e = ::tb200::radix_sort_async<UK, UV, HAS_V>(reinterpret_cast<UK*>(keys), reinterpret_cast<UK*>(tmp.at(wsb)), reinterpret_cast<UV*>(items),
                                                          reinterpret_cast<UV*>(tmp.at(wsb + kb)), n, coding, 0, 8 * (int)sizeof(K), tmp.at(),
                                                          cuda_cub::stream(policy));
    finish(policy, e, tmp.at(), "sort: radix sort failed");
  } else {
    // anything else: stable merge sort with the caller's comparator (sort.h:1544-1557)
    using VV = typename std::conditional<HAS_V, V, std::uint32_t>::type;
    const std::size_t wsb = up256(::tb200::merge_sort_workspace_bytes<K, VV, HAS_V>(n));
    scratch<Policy> tmp(policy, wsb + kb + vb);
    cudaError_t e = ::tb200::merge_sort_async<K, VV, HAS_V>(keys, reinterpret_cast<K*>(tmp.at(wsb)), reinterpret_cast<VV*>(items),
                                                          reinterpret_cast<VV*>(tmp.at(wsb + kb)), n, comp, tmp.at(), cuda_cub::stream(policy));
    finish(policy, e, tmp.at(), "sort: merge sort failed");
  }
}

// copies a non-contiguous range into a contiguous temporary and back (the reference's trivial_sequence, sort.h:1573-1607)
template <class Policy, class It> struct contiguous_copy {
  using T = value_t<It>;
  thrust::detail::temporary_array<T, Policy> buf;
  Policy& pol; It first; std::size_t n;
  contiguous_copy(Policy& policy, It f, std::size_t count) : buf(policy, f, f + count), pol(policy), first(f), n(count) {}
  T* data() { return thrust::raw_pointer_cast(buf.data()); }
  void write_back() { thrust::copy(pol, buf.begin(), buf.end(), first); }
};

template <class Policy, class KeysIt, class ItemsIt, bool HAS_V, class Comp>
void sort_any(Policy& policy, KeysIt keys_first, KeysIt keys_last, ItemsIt items_first, Comp comp) {
  using K = value_t<KeysIt>;
  const std::size_t n = (std::size_t)thrust::distance(keys_first, keys_last);
  if (n <= 1) return;
  if constexpr (thrust::is_contiguous_iterator<KeysIt>::value && (!HAS_V || thrust::is_contiguous_iterator<ItemsIt>::value)) {
    if constexpr (HAS_V) sort_raw<Policy, K, value_t<ItemsIt>, true>(policy, unwrap(keys_first), unwrap(items_first), n, comp);
    else sort_raw<Policy, K, std::uint32_t, false>(policy, unwrap(keys_first), (std::uint32_t*)nullptr, n, comp);
  } else if constexpr (HAS_V) {
    contiguous_copy<Policy, KeysIt> k(policy, keys_first, n);
    contiguous_copy<Policy, ItemsIt> v(policy, items_first, n);
    sort_raw<Policy, K, value_t<ItemsIt>, true>(policy, k.data(), v.data(), n, comp);
    k.write_back();
    v.write_back();
  } else {
    contiguous_copy<Policy, KeysIt> k(policy, keys_first, n);
    sort_raw<Policy, K, std::uint32_t, false>(policy, k.data(), (std::uint32_t*)nullptr, n, comp);
    k.write_back();
  }
}
}  // namespace tb200_overlay

template <class Policy, class It, class Comp, tb200_overlay::enable_for<Policy> = 0>
void stable_sort(Policy& policy, It first, It last, Comp comp) { tb200_overlay::sort_any<Policy, It, It, false>(policy, first, last, first, comp); }
template <class Policy, class It, class Comp, tb200_overlay::enable_for<Policy> = 0>
void sort(Policy& policy, It first, It last, Comp comp) { cuda_cub::stable_sort(policy, first, last, comp); }
template <class Policy, class It, tb200_overlay::enable_for<Policy> = 0>
void stable_sort(Policy& policy, It first, It last) { cuda_cub::stable_sort(policy, first, last, thrust::less<tb200_overlay::value_t<It>>()); }
template <class Policy, class It, tb200_overlay::enable_for<Policy> = 0>
void sort(Policy& policy, It first, It last) { cuda_cub::stable_sort(policy, first, last); }
template <class Policy, class KeysIt, class ValuesIt, class Comp, tb200_overlay::enable_for<Policy> = 0>
void stable_sort_by_key(Policy& policy, KeysIt keys_first, KeysIt keys_last, ValuesIt values, Comp comp) {
  tb200_overlay::sort_any<Policy, KeysIt, ValuesIt, true>(policy, keys_first, keys_last, values, comp);
}
template <class Policy, class KeysIt, class ValuesIt, class Comp, tb200_overlay::enable_for<Policy> = 0>
void sort_by_key(Policy& policy, KeysIt keys_first, KeysIt keys_last, ValuesIt values, Comp comp) {
  cuda_cub::stable_sort_by_key(policy, keys_first, keys_last, values, comp);
}
template <class Policy, class KeysIt, class ValuesIt, tb200_overlay::enable_for<Policy> = 0>
void stable_sort_by_key(Policy& policy, KeysIt keys_first, KeysIt keys_last, ValuesIt values) {
  cuda_cub::stable_sort_by_key(policy, keys_first, keys_last, values, thrust::less<tb200_overlay::value_t<KeysIt>>());
}
template <class Policy, class KeysIt, class ValuesIt, tb200_overlay::enable_for<Policy> = 0>
void sort_by_key(Policy& policy, KeysIt keys_first, KeysIt keys_last, ValuesIt values) {
  cuda_cub::stable_sort_by_key(policy, keys_first, keys_last, values);
}

// ------------------------------------------------------------------------------------- copy_if
// replaces cuda_cub::copy_if (thrust/system/cuda/detail/copy_if.h:780-853)
template <class Policy, class InputIt, class OutputIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
OutputIt copy_if(Policy& policy, InputIt first, InputIt last, OutputIt result, Pred pred) {
  namespace ov = tb200_overlay;
  using T = ov::value_t<InputIt>;
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return result;                                                           // copy_if.h:713-714
  ov::scratch<Policy> tmp(policy, ::tb200::select_workspace_bytes<T>(n));
  auto in = ov::unwrap(first);
  auto out = ov::unwrap(result);
  cudaError_t e = ::tb200::select_async<::tb200::SEL_PRED, false>(in, in, out, out, n, T(), pred, false, nullptr, tmp.at(), cuda_cub::stream(policy));
  return result + ov::finish(policy, e, tmp.at(), "copy_if failed");
}
template <class Policy, class InputIt, class StencilIt, class OutputIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
OutputIt copy_if(Policy& policy, InputIt first, InputIt last, StencilIt stencil, OutputIt result, Pred pred) {
  namespace ov = tb200_overlay;
  using T = ov::value_t<InputIt>;
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return result;
  ov::scratch<Policy> tmp(policy, ::tb200::select_workspace_bytes<T>(n));
  auto out = ov::unwrap(result);
  cudaError_t e = ::tb200::select_async<::tb200::SEL_STENCIL, false>(ov::unwrap(first), ov::unwrap(stencil), out, out, n, T(), pred, false, nullptr, tmp.at(),
                                                                   cuda_cub::stream(policy));
  return result + ov::finish(policy, e, tmp.at(), "copy_if failed");
}

// ------------------------------------------------------------------------------------- partition
// replaces cuda_cub::partition_copy / stable_partition_copy / partition / stable_partition (thrust/system/cuda/detail/partition.h:833-1132)
template <class Policy, class InputIt, class SelectedOutIt, class RejectedOutIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<SelectedOutIt, RejectedOutIt> stable_partition_copy(Policy& policy, InputIt first, InputIt last, SelectedOutIt selected, RejectedOutIt rejected, Pred pred) {
  namespace ov = tb200_overlay;
  using T = ov::value_t<InputIt>;
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return thrust::make_pair(selected, rejected);
  ov::scratch<Policy> tmp(policy, ::tb200::select_workspace_bytes<T>(n));
  auto in = ov::unwrap(first);
  cudaError_t e = ::tb200::select_async<::tb200::SEL_PRED, true>(in, in, ov::unwrap(selected), ov::unwrap(rejected), n, T(), pred, false, nullptr, tmp.at(),
                                                               cuda_cub::stream(policy));
  const std::size_t k = ov::finish(policy, e, tmp.at(), "partition_copy failed");
  return thrust::make_pair(selected + k, rejected + (n - k));
}
template <class Policy, class InputIt, class StencilIt, class SelectedOutIt, class RejectedOutIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<SelectedOutIt, RejectedOutIt> stable_partition_copy(Policy& policy, InputIt first, InputIt last, StencilIt stencil, SelectedOutIt selected,
                                                                  RejectedOutIt rejected, Pred pred) {
  namespace ov = tb200_overlay;
  using T = ov::value_t<InputIt>;
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return thrust::make_pair(selected, rejected);
  ov::scratch<Policy> tmp(policy, ::tb200::select_workspace_bytes<T>(n));
  cudaError_t e = ::tb200::select_async<::tb200::SEL_STENCIL, true>(ov::unwrap(first), ov::unwrap(stencil), ov::unwrap(selected), ov::unwrap(rejected), n, T(), pred,
                                                                  false, nullptr, tmp.at(), cuda_cub::stream(policy));
  const std::size_t k = ov::finish(policy, e, tmp.at(), "partition_copy failed");
  return thrust::make_pair(selected + k, rejected + (n - k));
}
template <class Policy, class InputIt, class SelectedOutIt, class RejectedOutIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<SelectedOutIt, RejectedOutIt> partition_copy(Policy& policy, InputIt first, InputIt last, SelectedOutIt selected, RejectedOutIt rejected, Pred pred) {
  return cuda_cub::stable_partition_copy(policy, first, last, selected, rejected, pred);
}
template <class Policy, class InputIt, class StencilIt, class SelectedOutIt, class RejectedOutIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<SelectedOutIt, RejectedOutIt> partition_copy(Policy& policy, InputIt first, InputIt last, StencilIt stencil, SelectedOutIt selected,
                                                           RejectedOutIt rejected, Pred pred) {
  return cuda_cub::stable_partition_copy(policy, first, last, stencil, selected, rejected, pred);
}
// in place: kept items first and dropped items mirrored into a scratch copy, then written back in
// order -- always the stable result, which also satisfies thrust::partition
template <class Policy, class It, class Pred, tb200_overlay::enable_for<Policy> = 0>
It stable_partition(Policy& policy, It first, It last, Pred pred) {
  namespace ov = tb200_overlay;
  using T = ov::value_t<It>;
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return first;
  const std::size_t wsb = ov::up256(::tb200::select_workspace_bytes<T>(n));
  ov::scratch<Policy> tmp(policy, wsb + n * sizeof(T));
  T* copy = reinterpret_cast<T*>(tmp.at(wsb));
  auto in = ov::unwrap(first);
  cudaError_t e = ::tb200::select_async<::tb200::SEL_PRED, true>(in, in, copy, copy, n, T(), pred, true, nullptr, tmp.at(), cuda_cub::stream(policy));
  cuda_cub::throw_on_error(e, "partition failed");
  const ::tb200::device_info& di = ::tb200::current_device_info();
  std::size_t grid = (n + 2047) / 2048;
  if (grid > (std::size_t)di.sm_count * 8) grid = (std::size_t)di.sm_count * 8;
  ::tb200::partition_finish_kernel<<<(unsigned)grid, 256, 0, cuda_cub::stream(policy)>>>(in, (const T*)copy, n, reinterpret_cast<const ::tb200::ws_header*>(tmp.at()));
  return first + ov::finish(policy, cudaGetLastError(), tmp.at(), "partition failed");
}
template <class Policy, class It, class StencilIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
It stable_partition(Policy& policy, It first, It last, StencilIt stencil, Pred pred) {
  namespace ov = tb200_overlay;
  using T = ov::value_t<It>;
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return first;
  const std::size_t wsb = ov::up256(::tb200::select_workspace_bytes<T>(n));
  ov::scratch<Policy> tmp(policy, wsb + n * sizeof(T));
  T* copy = reinterpret_cast<T*>(tmp.at(wsb));
  auto in = ov::unwrap(first);
  cudaError_t e = ::tb200::select_async<::tb200::SEL_STENCIL, true>(in, ov::unwrap(stencil), copy, copy, n, T(), pred, true, nullptr, tmp.at(), cuda_cub::stream(policy));
  cuda_cub::throw_on_error(e, "partition failed");
  const ::tb200::device_info& di = ::tb200::current_device_info();
  std::size_t grid = (n + 2047) / 2048;
  if (grid > (std::size_t)di.sm_count * 8) grid = (std::size_t)di.sm_count * 8;
  ::tb200::partition_finish_kernel<<<(unsigned)grid, 256, 0, cuda_cub::stream(policy)>>>(in, (const T*)copy, n, reinterpret_cast<const ::tb200::ws_header*>(tmp.at()));
  return first + ov::finish(policy, cudaGetLastError(), tmp.at(), "partition failed");
}
template <class Policy, class It, class Pred, tb200_overlay::enable_for<Policy> = 0>
It partition(Policy& policy, It first, It last, Pred pred) { return cuda_cub::stable_partition(policy, first, last, pred); }
template <class Policy, class It, class StencilIt, class Pred, tb200_overlay::enable_for<Policy> = 0>
It partition(Policy& policy, It first, It last, StencilIt stencil, Pred pred) { return cuda_cub::stable_partition(policy, first, last, stencil, pred); }

// ------------------------------------------------------------------------------------- unique
// replaces cuda_cub::unique / unique_copy (thrust/system/cuda/detail/unique.h:710-795)
template <class Policy, class InputIt, class OutputIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
OutputIt unique_copy(Policy& policy, InputIt first, InputIt last, OutputIt result, BinaryPred binary_pred) {
  namespace ov = tb200_overlay;
  using T = ov::value_t<InputIt>;
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return result;
  ov::scratch<Policy> tmp(policy, ::tb200::select_workspace_bytes<T>(n));
  auto in = ov::unwrap(first);
  auto out = ov::unwrap(result);
  cudaError_t e = ::tb200::select_async<::tb200::SEL_UNIQUE, false>(in, in, out, out, n, T(), binary_pred, false, nullptr, tmp.at(), cuda_cub::stream(policy));
  return result + ov::finish(policy, e, tmp.at(), "unique failed");
}
template <class Policy, class InputIt, class OutputIt, tb200_overlay::enable_for<Policy> = 0>
OutputIt unique_copy(Policy& policy, InputIt first, InputIt last, OutputIt result) {
  return cuda_cub::unique_copy(policy, first, last, result, thrust::equal_to<tb200_overlay::value_t<InputIt>>());
}
template <class Policy, class It, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
It unique(Policy& policy, It first, It last, BinaryPred binary_pred) { return cuda_cub::unique_copy(policy, first, last, first, binary_pred); }   // unique.h:772
template <class Policy, class It, tb200_overlay::enable_for<Policy> = 0>
It unique(Policy& policy, It first, It last) { return cuda_cub::unique(policy, first, last, thrust::equal_to<tb200_overlay::value_t<It>>()); }

// ------------------------------------------------------------------------------------- reduce_by_key
// replaces cuda_cub::reduce_by_key (thrust/system/cuda/detail/reduce_by_key.h:1063-1161)
template <class Policy, class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, class BinaryPred, class BinaryOp, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeyOutIt, ValOutIt> reduce_by_key(Policy& policy, KeyIt keys_first, KeyIt keys_last, ValIt values_first, KeyOutIt keys_output, ValOutIt values_output,
                                               BinaryPred binary_pred, BinaryOp binary_op) {
  namespace ov = tb200_overlay;
  using K = ov::value_t<KeyIt>;
  using V = ov::value_t<ValIt>;
  const std::size_t n = (std::size_t)thrust::distance(keys_first, keys_last);
  if (n == 0) return thrust::make_pair(keys_output, values_output);
  ov::scratch<Policy> tmp(policy, ::tb200::rbk_workspace_bytes<K, V>(n));
  cudaError_t e = ::tb200::reduce_by_key_async(ov::unwrap(keys_first), ov::unwrap(values_first), ov::unwrap(keys_output), ov::unwrap(values_output), n, K(), V(),
                                              binary_pred, ov::map_op<BinaryOp, V>::get(binary_op), nullptr, tmp.at(), cuda_cub::stream(policy));
  const std::size_t runs = ov::finish(policy, e, tmp.at(), "reduce_by_key failed");
  return thrust::make_pair(keys_output + runs, values_output + runs);
}
template <class Policy, class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeyOutIt, ValOutIt> reduce_by_key(Policy& policy, KeyIt keys_first, KeyIt keys_last, ValIt values_first, KeyOutIt keys_output, ValOutIt values_output,
                                               BinaryPred binary_pred) {
  return cuda_cub::reduce_by_key(policy, keys_first, keys_last, values_first, keys_output, values_output, binary_pred, thrust::plus<tb200_overlay::value_t<ValIt>>());
}
template <class Policy, class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeyOutIt, ValOutIt> reduce_by_key(Policy& policy, KeyIt keys_first, KeyIt keys_last, ValIt values_first, KeyOutIt keys_output, ValOutIt values_output) {
  return cuda_cub::reduce_by_key(policy, keys_first, keys_last, values_first, keys_output, values_output, thrust::equal_to<tb200_overlay::value_t<KeyIt>>());
}

// ------------------------------------------------------------------------------------- scan_by_key, unique_by_key
// replaces cuda_cub::inclusive_scan_by_key / exclusive_scan_by_key (thrust/system/cuda/detail/scan_by_key.h)
// and unique_by_key(_copy) (thrust/system/cuda/detail/unique_by_key.h): the first "next" components
template <class Policy, class KeyIt, class ValIt, class OutIt, class BinaryPred, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutIt inclusive_scan_by_key(Policy& policy, KeyIt key_first, KeyIt key_last, ValIt value_first, OutIt value_result, BinaryPred binary_pred, ScanOp scan_op) {
  namespace ov = tb200_overlay;
  using K = ov::value_t<KeyIt>;
  using V = ov::value_t<ValIt>;
  const std::size_t n = (std::size_t)thrust::distance(key_first, key_last);
  if (n == 0) return value_result;
  ov::scratch<Policy> tmp(policy, ::tb200::scan_by_key_workspace_bytes<K, V>(n));
  cudaError_t e = ::tb200::scan_by_key_async<true>(ov::unwrap(key_first), ov::unwrap(value_first), ov::unwrap(value_result), n, K(), V(), binary_pred,
                                                 ov::map_op<ScanOp, V>::get(scan_op), tmp.at(), cuda_cub::stream(policy));
  ov::finish(policy, e, tmp.at(), "inclusive_scan_by_key failed");
  return value_result + n;
}
template <class Policy, class KeyIt, class ValIt, class OutIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
OutIt inclusive_scan_by_key(Policy& policy, KeyIt key_first, KeyIt key_last, ValIt value_first, OutIt value_result, BinaryPred binary_pred) {
  return cuda_cub::inclusive_scan_by_key(policy, key_first, key_last, value_first, value_result, binary_pred, thrust::plus<>());
}
template <class Policy, class KeyIt, class ValIt, class OutIt, tb200_overlay::enable_for<Policy> = 0>
OutIt inclusive_scan_by_key(Policy& policy, KeyIt key_first, KeyIt key_last, ValIt value_first, OutIt value_result) {
  return cuda_cub::inclusive_scan_by_key(policy, key_first, key_last, value_first, value_result, thrust::equal_to<>());
}
template <class Policy, class KeyIt, class ValIt, class OutIt, class Init, class BinaryPred, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutIt exclusive_scan_by_key(Policy& policy, KeyIt key_first, KeyIt key_last, ValIt value_first, OutIt value_result, Init init, BinaryPred binary_pred, ScanOp scan_op) {
  namespace ov = tb200_overlay;
  using K = ov::value_t<KeyIt>;
  using V = Init;                                                                       // accumulates in the init type
  const std::size_t n = (std::size_t)thrust::distance(key_first, key_last);
  if (n == 0) return value_result;
  ov::scratch<Policy> tmp(policy, ::tb200::scan_by_key_workspace_bytes<K, V>(n));
  cudaError_t e = ::tb200::scan_by_key_async<false>(ov::unwrap(key_first), ov::unwrap(value_first), ov::unwrap(value_result), n, K(), init, binary_pred,
                                                  ov::map_op<ScanOp, V>::get(scan_op), tmp.at(), cuda_cub::stream(policy));
  ov::finish(policy, e, tmp.at(), "exclusive_scan_by_key failed");
  return value_result + n;
}
template <class Policy, class KeyIt, class ValIt, class OutIt, class Init, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
OutIt exclusive_scan_by_key(Policy& policy, KeyIt key_first, KeyIt key_last, ValIt value_first, OutIt value_result, Init init, BinaryPred binary_pred) {
  return cuda_cub::exclusive_scan_by_key(policy, key_first, key_last, value_first, value_result, init, binary_pred, thrust::plus<>());
}
template <class Policy, class KeyIt, class ValIt, class OutIt, class Init, tb200_overlay::enable_for<Policy> = 0>
OutIt exclusive_scan_by_key(Policy& policy, KeyIt key_first, KeyIt key_last, ValIt value_first, OutIt value_result, Init init) {
  return cuda_cub::exclusive_scan_by_key(policy, key_first, key_last, value_first, value_result, init, thrust::equal_to<>());
}
template <class Policy, class KeyIt, class ValIt, class OutIt, tb200_overlay::enable_for<Policy> = 0>
OutIt exclusive_scan_by_key(Policy& policy, KeyIt key_first, KeyIt key_last, ValIt value_first, OutIt value_result) {
  return cuda_cub::exclusive_scan_by_key(policy, key_first, key_last, value_first, value_result, tb200_overlay::value_t<ValIt>{});
}
template <class Policy, class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeyOutIt, ValOutIt> unique_by_key_copy(Policy& policy, KeyIt keys_first, KeyIt keys_last, ValIt values_first, KeyOutIt keys_result, ValOutIt values_result,
                                                    BinaryPred binary_pred) {
  return cuda_cub::reduce_by_key(policy, keys_first, keys_last, values_first, keys_result, values_result, binary_pred, ::tb200::first_op());
}
template <class Policy, class KeyIt, class ValIt, class KeyOutIt, class ValOutIt, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeyOutIt, ValOutIt> unique_by_key_copy(Policy& policy, KeyIt keys_first, KeyIt keys_last, ValIt values_first, KeyOutIt keys_result, ValOutIt values_result) {
  return cuda_cub::unique_by_key_copy(policy, keys_first, keys_last, values_first, keys_result, values_result, thrust::equal_to<tb200_overlay::value_t<KeyIt>>());
}
template <class Policy, class KeyIt, class ValIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeyIt, ValIt> unique_by_key(Policy& policy, KeyIt keys_first, KeyIt keys_last, ValIt values_first, BinaryPred binary_pred) {
  return cuda_cub::unique_by_key_copy(policy, keys_first, keys_last, values_first, keys_first, values_first, binary_pred);
}
template <class Policy, class KeyIt, class ValIt, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeyIt, ValIt> unique_by_key(Policy& policy, KeyIt keys_first, KeyIt keys_last, ValIt values_first) {
  return cuda_cub::unique_by_key(policy, keys_first, keys_last, values_first, thrust::equal_to<tb200_overlay::value_t<KeyIt>>());
}

// ------------------------------------------------------------------------------------- merge
// replaces cuda_cub::merge / merge_by_key (thrust/system/cuda/detail/merge.h:862-1013)
template <class Policy, class KeysIt1, class KeysIt2, class ItemsIt1, class ItemsIt2, class KeysOutIt, class ItemsOutIt, class Comp, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeysOutIt, ItemsOutIt> merge_by_key(Policy& policy, KeysIt1 keys1_first, KeysIt1 keys1_last, KeysIt2 keys2_first, KeysIt2 keys2_last, ItemsIt1 items1_first,
                                                 ItemsIt2 items2_first, KeysOutIt keys_result, ItemsOutIt items_result, Comp comp) {
  namespace ov = tb200_overlay;
  using K = ov::value_t<KeysIt1>;
  using V = ov::value_t<ItemsIt1>;
  const std::size_t na = (std::size_t)thrust::distance(keys1_first, keys1_last), nb = (std::size_t)thrust::distance(keys2_first, keys2_last);
  if (na + nb == 0) return thrust::make_pair(keys_result, items_result);
  ov::scratch<Policy> tmp(policy, ::tb200::merge_workspace_bytes<K, V, true>(na + nb));
  cudaError_t e = ::tb200::merge_async<K, V, true>(ov::unwrap(keys1_first), na, ov::unwrap(keys2_first), nb, ov::unwrap(items1_first), ov::unwrap(items2_first),
                                                 ov::unwrap(keys_result), ov::unwrap(items_result), comp, tmp.at(), cuda_cub::stream(policy));
  ov::finish(policy, e, tmp.at(), "merge_by_key failed");
  return thrust::make_pair(keys_result + (na + nb), items_result + (na + nb));
}
template <class Policy, class KeysIt1, class KeysIt2, class ItemsIt1, class ItemsIt2, class KeysOutIt, class ItemsOutIt, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KeysOutIt, ItemsOutIt> merge_by_key(Policy& policy, KeysIt1 keys1_first, KeysIt1 keys1_last, KeysIt2 keys2_first, KeysIt2 keys2_last, ItemsIt1 items1_first,
                                                 ItemsIt2 items2_first, KeysOutIt keys_result, ItemsOutIt items_result) {
  return cuda_cub::merge_by_key(policy, keys1_first, keys1_last, keys2_first, keys2_last, items1_first, items2_first, keys_result, items_result,
                                thrust::less<tb200_overlay::value_t<KeysIt1>>());
}
template <class Policy, class KeysIt1, class KeysIt2, class OutIt, class Comp, tb200_overlay::enable_for<Policy> = 0>
OutIt merge(Policy& policy, KeysIt1 keys1_first, KeysIt1 keys1_last, KeysIt2 keys2_first, KeysIt2 keys2_last, OutIt result, Comp comp) {
  namespace ov = tb200_overlay;
  using K = ov::value_t<KeysIt1>;
  const std::size_t na = (std::size_t)thrust::distance(keys1_first, keys1_last), nb = (std::size_t)thrust::distance(keys2_first, keys2_last);
  if (na + nb == 0) return result;
  ov::scratch<Policy> tmp(policy, ::tb200::merge_workspace_bytes<K, std::uint32_t, false>(na + nb));
  const std::uint32_t* none = nullptr;
  cudaError_t e = ::tb200::merge_async<K, std::uint32_t, false>(ov::unwrap(keys1_first), na, ov::unwrap(keys2_first), nb, none, none, ov::unwrap(result),
                                                              (std::uint32_t*)nullptr, comp, tmp.at(), cuda_cub::stream(policy));
  ov::finish(policy, e, tmp.at(), "merge failed");
  return result + (na + nb);
}
template <class Policy, class KeysIt1, class KeysIt2, class OutIt, tb200_overlay::enable_for<Policy> = 0>
OutIt merge(Policy& policy, KeysIt1 keys1_first, KeysIt1 keys1_last, KeysIt2 keys2_first, KeysIt2 keys2_last, OutIt result) {
  return cuda_cub::merge(policy, keys1_first, keys1_last, keys2_first, keys2_last, result, thrust::less<tb200_overlay::value_t<KeysIt1>>());
}

// ------------------------------------------------------------------------------------- extrema
// replaces cuda_cub::min_element / max_element / minmax_element (thrust/system/cuda/detail/extrema.h:412-565)
namespace tb200_overlay {
template <class Policy, class It, class BinaryPred>
thrust::pair<std::size_t, std::size_t> extrema_positions(Policy& policy, It first, std::size_t n, BinaryPred binary_pred) {
  using T = value_t<It>;
  scratch<Policy> tmp(policy, ::tb200::extrema_workspace_bytes<T>() + 256);
  unsigned long long* d_index = reinterpret_cast<unsigned long long*>(tmp.at(up256(::tb200::extrema_workspace_bytes<T>())));
  cudaError_t e = ::tb200::extrema_async(unwrap(first), n, T(), binary_pred, d_index, tmp.at(), cuda_cub::stream(policy));
  cuda_cub::throw_on_error(e, "extrema: launch failed");
  unsigned long long h[2];
  cuda_cub::throw_on_error(cudaMemcpyAsync(h, d_index, sizeof(h), cudaMemcpyDeviceToHost, cuda_cub::stream(policy)), "extrema: read-back failed");
  cuda_cub::throw_on_error(cudaStreamSynchronize(cuda_cub::stream(policy)), "extrema: synchronize failed");
  return thrust::make_pair((std::size_t)h[0], (std::size_t)h[1]);
}
}  // namespace tb200_overlay

template <class Policy, class ItemsIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
ItemsIt min_element(Policy& policy, ItemsIt first, ItemsIt last, BinaryPred binary_pred) {
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return last;
  return first + tb200_overlay::extrema_positions(policy, first, n, binary_pred).first;
}
template <class Policy, class ItemsIt, tb200_overlay::enable_for<Policy> = 0>
ItemsIt min_element(Policy& policy, ItemsIt first, ItemsIt last) {
  return cuda_cub::min_element(policy, first, last, thrust::less<tb200_overlay::value_t<ItemsIt>>());
}
template <class Policy, class ItemsIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
ItemsIt max_element(Policy& policy, ItemsIt first, ItemsIt last, BinaryPred binary_pred) {
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return last;
  return first + tb200_overlay::extrema_positions(policy, first, n, binary_pred).second;
}
template <class Policy, class ItemsIt, tb200_overlay::enable_for<Policy> = 0>
ItemsIt max_element(Policy& policy, ItemsIt first, ItemsIt last) {
  return cuda_cub::max_element(policy, first, last, thrust::less<tb200_overlay::value_t<ItemsIt>>());
}
template <class Policy, class ItemsIt, class BinaryPred, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<ItemsIt, ItemsIt> minmax_element(Policy& policy, ItemsIt first, ItemsIt last, BinaryPred binary_pred) {
  const std::size_t n = (std::size_t)thrust::distance(first, last);
  if (n == 0) return thrust::make_pair(last, last);
  const thrust::pair<std::size_t, std::size_t> p = tb200_overlay::extrema_positions(policy, first, n, binary_pred);
  return thrust::make_pair(first + p.first, first + p.second);
}
template <class Policy, class ItemsIt, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<ItemsIt, ItemsIt> minmax_element(Policy& policy, ItemsIt first, ItemsIt last) {
  return cuda_cub::minmax_element(policy, first, last, thrust::less<tb200_overlay::value_t<ItemsIt>>());
}

}  // namespace cuda_cub
THRUST_NAMESPACE_END

// ------------------------------------------------------------------------------------- set operations
// replaces cuda_cub::set_union / set_intersection / set_difference / set_symmetric_difference and their
// _by_key forms (thrust/system/cuda/detail/set_operations.h:1260-1760)
THRUST_NAMESPACE_BEGIN
namespace cuda_cub {
namespace tb200_overlay {
template <bool HAS_V, class Policy, class K1, class K2, class V1, class V2, class KO, class VO, class Comp>
thrust::pair<KO, VO> set_any(Policy& policy, int op, K1 k1, K1 k1_last, K2 k2, K2 k2_last, V1 v1, V2 v2, KO ko, VO vo, Comp comp) {
  using T = value_t<K1>;
  const std::size_t na = (std::size_t)thrust::distance(k1, k1_last), nb = (std::size_t)thrust::distance(k2, k2_last);
  scratch<Policy> tmp(policy, ::tb200::set_op_workspace_bytes(na, nb));
  cudaError_t e = ::tb200::set_operation_async<T, HAS_V>(op, unwrap(k1), na, unwrap(k2), nb, unwrap(v1), unwrap(v2), unwrap(ko), unwrap(vo), comp, nullptr,
                                                        tmp.at(), cuda_cub::stream(policy));
  const std::size_t m = finish(policy, e, tmp.at(), "set operation failed");
  return thrust::make_pair(ko + m, vo + m);
}
}  // namespace tb200_overlay

#define TB200_SET_OPERATION(NAME, OP)                                                                                                         \
  template <class Policy, class It1, class It2, class OutIt, class Comp, tb200_overlay::enable_for<Policy> = 0>                                \
  OutIt NAME(Policy& policy, It1 first1, It1 last1, It2 first2, It2 last2, OutIt result, Comp comp) {                                          \
    return tb200_overlay::set_any<false>(policy, OP, first1, last1, first2, last2, first1, first2, result, result, comp).first;                \
  }                                                                                                                                            \
  template <class Policy, class It1, class It2, class OutIt, tb200_overlay::enable_for<Policy> = 0>                                            \
  OutIt NAME(Policy& policy, It1 first1, It1 last1, It2 first2, It2 last2, OutIt result) {                                                     \
    return cuda_cub::NAME(policy, first1, last1, first2, last2, result, thrust::less<tb200_overlay::value_t<It1>>());                          \
  }
TB200_SET_OPERATION(set_union, ::tb200::SET_UNION)
TB200_SET_OPERATION(set_intersection, ::tb200::SET_INTERSECTION)
TB200_SET_OPERATION(set_difference, ::tb200::SET_DIFFERENCE)
TB200_SET_OPERATION(set_symmetric_difference, ::tb200::SET_SYMMETRIC_DIFFERENCE)
#undef TB200_SET_OPERATION

#define TB200_SET_OPERATION_BY_KEY(NAME, OP)                                                                                                  \
  template <class Policy, class K1, class K2, class V1, class V2, class KO, class VO, class Comp, tb200_overlay::enable_for<Policy> = 0>       \
  thrust::pair<KO, VO> NAME(Policy& policy, K1 k1, K1 k1_last, K2 k2, K2 k2_last, V1 v1, V2 v2, KO ko, VO vo, Comp comp) {                     \
    return tb200_overlay::set_any<true>(policy, OP, k1, k1_last, k2, k2_last, v1, v2, ko, vo, comp);                                           \
  }                                                                                                                                            \
  template <class Policy, class K1, class K2, class V1, class V2, class KO, class VO, tb200_overlay::enable_for<Policy> = 0>                   \
  thrust::pair<KO, VO> NAME(Policy& policy, K1 k1, K1 k1_last, K2 k2, K2 k2_last, V1 v1, V2 v2, KO ko, VO vo) {                                \
    return cuda_cub::NAME(policy, k1, k1_last, k2, k2_last, v1, v2, ko, vo, thrust::less<tb200_overlay::value_t<K1>>());                       \
  }
TB200_SET_OPERATION_BY_KEY(set_union_by_key, ::tb200::SET_UNION)
TB200_SET_OPERATION_BY_KEY(set_difference_by_key, ::tb200::SET_DIFFERENCE)
TB200_SET_OPERATION_BY_KEY(set_symmetric_difference_by_key, ::tb200::SET_SYMMETRIC_DIFFERENCE)
#undef TB200_SET_OPERATION_BY_KEY
// the intersection takes values from the first range only
template <class Policy, class K1, class K2, class V1, class KO, class VO, class Comp, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KO, VO> set_intersection_by_key(Policy& policy, K1 k1, K1 k1_last, K2 k2, K2 k2_last, V1 v1, KO ko, VO vo, Comp comp) {
  return tb200_overlay::set_any<true>(policy, ::tb200::SET_INTERSECTION, k1, k1_last, k2, k2_last, v1, v1, ko, vo, comp);
}
template <class Policy, class K1, class K2, class V1, class KO, class VO, tb200_overlay::enable_for<Policy> = 0>
thrust::pair<KO, VO> set_intersection_by_key(Policy& policy, K1 k1, K1 k1_last, K2 k2, K2 k2_last, V1 v1, KO ko, VO vo) {
  return cuda_cub::set_intersection_by_key(policy, k1, k1_last, k2, k2_last, v1, ko, vo, thrust::less<tb200_overlay::value_t<K1>>());
}

}  // namespace cuda_cub
THRUST_NAMESPACE_END

// ------------------------------------------------------------------------------------- callers of the above
// count / count_if, inner_product, transform_reduce, transform_inclusive_scan / transform_exclusive_scan
// and remove / remove_if / remove_copy(_if) are thin forwarders in the reference's backend
// (thrust/system/cuda/detail/{count.h:56, inner_product.h:64, transform_reduce.h:59, transform_scan.h,
// remove.h:38-134}); the stock ones hand their `execution_policy<Derived>&` on, which would reach the
// stock reduce_n / scan / copy_if, so they are restated here on the concrete policy types.
THRUST_NAMESPACE_BEGIN
namespace cuda_cub {

template <class Policy, class InputIt, class UnaryPred, tb200_overlay::enable_for<Policy> = 0>
typename thrust::iterator_traits<InputIt>::difference_type count_if(Policy& policy, InputIt first, InputIt last, UnaryPred unary_pred) {
  using size_type = typename thrust::iterator_traits<InputIt>::difference_type;
  using flags_t = thrust::transform_iterator<UnaryPred, InputIt, size_type, size_type>;
  return cuda_cub::reduce_n(policy, flags_t(first, unary_pred), thrust::distance(first, last), size_type(0), thrust::plus<size_type>());
}
template <class Policy, class InputIt, class Value, tb200_overlay::enable_for<Policy> = 0>
typename thrust::iterator_traits<InputIt>::difference_type count(Policy& policy, InputIt first, InputIt last, const Value& value) {
  return cuda_cub::count_if(policy, first, last, thrust::detail::equal_to_value<Value>(value));
}

template <class Policy, class InputIt1, class InputIt2, class T, class ReduceOp, class ProductOp, tb200_overlay::enable_for<Policy> = 0>
T inner_product(Policy& policy, InputIt1 first1, InputIt1 last1, InputIt2 first2, T init, ReduceOp reduce_op, ProductOp product_op) {
  const auto products = thrust::make_transform_iterator(thrust::make_zip_iterator(first1, first2), thrust::make_zip_function(product_op));
  return cuda_cub::reduce_n(policy, products, thrust::distance(first1, last1), init, reduce_op);
}
template <class Policy, class InputIt1, class InputIt2, class T, tb200_overlay::enable_for<Policy> = 0>
T inner_product(Policy& policy, InputIt1 first1, InputIt1 last1, InputIt2 first2, T init) {
  return cuda_cub::inner_product(policy, first1, last1, first2, init, thrust::plus<T>(), thrust::multiplies<T>());
}

template <class Policy, class InputIt, class TransformOp, class T, class ReduceOp, tb200_overlay::enable_for<Policy> = 0>
T transform_reduce(Policy& policy, InputIt first, InputIt last, TransformOp transform_op, T init, ReduceOp reduce_op) {
  using transformed_t = thrust::transform_iterator<TransformOp, InputIt, T, T>;       // accumulates in the type of init
  return cuda_cub::reduce_n(policy, transformed_t(first, transform_op), thrust::distance(first, last), init, reduce_op);
}

template <class Policy, class InputIt, class OutputIt, class TransformOp, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutputIt transform_inclusive_scan(Policy& policy, InputIt first, InputIt last, OutputIt result, TransformOp transform_op, ScanOp scan_op) {
  using value_type = ::cuda::std::remove_cvref_t<thrust::detail::invoke_result_t<TransformOp, typename thrust::iterator_value<InputIt>::type>>;
  using transformed_t = thrust::transform_iterator<TransformOp, InputIt, value_type, value_type>;   // the transformed value type (P0571)
  return cuda_cub::inclusive_scan_n(policy, transformed_t(first, transform_op), thrust::distance(first, last), result, scan_op);
}
template <class Policy, class InputIt, class OutputIt, class TransformOp, class InitialValueType, class ScanOp, tb200_overlay::enable_for<Policy> = 0>
OutputIt transform_exclusive_scan(Policy& policy, InputIt first, InputIt last, OutputIt result, TransformOp transform_op, InitialValueType init, ScanOp scan_op) {
  using result_type = ::cuda::std::remove_cvref_t<InitialValueType>;                  // the initial value's type (P0571)
  using transformed_t = thrust::transform_iterator<TransformOp, InputIt, result_type, result_type>;
  return cuda_cub::exclusive_scan_n(policy, transformed_t(first, transform_op), thrust::distance(first, last), result, init, scan_op);
}

template <class Policy, class InputIt, class Predicate, tb200_overlay::enable_for<Policy> = 0>
InputIt remove_if(Policy& policy, InputIt first, InputIt last, Predicate predicate) {
  return cuda_cub::copy_if(policy, first, last, first, thrust::not_fn(predicate));    // in place: stable compaction onto itself
}
template <class Policy, class InputIt, class StencilIt, class Predicate, tb200_overlay::enable_for<Policy> = 0>
InputIt remove_if(Policy& policy, InputIt first, InputIt last, StencilIt stencil, Predicate predicate) {
  return cuda_cub::copy_if(policy, first, last, stencil, first, thrust::not_fn(predicate));
}
template <class Policy, class InputIt, class T, tb200_overlay::enable_for<Policy> = 0>
InputIt remove(Policy& policy, InputIt first, InputIt last, const T& value) {
  return cuda_cub::remove_if(policy, first, last, thrust::detail::equal_to_value<T>(value));
}
template <class Policy, class InputIt, class OutputIt, class Predicate, tb200_overlay::enable_for<Policy> = 0>
OutputIt remove_copy_if(Policy& policy, InputIt first, InputIt last, OutputIt result, Predicate predicate) {
  return cuda_cub::copy_if(policy, first, last, result, thrust::not_fn(predicate));
}
template <class Policy, class InputIt, class StencilIt, class OutputIt, class Predicate, tb200_overlay::enable_for<Policy> = 0>
OutputIt remove_copy_if(Policy& policy, InputIt first, InputIt last, StencilIt stencil, OutputIt result, Predicate predicate) {
  return cuda_cub::copy_if(policy, first, last, stencil, result, thrust::not_fn(predicate));
}
template <class Policy, class InputIt, class OutputIt, class T, tb200_overlay::enable_for<Policy> = 0>
OutputIt remove_copy(Policy& policy, InputIt first, InputIt last, OutputIt result, const T& value) {
  return cuda_cub::remove_copy_if(policy, first, last, result, thrust::detail::equal_to_value<T>(value));
}

}  // namespace cuda_cub
THRUST_NAMESPACE_END

// thrust::async::{reduce, inclusive_scan, exclusive_scan, sort}: needs the installation's asynchronous algorithms (C++14)
#if !defined(THRUST_B200_NO_ASYNC_OVERLAY) && __has_include(<thrust/system/cuda/detail/async/customization.h>)
#include "thrust_async_overlay.cuh"
#endif
