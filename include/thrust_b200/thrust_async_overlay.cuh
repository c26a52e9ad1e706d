// thrust::async::reduce, inclusive_scan, exclusive_scan, sort / stable_sort on this library's kernels.
//
// The asynchronous algorithms of thrust/system/cuda/detail/async/{reduce,inclusive_scan,
// exclusive_scan,sort}.h are the synchronous ones without the final wait: they size and allocate
// temporary storage, enqueue the kernels on the policy's stream and hand back an event (or, for
// reduce, a future that owns the device-side result).  The kernels of this library are already
// stream-ordered and allocate nothing, so the overlay is the same few steps around them.  As in
// thrust_overlay.cuh, the overloads take the concrete policy type and are therefore preferred by
// overload resolution over the stock `execution_policy<Derived>&` ones; any other policy keeps the
// stock implementation.  The event / future keeps the temporary storage alive until the work is
// done, exactly as the stock implementation's does.  Included by thrust_overlay.cuh when the
// installation's Thrust has the asynchronous algorithms.
#pragma once

#include <thrust/system/cuda/detail/async/customization.h>
#include <thrust/system/cuda/future.h>

#include <tuple>

THRUST_NAMESPACE_BEGIN
namespace system { namespace cuda { namespace detail {

// event that owns `content` (temporary storage) and is bound to the policy's stream and dependencies
template <class Policy, class Content>
unique_eager_event tb200_dependent_event(Policy& policy, Content&& content) {
  cudaStream_t const user_raw_stream = thrust::cuda_cub::stream(policy);
  if (thrust::cuda_cub::default_stream() != user_raw_stream)
    return make_dependent_event(std::tuple_cat(std::make_tuple(std::move(content), unique_stream(nonowning, user_raw_stream)),
                                               extract_dependencies(std::move(thrust::detail::derived_cast(policy)))));
  return make_dependent_event(std::tuple_cat(std::make_tuple(std::move(content)), extract_dependencies(std::move(thrust::detail::derived_cast(policy)))));
}

template <class Policy, class ForwardIt, class Size, class T, class BinaryOp>
unique_eager_future<::cuda::std::remove_cvref_t<T>> tb200_async_reduce_n(Policy& policy, ForwardIt first, Size n, T init, BinaryOp op) {
  namespace ov = thrust::cuda_cub::tb200_overlay;
  using U = ::cuda::std::remove_cvref_t<T>;
  auto const device_alloc = get_async_device_allocator(policy);
  using pointer = typename thrust::detail::allocator_traits<decltype(device_alloc)>::template rebind_traits<U>::pointer;
  // [result | padding to 256 | workspace]
  const std::size_t head = ov::up256(sizeof(U)) + 256;
  auto content = uninitialized_allocate_unique_n<std::uint8_t>(device_alloc, head + ::tb200::reduce_workspace_bytes<U>());
  std::uint8_t* const raw = raw_pointer_cast(content.get());
  U* const ret_ptr = thrust::detail::aligned_reinterpret_cast<U*>(raw);
  std::uint8_t* const ws = reinterpret_cast<std::uint8_t*>((reinterpret_cast<std::uintptr_t>(raw) + sizeof(U) + 255) & ~std::uintptr_t(255));
  cudaStream_t const user_raw_stream = thrust::cuda_cub::stream(policy);
  unique_eager_future_promise_pair<U, pointer> fp;
  auto locate = [](decltype(content) const& c) { return pointer(thrust::detail::aligned_reinterpret_cast<U*>(raw_pointer_cast(c.get()))); };
  if (thrust::cuda_cub::default_stream() != user_raw_stream)
    fp = make_dependent_future<U, pointer>(locate, std::tuple_cat(std::make_tuple(std::move(content), unique_stream(nonowning, user_raw_stream)),
                                                                  extract_dependencies(std::move(thrust::detail::derived_cast(policy)))));
  else
    fp = make_dependent_future<U, pointer>(locate, std::tuple_cat(std::make_tuple(std::move(content)),
                                                                  extract_dependencies(std::move(thrust::detail::derived_cast(policy)))));
  ++ov::call_count();
  thrust::cuda_cub::throw_on_error(::tb200::reduce_async(ov::unwrap(first), (std::size_t)n, (U)init, ov::template map_op<BinaryOp, U>::get(op), ret_ptr, ws,
                                                         fp.future.stream().native_handle()),
                                   "async reduce: launch failed");
  return std::move(fp.future);
}

template <bool INCLUSIVE, class Policy, class ForwardIt, class Size, class OutputIt, class T, class BinaryOp>
unique_eager_event tb200_async_scan_n(Policy& policy, ForwardIt first, Size n, OutputIt out, T init, bool has_init, BinaryOp op) {
  namespace ov = thrust::cuda_cub::tb200_overlay;
  auto const device_alloc = get_async_device_allocator(policy);
  auto content = uninitialized_allocate_unique_n<std::uint8_t>(device_alloc, ::tb200::scan_workspace_bytes<T>((std::size_t)n) + 256);
  std::uint8_t* const ws = reinterpret_cast<std::uint8_t*>((reinterpret_cast<std::uintptr_t>(raw_pointer_cast(content.get())) + 255) & ~std::uintptr_t(255));
  unique_eager_event ev = tb200_dependent_event(policy, std::move(content));
  ++ov::call_count();
  thrust::cuda_cub::throw_on_error(::tb200::scan_async<INCLUSIVE>(ov::unwrap(first), ov::unwrap(out), (std::size_t)n, init, has_init,
                                                                  ov::template map_op<BinaryOp, T>::get(op), ws, ev.stream().native_handle()),
                                   "async scan: launch failed");
  return ev;
}

// radix-sortable keys in a contiguous range, ascending or descending
template <class Policy, class K>
unique_eager_event tb200_async_radix_sort_n(Policy& policy, K* keys, std::size_t n, bool descending) {
  namespace ov = thrust::cuda_cub::tb200_overlay;
  using UK = typename ov::template radix_key<K>::bits;
  auto const device_alloc = get_async_device_allocator(policy);
  const std::size_t wsb = ov::up256(::tb200::radix_workspace_bytes<sizeof(UK), 0>(n));
  auto content = uninitialized_allocate_unique_n<std::uint8_t>(device_alloc, wsb + ov::up256(n * sizeof(UK)) + 256);
  std::uint8_t* const ws = reinterpret_cast<std::uint8_t*>((reinterpret_cast<std::uintptr_t>(raw_pointer_cast(content.get())) + 255) & ~std::uintptr_t(255));
  unique_eager_event ev = tb200_dependent_event(policy, std::move(content));
  ++ov::call_count();
  ::tb200::key_coding coding;
  coding.kind = ov::template radix_key<K>::kind;
  coding.descending = descending ? 1 : 0;
  thrust::cuda_cub::throw_on_error(::tb200::radix_sort_async<UK, std::uint32_t, false>(reinterpret_cast<UK*>(keys), reinterpret_cast<UK*>(ws + wsb), nullptr, nullptr, n,
                                                                                        coding, 0, 8 * (int)sizeof(UK), ws, ev.stream().native_handle()),
                                   "async sort: launch failed");
  return ev;
}

}}}  // namespace system::cuda::detail

namespace cuda_cub {

// replaces cuda_cub::async_reduce (thrust/system/cuda/detail/async/reduce.h, ADL entry point)
template <class Policy, class ForwardIt, class Sentinel, class T, class BinaryOp, tb200_overlay::enable_for<Policy> = 0>
auto async_reduce(Policy& policy, ForwardIt first, Sentinel last, T init, BinaryOp op)
    THRUST_RETURNS(thrust::system::cuda::detail::tb200_async_reduce_n(policy, first, thrust::distance(first, last), init, op))

// replace cuda_cub::async_inclusive_scan / async_exclusive_scan (async/inclusive_scan.h, async/exclusive_scan.h)
template <class Policy, class ForwardIt, class Sentinel, class OutputIt, class BinaryOp, tb200_overlay::enable_for<Policy> = 0>
auto async_inclusive_scan(Policy& policy, ForwardIt first, Sentinel&& last, OutputIt&& out, BinaryOp&& op)
    THRUST_RETURNS(thrust::system::cuda::detail::tb200_async_scan_n<true>(policy, first, thrust::distance(first, last), out,
                                                                         typename thrust::iterator_traits<ForwardIt>::value_type(), false, op))
template <class Policy, class ForwardIt, class Sentinel, class OutputIt, class InitialValueType, class BinaryOp, tb200_overlay::enable_for<Policy> = 0>
auto async_exclusive_scan(Policy& policy, ForwardIt first, Sentinel&& last, OutputIt&& out, InitialValueType&& init, BinaryOp&& op)
    THRUST_RETURNS(thrust::system::cuda::detail::tb200_async_scan_n<false>(policy, first, thrust::distance(first, last), out,
                                                                          (typename ::cuda::std::remove_cvref_t<InitialValueType>)init, true, op))

// replaces cuda_cub::async_stable_sort for radix-sortable keys in contiguous ranges under less / greater
// (async/sort.h); anything else keeps the stock merge sort
template <class Policy, class ForwardIt, class Sentinel, class StrictWeakOrdering, tb200_overlay::enable_for<Policy> = 0,
          typename std::enable_if<thrust::is_contiguous_iterator<ForwardIt>::value &&
                                  tb200_overlay::radix_key<typename thrust::iterator_traits<ForwardIt>::value_type>::ok &&
                                  tb200_overlay::radix_order<StrictWeakOrdering, typename thrust::iterator_traits<ForwardIt>::value_type>::value >= 0, int>::type = 0>
auto async_stable_sort(Policy& policy, ForwardIt first, Sentinel last, StrictWeakOrdering)
    THRUST_RETURNS(thrust::system::cuda::detail::tb200_async_radix_sort_n(
        policy, thrust::raw_pointer_cast(&*first), (std::size_t)thrust::distance(first, last),
        tb200_overlay::radix_order<StrictWeakOrdering, typename thrust::iterator_traits<ForwardIt>::value_type>::value == 1))

}  // namespace cuda_cub
THRUST_NAMESPACE_END
