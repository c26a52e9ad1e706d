// Names that the reference's unit-test framework (Thrust 1.14.0, testing/unittest/*.h) takes from
// thrust::detail and that the CUDA toolkit's newer Thrust no longer provides.  Force-included, before
// the test sources, when those sources are compiled against the toolkit's Thrust plus this
// library's overlay (oracle/ref_tests/Makefile).  Test infrastructure only.
#pragma once
#include <thrust/detail/config.h>
#include <thrust/detail/type_traits.h>

#ifndef THRUST_DISABLE_MSVC_FORCING_VALUE_TO_BOOL_WARNING_BEGIN
#define THRUST_DISABLE_MSVC_FORCING_VALUE_TO_BOOL_WARNING_BEGIN
#define THRUST_DISABLE_MSVC_FORCING_VALUE_TO_BOOL_WARNING_END
#endif
#ifndef THRUST_IF_CONSTEXPR
#define THRUST_IF_CONSTEXPR if constexpr
#endif

#include <cstdint>
#include <type_traits>

THRUST_NAMESPACE_BEGIN
namespace detail {
using std::enable_if;
using std::is_floating_point;
using std::is_integral;
using std::is_same;
using std::is_const;
using std::is_pod;
using std::is_convertible;
using std::remove_const;
using std::remove_reference;
using std::add_const;
using std::conditional;
using ::std::int8_t; using ::std::int16_t; using ::std::int32_t; using ::std::int64_t;
using ::std::uint8_t; using ::std::uint16_t; using ::std::uint32_t; using ::std::uint64_t;
template <class A, class B> struct is_different : std::integral_constant<bool, !std::is_same<A, B>::value> {};
}  // namespace detail
THRUST_NAMESPACE_END
