// Compile-time loop: staticFor<N>(f) calls f(std::integral_constant<int, I>{}) for I = 0 .. N-1, in order.
//
// Parity: purlin::static_for of csrc/include/purlin/static_for.cuh:6-24 in the reference (a constexpr loop whose
// index is a constant expression inside the body, so it can select template arguments such as wait<I>()).
// Built on a fold over an index sequence: for N == 0 the functor is never instantiated with an index, it is
// taken by forwarding reference (a non-copyable functor works), and the call is constexpr when the body is.
#pragma once
#include <type_traits>
#include <utility>

#include "constants.hpp"

namespace purlin {

namespace detail {
template <class F, int... I>
PURLIN_HD constexpr void staticForImpl(F&& f, std::integer_sequence<int, I...>) {
  (static_cast<void>(f(std::integral_constant<int, I>{})), ...);
}
}  // namespace detail

template <int N, class F>
PURLIN_HD constexpr void staticFor(F&& f) {
  static_assert(N >= 0, "the trip count cannot be negative");
  if constexpr (N > 0) detail::staticForImpl(static_cast<F&&>(f), std::make_integer_sequence<int, N>{});
}

// Run-time value -> compile-time constant: calls f(integral_constant<int, v>) for the v in [0, N) that equals
// `value`; returns false when value is outside the range.
template <int N, class F>
PURLIN_HD constexpr bool staticSwitch(int value, F&& f) {
  bool hit = false;
  staticFor<N>([&](auto i) {
    if (!hit && value == decltype(i)::value) { f(i); hit = true; }
  });
  return hit;
}

}  // namespace purlin
