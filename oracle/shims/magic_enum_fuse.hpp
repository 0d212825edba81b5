// Test infrastructure (oracle build only): enum_fuse(a, b) folds two
// enumerators into one integer usable as a `case` label.
#pragma once
#include "magic_enum.hpp"

namespace magic_enum {

template <class A, class B>
constexpr std::optional<std::uintmax_t> enum_fuse(A a, B b) {
    const long long va = static_cast<long long>(a);
    const long long vb = static_cast<long long>(b);
    if (va < shim::MIN || va > shim::MAX || vb < shim::MIN || vb > shim::MAX) { return std::nullopt; }
    return static_cast<std::uintmax_t>(va - shim::MIN) * static_cast<std::uintmax_t>(shim::COUNT)
         + static_cast<std::uintmax_t>(vb - shim::MIN);
}

}  // namespace magic_enum
