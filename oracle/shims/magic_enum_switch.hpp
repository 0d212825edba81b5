// Test infrastructure (oracle build only): enum_switch(f, v) calls
// f(std::integral_constant<E, V>{}) for the enumerator V equal to v, and
// instantiates f only for values that name a real enumerator.
#pragma once
#include "magic_enum.hpp"

namespace magic_enum {

namespace shim {

template <class E, int I, class F, class R>
constexpr R switch_from(F &&f, E value) {
    if constexpr (I > MAX) {
        if constexpr (std::is_void_v<R>) { return; } else { return R{}; }
    } else {
        if constexpr (in_underlying_range<E, I>()) {
            if constexpr (!raw_name<E, static_cast<E>(I)>().empty()) {
                if (value == static_cast<E>(I)) {
                    return static_cast<R>(std::forward<F>(f)(std::integral_constant<E, static_cast<E>(I)>{}));
                }
            }
        }
        return switch_from<E, I + 1, F, R>(std::forward<F>(f), value);
    }
}

template <class E, int I>
constexpr int first_valid() {
    if constexpr (I > MAX) { return MAX + 1; }
    else if constexpr (in_underlying_range<E, I>()) {
        if constexpr (!raw_name<E, static_cast<E>(I)>().empty()) { return I; }
        else { return first_valid<E, I + 1>(); }
    } else { return first_valid<E, I + 1>(); }
}

}  // namespace shim

template <class F, class E>
constexpr auto enum_switch(F &&f, E value) {
    constexpr int first = shim::first_valid<E, shim::MIN>();
    static_assert(first <= shim::MAX, "enum has no enumerator in the supported range");
    using R = std::invoke_result_t<F, std::integral_constant<E, static_cast<E>(first)>>;
    return shim::switch_from<E, shim::MIN, F, R>(std::forward<F>(f), value);
}

}  // namespace magic_enum
