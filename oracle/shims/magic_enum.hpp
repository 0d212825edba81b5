// Test infrastructure (oracle build only): a small stand-in for the three
// magic_enum entry points the reference calls (enum_name, enum_switch,
// enum_fuse), written for GCC. Enumerator names come from
// __PRETTY_FUNCTION__ over the value range [MIN, MAX]; values outside the
// range have no name and are never dispatched to.
#pragma once
#include <array>
#include <cstdint>
#include <optional>
#include <string_view>
#include <type_traits>
#include <utility>

namespace magic_enum {

namespace shim {

constexpr int MIN = -8;
constexpr int MAX = 72;
constexpr int COUNT = MAX - MIN + 1;

template <class E, E V>
constexpr std::string_view raw_name() {
    // "... [with E = spy::NumberType; E V = spy::NumberType::FP32]"  (valid)
    // "... [with E = spy::NumberType; E V = (spy::NumberType)4]"      (invalid)
    std::string_view s = __PRETTY_FUNCTION__;
    const auto eq = s.rfind("V = ");
    s.remove_prefix(eq + 4);
    const auto end = s.find_first_of(";]");
    s = s.substr(0, end);
    if (!s.empty() && s.front() == '(') { return {}; }
    const auto colon = s.rfind("::");
    if (colon != std::string_view::npos) { s.remove_prefix(colon + 2); }
    return s;
}

template <class E, int I>
constexpr bool in_underlying_range() {
    using U = std::underlying_type_t<E>;
    if constexpr (std::is_same_v<U, bool>) { return I == 0 || I == 1; }
    else if constexpr (std::is_unsigned_v<U>) { return I >= 0; }
    else { return true; }
}

template <class E, int I>
constexpr std::string_view name_at() {
    if constexpr (in_underlying_range<E, I>()) { return raw_name<E, static_cast<E>(I)>(); }
    else { return {}; }
}

template <class E, std::size_t... Is>
constexpr auto make_names(std::index_sequence<Is...>) {
    return std::array<std::string_view, sizeof...(Is)>{ name_at<E, static_cast<int>(Is) + MIN>()... };
}

template <class E>
inline constexpr auto names = make_names<E>(std::make_index_sequence<COUNT>{});

template <class E>
constexpr bool is_valid(long long v) {
    return v >= MIN && v <= MAX && !names<E>[static_cast<std::size_t>(v - MIN)].empty();
}

}  // namespace shim

template <class E>
constexpr std::string_view enum_name(E value) {
    const long long v = static_cast<long long>(value);
    if (v < shim::MIN || v > shim::MAX) { return {}; }
    return shim::names<std::decay_t<E>>[static_cast<std::size_t>(v - shim::MIN)];
}

template <auto V>
using enum_constant = std::integral_constant<decltype(V), V>;

}  // namespace magic_enum
