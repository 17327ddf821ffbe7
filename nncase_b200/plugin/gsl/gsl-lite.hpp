// Minimal stand-in for the gsl-lite header that the nncase native sources include.
//
// BUILD SHIM. The nncase native runtime depends on gsl-lite 0.37 (a Conan package that
// is not vendored in its tree). This file provides just the surface its headers and
// sources use -- gsl::span, gsl::byte, gsl::cstring_span, make_span and four
// configuration macros -- written from scratch on top of the C++20 standard library,
// so that code can be compiled against the reference's headers where the package is
// not installed: the runtime plugin in this directory, and the CPU checker that
// compiles the reference's own kernels. With the real gsl-lite on the include path
// this file is not needed.
#pragma once
#include <algorithm>
#include <array>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <utility>
#include <iterator>
#include <string>
#include <type_traits>
#include <vector>

#define gsl_CPP17_OR_GREATER 1
#define gsl_NODISCARD [[nodiscard]]
#define gsl_NORETURN [[noreturn]]

#define gsl_DEFINE_ENUM_BITMASK_OPERATORS(E)                                                   \
    inline constexpr E operator|(E a, E b) noexcept {                                          \
        using U = std::underlying_type_t<E>;                                                   \
        return static_cast<E>(static_cast<U>(a) | static_cast<U>(b));                          \
    }                                                                                          \
    inline constexpr E operator&(E a, E b) noexcept {                                          \
        using U = std::underlying_type_t<E>;                                                   \
        return static_cast<E>(static_cast<U>(a) & static_cast<U>(b));                          \
    }                                                                                          \
    inline constexpr E operator^(E a, E b) noexcept {                                          \
        using U = std::underlying_type_t<E>;                                                   \
        return static_cast<E>(static_cast<U>(a) ^ static_cast<U>(b));                          \
    }                                                                                          \
    inline constexpr E operator~(E a) noexcept {                                               \
        using U = std::underlying_type_t<E>;                                                   \
        return static_cast<E>(~static_cast<U>(a));                                             \
    }                                                                                          \
    inline constexpr E &operator|=(E &a, E b) noexcept { return a = a | b; }                   \
    inline constexpr E &operator&=(E &a, E b) noexcept { return a = a & b; }                   \
    inline constexpr E &operator^=(E &a, E b) noexcept { return a = a ^ b; }

namespace gsl {

using byte = std::byte;

template <class T> class span {
  public:
    using element_type = T;
    using value_type = std::remove_cv_t<T>;
    using size_type = std::size_t;
    using index_type = std::size_t;
    using difference_type = std::ptrdiff_t;
    using pointer = T *;
    using const_pointer = const T *;
    using reference = T &;
    using const_reference = const T &;
    using iterator = T *;
    using const_iterator = const T *;
    using reverse_iterator = std::reverse_iterator<iterator>;

    constexpr span() noexcept = default;
    constexpr span(T *p, size_type n) noexcept : p_(p), n_(n) {}
    constexpr span(T *first, T *last) noexcept : p_(first), n_(size_type(last - first)) {}
    template <std::size_t N> constexpr span(T (&a)[N]) noexcept : p_(a), n_(N) {}
    template <class U, std::size_t N,
              class = std::enable_if_t<std::is_convertible_v<U (*)[], T (*)[]>>>
    constexpr span(std::array<U, N> &a) noexcept : p_(a.data()), n_(N) {}
    template <class U, std::size_t N,
              class = std::enable_if_t<std::is_convertible_v<const U (*)[], T (*)[]>>>
    constexpr span(const std::array<U, N> &a) noexcept : p_(a.data()), n_(N) {}
    // any contiguous container with data()/size() whose element pointer converts
    template <class C, class = std::enable_if_t<
                           !std::is_array_v<std::remove_reference_t<C>> &&
                           std::is_convertible_v<
                               std::remove_pointer_t<decltype(std::declval<C &>().data())> (*)[],
                               T (*)[]>>,
              class = decltype(std::declval<C &>().size())>
    constexpr span(C &&c) noexcept : p_(c.data()), n_(c.size()) {}
    template <class U, class = std::enable_if_t<std::is_convertible_v<U (*)[], T (*)[]>>>
    constexpr span(const span<U> &o) noexcept : p_(o.data()), n_(o.size()) {}
    constexpr span(std::initializer_list<value_type> il) noexcept
        requires std::is_const_v<T>
        : p_(il.begin()), n_(il.size()) {}

    constexpr pointer data() const noexcept { return p_; }
    constexpr size_type size() const noexcept { return n_; }
    constexpr size_type length() const noexcept { return n_; }
    constexpr size_type size_bytes() const noexcept { return n_ * sizeof(T); }
    constexpr bool empty() const noexcept { return n_ == 0; }
    constexpr reference operator[](size_type i) const noexcept { return p_[i]; }
    constexpr reference front() const noexcept { return p_[0]; }
    constexpr reference back() const noexcept { return p_[n_ - 1]; }
    constexpr iterator begin() const noexcept { return p_; }
    constexpr iterator end() const noexcept { return p_ + n_; }
    constexpr const_iterator cbegin() const noexcept { return p_; }
    constexpr const_iterator cend() const noexcept { return p_ + n_; }
    constexpr reverse_iterator rbegin() const noexcept { return reverse_iterator(end()); }
    constexpr reverse_iterator rend() const noexcept { return reverse_iterator(begin()); }

    constexpr span first(size_type n) const noexcept { return {p_, n}; }
    constexpr span last(size_type n) const noexcept { return {p_ + (n_ - n), n}; }
    constexpr span subspan(size_type off) const noexcept { return {p_ + off, n_ - off}; }
    constexpr span subspan(size_type off, size_type n) const noexcept { return {p_ + off, n}; }

    template <class U> span<U> as_span() const noexcept {
        return {reinterpret_cast<U *>(p_), size_bytes() / sizeof(U)};
    }

  private:
    T *p_ = nullptr;
    size_type n_ = 0;
};

template <class T, std::size_t N> span(T (&)[N]) -> span<T>;
template <class T, std::size_t N> span(std::array<T, N> &) -> span<T>;
template <class T, std::size_t N> span(const std::array<T, N> &) -> span<const T>;
template <class T> span(T *, std::size_t) -> span<T>;
template <class T> span(T *, T *) -> span<T>;
template <class C>
span(C &) -> span<std::remove_pointer_t<decltype(std::declval<C &>().data())>>;
template <class C>
span(const C &) -> span<std::remove_pointer_t<decltype(std::declval<const C &>().data())>>;

template <class T> constexpr span<T> make_span(T *p, std::size_t n) noexcept { return {p, n}; }
template <class T> constexpr span<T> make_span(T *f, T *l) noexcept { return {f, l}; }
template <class T, std::size_t N> constexpr span<T> make_span(T (&a)[N]) noexcept { return {a}; }
template <class C> constexpr auto make_span(C &c) noexcept {
    return span<std::remove_pointer_t<decltype(c.data())>>(c.data(), c.size());
}
template <class C> constexpr auto make_span(const C &c) noexcept {
    return span<std::remove_pointer_t<decltype(c.data())>>(c.data(), c.size());
}

// element-wise comparison, as gsl-lite defines for spans
template <class T, class U> constexpr bool operator==(span<T> a, span<U> b) noexcept {
    if (a.size() != b.size())
        return false;
    for (std::size_t i = 0; i < a.size(); i++)
        if (!(a[i] == b[i]))
            return false;
    return true;
}
template <class T, class U> constexpr bool operator!=(span<T> a, span<U> b) noexcept {
    return !(a == b);
}

template <class T> span<const byte> as_bytes(span<T> s) noexcept {
    return {reinterpret_cast<const byte *>(s.data()), s.size_bytes()};
}
template <class T> span<byte> as_writable_bytes(span<T> s) noexcept {
    return {reinterpret_cast<byte *>(s.data()), s.size_bytes()};
}

// read-only character span constructible from literals and std::string
class cstring_span : public span<const char> {
  public:
    using span<const char>::span;
    constexpr cstring_span() noexcept = default;
    template <std::size_t N>
    constexpr cstring_span(const char (&lit)[N]) noexcept : span<const char>(lit, N ? N - 1 : 0) {}
    cstring_span(const std::string &s) noexcept : span<const char>(s.data(), s.size()) {}
    constexpr cstring_span(span<const char> s) noexcept : span<const char>(s) {}
};

inline std::string to_string(cstring_span s) { return std::string(s.data(), s.size()); }

} // namespace gsl
