// See status.h in this folder.
#pragma once
#include <cstddef>
#include <initializer_list>
#include <type_traits>
#include <vector>

namespace absl {

// A view of contiguous elements; what std::span gives, plus construction from a braced
// list of constants, which the reference's callers use.
template <typename T>
class Span {
 public:
  using value_type = std::remove_cv_t<T>;
  using iterator = T*;
  using const_iterator = const T*;
  constexpr Span() = default;
  constexpr Span(T* data, size_t size) : data_(data), size_(size) {}
  template <typename C, typename = decltype(std::declval<C&>().data()),
            typename = decltype(std::declval<C&>().size())>
  constexpr Span(C& c) : data_(c.data()), size_(c.size()) {}                      // NOLINT
  template <typename C, typename = decltype(std::declval<const C&>().data()),
            typename = decltype(std::declval<const C&>().size()),
            typename = std::enable_if_t<std::is_const_v<T>, C>>
  constexpr Span(const C& c) : data_(c.data()), size_(c.size()) {}                // NOLINT
  template <typename U = T, typename = std::enable_if_t<std::is_const_v<U>>>
  constexpr Span(std::initializer_list<value_type> l) : data_(l.begin()), size_(l.size()) {}  // NOLINT
  constexpr T* data() const { return data_; }
  constexpr size_t size() const { return size_; }
  constexpr bool empty() const { return size_ == 0; }
  constexpr T& operator[](size_t i) const { return data_[i]; }
  constexpr T* begin() const { return data_; }
  constexpr T* end() const { return data_ + size_; }
  constexpr T& front() const { return data_[0]; }
  constexpr T& back() const { return data_[size_ - 1]; }
  constexpr Span subspan(size_t pos, size_t len = static_cast<size_t>(-1)) const {
    const size_t n = size_ - pos;
    return Span(data_ + pos, len < n ? len : n);
  }

 private:
  T* data_ = nullptr;
  size_t size_ = 0;
};

template <typename C>
constexpr auto MakeConstSpan(const C& c) {
  return Span<const std::remove_pointer_t<decltype(c.data())>>(c.data(), c.size());
}
template <typename T>
constexpr Span<const T> MakeConstSpan(const T* data, size_t size) {
  return Span<const T>(data, size);
}
template <typename C>
constexpr auto MakeSpan(C& c) {
  return Span<std::remove_pointer_t<decltype(c.data())>>(c.data(), c.size());
}
template <typename T>
constexpr Span<T> MakeSpan(T* data, size_t size) {
  return Span<T>(data, size);
}

template <typename T>
bool operator==(Span<T> a, Span<T> b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (!(a[i] == b[i])) return false;
  return true;
}

}  // namespace absl
