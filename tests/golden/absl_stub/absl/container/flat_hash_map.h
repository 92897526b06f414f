// See status.h in this folder.  A map keyed by strings can be searched with a string_view.
#pragma once
#include <functional>
#include <string>
#include <string_view>
#include <unordered_map>

namespace absl {
namespace stub_internal {

template <typename K>
struct Hash : std::hash<K> {};
template <>
struct Hash<std::string> {
  using is_transparent = void;
  size_t operator()(std::string_view s) const { return std::hash<std::string_view>{}(s); }
};
template <typename K>
struct Eq : std::equal_to<K> {};
template <>
struct Eq<std::string> {
  using is_transparent = void;
  bool operator()(std::string_view a, std::string_view b) const { return a == b; }
};

}  // namespace stub_internal

template <typename K, typename V, typename H = stub_internal::Hash<K>,
          typename E = stub_internal::Eq<K>>
using flat_hash_map = std::unordered_map<K, V, H, E>;

}  // namespace absl
