// See status.h in this folder.
#pragma once
#include <unordered_map>

namespace absl {

template <typename K, typename V, typename H = std::hash<K>, typename E = std::equal_to<K>>
using flat_hash_map = std::unordered_map<K, V, H, E>;

}  // namespace absl
