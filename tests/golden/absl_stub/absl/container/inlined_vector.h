// See status.h in this folder.
#pragma once
#include <cstddef>
#include <vector>

namespace absl {

template <typename T, size_t N>
using InlinedVector = std::vector<T>;

}  // namespace absl
