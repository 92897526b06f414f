// See status.h in this folder.
#pragma once
#include <sstream>
#include <string>

namespace absl {

template <typename Range>
std::string StrJoin(const Range& range, const char* separator) {
  std::ostringstream os;
  bool first = true;
  for (const auto& v : range) {
    if (!first) os << separator;
    os << v;
    first = false;
  }
  return os.str();
}

}  // namespace absl
