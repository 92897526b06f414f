// See status.h in this folder.
#pragma once
#include <sstream>
#include <string>

namespace absl {

template <typename... Args>
std::string StrCat(const Args&... args) {
  std::ostringstream os;
  (os << ... << args);
  return os.str();
}

template <typename... Args>
void StrAppend(std::string* dest, const Args&... args) {
  dest->append(StrCat(args...));
}

}  // namespace absl
