// See status.h in this folder.
#pragma once
#include <cstdint>
#include <ostream>
#include <sstream>
#include <string>

namespace absl {

// absl::Hex(v): the value in hexadecimal when streamed
struct Hex {
  unsigned long long value;
  template <typename T>
  explicit Hex(T v) : value(static_cast<unsigned long long>(v)) {}
};
inline std::ostream& operator<<(std::ostream& os, const Hex& h) {
  const auto flags = os.flags();
  os << std::hex << h.value;
  os.flags(flags);
  return os;
}

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
