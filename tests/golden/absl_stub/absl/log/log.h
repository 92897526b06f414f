// See status.h in this folder.  LOG(...) << ... goes to stderr; FATAL aborts.
#pragma once
#include <cstdlib>
#include <iostream>
#include <sstream>

namespace absl_stub {
class LogLine {
 public:
  explicit LogLine(bool fatal) : fatal_(fatal) {}
  ~LogLine() {
    std::cerr << os_.str() << std::endl;
    if (fatal_) std::abort();
  }
  template <typename T>
  LogLine& operator<<(const T& v) {
    os_ << v;
    return *this;
  }

 private:
  bool fatal_;
  std::ostringstream os_;
};
struct Voidify {
  void operator&(const LogLine&) {}
};
}  // namespace absl_stub

#define INFERX_STUB_LOG_INFO ::absl_stub::LogLine(false)
#define INFERX_STUB_LOG_WARNING ::absl_stub::LogLine(false)
#define INFERX_STUB_LOG_ERROR ::absl_stub::LogLine(false)
#define INFERX_STUB_LOG_FATAL ::absl_stub::LogLine(true)
#define LOG(severity) INFERX_STUB_LOG_##severity
#define VLOG(n) \
  if (true) {   \
  } else        \
    ::absl_stub::LogLine(false)
