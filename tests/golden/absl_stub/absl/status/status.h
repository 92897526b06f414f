// A stand-in for the few abseil names the reference's scheduler, cache pool and host
// sampler use, so that those files compile on a machine without abseil.  Only what they
// call is here; nothing of abseil's own code.
#pragma once
#include <ostream>
#include <string>
#include <utility>

namespace absl {

enum class StatusCode {
  kOk = 0, kInvalidArgument = 3, kNotFound = 5, kResourceExhausted = 8,
  kFailedPrecondition = 9, kOutOfRange = 11, kUnimplemented = 12, kInternal = 13,
  kUnavailable = 14, kDeadlineExceeded = 4, kCancelled = 1, kUnknown = 2,
  kAlreadyExists = 6, kPermissionDenied = 7, kAborted = 10, kDataLoss = 15,
  kUnauthenticated = 16,
};

class Status {
 public:
  Status() = default;
  Status(StatusCode code, std::string message) : code_(code), message_(std::move(message)) {}
  bool ok() const { return code_ == StatusCode::kOk; }
  StatusCode code() const { return code_; }
  const std::string& message() const { return message_; }
  std::string ToString() const { return ok() ? "OK" : message_; }
  void IgnoreError() const {}
  friend bool operator==(const Status& a, const Status& b) {
    return a.code_ == b.code_ && a.message_ == b.message_;
  }
  friend bool operator!=(const Status& a, const Status& b) { return !(a == b); }
  friend std::ostream& operator<<(std::ostream& os, const Status& s) { return os << s.ToString(); }

 private:
  StatusCode code_ = StatusCode::kOk;
  std::string message_;
};

inline Status OkStatus() { return Status(); }

#define INFERX_STUB_ERROR(Name, Code)                                             \
  inline Status Name(std::string message) { return Status(StatusCode::Code, std::move(message)); } \
  inline bool Is##Name##Impl(const Status& s) { return s.code() == StatusCode::Code; }
INFERX_STUB_ERROR(InvalidArgumentError, kInvalidArgument)
INFERX_STUB_ERROR(NotFoundError, kNotFound)
INFERX_STUB_ERROR(ResourceExhaustedError, kResourceExhausted)
INFERX_STUB_ERROR(FailedPreconditionError, kFailedPrecondition)
INFERX_STUB_ERROR(OutOfRangeError, kOutOfRange)
INFERX_STUB_ERROR(UnimplementedError, kUnimplemented)
INFERX_STUB_ERROR(InternalError, kInternal)
INFERX_STUB_ERROR(UnavailableError, kUnavailable)
INFERX_STUB_ERROR(DeadlineExceededError, kDeadlineExceeded)
INFERX_STUB_ERROR(CancelledError, kCancelled)
INFERX_STUB_ERROR(UnknownError, kUnknown)
INFERX_STUB_ERROR(AlreadyExistsError, kAlreadyExists)
INFERX_STUB_ERROR(PermissionDeniedError, kPermissionDenied)
INFERX_STUB_ERROR(AbortedError, kAborted)
INFERX_STUB_ERROR(DataLossError, kDataLoss)
INFERX_STUB_ERROR(UnauthenticatedError, kUnauthenticated)
#undef INFERX_STUB_ERROR

inline bool IsResourceExhausted(const Status& s) { return s.code() == StatusCode::kResourceExhausted; }
inline bool IsInvalidArgument(const Status& s) { return s.code() == StatusCode::kInvalidArgument; }
inline bool IsNotFound(const Status& s) { return s.code() == StatusCode::kNotFound; }
inline bool IsFailedPrecondition(const Status& s) { return s.code() == StatusCode::kFailedPrecondition; }
inline bool IsOutOfRange(const Status& s) { return s.code() == StatusCode::kOutOfRange; }
inline bool IsUnimplemented(const Status& s) { return s.code() == StatusCode::kUnimplemented; }
inline bool IsInternal(const Status& s) { return s.code() == StatusCode::kInternal; }
inline bool IsUnavailable(const Status& s) { return s.code() == StatusCode::kUnavailable; }

}  // namespace absl
