// See status.h in this folder.
#pragma once
#include <optional>
#include <utility>

#include "absl/status/status.h"

namespace absl {

template <typename T>
class StatusOr {
 public:
  StatusOr(const Status& status) : status_(status) {}                 // NOLINT
  StatusOr(Status&& status) : status_(std::move(status)) {}            // NOLINT
  StatusOr(const T& value) : value_(value) {}                          // NOLINT
  StatusOr(T&& value) : value_(std::move(value)) {}                    // NOLINT
  template <typename U, typename = std::enable_if_t<std::is_constructible_v<T, U&&> &&
                                                    !std::is_same_v<std::decay_t<U>, StatusOr> &&
                                                    !std::is_same_v<std::decay_t<U>, Status> &&
                                                    !std::is_same_v<std::decay_t<U>, T>>>
  StatusOr(U&& value) : value_(std::in_place, std::forward<U>(value)) {}   // NOLINT
  bool ok() const { return value_.has_value(); }
  const Status& status() const { return status_; }
  T& value() & { return *value_; }
  const T& value() const& { return *value_; }
  T&& value() && { return *std::move(value_); }
  T& operator*() & { return *value_; }
  const T& operator*() const& { return *value_; }
  T&& operator*() && { return *std::move(value_); }
  T* operator->() { return &*value_; }
  const T* operator->() const { return &*value_; }

 private:
  Status status_;
  std::optional<T> value_;
};

}  // namespace absl
