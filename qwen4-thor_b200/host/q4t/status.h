// q4t::Status as the engine uses it (reference include/q4t/status.h:13-27): an
// empty message means success; fallible operators return it instead of throwing.
#pragma once
#include <string>
#include <utility>

namespace q4t {
class Status {
 public:
  Status() = default;
  Status(std::string msg) : message_(std::move(msg)) {}
  bool ok() const { return message_.empty(); }
  explicit operator bool() const { return ok(); }
  const std::string& message() const { return message_; }
  static Status Fail(std::string msg) { return Status(std::move(msg)); }

 private:
  std::string message_;
};
}  // namespace q4t
