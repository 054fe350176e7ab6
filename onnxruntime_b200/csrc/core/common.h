// Status codes, the exception type that carries them, and ENFORCE macros.
//
// Error categories follow the reference's common::StatusCode
// (include/onnxruntime/core/common/status.h) so that the Python layer can map
// them onto the same exception classes (Fail, InvalidArgument, NoSuchFile, ...).
#pragma once
#include <sstream>
#include <stdexcept>
#include <string>

namespace ortb {

enum class StatusCode : int {
  OK = 0,
  FAIL = 1,
  INVALID_ARGUMENT = 2,
  NO_SUCHFILE = 3,
  NO_MODEL = 4,
  ENGINE_ERROR = 5,
  RUNTIME_EXCEPTION = 6,
  INVALID_PROTOBUF = 7,
  MODEL_LOADED = 8,
  NOT_IMPLEMENTED = 9,
  INVALID_GRAPH = 10,
  EP_FAIL = 11,
  MODEL_LOAD_CANCELED = 12,
  MODEL_REQUIRES_COMPILATION = 13,
  NOT_FOUND = 14,
};

const char* StatusCodeName(StatusCode c);

class Status {
 public:
  Status() = default;
  Status(StatusCode code, std::string msg) : code_(code), msg_(std::move(msg)) {}
  static Status OK() { return Status(); }
  bool IsOK() const { return code_ == StatusCode::OK; }
  StatusCode Code() const { return code_; }
  const std::string& ErrorMessage() const { return msg_; }
  std::string ToString() const;

 private:
  StatusCode code_ = StatusCode::OK;
  std::string msg_;
};

class OrtError : public std::runtime_error {
 public:
  OrtError(StatusCode code, const std::string& msg) : std::runtime_error(msg), code_(code) {}
  StatusCode code() const { return code_; }
  Status ToStatus() const { return Status(code_, what()); }

 private:
  StatusCode code_;
};

template <typename... Args>
std::string MakeString(const Args&... args) {
  std::ostringstream ss;
  (ss << ... << args);
  return ss.str();
}

#define ORTB_THROW(code, ...) throw ::ortb::OrtError(::ortb::StatusCode::code, ::ortb::MakeString(__VA_ARGS__))
#define ORTB_ENFORCE(cond, ...)                                                          \
  do {                                                                                   \
    if (!(cond)) ORTB_THROW(FAIL, __FILE__, ":", __LINE__, " ", #cond, " was false. ", __VA_ARGS__); \
  } while (0)
#define ORTB_ENFORCE_ARG(cond, ...)                              \
  do {                                                           \
    if (!(cond)) ORTB_THROW(INVALID_ARGUMENT, __VA_ARGS__);      \
  } while (0)
#define ORTB_NOT_IMPLEMENTED(...) ORTB_THROW(NOT_IMPLEMENTED, __VA_ARGS__)

}  // namespace ortb
