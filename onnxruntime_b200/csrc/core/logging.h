// Logging: a process-wide manager with a default severity / verbosity and a replaceable sink, and per-session
// loggers that carry their own id and severity threshold (SessionOptions.logid / log_severity_level; RunOptions
// may lower or raise the threshold for one run).  Severities are the reference's: 0 VERBOSE, 1 INFO, 2 WARNING,
// 3 ERROR, 4 FATAL (onnxruntime/core/common/logging/logging.h, severity.h).  Line format of the default sink:
//   2026-01-02 03:04:05.678 [W:ortb200:<logid>, <file>:<line> <function>] message
#pragma once
#include <functional>
#include <mutex>
#include <sstream>
#include <string>

namespace ortb {
namespace logging {

enum Severity { kVerbose = 0, kInfo = 1, kWarning = 2, kError = 3, kFatal = 4 };

struct Record {
  Severity severity;
  std::string logger_id, file, function, message;
  int line;
};

using Sink = std::function<void(const Record&)>;

class Manager {
 public:
  static Manager& Get();
  int default_severity() const { return default_severity_; }
  int default_verbosity() const { return default_verbosity_; }
  void set_default_severity(int s) { default_severity_ = s; }
  void set_default_verbosity(int v) { default_verbosity_ = v; }
  // nullptr restores the stderr sink
  void SetSink(Sink sink);
  void Emit(const Record& r);
  static std::string Format(const Record& r);

 private:
  Manager() = default;
  int default_severity_ = kWarning, default_verbosity_ = 0;
  std::mutex mu_;
  Sink sink_;
};

class Logger {
 public:
  Logger() = default;
  Logger(std::string id, int severity, int verbosity) : id_(std::move(id)), severity_(severity), verbosity_(verbosity) {}
  // a negative threshold means "use the process default"
  int threshold() const { return severity_ >= 0 ? severity_ : Manager::Get().default_severity(); }
  int verbosity() const { return verbosity_ >= 0 ? verbosity_ : Manager::Get().default_verbosity(); }
  bool Enabled(Severity s) const { return static_cast<int>(s) >= threshold(); }
  const std::string& id() const { return id_; }
  void set_severity(int s) { severity_ = s; }

 private:
  std::string id_;
  int severity_ = -1, verbosity_ = -1;
};

// Collects one message and emits it when it goes out of scope.
class Capture {
 public:
  Capture(const Logger& logger, Severity s, const char* file, int line, const char* function)
      : rec_{s, logger.id(), file, function, "", line} {}
  ~Capture();
  std::ostringstream& stream() { return os_; }

 private:
  Record rec_;
  std::ostringstream os_;
};

}  // namespace logging
}  // namespace ortb

#define ORTB_LOG(logger, sev)                                 \
  if (!(logger).Enabled(::ortb::logging::sev)) {              \
  } else                                                      \
    ::ortb::logging::Capture((logger), ::ortb::logging::sev, __FILE__, __LINE__, __func__).stream()

#define ORTB_VLOG(logger, level)                                                                    \
  if (!((logger).Enabled(::ortb::logging::kVerbose) && (level) <= (logger).verbosity())) {         \
  } else                                                                                            \
    ::ortb::logging::Capture((logger), ::ortb::logging::kVerbose, __FILE__, __LINE__, __func__).stream()
