#include "logging.h"

#include <chrono>
#include <cstdio>
#include <ctime>

namespace ortb {
namespace logging {

Manager& Manager::Get() {
  static Manager m;
  return m;
}

void Manager::SetSink(Sink sink) {
  std::lock_guard<std::mutex> lock(mu_);
  sink_ = std::move(sink);
}

std::string Manager::Format(const Record& r) {
  using namespace std::chrono;
  const auto now = system_clock::now();
  const std::time_t t = system_clock::to_time_t(now);
  const int ms = static_cast<int>(duration_cast<milliseconds>(now.time_since_epoch()).count() % 1000);
  std::tm tm{};
  gmtime_r(&t, &tm);
  char stamp[64];
  std::snprintf(stamp, sizeof(stamp), "%04d-%02d-%02d %02d:%02d:%02d.%03d", tm.tm_year + 1900, tm.tm_mon + 1, tm.tm_mday,
                tm.tm_hour, tm.tm_min, tm.tm_sec, ms);
  static const char kLetters[] = "VIWEF";
  std::string file = r.file;
  const size_t slash = file.find_last_of('/');
  if (slash != std::string::npos) file = file.substr(slash + 1);
  std::ostringstream os;
  os << stamp << " [" << kLetters[r.severity] << ":ortb200:" << r.logger_id << ", " << file << ":" << r.line << " " << r.function
     << "] " << r.message;
  return os.str();
}

void Manager::Emit(const Record& r) {
  std::lock_guard<std::mutex> lock(mu_);
  if (sink_) {
    sink_(r);
    return;
  }
  const std::string line = Format(r);
  std::fprintf(stderr, "%s\n", line.c_str());
  std::fflush(stderr);
}

Capture::~Capture() {
  rec_.message = os_.str();
  Manager::Get().Emit(rec_);
}

}  // namespace logging
}  // namespace ortb
