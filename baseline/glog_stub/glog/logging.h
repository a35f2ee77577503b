// Minimal stand-in for <glog/logging.h> so that the reference's sources compile unmodified
// on an image without glog.  Only what the reference uses: LOG / LOG_IF / CHECK_GE streams,
// the two FLAGS it sets, Init / Shutdown / InstallFailureSignalHandler.  FATAL aborts.
#pragma once
#include <cstdlib>
#include <iostream>
#include <sstream>

static bool FLAGS_colorlogtostderr = false;
static bool FLAGS_logtostderr = false;

namespace google {
inline void InitGoogleLogging(const char*) { (void)FLAGS_colorlogtostderr; (void)FLAGS_logtostderr; }
inline void ShutdownGoogleLogging() {}
inline void InstallFailureSignalHandler() {}
}  // namespace google

namespace glog_stub {
enum Severity { INFO = 0, WARNING = 1, ERROR = 2, FATAL = 3 };
class Message {
 public:
  Message(int sev, const char* file, int line) : sev_(sev) {
    static const char tag[] = "IWEF";
    os_ << tag[sev] << " " << file << ":" << line << "] ";
  }
  ~Message() {
    os_ << "\n";
    if (sev_ >= WARNING || std::getenv("GLOG_STUB_VERBOSE")) std::cerr << os_.str();
    if (sev_ == FATAL) std::abort();
  }
  std::ostream& stream() { return os_; }
 private:
  int sev_;
  std::ostringstream os_;
};
struct Voidify { void operator&(std::ostream&) {} };
}  // namespace glog_stub

#define LOG(sev) glog_stub::Message(glog_stub::sev, __FILE__, __LINE__).stream()
#define LOG_IF(sev, cond) !(cond) ? (void)0 : glog_stub::Voidify() & LOG(sev)
#define CHECK_GE(a, b) LOG_IF(FATAL, !((a) >= (b))) << "Check failed: " #a " >= " #b " "
#define CHECK(c) LOG_IF(FATAL, !(c)) << "Check failed: " #c " "
