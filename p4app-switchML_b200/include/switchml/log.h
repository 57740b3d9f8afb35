// Minimal logging layer with the verbosity convention of the reference
// (CONTRIBUTING.md:75-92: 0 = always-on info, 1 = per-context/job summaries such as the
// stats report, 2 = per-job detail, 3 = per-packet/tile, 4 = per-element dumps) without
// depending on glog (reference glog_fix.h:29-49 wraps glog for the same purpose).
//
//   SML_LOG(INFO|WARNING|ERROR|FATAL) << ...;   FATAL throws switchml::FatalError
//   SML_VLOG(n) << ...;                         printed when n <= verbosity
//   SML_CHECK(cond) << ...;                     FATAL when cond is false
//
//   SML_DVLOG(n), SML_DVLOG_IF(n, cond)         the same, but compiled in only with
//                                               -DSWITCHML_DEBUG (DEBUG=1 builds), like glog's DVLOG
//
// Verbosity comes from the environment variable SWITCHML_V (default 0) or
// SetVerbosity(). Single source files can be given their own level, like glog's --vmodule
// that the reference exposes: SWITCHML_VMODULE="udp_backend=3,control=2" or SetVModule();
// a module is the file's name without directory and extension. FATAL raises an exception instead of aborting so that language
// bindings can surface the message; uncaught it still terminates the process.
#ifndef SWITCHML_LOG_H_
#define SWITCHML_LOG_H_

#include <sstream>
#include <stdexcept>
#include <string>

namespace switchml {

class FatalError : public std::runtime_error {
 public:
  explicit FatalError(const std::string& what) : std::runtime_error(what) {}
};

enum LogSeverity { LOG_INFO = 0, LOG_WARNING = 1, LOG_ERROR = 2, LOG_FATAL = 3 };

int GetVerbosity();
void SetVerbosity(int v);
// Per-file levels: "name=level,name=level"; an empty string removes them all.
void SetVModule(const char* spec);
// True if a SML_VLOG(n) in `file` prints.
bool VlogIsOn(const char* file, int n);
// Redirect log lines to a callback (used by tests); nullptr restores stderr.
void SetLogSink(void (*sink)(int severity, const char* line));

class LogMessage {
 public:
  LogMessage(const char* file, int line, int severity);
  ~LogMessage() noexcept(false);
  std::ostream& stream() { return ss_; }

 private:
  std::ostringstream ss_;
  const char* file_;
  int line_;
  int severity_;
};

// Swallows a stream expression when the log statement is disabled.
struct LogVoidify {
  void operator&(std::ostream&) {}
};

}  // namespace switchml

#define SML_LOG_INFO ::switchml::LogMessage(__FILE__, __LINE__, ::switchml::LOG_INFO).stream()
#define SML_LOG_WARNING ::switchml::LogMessage(__FILE__, __LINE__, ::switchml::LOG_WARNING).stream()
#define SML_LOG_ERROR ::switchml::LogMessage(__FILE__, __LINE__, ::switchml::LOG_ERROR).stream()
#define SML_LOG_FATAL ::switchml::LogMessage(__FILE__, __LINE__, ::switchml::LOG_FATAL).stream()
#define SML_LOG(sev) SML_LOG_##sev

#define SML_VLOG_IS_ON(n) (::switchml::VlogIsOn(__FILE__, (n)))
#define SML_VLOG(n) \
  !SML_VLOG_IS_ON(n) ? (void)0 : ::switchml::LogVoidify() & SML_LOG(INFO)
#define SML_VLOG_IF(n, cond) \
  !(SML_VLOG_IS_ON(n) && (cond)) ? (void)0 : ::switchml::LogVoidify() & SML_LOG(INFO)
#ifdef SWITCHML_DEBUG
#define SML_DVLOG(n) SML_VLOG(n)
#define SML_DVLOG_IF(n, cond) SML_VLOG_IF(n, cond)
#else
#define SML_DVLOG(n) true ? (void)0 : ::switchml::LogVoidify() & SML_LOG(INFO)
#define SML_DVLOG_IF(n, cond) true ? (void)0 : ::switchml::LogVoidify() & SML_LOG(INFO)
#endif
#define SML_CHECK(cond) \
  (cond) ? (void)0 : ::switchml::LogVoidify() & SML_LOG(FATAL) << "Check failed: " #cond " "

#endif  // SWITCHML_LOG_H_
