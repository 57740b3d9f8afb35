// Logging sink and verbosity control; see switchml/log.h for the conventions.
#include "switchml/log.h"

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace switchml {

namespace {
std::atomic<int> g_verbosity{-1};
std::atomic<void (*)(int, const char*)> g_sink{nullptr};
std::mutex g_print_mu;

const char* Basename(const char* path) {
  const char* s = strrchr(path, '/');
  return s ? s + 1 : path;
}
}  // namespace

int GetVerbosity() {
  int v = g_verbosity.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = getenv("SWITCHML_V");
    v = e ? atoi(e) : 0;
    if (v < 0) v = 0;
    g_verbosity.store(v, std::memory_order_relaxed);
  }
  return v;
}

void SetVerbosity(int v) { g_verbosity.store(v < 0 ? 0 : v, std::memory_order_relaxed); }

void SetLogSink(void (*sink)(int, const char*)) { g_sink.store(sink); }

LogMessage::LogMessage(const char* file, int line, int severity)
    : file_(file), line_(line), severity_(severity) {}

LogMessage::~LogMessage() noexcept(false) {
  static const char kTag[] = {'I', 'W', 'E', 'F'};
  std::string body = ss_.str();
  char head[160];
  auto now = std::chrono::system_clock::now().time_since_epoch();
  long long us = std::chrono::duration_cast<std::chrono::microseconds>(now).count();
  snprintf(head, sizeof(head), "%c %lld.%06lld %s:%d] ", kTag[severity_], us / 1000000,
           us % 1000000, Basename(file_), line_);
  std::string line = std::string(head) + body;
  auto sink = g_sink.load();
  if (sink) {
    sink(severity_, line.c_str());
  } else {
    std::lock_guard<std::mutex> lk(g_print_mu);
    fprintf(stderr, "%s\n", line.c_str());
    fflush(stderr);
  }
  if (severity_ == LOG_FATAL) {
    throw FatalError(body);
  }
}

}  // namespace switchml
