// Logging sink and verbosity control; see switchml/log.h for the conventions.
#include "switchml/log.h"

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

namespace switchml {

namespace {
std::atomic<int> g_verbosity{-1};
std::atomic<void (*)(int, const char*)> g_sink{nullptr};
std::mutex g_print_mu;

const char* Basename(const char* path) {
  const char* s = strrchr(path, '/');
  return s ? s + 1 : path;
}

// Per-module levels. Readers take a snapshot of the shared pointer; SetVModule swaps it.
typedef std::vector<std::pair<std::string, int>> VModule;
std::mutex g_vmodule_mu;
std::shared_ptr<const VModule> g_vmodule;
std::atomic<int> g_vmodule_state{-1};  // -1: environment not read yet, 0: none, 1: some

std::shared_ptr<const VModule> ParseVModule(const char* spec) {
  auto v = std::make_shared<VModule>();
  std::string s = spec ? spec : "";
  size_t pos = 0;
  while (pos < s.size()) {
    size_t end = s.find(',', pos);
    if (end == std::string::npos) end = s.size();
    std::string item = s.substr(pos, end - pos);
    size_t eq = item.find('=');
    if (eq != std::string::npos && eq > 0) v->emplace_back(item.substr(0, eq), atoi(item.c_str() + eq + 1));
    pos = end + 1;
  }
  return v;
}
}  // namespace

void SetVModule(const char* spec) {
  std::shared_ptr<const VModule> v = ParseVModule(spec);
  std::lock_guard<std::mutex> lk(g_vmodule_mu);
  g_vmodule = v;
  g_vmodule_state.store(v->empty() ? 0 : 1, std::memory_order_release);
}

bool VlogIsOn(const char* file, int n) {
  int state = g_vmodule_state.load(std::memory_order_acquire);
  if (state < 0) {
    SetVModule(getenv("SWITCHML_VMODULE"));
    state = g_vmodule_state.load(std::memory_order_acquire);
  }
  if (state == 0) return n <= GetVerbosity();
  std::shared_ptr<const VModule> v;
  {
    std::lock_guard<std::mutex> lk(g_vmodule_mu);
    v = g_vmodule;
  }
  const char* base = Basename(file);
  const char* dot = strrchr(base, '.');
  size_t len = dot ? static_cast<size_t>(dot - base) : strlen(base);
  for (const auto& m : *v)
    if (m.first.size() == len && memcmp(m.first.data(), base, len) == 0) return n <= m.second;
  return n <= GetVerbosity();
}

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
