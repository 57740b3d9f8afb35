// Barrier and process helpers. Parity: reference client_lib/src/utils.cc:29-72.
#include "switchml/utils.h"

#include <pthread.h>
#include <sched.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace switchml {

Barrier::Barrier(int num_participants) : num_participants_(num_participants) {}

bool Barrier::Wait() {
  std::unique_lock<std::mutex> lk(mu_);
  if (destroyed_) return false;
  unsigned long gen = generation_;
  if (++waiting_ == num_participants_) {
    waiting_ = 0;
    ++generation_;
    cv_.notify_all();
    return true;
  }
  cv_.wait(lk, [&] { return gen != generation_ || destroyed_; });
  return gen != generation_;
}

void Barrier::Destroy() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    destroyed_ = true;
  }
  cv_.notify_all();
}

std::string Execute(const char* cmd) {
  std::string out;
  FILE* p = popen(cmd, "r");
  if (!p) return out;
  char buf[256];
  while (fgets(buf, sizeof(buf), p)) out += buf;
  pclose(p);
  return out;
}

bool ParseCoreList(const std::string& spec, std::string* error, int* out, int max_out,
                   int* count) {
  *count = 0;
  size_t pos = 0;
  while (pos < spec.size()) {
    size_t comma = spec.find(',', pos);
    std::string tok = spec.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
    pos = comma == std::string::npos ? spec.size() : comma + 1;
    if (tok.empty()) continue;
    char* end = nullptr;
    long a = strtol(tok.c_str(), &end, 10), b = a;
    if (end == tok.c_str()) { if (error) *error = "bad core '" + tok + "'"; return false; }
    if (*end == '-') {
      const char* s = end + 1;
      b = strtol(s, &end, 10);
      if (end == s) { if (error) *error = "bad range '" + tok + "'"; return false; }
    }
    if (*end != '\0' || a < 0 || b < a) { if (error) *error = "bad range '" + tok + "'"; return false; }
    for (long c = a; c <= b; c++) {
      if (*count >= max_out) { if (error) *error = "too many cores"; return false; }
      out[(*count)++] = static_cast<int>(c);
    }
  }
  return true;
}

bool BindToCore(int core) {
  cpu_set_t set;
  CPU_ZERO(&set);
  CPU_SET(core, &set);
  return pthread_setaffinity_np(pthread_self(), sizeof(set), &set) == 0;
}

int GetDeviceNuma(const std::string& pci_bus_id) {
  std::string path = "/sys/bus/pci/devices/" + pci_bus_id + "/numa_node";
  FILE* f = fopen(path.c_str(), "r");
  if (!f) return -1;
  int node = -1;
  if (fscanf(f, "%d", &node) != 1) node = -1;
  fclose(f);
  return node;
}

bool GetCoresNuma(int node, int* out, int max_out, int* count) {
  *count = 0;
  if (node < 0) return false;
  std::string path = "/sys/devices/system/node/node" + std::to_string(node) + "/cpulist";
  FILE* f = fopen(path.c_str(), "r");
  if (!f) return false;
  char buf[4096];
  size_t n = fread(buf, 1, sizeof(buf) - 1, f);
  fclose(f);
  buf[n] = 0;
  std::string spec(buf);
  while (!spec.empty() && (spec.back() == '\n' || spec.back() == ' ')) spec.pop_back();
  std::string err;
  return ParseCoreList(spec, &err, out, max_out, count) && *count > 0;
}

bool BindToNumaNode(int node) {
  int ids[1024], count = 0;
  if (!GetCoresNuma(node, ids, 1024, &count)) return false;
  cpu_set_t set;
  CPU_ZERO(&set);
  for (int i = 0; i < count; i++)
    if (ids[i] >= 0 && ids[i] < CPU_SETSIZE) CPU_SET(ids[i], &set);
  return sched_setaffinity(0, sizeof(set), &set) == 0;
}

}  // namespace switchml
