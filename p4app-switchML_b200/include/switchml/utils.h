// Small host-side helpers.
// Parity: reference client_lib/src/utils.h:38-101 (reusable thread Barrier with
// Destroy(), Execute(cmd) popen helper).
#ifndef SWITCHML_UTILS_H_
#define SWITCHML_UTILS_H_

#include <condition_variable>
#include <mutex>
#include <string>

namespace switchml {

// Reusable barrier for a fixed number of threads. Destroy() releases every waiter and
// makes all later Wait() calls return immediately (used to unblock workers at Stop()).
class Barrier {
 public:
  explicit Barrier(int num_participants);
  Barrier(const Barrier&) = delete;
  void operator=(const Barrier&) = delete;
  // Returns true for a normal release, false if the barrier was destroyed.
  bool Wait();
  void Destroy();

 private:
  const int num_participants_;
  int waiting_ = 0;
  unsigned long generation_ = 0;
  bool destroyed_ = false;
  std::mutex mu_;
  std::condition_variable cv_;
};

// Run a shell command and return its standard output.
std::string Execute(const char* cmd);

// Parse "a-b,c" style core lists ("0-3", "0,2,4-6") into ids; empty on syntax error.
bool ParseCoreList(const std::string& spec, std::string* error, int* out, int max_out, int* count);

}  // namespace switchml
#endif  // SWITCHML_UTILS_H_
