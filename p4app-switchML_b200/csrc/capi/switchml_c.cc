// C interface: see switchml/switchml_c.h.
#include "switchml/switchml_c.h"

#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "backends/cuda/cuda_backend.h"
#include "ppp/cpu_exponent_quantizer_ppp.h"
#include "rendezvous/control.h"
#include "switchml/context.h"
#include "switchml/log.h"
#include "switchml/version.h"

using namespace switchml;

namespace {
thread_local std::string g_error;
std::mutex g_jobs_mu;
std::map<int64_t, std::shared_ptr<Job>> g_jobs;
int64_t g_next_handle = 1;

int Fail(const std::string& what) {
  g_error = what;
  return -1;
}

int CopyOut(const std::string& s, char* buf, size_t len) {
  if (!buf || len == 0) return static_cast<int>(s.size());
  size_t n = s.size() < len - 1 ? s.size() : len - 1;
  memcpy(buf, s.data(), n);
  buf[n] = '\0';
  return static_cast<int>(s.size());
}

std::shared_ptr<Job> Lookup(int64_t h) {
  std::lock_guard<std::mutex> lk(g_jobs_mu);
  auto it = g_jobs.find(h);
  return it == g_jobs.end() ? nullptr : it->second;
}

CudaBackendInterface* Cuda() {
  Context& c = Context::GetInstance();
  if (c.GetContextState() != Context::RUNNING) return nullptr;
  return dynamic_cast<CudaBackendInterface*>(c.GetBackend());
}
}  // namespace

extern "C" {

const char* sml_version(void) { return SWITCHML_VERSION; }
const char* sml_last_error(void) { return g_error.c_str(); }
int sml_checked_build(void) { return KernelsCheckedBuild() ? 1 : 0; }
void sml_set_verbosity(int v) { SetVerbosity(v); }
void sml_set_vmodule(const char* spec) { SetVModule(spec); }

int sml_start(const char* ini_text, int apply_env) {
  try {
    Context& ctx = Context::GetInstance();
    if (!ini_text || !*ini_text) {
      return ctx.Start(nullptr) ? 0 : Fail("Context::Start failed (see log)");
    }
    Config cfg;
    if (!cfg.LoadFromString(ini_text)) return Fail("configuration does not parse");
    if (apply_env) cfg.ApplyEnvOverrides();
    return ctx.Start(&cfg) ? 0 : Fail("Context::Start failed (see log)");
  } catch (const std::exception& e) {
    return Fail(e.what());
  }
}

int sml_start_file(const char* path) {
  try {
    Config cfg;
    if (!cfg.LoadFromFile(path ? path : "")) return Fail("cannot load configuration file");
    cfg.ApplyEnvOverrides();
    return Context::GetInstance().Start(&cfg) ? 0 : Fail("Context::Start failed (see log)");
  } catch (const std::exception& e) {
    return Fail(e.what());
  }
}

int sml_stop(void) {
  try {
    // Job handles outlive the context: Stop() fails what is still queued or running, and the
    // caller must be able to read the status and the reason afterwards. sml_job_release()
    // is what frees a handle.
    Context::GetInstance().Stop();
    return 0;
  } catch (const std::exception& e) {
    return Fail(e.what());
  }
}

int sml_state(void) { return static_cast<int>(Context::GetInstance().GetContextState()); }

int sml_config_dump(char* buf, size_t len) {
  return CopyOut(Context::GetInstance().GetConfig().ToString(), buf, len);
}

int sml_config_check(const char* ini_text, char* buf, size_t len) {
  try {
    Config cfg;
    if (!cfg.LoadFromString(ini_text ? ini_text : "")) return Fail("configuration does not parse");
    cfg.Validate();
    return CopyOut(cfg.ToString(), buf, len);
  } catch (const std::exception& e) {
    return Fail(e.what());
  }
}

int64_t sml_allreduce_async(void* in, void* out, uint64_t numel, int dtype, void* stream) {
  try {
    if (dtype < 0 || dtype > 3) return Fail("bad dtype");
    std::shared_ptr<Job> job = Context::GetInstance().AllReduceAsync(
        in, out, numel, static_cast<DataType>(dtype), SUM, stream);
    std::lock_guard<std::mutex> lk(g_jobs_mu);
    int64_t h = g_next_handle++;
    g_jobs[h] = job;
    return h;
  } catch (const std::exception& e) {
    return Fail(e.what());
  }
}

int64_t sml_broadcast_async(void* ptr, uint64_t numel, int dtype, int root, void* stream) {
  try {
    if (dtype < 0 || dtype > 3) return Fail("bad dtype");
    std::shared_ptr<Job> job =
        Context::GetInstance().BroadcastAsync(ptr, numel, static_cast<DataType>(dtype), root, stream);
    std::lock_guard<std::mutex> lk(g_jobs_mu);
    int64_t h = g_next_handle++;
    g_jobs[h] = job;
    return h;
  } catch (const std::exception& e) {
    return Fail(e.what());
  }
}

int sml_allreduce(void* in, void* out, uint64_t numel, int dtype) {
  try {
    if (dtype < 0 || dtype > 3) return Fail("bad dtype");
    std::shared_ptr<Job> job =
        Context::GetInstance().AllReduce(in, out, numel, static_cast<DataType>(dtype), SUM);
    if (job->GetJobStatus() != FINISHED) return Fail("job failed: " + job->failure_reason_);
    return 0;
  } catch (const std::exception& e) {
    return Fail(e.what());
  }
}

int sml_job_wait(int64_t h, double timeout_ms) {
  std::shared_ptr<Job> job = Lookup(h);
  if (!job) return Fail("unknown job handle");
  if (timeout_ms < 0) job->WaitToComplete();
  else job->WaitToCompleteFor(timeout_ms);
  return static_cast<int>(job->GetJobStatus());
}

int sml_job_status(int64_t h) {
  std::shared_ptr<Job> job = Lookup(h);
  if (!job) return Fail("unknown job handle");
  return static_cast<int>(job->GetJobStatus());
}

int sml_job_stream_wait(int64_t h, void* stream) {
  std::shared_ptr<Job> job = Lookup(h);
  if (!job) return Fail("unknown job handle");
  return job->StreamWait(stream) ? 0 : Fail("job failed: " + job->failure_reason_);
}

int sml_job_error(int64_t h, char* buf, size_t len) {
  std::shared_ptr<Job> job = Lookup(h);
  if (!job) return Fail("unknown job handle");
  return CopyOut(job->failure_reason_, buf, len);
}

void sml_job_release(int64_t h) {
  std::lock_guard<std::mutex> lk(g_jobs_mu);
  g_jobs.erase(h);
}

void sml_wait_all(void) {
  try {
    Context::GetInstance().WaitForAllJobs();
  } catch (const std::exception& e) {
    Fail(e.what());
  }
}

int sml_stats_json(char* buf, size_t len) {
  Context& c = Context::GetInstance();
  std::string s = c.GetStats().ToJson();
  std::string extra = c.GetBackend() ? c.GetBackend()->ExtraStatsJson() : "{}";
  s.pop_back();
  s += ",\"backend\":" + extra + "}";
  return CopyOut(s, buf, len);
}

int sml_stats_report(char* buf, size_t len) {
  return CopyOut(Context::GetInstance().GetStats().Report(), buf, len);
}

void sml_stats_reset(void) { Context::GetInstance().GetStats().ResetStats(); }

void* sml_symm_alloc(size_t bytes) {
  CudaBackendInterface* b = Cuda();
  return b ? b->SymmetricAlloc(bytes) : nullptr;
}

void sml_symm_reset(void) {
  CudaBackendInterface* b = Cuda();
  if (b) b->SymmetricReset();
}

int sml_uses_multimem(void) {
  CudaBackendInterface* b = Cuda();
  return b && b->UsesMultimem() ? 1 : 0;
}

int sml_symm_info(void** local, void** peers, void** multicast, size_t* bytes) {
  CudaBackendInterface* b = Cuda();
  if (!b || !b->SymmetricHeapInfo(local, peers, multicast, bytes)) return Fail("no symmetric heap");
  return 0;
}

int sml_device(void) {
  CudaBackendInterface* b = Cuda();
  return b ? b->Device() : -1;
}

int sml_wait_probe(double budget_ms) {
  CudaBackendInterface* b = Cuda();
  if (!b) return Fail("the cuda backend is not running");
  return b->RunWaitProbe(budget_ms);
}

void sml_oracle_quant_allreduce(const float* const* inputs, int num_workers, uint64_t numel,
                                uint64_t block_numel, float* out) {
  OracleQuantAllReduce(inputs, num_workers, numel, block_numel, out);
}

void sml_oracle_int_allreduce(const int32_t* const* inputs, int num_workers, uint64_t numel,
                              int32_t* out) {
  OracleIntAllReduce(inputs, num_workers, numel, out);
}

void sml_static_slice(uint64_t numel, int parts, int index, uint64_t* offset, uint64_t* length) {
  Numel o, l;
  StaticSlice(numel, parts, index, &o, &l);
  *offset = o;
  *length = l;
}

int sml_emu_allreduce(int nranks, void* const* in_ptrs, void* const* out_ptrs, uint64_t numel,
                      int elem_type, int mode, int algo, int block_numel, uint64_t slot_bytes,
                      int slots_per_channel, int channels, float post_scale, int repeats,
                      int exponent_lookahead) {
  std::string err;
  int r = EmulatedAllReduce(nranks, in_ptrs, out_ptrs, numel, elem_type, mode, algo, block_numel,
                            slot_bytes, slots_per_channel, channels, post_scale, repeats,
                            exponent_lookahead, &err);
  if (r != 0) g_error = err;
  return r;
}

int sml_convert_u8(int widen, const void* in, void* out, uint64_t numel, void* stream) {
  std::string err;
  int r = ConvertU8OnDevice(widen != 0, in, out, numel, stream, &err);
  if (r != 0) g_error = err;
  return r;
}

void* sml_controller_start(const char* ip, int port, int udp_port) {
  return sml_controller_start_pipes(ip, port, udp_port, 1);
}

void* sml_controller_start_pipes(const char* ip, int port, int udp_port, int pipes) {
  ControlServer* s = new ControlServer();
  if (!s->Start(ip ? ip : "127.0.0.1", static_cast<uint16_t>(port), static_cast<uint16_t>(udp_port), pipes)) {
    delete s;
    Fail("cannot start the controller");
    return nullptr;
  }
  return s;
}

int sml_controller_port(void* server) { return static_cast<ControlServer*>(server)->port(); }
int sml_controller_udp_port(void* server) { return static_cast<ControlServer*>(server)->udp_port(); }

void sml_controller_stop(void* server) {
  ControlServer* s = static_cast<ControlServer*>(server);
  s->Stop();
  delete s;
}

int sml_controller_command(const char* ip, int port, const char* line, char* buf, size_t len) {
  ControlClient c;
  if (!c.Connect(ip ? ip : "127.0.0.1", static_cast<uint16_t>(port), 2000)) return Fail("controller unreachable");
  std::string reply;
  if (!c.Command(line, &reply)) return Fail("command failed");
  return CopyOut(reply, buf, len);
}

}  // extern "C"
