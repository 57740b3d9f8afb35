// collnet_harness: drives libnccl-net-switchml.so the way NCCL's proxy thread does, without
// NCCL: dlopen, look up ncclCollNetPlugin_v8, init, devices, getProperties, reduceSupport,
// listen, exchange of the handles (through files in a directory every rank can see),
// connect, regMr, iallreduce + test for float32 / int32 / uint8, iflush, deregMr, closeColl,
// closeListen. Every rank is one process; rank and session size come from the SwitchML
// configuration (switchml.cfg, SWITCHML_RANK, SWITCHML_NUM_WORKERS).
//
//   collnet_harness --plugin lib/libnccl-net-switchml.so --exchange-dir /tmp/x [--numel 5000]
//                   [--device cpu|pinned|gpu] [--rounds 3]
//
// Prints "collnet harness ok" and exits 0 when every result equals the expected sum.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <unistd.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <thread>
#include <vector>

#include "nccl/nccl_net_abi.h"
#include "switchml/cli_flags.h"
#include "switchml/context.h"

namespace {

int g_log_lines = 0;

enum Memory { kHost, kPinned, kDevice };

void Logger(smlNcclDebugLogLevel level, unsigned long flags, const char* file, int line, const char* fmt, ...) {
  ++g_log_lines;
  if (level != SML_NCCL_LOG_WARN && getenv("COLLNET_HARNESS_TRACE") == nullptr) return;
  va_list ap;
  va_start(ap, fmt);
  fprintf(stderr, "[plugin %s] ", level == SML_NCCL_LOG_WARN ? "WARN" : "TRACE");
  vfprintf(stderr, fmt, ap);
  fprintf(stderr, "\n");
  va_end(ap);
}

#define CHECK_OK(call)                                                               \
  do {                                                                               \
    smlNcclResult_t sml_r = (call);                                                  \
    if (sml_r != smlNcclSuccess) {                                                   \
      fprintf(stderr, "%s:%d: %s returned %d\n", __FILE__, __LINE__, #call, sml_r);  \
      return 1;                                                                      \
    }                                                                                \
  } while (0)

#define EXPECT(cond)                                                         \
  do {                                                                       \
    if (!(cond)) {                                                           \
      fprintf(stderr, "%s:%d: expected %s\n", __FILE__, __LINE__, #cond);    \
      return 1;                                                              \
    }                                                                        \
  } while (0)

bool WaitDone(smlNcclCollNet_v8_t* net, void* request, int* size, double limit_s) {
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    int done = 0;
    if (net->test(request, &done, size) != smlNcclSuccess) return false;
    if (done) return true;
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit_s) return false;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

// Run one allreduce of `count` elements of T whose value on rank r is base + r.
template <typename T>
int OneRound(smlNcclCollNet_v8_t* net, void* comm, smlNcclDataType_t type, int count, int rank, int nranks, int base,
             Memory mem) {
  const bool gpu = mem == kDevice;
  std::vector<T> send(count), recv(count, T(0));
  for (int i = 0; i < count; ++i) send[i] = static_cast<T>(base + rank + (i % 3));
  void* s = send.data();
  void* r = recv.data();
  const size_t bytes = sizeof(T) * count;
  if (gpu) {
    EXPECT(cudaMalloc(&s, bytes) == cudaSuccess && cudaMalloc(&r, bytes) == cudaSuccess);
    EXPECT(cudaMemcpy(s, send.data(), bytes, cudaMemcpyHostToDevice) == cudaSuccess);
    EXPECT(cudaMemset(r, 0, bytes) == cudaSuccess);
  } else if (mem == kPinned) {
    // What NCCL hands a plugin as NCCL_PTR_HOST: page-locked memory the GPU can reach.
    EXPECT(cudaHostAlloc(&s, bytes, cudaHostAllocMapped) == cudaSuccess);
    EXPECT(cudaHostAlloc(&r, bytes, cudaHostAllocMapped) == cudaSuccess);
    memcpy(s, send.data(), bytes);
    memset(r, 0, bytes);
  }
  const int ptr_type = gpu ? SML_NCCL_PTR_CUDA : SML_NCCL_PTR_HOST;
  void *smh = nullptr, *rmh = nullptr, *req = nullptr;
  CHECK_OK(net->regMr(comm, s, bytes, ptr_type, &smh));
  CHECK_OK(net->regMr(comm, r, bytes, ptr_type, &rmh));
  CHECK_OK(net->iallreduce(comm, s, r, count, type, smlNcclSum, smh, rmh, &req));
  EXPECT(req != nullptr);
  int size = -1;
  EXPECT(WaitDone(net, req, &size, 60.0));
  EXPECT(size == static_cast<int>(bytes));
  void* freq = nullptr;
  CHECK_OK(net->iflush(comm, r, static_cast<int>(bytes), rmh, &freq));
  if (freq) EXPECT(WaitDone(net, freq, &size, 5.0));
  if (gpu) EXPECT(cudaMemcpy(recv.data(), r, bytes, cudaMemcpyDeviceToHost) == cudaSuccess);
  if (mem == kPinned) memcpy(recv.data(), r, bytes);
  for (int i = 0; i < count; ++i) {
    long expect = static_cast<long>(nranks) * (base + (i % 3)) + static_cast<long>(nranks) * (nranks - 1) / 2;
    if (type == smlNcclUint8) expect &= 0xff;
    const double got = static_cast<double>(recv[i]);
    const double tol = sizeof(T) == 4 && type == smlNcclFloat32 ? 1e-2 * expect + 1e-3 : 0.0;
    if (got < expect - tol || got > expect + tol) {
      fprintf(stderr, "type %d element %d: got %f, expected %ld\n", static_cast<int>(type), i, got, expect);
      return 1;
    }
  }
  CHECK_OK(net->deregMr(comm, smh));
  CHECK_OK(net->deregMr(comm, rmh));
  if (gpu) {
    cudaFree(s);
    cudaFree(r);
  } else if (mem == kPinned) {
    cudaFreeHost(s);
    cudaFreeHost(r);
  }
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  switchml::CliFlags flags;
  flags.Add("plugin", "lib/libnccl-net-switchml.so", "Path of the plugin.")
      .Add("exchange-dir", "", "Directory visible to every rank, used to pass the listen handles around.")
      .Add("numel", "5000", "Elements per allreduce.")
      .Add("rounds", "3", "Allreduces per data type.")
      .Add("device", "cpu", "Where the buffers live: cpu (ordinary host memory), pinned (page-locked host memory, "
                            "the only host memory backend = cuda accepts) or gpu.");
  if (!flags.Parse(argc, argv, "collnet_harness: drives the NCCL collective-network plugin without NCCL")) return 2;
  const std::string dir = flags.Str("exchange-dir");
  const int count = static_cast<int>(flags.U64("numel"));
  const int rounds = static_cast<int>(flags.U64("rounds"));
  const std::string where = flags.Str("device");
  const Memory mem = where == "gpu" ? kDevice : where == "pinned" ? kPinned : kHost;
  const bool gpu = mem == kDevice;

  void* lib = dlopen(flags.Str("plugin").c_str(), RTLD_NOW | RTLD_LOCAL);
  if (lib == nullptr) {
    fprintf(stderr, "dlopen: %s\n", dlerror());
    return 1;
  }
  auto* net = static_cast<smlNcclCollNet_v8_t*>(dlsym(lib, "ncclCollNetPlugin_v8"));
  if (net == nullptr) {
    fprintf(stderr, "the plugin does not export ncclCollNetPlugin_v8\n");
    return 1;
  }
  printf("plugin name: %s\n", net->name);

  CHECK_OK(net->init(Logger));
  int ndev = 0;
  CHECK_OK(net->devices(&ndev));
  EXPECT(ndev == 1);
  smlNcclNetProperties_v8_t props;
  CHECK_OK(net->getProperties(0, &props));
  printf("device 0: %s, ptrSupport 0x%x, speed %d Mbps, maxComms %d\n", props.name, props.ptrSupport, props.speed,
         props.maxComms);
  EXPECT(props.ptrSupport & SML_NCCL_PTR_HOST);
  if (gpu) EXPECT(props.ptrSupport & SML_NCCL_PTR_CUDA);

  int ok = 0;
  CHECK_OK(net->reduceSupport(smlNcclFloat32, smlNcclSum, &ok));
  EXPECT(ok == 1);
  CHECK_OK(net->reduceSupport(smlNcclInt32, smlNcclSum, &ok));
  EXPECT(ok == 1);
  CHECK_OK(net->reduceSupport(smlNcclUint8, smlNcclSum, &ok));
  EXPECT(ok == 1);
  CHECK_OK(net->reduceSupport(smlNcclFloat64, smlNcclSum, &ok));
  EXPECT(ok == 0);
  CHECK_OK(net->reduceSupport(smlNcclFloat32, smlNcclMax, &ok));
  EXPECT(ok == 0);

  // The plugin started the context; the session's shape is read back from it.
  const auto& general = switchml::Context::GetInstance().GetConfig().general_;
  const int rank = static_cast<int>(general.rank);
  const int nranks = static_cast<int>(general.num_workers);

  char handle[SML_NCCL_NET_HANDLE_MAXSIZE];
  void* listen_comm = nullptr;
  CHECK_OK(net->listen(0, handle, &listen_comm));

  std::vector<std::vector<char>> all(nranks, std::vector<char>(SML_NCCL_NET_HANDLE_MAXSIZE));
  memcpy(all[rank].data(), handle, sizeof(handle));
  if (nranks > 1) {
    EXPECT(!dir.empty());
    const std::string mine = dir + "/handle." + std::to_string(rank);
    {
      std::ofstream f(mine + ".tmp", std::ios::binary);
      f.write(handle, sizeof(handle));
    }
    EXPECT(rename((mine + ".tmp").c_str(), mine.c_str()) == 0);
    for (int r = 0; r < nranks; ++r) {
      if (r == rank) continue;
      const std::string theirs = dir + "/handle." + std::to_string(r);
      bool got = false;
      for (int tries = 0; tries < 6000 && !got; ++tries) {
        std::ifstream f(theirs, std::ios::binary);
        if (f && f.read(all[r].data(), SML_NCCL_NET_HANDLE_MAXSIZE)) got = true;
        else std::this_thread::sleep_for(std::chrono::milliseconds(10));
      }
      EXPECT(got);
    }
  }
  std::vector<void*> handles(nranks);
  for (int r = 0; r < nranks; ++r) handles[r] = all[r].data();

  // A foreign handle must be refused.
  {
    std::vector<char> bogus(SML_NCCL_NET_HANDLE_MAXSIZE, 0);
    std::vector<void*> bad = handles;
    bad[0] = bogus.data();
    void* none = nullptr;
    EXPECT(net->connect(bad.data(), nranks, rank, listen_comm, &none) != smlNcclSuccess);
  }
  void* comm = nullptr;
  CHECK_OK(net->connect(handles.data(), nranks, rank, listen_comm, &comm));
  EXPECT(comm != nullptr);

  for (int i = 0; i < rounds; ++i) {
    if (OneRound<float>(net, comm, smlNcclFloat32, count, rank, nranks, 1 + i, mem)) return 1;
    if (OneRound<int32_t>(net, comm, smlNcclInt32, count, rank, nranks, 100 + i, mem)) return 1;
    if (OneRound<uint8_t>(net, comm, smlNcclUint8, count, rank, nranks, 1 + i, mem)) return 1;
  }

  // Unsupported requests come back as errors, not as jobs.
  if (mem == kHost) {
    std::vector<double> d(8, 1.0);
    void *mh = nullptr, *req = nullptr;
    CHECK_OK(net->regMr(comm, d.data(), 64, SML_NCCL_PTR_HOST, &mh));
    EXPECT(net->iallreduce(comm, d.data(), d.data(), 8, smlNcclFloat64, smlNcclSum, mh, mh, &req) != smlNcclSuccess);
    EXPECT(net->iallreduce(comm, d.data(), d.data(), 64, smlNcclFloat32, smlNcclSum, mh, mh, &req) != smlNcclSuccess);
    CHECK_OK(net->deregMr(comm, mh));
  }

  CHECK_OK(net->closeColl(comm));
  CHECK_OK(net->closeListen(listen_comm));
  EXPECT(switchml::Context::GetInstance().GetContextState() != switchml::Context::RUNNING);
  printf("collnet harness ok: rank %d of %d, %d rounds of %d elements on the %s, %d log lines\n", rank, nranks, rounds,
         count, gpu ? "gpu" : (mem == kPinned ? "pinned host memory" : "cpu"), g_log_lines);
  return 0;
}
