// libnccl-net-switchml.so: a collective-network plugin that hands NCCL's in-network
// allreduce to the SwitchML context.
//
// Counterpart of the reference's frameworks_integration/nccl_plugin/switchml_plugin.cc
// (init starts the context :135-141, one device :147-151, reduceSupport :247-253, regMr as a
// book-keeping no-op :258-287, iallreduce -> AllReduceAsync with uint8 widened to int32
// :293-343, test polls the job :361-387; the widening lives in the context here, on the
// host for the CPU backends and in a kernel for backend = cuda). Differences, all deliberate:
//   * written against version 8 of NCCL's plugin interface, which a stock NCCL loads; the
//     reference needs a patched NCCL 2.8;
//   * listen/connect need no point-to-point ring of NCCL's own transport: the context has
//     its own rendezvous, so a handle only carries a magic number, the session and the rank,
//     and connect() checks them;
//   * with backend = cuda, device pointers are accepted (NCCL_PTR_CUDA) and bfloat16 sums
//     are offered; the reference takes host pointers only;
//   * a FAILED job makes test() return an error instead of polling forever;
//   * the context is stopped again when the last collective communicator is closed.
// iallgather and ireducescatter are not offered (the switch only aggregates).
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "nccl/nccl_net_abi.h"
#include "switchml/context.h"
#include "switchml/log.h"

namespace {

using switchml::Context;

constexpr uint32_t kHandleMagic = 0x534d4c38;  // "SML8"

struct Handle {  // travels through NCCL's bootstrap, at most SML_NCCL_NET_HANDLE_MAXSIZE bytes
  uint32_t magic;
  uint32_t rank;         // SwitchML rank of the listener
  uint32_t num_workers;  // size of its SwitchML session
  uint32_t backend_is_cuda;
};
static_assert(sizeof(Handle) <= SML_NCCL_NET_HANDLE_MAXSIZE, "handle too large");

struct ListenComm {
  int dev;
};

struct CollComm {
  int rank;
  int nranks;
};

struct MemHandle {
  int type;  // SML_NCCL_PTR_HOST or SML_NCCL_PTR_CUDA
  void* base;
  size_t size;
};

struct Request {
  enum Kind { kAllReduce, kFlush } kind = kAllReduce;
  smlNcclDataType_t data_type = smlNcclFloat32;
  void* recv = nullptr;
  int count = 0;
  std::shared_ptr<switchml::Job> job;
};

smlNcclDebugLogger_t g_logger = nullptr;
std::mutex g_mutex;
bool g_started_here = false;
int g_open_comms = 0;
std::atomic<uint64_t> g_requests{0};

double NowMs() {
  using namespace std::chrono;
  return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

// Tracing like the reference's TRACE macro (nccl_plugin/utils.h:33-48): through NCCL's logger
// when there is one, with a millisecond timestamp; also to the library's own log at -v 3.
#define PLUGIN_TRACE(...)                                                                        \
  do {                                                                                           \
    char sml_trace_buf[256];                                                                     \
    snprintf(sml_trace_buf, sizeof(sml_trace_buf), __VA_ARGS__);                                 \
    if (g_logger)                                                                                \
      g_logger(SML_NCCL_LOG_TRACE, SML_NCCL_INIT | SML_NCCL_NET, __FILE__, __LINE__, "[%.3f] %s", \
               NowMs(), sml_trace_buf);                                                          \
    SML_VLOG(3) << "nccl plugin: " << sml_trace_buf;                                             \
  } while (0)

#define PLUGIN_WARN(...)                                                                          \
  do {                                                                                            \
    char sml_warn_buf[256];                                                                       \
    snprintf(sml_warn_buf, sizeof(sml_warn_buf), __VA_ARGS__);                                    \
    if (g_logger) g_logger(SML_NCCL_LOG_WARN, ~0ul, __FILE__, __LINE__, "%s", sml_warn_buf);      \
    SML_LOG(WARNING) << "nccl plugin: " << sml_warn_buf;                                          \
  } while (0)

bool BackendIsCuda() { return Context::GetInstance().GetConfig().general_.backend == "cuda"; }

smlNcclResult_t EnsureStarted() {
  std::lock_guard<std::mutex> lock(g_mutex);
  Context& ctx = Context::GetInstance();
  if (ctx.GetContextState() == Context::RUNNING) return smlNcclSuccess;
  try {
    if (!ctx.Start()) return smlNcclSystemError;
  } catch (const std::exception& e) {
    PLUGIN_WARN("the SwitchML context did not start: %s", e.what());
    return smlNcclSystemError;
  }
  g_started_here = true;
  return smlNcclSuccess;
}

int TypeSize(smlNcclDataType_t t) {
  switch (t) {
    case smlNcclInt8: case smlNcclUint8: return 1;
    case smlNcclFloat16: case smlNcclBfloat16: return 2;
    case smlNcclInt32: case smlNcclUint32: case smlNcclFloat32: return 4;
    case smlNcclInt64: case smlNcclUint64: case smlNcclFloat64: return 8;
  }
  return -1;
}

bool TypeSupported(smlNcclDataType_t t) {
  switch (t) {
    case smlNcclInt32: case smlNcclFloat32: return true;
    case smlNcclUint8: return true;  // PyTorch reduces uint8 flags across workers; summed as int32
    case smlNcclBfloat16: return BackendIsCuda();
    default: return false;
  }
}

smlNcclResult_t PluginInit(smlNcclDebugLogger_t log_function) {
  g_logger = log_function;
  PLUGIN_TRACE("init");
  return EnsureStarted();
}

smlNcclResult_t PluginDevices(int* ndev) {
  *ndev = 1;
  return smlNcclSuccess;
}

smlNcclResult_t PluginGetProperties(int dev, smlNcclNetProperties_v8_t* props) {
  if (dev != 0 || props == nullptr) return smlNcclInvalidArgument;
  static char name[] = "SwitchML";
  const bool cuda = BackendIsCuda();
  memset(props, 0, sizeof(*props));
  props->name = name;
  props->pciPath = nullptr;
  props->guid = 0x5357495443484d4cull;  // "SWITCHML"
  props->ptrSupport = SML_NCCL_PTR_HOST | (cuda ? SML_NCCL_PTR_CUDA : 0);
  props->regIsGlobal = 1;  // registration keeps no per-communicator state
  props->speed = cuda ? 7200000 : 100000;  // Mbps: 900 GB/s of NVLink per direction, or a 100G port
  props->port = 0;
  props->latency = cuda ? 5.0f : 20.0f;
  props->maxComms = 1;  // one session per process, like the reference (:157)
  props->maxRecvs = 1;
  props->netDeviceType = SML_NCCL_NET_DEVICE_HOST;
  props->netDeviceVersion = 0;
  return smlNcclSuccess;
}

smlNcclResult_t PluginListen(int dev, void* handle, void** listen_comm) {
  if (dev != 0 || handle == nullptr || listen_comm == nullptr) return smlNcclInvalidArgument;
  smlNcclResult_t r = EnsureStarted();
  if (r != smlNcclSuccess) return r;
  const auto& general = Context::GetInstance().GetConfig().general_;
  Handle h{kHandleMagic, static_cast<uint32_t>(general.rank), static_cast<uint32_t>(general.num_workers),
           BackendIsCuda() ? 1u : 0u};
  memset(handle, 0, SML_NCCL_NET_HANDLE_MAXSIZE);
  memcpy(handle, &h, sizeof(h));
  *listen_comm = new ListenComm{dev};
  PLUGIN_TRACE("listen: SwitchML rank %u of %u", h.rank, h.num_workers);
  return smlNcclSuccess;
}

smlNcclResult_t PluginConnect(void* handles[], int nranks, int rank, void* listen_comm, void** coll_comm) {
  if (handles == nullptr || listen_comm == nullptr || coll_comm == nullptr) return smlNcclInvalidArgument;
  if (rank < 0 || rank >= nranks) {
    PLUGIN_WARN("connect: rank %d is not in [0, %d)", rank, nranks);
    return smlNcclInternalError;
  }
  const auto& general = Context::GetInstance().GetConfig().general_;
  if (static_cast<uint32_t>(nranks) != general.num_workers) {
    PLUGIN_WARN("connect: NCCL brings %d ranks, the SwitchML session has %u workers", nranks,
                static_cast<unsigned>(general.num_workers));
    return smlNcclInvalidUsage;
  }
  uint64_t seen = 0;
  for (int i = 0; i < nranks; ++i) {
    Handle h;
    memcpy(&h, handles[i], sizeof(h));
    if (h.magic != kHandleMagic || h.num_workers != general.num_workers || h.rank >= h.num_workers) {
      PLUGIN_WARN("connect: the handle of rank %d does not come from a worker of this session", i);
      return smlNcclInvalidUsage;
    }
    if (seen & (1ull << h.rank)) {
      PLUGIN_WARN("connect: two NCCL ranks use SwitchML rank %u", h.rank);
      return smlNcclInvalidUsage;
    }
    seen |= 1ull << h.rank;
  }
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    ++g_open_comms;
  }
  *coll_comm = new CollComm{rank, nranks};
  PLUGIN_TRACE("connect: rank %d of %d", rank, nranks);
  return smlNcclSuccess;
}

smlNcclResult_t PluginReduceSupport(smlNcclDataType_t type, smlNcclRedOp_t op, int* supported) {
  *supported = (op == smlNcclSum && TypeSupported(type)) ? 1 : 0;
  return smlNcclSuccess;
}

smlNcclResult_t PluginRegMr(void* coll_comm, void* data, size_t size, int type, void** mhandle) {
  if (mhandle == nullptr) return smlNcclInvalidArgument;
  if (type == SML_NCCL_PTR_CUDA && !BackendIsCuda()) {
    PLUGIN_WARN("regMr: device memory needs backend = cuda");
    return smlNcclInvalidUsage;
  }
  if (type != SML_NCCL_PTR_HOST && type != SML_NCCL_PTR_CUDA) return smlNcclInvalidArgument;
  *mhandle = new MemHandle{type, data, size};
  PLUGIN_TRACE("regMr: %zu bytes of %s memory", size, type == SML_NCCL_PTR_HOST ? "host" : "device");
  return smlNcclSuccess;
}

smlNcclResult_t PluginRegMrDmaBuf(void*, void*, size_t, int, uint64_t, int, void**) {
  return smlNcclInternalError;  // ptrSupport does not advertise dma-buf
}

smlNcclResult_t PluginDeregMr(void* coll_comm, void* mhandle) {
  delete static_cast<MemHandle*>(mhandle);
  return smlNcclSuccess;
}

bool Covers(const MemHandle* mh, const void* p, size_t bytes) {
  if (mh == nullptr) return true;  // NCCL may pass no handle for unregistered host memory
  const char* b = static_cast<const char*>(mh->base);
  const char* q = static_cast<const char*>(p);
  return q >= b && q + bytes <= b + mh->size;
}

smlNcclResult_t PluginIallreduce(void* coll_comm, void* send, void* recv, int count, smlNcclDataType_t type,
                                 smlNcclRedOp_t op, void* send_mh, void* recv_mh, void** request) {
  if (request == nullptr || count < 0) return smlNcclInvalidArgument;
  if (op != smlNcclSum || !TypeSupported(type)) return smlNcclInvalidArgument;
  const auto* smh = static_cast<const MemHandle*>(send_mh);
  const auto* rmh = static_cast<const MemHandle*>(recv_mh);
  const size_t bytes = static_cast<size_t>(count) * TypeSize(type);
  if (!Covers(smh, send, bytes) || !Covers(rmh, recv, bytes)) {
    PLUGIN_WARN("iallreduce: the buffers lie outside their registered regions");
    return smlNcclInvalidArgument;
  }
  auto req = std::make_unique<Request>();
  req->data_type = type;
  req->recv = recv;
  req->count = count;
  switchml::DataType dt = switchml::FLOAT32;
  switch (type) {
    case smlNcclFloat32: dt = switchml::FLOAT32; break;
    case smlNcclInt32: dt = switchml::INT32; break;
    case smlNcclBfloat16: dt = switchml::BFLOAT16; break;
    case smlNcclUint8: dt = switchml::UINT8; break;  // widened to int32 inside the context
    default: return smlNcclInvalidArgument;
  }
  try {
    req->job = Context::GetInstance().AllReduceAsync(send, recv, static_cast<uint64_t>(count), dt, switchml::SUM);
  } catch (const std::exception& e) {
    PLUGIN_WARN("iallreduce: %s", e.what());
    return smlNcclInternalError;
  }
  if (!req->job) return smlNcclInternalError;
  g_requests.fetch_add(1, std::memory_order_relaxed);
  PLUGIN_TRACE("iallreduce: job %llu, %d elements of type %d", static_cast<unsigned long long>(req->job->id_),
               count, static_cast<int>(type));
  *request = req.release();
  return smlNcclSuccess;
}

smlNcclResult_t PluginIallgather(void*, void*, int, smlNcclNetSGE_v8_t*, size_t, size_t, size_t, void*,
                                 void** request) {
  if (request) *request = nullptr;
  PLUGIN_WARN("iallgather is not offered: the switch only aggregates");
  return smlNcclInternalError;
}

smlNcclResult_t PluginIreducescatter(void*, int, smlNcclNetSGE_v8_t*, void*, size_t, size_t, size_t,
                                     smlNcclDataType_t, smlNcclRedOp_t, void*, void** request) {
  if (request) *request = nullptr;
  PLUGIN_WARN("ireducescatter is not offered: the switch only aggregates");
  return smlNcclInternalError;
}

smlNcclResult_t PluginIflush(void* coll_comm, void* data, int size, void* mhandle, void** request) {
  // A finished job's result is already visible to the GPU: device results are written by
  // kernels of this process, host results by its worker threads. Nothing to flush.
  if (request == nullptr) return smlNcclInvalidArgument;
  auto* req = new Request();
  req->kind = Request::kFlush;
  req->count = size;
  *request = req;
  return smlNcclSuccess;
}

smlNcclResult_t PluginTest(void* request, int* done, int* size) {
  auto* req = static_cast<Request*>(request);
  if (req == nullptr || done == nullptr) return smlNcclInvalidArgument;
  if (req->kind == Request::kFlush) {
    *done = 1;
    if (size) *size = req->count;
    delete req;
    return smlNcclSuccess;
  }
  const switchml::JobStatus st = req->job->GetJobStatus();
  if (st == switchml::FAILED) {
    PLUGIN_WARN("job %llu failed", static_cast<unsigned long long>(req->job->id_));
    *done = 0;
    delete req;
    return smlNcclRemoteError;
  }
  if (st != switchml::FINISHED) {
    *done = 0;
    return smlNcclSuccess;
  }
  *done = 1;
  if (size) *size = req->count * TypeSize(req->data_type);
  PLUGIN_TRACE("test: job %llu finished", static_cast<unsigned long long>(req->job->id_));
  delete req;
  return smlNcclSuccess;
}

smlNcclResult_t PluginCloseColl(void* coll_comm) {
  delete static_cast<CollComm*>(coll_comm);
  bool stop = false;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_open_comms > 0 && --g_open_comms == 0 && g_started_here) {
      stop = true;
      g_started_here = false;
    }
  }
  if (stop) {
    PLUGIN_TRACE("closeColl: last communicator, stopping the context after %llu requests",
                 static_cast<unsigned long long>(g_requests.load()));
    Context::GetInstance().Stop();
  }
  return smlNcclSuccess;
}

smlNcclResult_t PluginCloseListen(void* listen_comm) {
  delete static_cast<ListenComm*>(listen_comm);
  return smlNcclSuccess;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) smlNcclCollNet_v8_t ncclCollNetPlugin_v8 = {
    "SWITCHMLv8",      PluginInit,        PluginDevices,    PluginGetProperties, PluginListen,
    PluginConnect,     PluginReduceSupport, PluginRegMr,    PluginRegMrDmaBuf,   PluginDeregMr,
    PluginIallreduce,  PluginIallgather,  PluginIreducescatter, PluginIflush,    PluginTest,
    PluginCloseColl,   PluginCloseListen,
};
