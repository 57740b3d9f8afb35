// The slice of NCCL's public external-network plugin interface that a collective-network
// plugin needs, version 8 of that interface (NCCL 2.19 and later look up the symbol
// `ncclCollNetPlugin_v8` in libnccl-net-<name>.so). Declared here, from the published
// interface, so that the plugin builds without NCCL's source tree; the values of the
// enums are those of nccl.h.
#ifndef SWITCHML_NCCL_NET_ABI_H_
#define SWITCHML_NCCL_NET_ABI_H_

#include <stddef.h>
#include <stdint.h>

extern "C" {

typedef enum {
  smlNcclSuccess = 0,
  smlNcclUnhandledCudaError = 1,
  smlNcclSystemError = 2,
  smlNcclInternalError = 3,
  smlNcclInvalidArgument = 4,
  smlNcclInvalidUsage = 5,
  smlNcclRemoteError = 6,
  smlNcclInProgress = 7,
} smlNcclResult_t;

typedef enum {
  smlNcclInt8 = 0,
  smlNcclUint8 = 1,
  smlNcclInt32 = 2,
  smlNcclUint32 = 3,
  smlNcclInt64 = 4,
  smlNcclUint64 = 5,
  smlNcclFloat16 = 6,
  smlNcclFloat32 = 7,
  smlNcclFloat64 = 8,
  smlNcclBfloat16 = 9,
} smlNcclDataType_t;

typedef enum {
  smlNcclSum = 0,
  smlNcclProd = 1,
  smlNcclMax = 2,
  smlNcclMin = 3,
  smlNcclAvg = 4,
} smlNcclRedOp_t;

typedef enum { SML_NCCL_LOG_NONE = 0, SML_NCCL_LOG_VERSION, SML_NCCL_LOG_WARN, SML_NCCL_LOG_INFO,
               SML_NCCL_LOG_ABORT, SML_NCCL_LOG_TRACE } smlNcclDebugLogLevel;

typedef void (*smlNcclDebugLogger_t)(smlNcclDebugLogLevel level, unsigned long flags, const char* file,
                                     int line, const char* fmt, ...);

#define SML_NCCL_INIT 0x1
#define SML_NCCL_NET 0x10
#define SML_NCCL_NET_HANDLE_MAXSIZE 128
#define SML_NCCL_PTR_HOST 0x1
#define SML_NCCL_PTR_CUDA 0x2
#define SML_NCCL_PTR_DMABUF 0x4
#define SML_NCCL_NET_DEVICE_HOST 0

typedef struct {
  char* name;
  char* pciPath;
  uint64_t guid;
  int ptrSupport;
  int regIsGlobal;
  int speed;      // Mbps
  int port;
  float latency;  // us
  int maxComms;
  int maxRecvs;
  int netDeviceType;
  int netDeviceVersion;
} smlNcclNetProperties_v8_t;

typedef struct {
  void* mhandle;
  void* address;
  uint32_t size;
} smlNcclNetSGE_v8_t;

typedef struct {
  const char* name;
  smlNcclResult_t (*init)(smlNcclDebugLogger_t logFunction);
  smlNcclResult_t (*devices)(int* ndev);
  smlNcclResult_t (*getProperties)(int dev, smlNcclNetProperties_v8_t* props);
  smlNcclResult_t (*listen)(int dev, void* handle, void** listenComm);
  smlNcclResult_t (*connect)(void* handles[], int nranks, int rank, void* listenComm, void** collComm);
  smlNcclResult_t (*reduceSupport)(smlNcclDataType_t dataType, smlNcclRedOp_t redOp, int* supported);
  smlNcclResult_t (*regMr)(void* collComm, void* data, size_t size, int type, void** mhandle);
  smlNcclResult_t (*regMrDmaBuf)(void* collComm, void* data, size_t size, int type, uint64_t offset,
                                 int fd, void** mhandle);
  smlNcclResult_t (*deregMr)(void* collComm, void* mhandle);
  smlNcclResult_t (*iallreduce)(void* collComm, void* sendData, void* recvData, int count,
                                smlNcclDataType_t dataType, smlNcclRedOp_t redOp, void* sendMhandle,
                                void* recvMhandle, void** request);
  smlNcclResult_t (*iallgather)(void* collComm, void* sendData, int nRecvParts, smlNcclNetSGE_v8_t* recvParts,
                                size_t bytesPerRank, size_t windowOffset, size_t windowBytes,
                                void* sendMhandle, void** request);
  smlNcclResult_t (*ireducescatter)(void* collComm, int nSendParts, smlNcclNetSGE_v8_t* sendParts,
                                    void* recvData, size_t bytesPerRank, size_t windowOffset,
                                    size_t windowBytes, smlNcclDataType_t dataType, smlNcclRedOp_t redOp,
                                    void* recvMhandle, void** request);
  smlNcclResult_t (*iflush)(void* collComm, void* data, int size, void* mhandle, void** request);
  smlNcclResult_t (*test)(void* request, int* done, int* size);
  smlNcclResult_t (*closeColl)(void* collComm);
  smlNcclResult_t (*closeListen)(void* listenComm);
} smlNcclCollNet_v8_t;

}  // extern "C"

#endif  // SWITCHML_NCCL_NET_ABI_H_
