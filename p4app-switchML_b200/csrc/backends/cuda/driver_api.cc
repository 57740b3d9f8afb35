// See driver_api.h.
#include "backends/cuda/driver_api.h"

#include <cuda_runtime.h>

#include <mutex>

namespace switchml {

namespace {
template <typename F>
bool Load(const char* name, F* fn, std::string* err) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    if (err) *err = std::string("driver symbol ") + name + " unavailable: " + cudaGetErrorString(e);
    cudaGetLastError();
    return false;
  }
  *fn = reinterpret_cast<F>(p);
  return true;
}
}  // namespace

const DriverApi* DriverApi::Get(std::string* error) {
  static DriverApi api;
  static bool ok = false;
  static std::string err;
  static std::once_flag once;
  std::call_once(once, [] {
    ok = Load("cuMemCreate", &api.MemCreate, &err) && Load("cuMemRelease", &api.MemRelease, &err) &&
         Load("cuMemAddressReserve", &api.MemAddressReserve, &err) &&
         Load("cuMemAddressFree", &api.MemAddressFree, &err) && Load("cuMemMap", &api.MemMap, &err) &&
         Load("cuMemUnmap", &api.MemUnmap, &err) && Load("cuMemSetAccess", &api.MemSetAccess, &err) &&
         Load("cuMemGetAllocationGranularity", &api.MemGetAllocationGranularity, &err) &&
         Load("cuMemExportToShareableHandle", &api.MemExportToShareableHandle, &err) &&
         Load("cuMemImportFromShareableHandle", &api.MemImportFromShareableHandle, &err) &&
         Load("cuMulticastCreate", &api.MulticastCreate, &err) &&
         Load("cuMulticastAddDevice", &api.MulticastAddDevice, &err) &&
         Load("cuMulticastBindMem", &api.MulticastBindMem, &err) &&
         Load("cuMulticastUnbind", &api.MulticastUnbind, &err) &&
         Load("cuMulticastGetGranularity", &api.MulticastGetGranularity, &err) &&
         Load("cuDeviceGet", &api.DeviceGet, &err) &&
         Load("cuDeviceGetAttribute", &api.DeviceGetAttribute, &err) &&
         Load("cuGetErrorString", &api.GetErrorString, &err);
  });
  if (!ok) {
    if (error) *error = err;
    return nullptr;
  }
  return &api;
}

std::string DriverApi::ErrorString(CUresult r) const {
  const char* s = nullptr;
  if (GetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUresult " + std::to_string(static_cast<int>(r));
}

}  // namespace switchml
