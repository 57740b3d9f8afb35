// See symmetric_memory.h.
#include "backends/cuda/symmetric_memory.h"

#include <cuda_runtime.h>
#include <unistd.h>

#include <cstring>

#include "backends/cuda/driver_api.h"
#include "switchml/log.h"

namespace switchml {

#define SML_CU(call, what)                                                      \
  do {                                                                          \
    CUresult _r = (call);                                                       \
    if (_r != CUDA_SUCCESS) {                                                   \
      if (error) *error = std::string(what) + ": " + api->ErrorString(_r);      \
      return false;                                                             \
    }                                                                           \
  } while (0)

SymmetricAllocator::SymmetricAllocator(int rank, int num_workers, int device,
                                       ControlClient* control, FdChannel* fds)
    : rank_(rank), n_(num_workers), device_(device), control_(control), fds_(fds) {}

bool SymmetricAllocator::DeviceSupportsMulticast() const {
  const DriverApi* api = DriverApi::Get();
  if (!api) return false;
  CUdevice dev;
  int v = 0;
  if (api->DeviceGet(&dev, device_) != CUDA_SUCCESS) return false;
  if (api->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS)
    return false;
  return v != 0;
}

namespace {

// All ranks learn whether everybody said yes.
bool AllAgree(ControlClient* c, int n, int rank, bool mine) {
  if (n == 1) return mine;
  std::vector<std::string> all;
  if (!c->AllGather(n, rank, mine ? "1" : "0", &all)) return false;
  for (const std::string& s : all) {
    if (s != "1") return false;
  }
  return true;
}

bool MapHandle(const DriverApi* api, CUmemGenericAllocationHandle h, size_t size, size_t gran,
               int device, void** va, std::string* error) {
  CUdeviceptr p = 0;
  SML_CU(api->MemAddressReserve(&p, size, gran, 0, 0), "cuMemAddressReserve");
  CUresult r = api->MemMap(p, size, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    api->MemAddressFree(p, size);
    if (error) *error = "cuMemMap: " + api->ErrorString(r);
    return false;
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = api->MemSetAccess(p, size, &acc, 1);
  if (r != CUDA_SUCCESS) {
    api->MemUnmap(p, size);
    api->MemAddressFree(p, size);
    if (error) *error = "cuMemSetAccess: " + api->ErrorString(r);
    return false;
  }
  *va = reinterpret_cast<void*>(p);
  return true;
}

void UnmapVa(const DriverApi* api, void* va, size_t size) {
  if (!va) return;
  api->MemUnmap(reinterpret_cast<CUdeviceptr>(va), size);
  api->MemAddressFree(reinterpret_cast<CUdeviceptr>(va), size);
}

}  // namespace

bool SymmetricAllocator::Create(size_t bytes, bool want_multicast, SymmetricRegion* out,
                                std::string* error) {
  std::string derr;
  const DriverApi* api = DriverApi::Get(&derr);
  if (!api) {
    if (error) *error = derr;
    return false;
  }
  cudaSetDevice(device_);
  cudaFree(0);  // make sure the primary context exists
  CUdevice dev;
  SML_CU(api->DeviceGet(&dev, device_), "cuDeviceGet");

  bool use_mc = want_multicast && n_ > 1 &&
                AllAgree(control_, n_, rank_, DeviceSupportsMulticast());
  if (want_multicast && n_ > 1 && !use_mc) {
    SML_VLOG(1) << "NVLink multicast is not available on every rank; using peer mappings only";
  }

  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  SML_CU(api->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
         "cuMemGetAllocationGranularity");
  CUmulticastObjectProp mprop;
  memset(&mprop, 0, sizeof(mprop));
  if (use_mc) {
    mprop.numDevices = static_cast<unsigned>(n_);
    mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mprop.size = bytes;
    size_t mgran = 0;
    CUresult r = api->MulticastGetGranularity(&mgran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (r == CUDA_SUCCESS && mgran > gran) gran = mgran;
  }
  size_t size = (bytes + gran - 1) / gran * gran;
  mprop.size = size;

  SymmetricRegion reg;
  reg.bytes = bytes;
  reg.mapped_bytes = size;
  reg.peers.assign(n_, nullptr);
  reg.peer_handles.assign(n_, 0);
  SML_CU(api->MemCreate(&reg.handle, size, &prop, 0), "cuMemCreate");
  if (!MapHandle(api, reg.handle, size, gran, device_, &reg.local, error)) return false;
  reg.peers[rank_] = reg.local;
  reg.peer_handles[rank_] = reg.handle;
  cudaMemset(reg.local, 0, size);
  cudaDeviceSynchronize();

  int tag = next_tag_;
  next_tag_ += 2;
  if (n_ > 1) {
    int fd = -1;
    SML_CU(api->MemExportToShareableHandle(&fd, reg.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
           "cuMemExportToShareableHandle");
    bool ok = true;
    for (int p = 0; p < n_ && ok; p++) {
      if (p != rank_) ok = fds_->SendTo(p, rank_, tag, fd);
    }
    close(fd);
    for (int i = 0; i < n_ - 1 && ok; i++) {
      int from = -1, t = 0, pfd = -1;
      ok = fds_->Recv(&from, &t, &pfd);
      if (!ok) break;
      if (t != tag || from < 0 || from >= n_ || from == rank_) {
        close(pfd);
        ok = false;
        break;
      }
      CUresult r = api->MemImportFromShareableHandle(
          &reg.peer_handles[from], reinterpret_cast<void*>(static_cast<uintptr_t>(pfd)),
          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(pfd);
      std::string merr;
      if (r != CUDA_SUCCESS ||
          !MapHandle(api, reg.peer_handles[from], size, gran, device_, &reg.peers[from], &merr)) {
        SML_LOG(ERROR) << "cannot map the memory of rank " << from << ": "
                       << (r != CUDA_SUCCESS ? api->ErrorString(r) : merr);
        ok = false;
      }
    }
    if (!AllAgree(control_, n_, rank_, ok)) {
      if (error) *error = "exchange of memory handles failed on at least one rank";
      *out = reg;
      Destroy(out, false);
      return false;
    }
  }

  if (use_mc) {
    // Rank 0 creates the multicast object and hands it to everybody.
    bool ok = true;
    std::string why;
    if (rank_ == 0) {
      CUresult r = api->MulticastCreate(&reg.mc_handle, &mprop);
      if (r != CUDA_SUCCESS) {
        ok = false;
        why = "cuMulticastCreate: " + api->ErrorString(r);
      }
      uint64_t created = ok ? 1 : 0;
      control_->Broadcast(n_, rank_, 0, &created);
      if (ok) {
        int fd = -1;
        r = api->MemExportToShareableHandle(&fd, reg.mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
        if (r != CUDA_SUCCESS) { ok = false; why = "export multicast handle: " + api->ErrorString(r); }
        for (int p = 1; p < n_; p++) {
          // If the export failed there is nothing to send; the peers' receive then times
          // out and all ranks agree below to fall back to peer mappings.
          if (fd >= 0) fds_->SendTo(p, rank_, tag + 1, fd);
        }
        if (fd >= 0) close(fd);
      }
    } else {
      uint64_t created = 0;
      control_->Broadcast(n_, rank_, 0, &created);
      if (!created) {
        ok = false;
        why = "rank 0 could not create a multicast object";
      } else {
        int from = -1, t = 0, pfd = -1;
        if (!fds_->Recv(&from, &t, &pfd) || t != tag + 1) {
          ok = false;
          why = "did not receive the multicast handle";
          if (pfd >= 0) close(pfd);
        } else {
          CUresult r = api->MemImportFromShareableHandle(
              &reg.mc_handle, reinterpret_cast<void*>(static_cast<uintptr_t>(pfd)),
              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
          close(pfd);
          if (r != CUDA_SUCCESS) { ok = false; why = "import multicast handle: " + api->ErrorString(r); }
        }
      }
    }
    if (ok) {
      CUresult r = api->MulticastAddDevice(reg.mc_handle, dev);
      if (r != CUDA_SUCCESS) { ok = false; why = "cuMulticastAddDevice: " + api->ErrorString(r); }
    }
    // Binding may only start once every device was added.
    bool all = AllAgree(control_, n_, rank_, ok);
    if (all) {
      CUresult r = api->MulticastBindMem(reg.mc_handle, 0, reg.handle, 0, size, 0);
      if (r != CUDA_SUCCESS) { ok = false; why = "cuMulticastBindMem: " + api->ErrorString(r); }
      else reg.mc_bound = true;
      if (ok && !MapHandle(api, reg.mc_handle, size, gran, device_, &reg.multicast, &why)) ok = false;
      all = AllAgree(control_, n_, rank_, ok);
    }
    if (!all) {
      SML_LOG(WARNING) << "NVLink multicast setup failed"
                       << (why.empty() ? std::string(" on another rank") : ": " + why)
                       << "; falling back to peer mappings";
      if (reg.multicast) UnmapVa(api, reg.multicast, size);
      reg.multicast = nullptr;
      if (reg.mc_bound) api->MulticastUnbind(reg.mc_handle, dev, 0, size);
      reg.mc_bound = false;
      if (reg.mc_handle) api->MemRelease(reg.mc_handle);
      reg.mc_handle = 0;
      if (n_ > 1) control_->Barrier(n_);
    }
  }
  if (n_ > 1) control_->Barrier(n_);
  *out = reg;
  return true;
}

void SymmetricAllocator::Destroy(SymmetricRegion* r, bool peers_alive) {
  const DriverApi* api = DriverApi::Get();
  if (!api || !r->local) return;
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  CUdevice dev;
  api->DeviceGet(&dev, device_);
  // Nobody may still be reducing through the multicast object when a rank leaves it.
  if (peers_alive && n_ > 1 && !control_->Barrier(n_, 10000)) peers_alive = false;
  if (r->multicast) UnmapVa(api, r->multicast, r->mapped_bytes);
  r->multicast = nullptr;
  if (r->mc_bound) api->MulticastUnbind(r->mc_handle, dev, 0, r->mapped_bytes);
  r->mc_bound = false;
  if (r->mc_handle) api->MemRelease(r->mc_handle);
  r->mc_handle = 0;
  if (peers_alive && n_ > 1 && !control_->Barrier(n_, 10000)) peers_alive = false;
  for (int p = 0; p < static_cast<int>(r->peers.size()); p++) {
    if (p == rank_ || !r->peers[p]) continue;
    UnmapVa(api, r->peers[p], r->mapped_bytes);
    if (r->peer_handles[p]) api->MemRelease(r->peer_handles[p]);
    r->peers[p] = nullptr;
  }
  if (peers_alive && n_ > 1) control_->Barrier(n_, 10000);
  UnmapVa(api, r->local, r->mapped_bytes);
  api->MemRelease(r->handle);
  r->local = nullptr;
  r->handle = 0;
}

}  // namespace switchml
