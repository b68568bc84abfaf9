// VMM-based symmetric heap (see b2/symm_heap.h). Driver entry points are fetched through the runtime
// (cudaGetDriverEntryPoint), like the tensor-map encoder, so the library still loads on a machine without a GPU.
#include "b2/symm_heap.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <string>

namespace b2 {
namespace symm {
namespace {

template <class Fn>
Fn entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
  return reinterpret_cast<Fn>(p);
}

struct Api {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  bool ok = false;
  Api() {
#define B2_ENTRY(field, name) field = entry<decltype(field)>(name)
    B2_ENTRY(MemCreate, "cuMemCreate");
    B2_ENTRY(MemRelease, "cuMemRelease");
    B2_ENTRY(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    B2_ENTRY(MemExportToShareableHandle, "cuMemExportToShareableHandle");
    B2_ENTRY(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    B2_ENTRY(MemAddressReserve, "cuMemAddressReserve");
    B2_ENTRY(MemAddressFree, "cuMemAddressFree");
    B2_ENTRY(MemMap, "cuMemMap");
    B2_ENTRY(MemUnmap, "cuMemUnmap");
    B2_ENTRY(MemSetAccess, "cuMemSetAccess");
    B2_ENTRY(MulticastCreate, "cuMulticastCreate");
    B2_ENTRY(MulticastAddDevice, "cuMulticastAddDevice");
    B2_ENTRY(MulticastBindMem, "cuMulticastBindMem");
    B2_ENTRY(MulticastGetGranularity, "cuMulticastGetGranularity");
    B2_ENTRY(DeviceGet, "cuDeviceGet");
    B2_ENTRY(DeviceGetAttribute, "cuDeviceGetAttribute");
#undef B2_ENTRY
    ok = MemCreate && MemRelease && MemGetAllocationGranularity && MemExportToShareableHandle && MemImportFromShareableHandle &&
         MemAddressReserve && MemAddressFree && MemMap && MemUnmap && MemSetAccess && DeviceGet && DeviceGetAttribute;
  }
};

const Api& api() {
  static const Api a;
  return a;
}

std::string fail(const char* what, CUresult r) { return std::string("symm heap: ") + what + " failed with CUresult " + std::to_string(static_cast<int>(r)); }

CUmemAllocationProp local_prop(int device) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

size_t round_up(size_t n, size_t g) { return g == 0 ? n : (n + g - 1) / g * g; }

// Reserve a range, map `handle` there and open it for this device.
std::string map_handle(const Api& a, int device, CUmemGenericAllocationHandle handle, size_t bytes, size_t gran, uint64_t* va_out) {
  CUdeviceptr va = 0;
  CUresult r = a.MemAddressReserve(&va, bytes, gran, 0, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemAddressReserve", r);
  r = a.MemMap(va, bytes, 0, handle, 0);
  if (r != CUDA_SUCCESS) {
    a.MemAddressFree(va, bytes);
    return fail("cuMemMap", r);
  }
  CUmemAccessDesc d{};
  d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  d.location.id = device;
  d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = a.MemSetAccess(va, bytes, &d, 1);
  if (r != CUDA_SUCCESS) {
    a.MemUnmap(va, bytes);
    a.MemAddressFree(va, bytes);
    return fail("cuMemSetAccess", r);
  }
  *va_out = static_cast<uint64_t>(va);
  return "";
}

}  // namespace

HeapSegment::~HeapSegment() { close(); }

std::string HeapSegment::create(int device, int rank, int world, size_t bytes, bool multicast) {
  const Api& a = api();
  if (!a.ok) return "symm heap: the CUDA driver does not offer the virtual memory management entry points";
  if (have_local_) return "symm heap: segment already created";
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || bytes == 0) return "symm heap: bad rank / world / size";
  if (cudaSetDevice(device) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) return "symm heap: cannot make the device current";
  device_ = device;
  rank_ = rank;
  world_ = world;
  const CUmemAllocationProp prop = local_prop(device);
  size_t gran = 0;
  CUresult r = a.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return fail("cuMemGetAllocationGranularity", r);
  mc_supported_ = false;
  if (multicast && world > 1 && a.MulticastCreate && a.MulticastAddDevice && a.MulticastBindMem && a.MulticastGetGranularity) {
    CUdevice dev;
    int has = 0;
    if (a.DeviceGet(&dev, device) == CUDA_SUCCESS && a.DeviceGetAttribute(&has, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS && has) {
      CUmulticastObjectProp mp{};
      mp.numDevices = static_cast<unsigned>(world);
      mp.size = round_up(bytes, gran);
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t mgran = 0;
      if (a.MulticastGetGranularity(&mgran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran > 0) {
        gran = gran > mgran ? gran : mgran;
        mc_supported_ = true;
      }
    }
  }
  gran_ = gran;
  bytes_ = round_up(bytes, gran);
  CUmemGenericAllocationHandle h = 0;
  r = a.MemCreate(&h, bytes_, &prop, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemCreate", r);
  local_handle_ = h;
  have_local_ = true;
  std::string e = map_handle(a, device_, h, bytes_, gran_, &va_[rank]);
  if (!e.empty()) return e;
  peer_mapped_[rank] = true;
  if (cudaMemset(reinterpret_cast<void*>(va_[rank]), 0, bytes_) != cudaSuccess) return "symm heap: clearing the allocation failed";
  return "";
}

int HeapSegment::export_fd(std::string* err) {
  const Api& a = api();
  int fd = -1;
  const CUresult r = a.MemExportToShareableHandle(&fd, local_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    if (err) *err = fail("cuMemExportToShareableHandle", r);
    return -1;
  }
  return fd;
}

std::string HeapSegment::map_peer(int peer, int fd) {
  const Api& a = api();
  if (peer < 0 || peer >= world_ || peer == rank_ || peer_mapped_[peer]) {
    ::close(fd);
    return "symm heap: bad peer index";
  }
  CUmemGenericAllocationHandle h = 0;
  const CUresult r = a.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  ::close(fd);
  if (r != CUDA_SUCCESS) return fail("cuMemImportFromShareableHandle", r);
  peer_handle_[peer] = h;
  std::string e = map_handle(a, device_, h, bytes_, gran_, &va_[peer]);
  if (!e.empty()) {
    a.MemRelease(h);
    peer_handle_[peer] = 0;
    return e;
  }
  peer_mapped_[peer] = true;
  return "";
}

int HeapSegment::mc_create(std::string* err) {
  const Api& a = api();
  if (!mc_supported_) {
    if (err) *err = "symm heap: no multicast support";
    return -1;
  }
  CUmulticastObjectProp mp{};
  mp.numDevices = static_cast<unsigned>(world_);
  mp.size = bytes_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = a.MulticastCreate(&h, &mp);
  if (r != CUDA_SUCCESS) {
    if (err) *err = fail("cuMulticastCreate", r);
    return -1;
  }
  mc_handle_ = h;
  have_mc_ = true;
  int fd = -1;
  r = a.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    if (err) *err = fail("cuMemExportToShareableHandle (multicast)", r);
    return -1;
  }
  return fd;
}

std::string HeapSegment::mc_import(int fd) {
  const Api& a = api();
  CUmemGenericAllocationHandle h = 0;
  const CUresult r = a.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  ::close(fd);
  if (r != CUDA_SUCCESS) return fail("cuMemImportFromShareableHandle (multicast)", r);
  mc_handle_ = h;
  have_mc_ = true;
  return "";
}

std::string HeapSegment::mc_add_device() {
  const Api& a = api();
  if (!have_mc_) return "symm heap: no multicast object";
  CUdevice dev;
  CUresult r = a.DeviceGet(&dev, device_);
  if (r != CUDA_SUCCESS) return fail("cuDeviceGet", r);
  r = a.MulticastAddDevice(mc_handle_, dev);
  return r == CUDA_SUCCESS ? "" : fail("cuMulticastAddDevice", r);
}

std::string HeapSegment::mc_bind_and_map() {
  const Api& a = api();
  if (!have_mc_) return "symm heap: no multicast object";
  CUresult r = a.MulticastBindMem(mc_handle_, 0, local_handle_, 0, bytes_, 0);
  if (r != CUDA_SUCCESS) return fail("cuMulticastBindMem", r);
  mc_bound_ = true;
  return map_handle(a, device_, mc_handle_, bytes_, gran_, &mc_va_);
}

void HeapSegment::close() {
  const Api& a = api();
  if (!a.ok) return;
  if (mc_va_ != 0) {
    a.MemUnmap(static_cast<CUdeviceptr>(mc_va_), bytes_);
    a.MemAddressFree(static_cast<CUdeviceptr>(mc_va_), bytes_);
    mc_va_ = 0;
  }
  if (have_mc_) {
    a.MemRelease(mc_handle_);   // the object goes away when the last rank has released it
    have_mc_ = false;
  }
  for (int i = 0; i < kMaxRanks; ++i) {
    if (peer_mapped_[i]) {
      a.MemUnmap(static_cast<CUdeviceptr>(va_[i]), bytes_);
      a.MemAddressFree(static_cast<CUdeviceptr>(va_[i]), bytes_);
      peer_mapped_[i] = false;
      va_[i] = 0;
    }
    if (peer_handle_[i] != 0) {
      a.MemRelease(peer_handle_[i]);
      peer_handle_[i] = 0;
    }
  }
  if (have_local_) {
    a.MemRelease(local_handle_);
    have_local_ = false;
  }
}

}  // namespace symm
}  // namespace b2
