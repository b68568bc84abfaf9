// Device capability probe: the runtime counterpart of the reference's compile-time target predicates
// (stdlib/src/sys/info.mojo:423-480 `is_nvidia_gpu`/`_is_sm_9x`, :872-899 `has_nvidia_gpu_accelerator`) and of
// examples/deviceinfo.mojo:38-80. One target only: compute capability 10.0.
#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>
#include "b2/api.h"

extern "C" int b2_device_caps(int device, B2DeviceCaps* out) {
  if (out == nullptr) return -b2::kBadArgument;
  std::memset(out, 0, sizeof(*out));
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
    cudaGetLastError();
    return -b2::kBadArgument;
  }
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return -b2::kBadArgument;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->sm_count = p.multiProcessorCount;
  out->smem_per_block_optin = static_cast<int>(p.sharedMemPerBlockOptin);
  out->l2_bytes = p.l2CacheSize;
  out->total_mem = static_cast<int64_t>(p.totalGlobalMem);
  std::strncpy(out->name, p.name, sizeof(out->name) - 1);
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device) == cudaSuccess) out->clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, device) == cudaSuccess) out->mem_clock_khz = v;
  out->max_cluster = p.major >= 9 ? 8 : 1;
  // Peer access to any other visible device.
  for (int d = 0; d < count; ++d) {
    if (d == device) continue;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, device, d) == cudaSuccess && can) out->can_map_peer = 1;
  }
  // Multicast (NVLS) support is a driver attribute; query it through the runtime-provided entry point.
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuDeviceGetAttribute", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess && fn != nullptr) {
    using AttrFn = CUresult (*)(int*, CUdevice_attribute, CUdevice);
    int mc = 0;
    if (reinterpret_cast<AttrFn>(fn)(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) == CUDA_SUCCESS)
      out->multicast_supported = mc;
  }
  cudaGetLastError();
  return 0;
}
