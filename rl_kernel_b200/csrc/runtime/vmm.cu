// Device allocations that another process of the same machine can map: CUDA virtual-memory
// management (cuMemCreate) with a POSIX file descriptor as the shareable handle.
//
// This is the native half of the weight bridge's "cuda-vmm" transport (the reference drives the
// same driver calls through ctypes, rl_engine/integrations/common/weights.py:985-1330): the
// trainer packs a state into ONE allocation, exports its descriptor over a unix socket, and a
// rollout process on the same GPU maps the very same physical memory -- no copy, no staging.
// The driver API is reached through cudaGetDriverEntryPoint, so the library keeps its single link
// dependency on the CUDA runtime.
#include "rlk/host.h"

#include <mutex>
#include <unistd.h>

namespace rlk {

struct VmmApi {
  CUresult (*GetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*Export)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*Import)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*Reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*Unmap)(CUdeviceptr, size_t);
  CUresult (*AddressFree)(CUdeviceptr, size_t);
  CUresult (*Release)(CUmemGenericAllocationHandle);
  bool ok;
};

static const VmmApi& vmm_api() {
  static VmmApi api{};
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char* name) -> void* {
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        return nullptr;
      return p;
    };
    api.GetGranularity = reinterpret_cast<decltype(api.GetGranularity)>(get("cuMemGetAllocationGranularity"));
    api.Create = reinterpret_cast<decltype(api.Create)>(get("cuMemCreate"));
    api.Export = reinterpret_cast<decltype(api.Export)>(get("cuMemExportToShareableHandle"));
    api.Import = reinterpret_cast<decltype(api.Import)>(get("cuMemImportFromShareableHandle"));
    api.Reserve = reinterpret_cast<decltype(api.Reserve)>(get("cuMemAddressReserve"));
    api.Map = reinterpret_cast<decltype(api.Map)>(get("cuMemMap"));
    api.SetAccess = reinterpret_cast<decltype(api.SetAccess)>(get("cuMemSetAccess"));
    api.Unmap = reinterpret_cast<decltype(api.Unmap)>(get("cuMemUnmap"));
    api.AddressFree = reinterpret_cast<decltype(api.AddressFree)>(get("cuMemAddressFree"));
    api.Release = reinterpret_cast<decltype(api.Release)>(get("cuMemRelease"));
    api.ok = api.GetGranularity && api.Create && api.Export && api.Import && api.Reserve && api.Map &&
             api.SetAccess && api.Unmap && api.AddressFree && api.Release;
  });
  return api;
}

#define RLK_CHECK_CU(expr)                                                                         \
  do {                                                                                             \
    CUresult _r = (expr);                                                                          \
    if (_r != CUDA_SUCCESS)                                                                        \
      return ::rlk::set_error(RLK_ERR_CUDA, "%s failed with driver error %d (%s:%d)", #expr, (int)_r, \
                              __FILE__, __LINE__);                                                 \
  } while (0)

static CUmemAllocationProp vmm_prop(int dev) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

static int map_rw(const VmmApi& api, CUmemGenericAllocationHandle h, size_t bytes, size_t gran, int dev,
                  CUdeviceptr* out) {
  CUdeviceptr va = 0;
  RLK_CHECK_CU(api.Reserve(&va, bytes, gran, 0, 0));
  CUresult r = api.Map(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    api.AddressFree(va, bytes);
    return set_error(RLK_ERR_CUDA, "cuMemMap failed with driver error %d", (int)r);
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = api.SetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    api.Unmap(va, bytes);
    api.AddressFree(va, bytes);
    return set_error(RLK_ERR_CUDA, "cuMemSetAccess failed with driver error %d", (int)r);
  }
  *out = va;
  return RLK_OK;
}

}  // namespace rlk

// 1 when the driver offers virtual-memory management with POSIX descriptors on the current device.
RLK_API int rlk_vmm_supported() {
  using namespace rlk;
  if (!vmm_api().ok) return 0;
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryPoolSupportedHandleTypes, dev) != cudaSuccess) return 0;
  return (v & cudaMemHandleTypePosixFileDescriptor) ? 1 : 0;
}

// Allocates at least `bytes` on the current device, maps it read/write and exports it.
//   *out_ptr    device address in this process
//   *out_mapped size actually allocated (a multiple of the allocation granularity): pass it to
//               rlk_vmm_import and rlk_vmm_release
//   *out_handle opaque allocation handle (needed for release)
//   *out_fd     POSIX descriptor to hand to the importing process (SCM_RIGHTS); the caller closes it
RLK_API int rlk_vmm_create(long long bytes, void** out_ptr, long long* out_mapped, unsigned long long* out_handle,
                           int* out_fd) {
  using namespace rlk;
  RLK_REQUIRE(bytes > 0 && out_ptr && out_mapped && out_handle && out_fd, "vmm_create: bad arguments");
  const VmmApi& api = vmm_api();
  if (!api.ok) return set_error(RLK_ERR_UNSUPPORTED, "vmm_create: the driver's virtual-memory entry points are unavailable");
  RLK_CHECK_CUDA(cudaFree(nullptr));      // make sure the primary context exists
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  CUmemAllocationProp prop = vmm_prop(dev);
  size_t gran = 0;
  RLK_CHECK_CU(api.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  const size_t mapped = (static_cast<size_t>(bytes) + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h = 0;
  RLK_CHECK_CU(api.Create(&h, mapped, &prop, 0));
  CUdeviceptr va = 0;
  int rc = map_rw(api, h, mapped, gran, dev, &va);
  if (rc) { api.Release(h); return rc; }
  int fd = -1;
  CUresult r = api.Export(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    api.Unmap(va, mapped);
    api.AddressFree(va, mapped);
    api.Release(h);
    return set_error(RLK_ERR_CUDA, "cuMemExportToShareableHandle failed with driver error %d", (int)r);
  }
  *out_ptr = reinterpret_cast<void*>(va);
  *out_mapped = static_cast<long long>(mapped);
  *out_handle = h;
  *out_fd = fd;
  return RLK_OK;
}

// Maps an allocation received as a descriptor into this process (current device = the device
// that owns the memory).  The descriptor may be closed afterwards.
RLK_API int rlk_vmm_import(int fd, long long mapped_bytes, void** out_ptr, unsigned long long* out_handle) {
  using namespace rlk;
  RLK_REQUIRE(fd >= 0 && mapped_bytes > 0 && out_ptr && out_handle, "vmm_import: bad arguments");
  const VmmApi& api = vmm_api();
  if (!api.ok) return set_error(RLK_ERR_UNSUPPORTED, "vmm_import: the driver's virtual-memory entry points are unavailable");
  RLK_CHECK_CUDA(cudaFree(nullptr));
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  CUmemAllocationProp prop = vmm_prop(dev);
  size_t gran = 0;
  RLK_CHECK_CU(api.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  RLK_REQUIRE(static_cast<size_t>(mapped_bytes) % gran == 0, "vmm_import: %lld bytes is not a multiple of the granularity %zu",
              mapped_bytes, gran);
  CUmemGenericAllocationHandle h = 0;
  RLK_CHECK_CU(api.Import(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  CUdeviceptr va = 0;
  int rc = map_rw(api, h, static_cast<size_t>(mapped_bytes), gran, dev, &va);
  if (rc) { api.Release(h); return rc; }
  *out_ptr = reinterpret_cast<void*>(va);
  *out_handle = h;
  return RLK_OK;
}

// Unmaps and drops this process's reference (creator or importer).  The physical memory goes away
// when the last process has released it.
RLK_API int rlk_vmm_release(void* ptr, long long mapped_bytes, unsigned long long handle) {
  using namespace rlk;
  RLK_REQUIRE(ptr != nullptr && mapped_bytes > 0, "vmm_release: bad arguments");
  const VmmApi& api = vmm_api();
  if (!api.ok) return set_error(RLK_ERR_UNSUPPORTED, "vmm_release: the driver's virtual-memory entry points are unavailable");
  RLK_CHECK_CUDA(cudaDeviceSynchronize());
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  RLK_CHECK_CU(api.Unmap(va, static_cast<size_t>(mapped_bytes)));
  RLK_CHECK_CU(api.AddressFree(va, static_cast<size_t>(mapped_bytes)));
  RLK_CHECK_CU(api.Release(handle));
  return RLK_OK;
}

RLK_API int rlk_close_fd(int fd) { return fd >= 0 ? ::close(fd) : 0; }
