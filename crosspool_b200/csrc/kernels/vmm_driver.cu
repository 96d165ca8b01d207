// The real CUDA driver behind xpool/kv_vmm.hpp's DriverApi table: cuMemAddressReserve /
// cuMemCreate / cuMemMap / cuMemSetAccess / cuMemUnmap / cuMemRelease, resolved through
// the runtime so that the library does not link libcuda.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include "xpool/kv_vmm.hpp"

namespace {

template <typename Fn>
Fn entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

int rc_of(CUresult r) { return r == CUDA_SUCCESS ? 0 : static_cast<int>(r); }  // CUDA_ERROR_OUT_OF_MEMORY == 2

int d_gran(void*, int device, uint64_t* out) {
  static auto fn = entry<CUresult (*)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags)>(
      "cuMemGetAllocationGranularity");
  if (!fn) return -1;
  CUmemAllocationProp prop = prop_for(device);
  size_t g = 0;
  CUresult r = fn(&g, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  *out = g;
  return rc_of(r);
}
int d_reserve(void*, uint64_t bytes, uint64_t alignment, uint64_t* va) {
  static auto fn = entry<CUresult (*)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long)>("cuMemAddressReserve");
  if (!fn) return -1;
  CUdeviceptr p = 0;
  CUresult r = fn(&p, bytes, alignment, 0, 0);
  *va = static_cast<uint64_t>(p);
  return rc_of(r);
}
int d_release_va(void*, uint64_t va, uint64_t bytes) {
  static auto fn = entry<CUresult (*)(CUdeviceptr, size_t)>("cuMemAddressFree");
  return fn ? rc_of(fn(static_cast<CUdeviceptr>(va), bytes)) : -1;
}
int d_create(void*, int device, uint64_t bytes, uint64_t* handle) {
  static auto fn = entry<CUresult (*)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long)>(
      "cuMemCreate");
  if (!fn) return -1;
  CUmemAllocationProp prop = prop_for(device);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = fn(&h, bytes, &prop, 0);
  *handle = static_cast<uint64_t>(h);
  return rc_of(r);
}
int d_release(void*, uint64_t handle) {
  static auto fn = entry<CUresult (*)(CUmemGenericAllocationHandle)>("cuMemRelease");
  return fn ? rc_of(fn(static_cast<CUmemGenericAllocationHandle>(handle))) : -1;
}
int d_map(void*, uint64_t va, uint64_t bytes, uint64_t handle) {
  static auto fn = entry<CUresult (*)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long)>("cuMemMap");
  return fn ? rc_of(fn(static_cast<CUdeviceptr>(va), bytes, 0, static_cast<CUmemGenericAllocationHandle>(handle), 0)) : -1;
}
int d_unmap(void*, uint64_t va, uint64_t bytes) {
  static auto fn = entry<CUresult (*)(CUdeviceptr, size_t)>("cuMemUnmap");
  return fn ? rc_of(fn(static_cast<CUdeviceptr>(va), bytes)) : -1;
}
int d_access(void*, uint64_t va, uint64_t bytes, int device) {
  static auto fn = entry<CUresult (*)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t)>("cuMemSetAccess");
  if (!fn) return -1;
  CUmemAccessDesc d;
  memset(&d, 0, sizeof(d));
  d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  d.location.id = device;
  d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return rc_of(fn(static_cast<CUdeviceptr>(va), bytes, &d, 1));
}

}  // namespace

// Copies the real driver's function table into `out` (sizeof(DriverApi) bytes).
extern "C" void xp_vmm_driver_api(void* out) {
  xpool::vmm::DriverApi a{nullptr, d_gran, d_reserve, d_release_va, d_create, d_release, d_map, d_unmap, d_access};
  *static_cast<xpool::vmm::DriverApi*>(out) = a;
}
