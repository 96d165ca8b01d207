// ABI version and small device utilities shared by every kernel file.
#include "xpool/api.h"
#include "xpool/protocol.hpp"

#include <cuda_runtime.h>

extern "C" int xp_abi_version(void) { return XP_ABI_VERSION; }

// Device mirror of the process's debug options (see xpool::DebugOptions): set once at bootstrap, readable by device
// code of this library as `xpool::g_debug_options_d`.
namespace xpool {
__constant__ DebugOptions g_debug_options_d;
}

extern "C" int xp_debug_options_set(const uint32_t* four) {
  xpool::DebugOptions o{four[0], four[1], four[2], four[3]};
  return cudaMemcpyToSymbol(xpool::g_debug_options_d, &o, sizeof(o)) == cudaSuccess ? 0 : -100;
}

extern "C" int xp_debug_options_get(uint32_t* four) {
  xpool::DebugOptions o{};
  if (cudaMemcpyFromSymbol(&o, xpool::g_debug_options_d, sizeof(o)) != cudaSuccess) return -100;
  four[0] = o.transport_observer, four[1] = o.fabric_observer, four[2] = o.graph_observer, four[3] = o.ffn_routing_observer;
  return 0;
}

namespace {
__global__ void fill_u32_kernel(uint32_t* p, uint32_t v, size_t n) {
  for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += gridDim.x * 256ull) p[i] = v;
}
// Writes more than the 126 MB L2 so that the next timed kernel starts cold.
__global__ void l2_flush_kernel(uint4* p, size_t n) {
  for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += gridDim.x * 256ull)
    p[i] = make_uint4(static_cast<uint32_t>(i), 0, 0, 0);
}
}  // namespace

extern "C" int xp_fill_u32(void* p, uint32_t v, size_t n, void* stream) {
  fill_u32_kernel<<<148, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint32_t*>(p), v, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

extern "C" int xp_l2_flush(void* p, size_t bytes, void* stream) {
  l2_flush_kernel<<<148 * 4, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint4*>(p), bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}
