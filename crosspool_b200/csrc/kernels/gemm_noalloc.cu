// xp_gemm_noalloc: the split-K GEMM with its scratch in the library image
// (contract and caveats in xpool/gemm_noalloc.h).
#include <cuda_runtime.h>

#include <atomic>

#include "xpool/api.h"
#include "xpool/gemm_noalloc.h"

namespace {

// Workspace first, then the tile counters, then one status word (in a 256-byte block of its own). In host code
// this name is only a stand-in for the symbol: the device address comes from cudaGetSymbolAddress.
constexpr size_t kStatusOffset = XP_NOALLOC_WS_BYTES + XP_NOALLOC_COUNTER_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kStatusOffset + 256];

constexpr int kMaxDevices = 64;
// Two host threads making the first call on one device at once both look the address up and store the same
// value; the atomic makes that race well defined.
std::atomic<void*> g_scratch_addr[kMaxDevices];

// Device address of the array on the current device; looked up once per device.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return XP_NOALLOC_E_SYMBOL;
  void* p = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return XP_NOALLOC_E_SYMBOL;
    }
    g_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = static_cast<unsigned char*>(p);
  return 0;
}

void fill_args(XpGemmArgs* a, const void* w, const void* x, void* out, int n_out, int k, int rows, int splits) {
  *a = XpGemmArgs{};
  a->w = w;
  a->x = x;
  a->out = out;
  a->n_out = n_out;
  a->k = k;
  a->rows = rows;
  a->splits = splits;
  a->epilogue = 0;
  a->w_evict_first = rows <= 64;
}

}  // namespace

extern "C" long long xp_gemm_noalloc_required_bytes(int n_out, int k, int rows, int splits) {
  if (n_out <= 0 || k <= 0 || rows <= 0 || splits < 1) return XP_NOALLOC_E_ARGUMENT;
  XpGemmArgs a;
  fill_args(&a, nullptr, nullptr, nullptr, n_out, k, rows, splits);
  // plan as if the full scratch were available, so that the requested split factor is honoured
  a.ws = reinterpret_cast<float*>(1);
  a.counters = reinterpret_cast<uint32_t*>(1);
  a.ws_bytes = static_cast<size_t>(1) << 40;
  a.counter_bytes = static_cast<size_t>(1) << 40;
  XpGemmPlan plan;
  const int rc = xp_gemm_plan(&a, &plan);
  if (rc != 0) return rc;
  if (plan.counter_bytes > XP_NOALLOC_COUNTER_BYTES) return static_cast<long long>(XP_NOALLOC_WS_BYTES) + 1;
  return static_cast<long long>(plan.ws_bytes);
}

extern "C" int xp_gemm_noalloc(const void* w, const void* x, void* out, int n_out, int k, int rows, int splits,
                               void* stream) {
  if (w == nullptr || x == nullptr || out == nullptr || splits < 1) return XP_NOALLOC_E_ARGUMENT;
  const long long need = xp_gemm_noalloc_required_bytes(n_out, k, rows, splits);
  if (need < 0) return static_cast<int>(need);
  if (need > static_cast<long long>(XP_NOALLOC_WS_BYTES)) return XP_NOALLOC_E_TOO_LARGE;
  unsigned char* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  unsigned char* counters = scratch + XP_NOALLOC_WS_BYTES;
  // the counters and the status word must start at zero; the previous call may have been cut short
  if (cudaMemsetAsync(counters, 0, XP_NOALLOC_COUNTER_BYTES + 256, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
    cudaGetLastError();
    return XP_NOALLOC_E_CLEAR;
  }
  XpGemmArgs a;
  fill_args(&a, w, x, out, n_out, k, rows, splits);
  a.ws = reinterpret_cast<float*>(scratch);
  a.counters = reinterpret_cast<uint32_t*>(counters);
  a.ws_bytes = XP_NOALLOC_WS_BYTES;
  a.counter_bytes = XP_NOALLOC_COUNTER_BYTES;
  a.status = reinterpret_cast<uint32_t*>(scratch + kStatusOffset);   // a pipeline wait that runs out is recorded here
  a.stream = stream;
  return xp_gemm(&a);
}

extern "C" int xp_gemm_noalloc_status(unsigned int* out, void* stream) {
  if (out == nullptr) return XP_NOALLOC_E_ARGUMENT;
  unsigned char* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(out, scratch + kStatusOffset, sizeof(unsigned int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return XP_NOALLOC_E_CLEAR;
  }
  return 0;
}

extern "C" const char* xp_gemm_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case XP_NOALLOC_E_TOO_LARGE:
      return "problem needs more split-K scratch than the fixed in-library array (XP_NOALLOC_WS_BYTES) holds; "
             "use fewer splits, fewer rows, or the allocating entry point xp_gemm";
    case XP_NOALLOC_E_SYMBOL: return "could not obtain the device address of the in-library scratch array";
    case XP_NOALLOC_E_ARGUMENT: return "null pointer, non-positive size, or splits < 1";
    case XP_NOALLOC_E_CLEAR: return "clearing or reading the in-library counters / status word failed";
    default: return "error from xp_gemm (see xpool/api.h)";
  }
}
