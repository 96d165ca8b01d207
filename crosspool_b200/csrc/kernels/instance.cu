// Instance-side entry of the FFN boundary for an engine that is not this repository's own: the op an external
// serving engine calls in place of a decoder MLP (reference: xpool::instance::ffn_shim -> InstanceRankRuntime::submit,
// src/cext/instance.cpp, src/cext/transport/instance.cpp, and the request kernel src/cext/transport/instance.cu:35-201).
//
// submit() enqueues three kernels on the caller's stream, all capturable into a CUDA graph:
//   1. publish_rows_kernel: copies the caller's hidden states straight into every FFN TP rank's input buffer (peer
//      stores), then the last CTA writes the invocation record and releases the slot's sequence word;
//   2. the bounded completion wait (xp_wait_flags; its cancel word is the Instance's failure slot);
//   3. fold_parts_kernel: sums the TP ranks' partial outputs in rank order with fp32 accumulation into the caller's
//      output tensor (NaN-poisoned when the wait did not end with a completion, like the reference).
// The own engine fuses 1 with its add-RMSNorm and 3 with the next one (norm.cu); an external engine keeps its own
// norm kernels, so here both are plain copies.
#include <mutex>
#include <vector>

#include "xpool/api.h"
#include "xpool/hooks.cuh"
#include "xpool/sm100.cuh"

namespace xpool {
namespace instance {

struct Binding {
  XpInstanceBinding b;
  uint32_t* done_counter = nullptr;   // device word: finds the last CTA of a publish
  uint32_t* seq = nullptr;            // device word: invocation sequence (advanced by every publish)
};

__global__ void __launch_bounds__(256)
publish_rows_kernel(XpInstanceBinding b, const __nv_bfloat16* __restrict__ x, int ld, int rows, uint32_t layer, uint32_t mode,
                    uint32_t requirement, uint32_t dp_layout, uint32_t* done_counter, uint32_t* seq_word) {
  const int row = blockIdx.x;
  const int nvec = b.hidden / 8;
  if (row < rows) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ld);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 val = src[v];
      for (int d = 0; d < b.n_peers; ++d)
        reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(b.peer_inputs[d]) + static_cast<size_t>(row) * b.hidden)[v] = val;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;
      const uint32_t seq = *seq_word + 1;
      *seq_word = seq;
      __threadfence_system();
      for (int d = 0; d < b.n_peers; ++d) {
        uint32_t* rec = reinterpret_cast<uint32_t*>(b.peer_records[d]);
        rec[0] = static_cast<uint32_t>(rows);
        rec[1] = layer;
        rec[2] = mode;
        rec[3] = 0;
        rec[4] = requirement;
        rec[5] = dp_layout;
        sm100::st_release_sys(reinterpret_cast<uint32_t*>(b.peer_flags[d]), seq);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
fold_parts_kernel(XpInstanceBinding b, __nv_bfloat16* __restrict__ out, int ld_out, int rows, const uint32_t* seq_word) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  // every completion word must have reached this invocation's sequence; otherwise the wait gave up
  bool complete = true;
  const uint32_t want = *seq_word;
  for (int p = 0; p < b.n_parts; ++p)
    if (static_cast<int32_t>(sm100::ld_acquire_sys(reinterpret_cast<const uint32_t*>(b.done_flags[p])) - want) < 0) complete = false;
  const int nvec = b.hidden / 8;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < b.n_parts; ++p) {
      const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(b.parts[p]) +
                                                               static_cast<size_t>(row) * b.hidden) + v);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      oh[j] = complete ? __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1])
                       : __floats2bfloat162_rn(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
    reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * ld_out)[v] = o;
  }
}

static std::mutex g_mu;
static std::vector<Binding*> g_bindings;
static int g_current = -1;

}  // namespace instance
}  // namespace xpool

using xpool::instance::Binding;

// Registers the transport of one Instance rank. Returns a handle >= 0, or a negative code.
extern "C" int xp_instance_create(const XpInstanceBinding* b) {
  if (b == nullptr || b->n_peers < 1 || b->n_peers > 8 || b->n_parts < 1 || b->n_parts > 8 || b->hidden % 8 != 0 ||
      b->capacity_rows < 1)
    return -1;
  auto* x = new Binding();
  x->b = *b;
  if (cudaMalloc(&x->done_counter, 256) != cudaSuccess) return -2;
  cudaMemset(x->done_counter, 0, 256);
  x->seq = x->done_counter + 16;
  std::lock_guard<std::mutex> g(xpool::instance::g_mu);
  xpool::instance::g_bindings.push_back(x);
  return static_cast<int>(xpool::instance::g_bindings.size()) - 1;
}

// Chooses the Instance that torch.ops.xpool.ffn_shim submits to in this process (one Instance rank per process).
extern "C" int xp_instance_set_current(int handle) {
  std::lock_guard<std::mutex> g(xpool::instance::g_mu);
  if (handle >= static_cast<int>(xpool::instance::g_bindings.size())) return -1;
  xpool::instance::g_current = handle;
  return 0;
}
extern "C" int xp_instance_current(void) { return xpool::instance::g_current; }

extern "C" int xp_instance_submit(int handle, const void* hidden, int rows, int ld, void* out, int ld_out, int layer, int mode,
                                  int requirement, int dp_layout, void* stream) {
  Binding* x = nullptr;
  {
    std::lock_guard<std::mutex> g(xpool::instance::g_mu);
    if (handle < 0 || handle >= static_cast<int>(xpool::instance::g_bindings.size())) return -1;
    x = xpool::instance::g_bindings[handle];
  }
  if (x == nullptr) return -1;
  const XpInstanceBinding& b = x->b;
  if (rows < 0 || rows > b.capacity_rows || ld < b.hidden || ld_out < b.hidden) return -2;
  if ((reinterpret_cast<uintptr_t>(hidden) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0 || (ld & 7) != 0 || (ld_out & 7) != 0)
    return -3;
  if (dp_layout != 0) return -4;   // rows of several data-parallel ranks in one invocation are not merged here
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = rows > 0 ? rows : 1;   // Idle mode publishes an empty invocation so that sequences stay in step
  xpool::instance::publish_rows_kernel<<<grid, 256, 0, s>>>(b, static_cast<const __nv_bfloat16*>(hidden), ld, rows,
                                                            static_cast<uint32_t>(layer), static_cast<uint32_t>(mode),
                                                            static_cast<uint32_t>(requirement), static_cast<uint32_t>(dp_layout),
                                                            x->done_counter, x->seq);
  XpWaitArgs w{};
  for (int p = 0; p < b.n_parts; ++p) w.flags[p] = reinterpret_cast<const uint32_t*>(b.done_flags[p]);
  w.n = b.n_parts;
  w.want_ptr = x->seq;
  w.cancel = reinterpret_cast<const uint32_t*>(b.failure);
  w.status = reinterpret_cast<uint32_t*>(b.status);
  w.wait_ns = b.wait_ns != 0 ? b.wait_ns : 5000000000ull;
  w.failure = b.failure;
  for (int d = 0; d < b.n_peers; ++d) w.peer_failures[d] = b.peer_failures[d];
  w.n_peer_failures = b.n_peers;
  w.origin_pe = b.origin_pe;
  const int rc = xp_wait_flags(&w, stream);
  if (rc != 0) return rc;
  if (rows > 0)
    xpool::instance::fold_parts_kernel<<<rows, 256, 0, s>>>(b, static_cast<__nv_bfloat16*>(out), ld_out, rows, x->seq);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" void xp_instance_destroy(int handle) {
  std::lock_guard<std::mutex> g(xpool::instance::g_mu);
  if (handle < 0 || handle >= static_cast<int>(xpool::instance::g_bindings.size())) return;
  Binding* x = xpool::instance::g_bindings[handle];
  if (x != nullptr) {
    cudaFree(x->done_counter);
    delete x;
    xpool::instance::g_bindings[handle] = nullptr;
  }
  if (xpool::instance::g_current == handle) xpool::instance::g_current = -1;
}
