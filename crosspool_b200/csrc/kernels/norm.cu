// Row-wise kernels of the attention side: the fused
//   [wait for FFN partials] -> fixed-order fp32 sum -> residual add -> RMSNorm
//   -> store locally and/or push to FFN ranks' input buffers -> release flags
// transport producer, plus a plain SwiGLU used by the unfused baseline path.
//
// In the reference the same work is spread over SGLang's add-RMSNorm kernel, the
// Instance request kernel (src/cext/transport/instance.cu:35-201), the AtnAgent
// resident kernel (src/cext/transport/atnagent.cu:126-193) and the delivery
// reduction (src/cext/ffnagent/delivery.cu:85-127). Here the kernel that
// produces the normalised hidden states is the transport producer: rows go
// straight into each FFN rank's own memory with ordinary peer stores, followed
// by a system-scope release of a sequence word.
#include "xpool/api.h"
#include "xpool/hooks.cuh"
#include "xpool/sm100.cuh"

namespace xpool {
namespace norm {

constexpr int kThreads = 256;

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (kThreads >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// One CTA per row; hidden % 8 == 0; hidden <= 8 * kThreads * kMaxVec.
constexpr int kMaxVec = 4;  // 256 threads * 8 elems * 4 = 8192 hidden max

__global__ void __launch_bounds__(kThreads)
norm_publish_kernel(XpNormArgs a) {
  __shared__ float red[kThreads / 32];
  __shared__ uint32_t s_fail;
  const int row = blockIdx.x;
  const int hidden = a.hidden;
  const int nvec = hidden / 8;

  // 1. bounded wait for the producers of the partial inputs (FFN ranks).
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (a.wait_seq != 0 && threadIdx.x < a.nparts && a.wait_flags[threadIdx.x] != nullptr) {
    const uint64_t deadline = sm100::global_timer_ns() + a.wait_ns;
    int rc = sm100::wait_flag_ge(a.wait_flags[threadIdx.x], a.wait_seq, deadline, a.cancel);
    if (rc != 0) {
      s_fail = 1;
      const trace::BufferView tv{static_cast<trace::Event*>(a.trace_events), static_cast<trace::BufferState*>(a.trace_state),
                                 a.trace_capacity, 0};
      hooks::Point<hooks::AtnFoldWaitTimedOut>::hooks({tv, static_cast<uint32_t>(row), a.wait_seq});
    }
  }
  __syncthreads();
  const bool failed = s_fail != 0;
  if (failed && threadIdx.x == 0 && a.status != nullptr) atomicCAS(a.status, 0u, 4u /*flag timeout*/);

  // 2. fixed-order fp32 fold of the partials (+ residual), sum of squares.
  float vals[kMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int v = threadIdx.x + it * kThreads;
    if (v >= nvec) break;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < a.nparts; ++p) {
      const Bf16x8* src = reinterpret_cast<const Bf16x8*>(
          reinterpret_cast<const __nv_bfloat16*>(a.parts[p]) + static_cast<size_t>(row) * a.ld_parts);
      // partials written by a peer GPU: bypass L1
      Bf16x8 x;
      *reinterpret_cast<uint4*>(&x) = __ldcg(reinterpret_cast<const uint4*>(&src[v]));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(x.v[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (failed) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __int_as_float(0x7fc00000);  // poison, like the reference
    }
    if (a.nparts > 1) {
      // the reduced FFN output is rounded once to the payload dtype
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(__float2bfloat16_rn(acc[j]));
    }
    if (a.resid != nullptr) {
      Bf16x8* r = reinterpret_cast<Bf16x8*>(reinterpret_cast<__nv_bfloat16*>(a.resid) +
                                            static_cast<size_t>(row) * hidden);
      Bf16x8 x = r[v];
      Bf16x8 y;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(x.v[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
        y.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        // the normalisation sees the rounded residual stream, as an unfused add would
        float2 b = __bfloat1622float2(y.v[j]);
        acc[2 * j] = b.x;
        acc[2 * j + 1] = b.y;
      }
      r[v] = y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      vals[it][j] = acc[j];
      ss += acc[j] * acc[j];
    }
  }
  if (a.weight == nullptr) return;  // residual-add only
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / static_cast<float>(hidden) + a.eps);

  // 3. normalise, store locally and push to the FFN ranks.
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int v = threadIdx.x + it * kThreads;
    if (v >= nvec) break;
    Bf16x8 w = reinterpret_cast<const Bf16x8*>(a.weight)[v];
    Bf16x8 y;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 wf = __bfloat1622float2(w.v[j]);
      // x * inv is rounded to bf16 before the weight multiply (HF RMSNorm order)
      float n0 = __bfloat162float(__float2bfloat16_rn(vals[it][2 * j] * inv));
      float n1 = __bfloat162float(__float2bfloat16_rn(vals[it][2 * j + 1] * inv));
      y.v[j] = __floats2bfloat162_rn(n0 * wf.x, n1 * wf.y);
    }
    if (a.out_local != nullptr)
      reinterpret_cast<Bf16x8*>(reinterpret_cast<__nv_bfloat16*>(a.out_local) +
                                static_cast<size_t>(row) * a.ld_out)[v] = y;
    for (int d = 0; d < a.npeers; ++d)
      reinterpret_cast<Bf16x8*>(reinterpret_cast<__nv_bfloat16*>(a.out_peers[d]) +
                                static_cast<size_t>(row) * a.ld_out)[v] = y;
  }

  // 4. last CTA releases the sequence word on every destination.
  if (a.npeers > 0 && (a.publish_seq != 0 || a.seq_counter != nullptr)) {
    // The CTA barrier orders every thread's row stores before thread 0; its system-scope fence is cumulative, so one
    // fence per CTA (not one per thread: 256 x rows membar.sys were the kernel's top stall) publishes the whole row.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const uint32_t prev = atomicAdd(a.done_counter, 1u);
      if (prev == gridDim.x - 1) {
        *a.done_counter = 0;
        uint32_t seq = a.publish_seq;
        if (a.seq_counter != nullptr) {
          seq = *a.seq_counter + 1;
          *a.seq_counter = seq;
        }
        __threadfence_system();
        for (int d = 0; d < a.npeers; ++d) {
          if (a.peer_meta[d] != nullptr) {
            // invocation record: rows, layer, forward mode; written before the flag
            a.peer_meta[d][0] = static_cast<uint32_t>(gridDim.x);
            a.peer_meta[d][1] = a.meta_layer;
            a.peer_meta[d][2] = a.meta_mode;
            a.peer_meta[d][3] = a.meta_deadline_ptr != nullptr ? *a.meta_deadline_ptr : a.meta_deadline_us;
          }
          sm100::st_release_sys(a.peer_flags[d], seq);
        }
        const trace::BufferView tv{static_cast<trace::Event*>(a.trace_events), static_cast<trace::BufferState*>(a.trace_state),
                                   a.trace_capacity, 0};
        hooks::Point<hooks::AtnPublished>::hooks({tv, a.meta_layer, static_cast<uint32_t>(gridDim.x), seq});
      }
    }
  }
}

__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows,
              int inter, float limit, float up_add, float alpha) {
  const size_t n = static_cast<size_t>(rows) * inter;
  for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += gridDim.x * 256ull) {
    const size_t r = i / inter, c = i % inter;
    float g = __bfloat162float(gu[r * 2 * inter + c]);
    float u = __bfloat162float(gu[r * 2 * inter + inter + c]);
    if (limit > 0.f) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
    }
    const float al = alpha == 0.f ? 1.f : alpha;
    out[i] = __float2bfloat16_rn(g / (1.f + __expf(-al * g)) * (u + up_add));
  }
}

}  // namespace norm
}  // namespace xpool

extern "C" int xp_norm_publish(const XpNormArgs* a, void* stream) {
  if (a->hidden % 8 != 0 || a->hidden > 8 * xpool::norm::kThreads * xpool::norm::kMaxVec) return -10;
  if (a->rows <= 0 || a->nparts < 1 || a->nparts > 8 || a->npeers < 0 || a->npeers > 8) return -11;
  xpool::norm::norm_publish_kernel<<<a->rows, xpool::norm::kThreads, 0,
                                     reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" int xp_swiglu(const void* gate_up, void* out, int rows, int inter, float limit,
                         float up_add, float alpha, void* stream) {
  const size_t n = static_cast<size_t>(rows) * inter;
  int blocks = static_cast<int>((n + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  xpool::norm::swiglu_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gate_up), reinterpret_cast<__nv_bfloat16*>(out), rows,
      inter, limit, up_add, alpha);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
