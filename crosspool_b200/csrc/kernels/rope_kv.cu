// Per-token attention pre-processing in one pass over the fused QKV projection:
// optional per-head RMSNorm of q and k (Qwen3), rotary embedding (rotate-half
// convention, base theta), and the scatter of k and v into the paged KV cache.
// The reference leaves all of this to SGLang (its KV store hook only delegates,
// src/xpool/integrations/sglang/ecs/pool.py:116-121).
//
// KV cache layout per layer: [num_pages, page_size, kv_heads, head_dim] for K and
// for V; `slots[row]` = page * page_size + offset, or -1 for padding rows.
#include "xpool/api.h"
#include "xpool/sm100.cuh"

namespace xpool {
namespace rope {

template <int D>
__global__ void __launch_bounds__(256)
rope_kv_kernel(XpRopeArgs a) {
  constexpr int PER = D / 64;  // elements per lane in each half
  const int row = blockIdx.x;
  const int head = blockIdx.y * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads_total = a.q_heads + 2 * a.kv_heads;
  if (head >= heads_total) return;
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.qkv) +
                             static_cast<size_t>(row) * a.ld_qkv + static_cast<size_t>(head) * D;
  const bool is_q = head < a.q_heads;
  const bool is_k = !is_q && head < a.q_heads + a.kv_heads;
  float x1[PER], x2[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    x1[i] = __bfloat162float(src[lane * PER + i]);
    x2[i] = __bfloat162float(src[D / 2 + lane * PER + i]);
  }
  if (is_q || is_k) {
    const __nv_bfloat16* nw =
        reinterpret_cast<const __nv_bfloat16*>(is_q ? a.q_norm_weight : a.k_norm_weight);
    if (nw != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) ss += x1[i] * x1[i] + x2[i] * x2[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = rsqrtf(ss / D + a.eps);
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        float n1 = __bfloat162float(__float2bfloat16_rn(x1[i] * inv));
        float n2 = __bfloat162float(__float2bfloat16_rn(x2[i] * inv));
        x1[i] = __bfloat162float(__float2bfloat16_rn(n1 * __bfloat162float(nw[lane * PER + i])));
        x2[i] = __bfloat162float(__float2bfloat16_rn(n2 * __bfloat162float(nw[D / 2 + lane * PER + i])));
      }
    }
    const float pos = static_cast<float>(a.positions[row]);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int idx = lane * PER + i;
      const float inv_freq = exp2f(-(2.f * idx / D) * a.log2_theta);
      float s, c;
      sincosf(pos * inv_freq, &s, &c);
      const float r1 = x1[i] * c - x2[i] * s;
      const float r2 = x2[i] * c + x1[i] * s;
      x1[i] = r1;
      x2[i] = r2;
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = reinterpret_cast<__nv_bfloat16*>(a.q_out) + static_cast<size_t>(row) * a.q_heads * D +
          static_cast<size_t>(head) * D;
  } else {
    const int slot = a.slots[row];
    if (slot < 0) return;
    const int hk = is_k ? head - a.q_heads : head - a.q_heads - a.kv_heads;
    __nv_bfloat16* cache = reinterpret_cast<__nv_bfloat16*>(is_k ? a.k_cache : a.v_cache);
    dst = cache + (static_cast<size_t>(slot) * a.kv_heads + hk) * D;
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    dst[lane * PER + i] = __float2bfloat16_rn(x1[i]);
    dst[D / 2 + lane * PER + i] = __float2bfloat16_rn(x2[i]);
  }
}

}  // namespace rope
}  // namespace xpool

extern "C" int xp_rope_kv(const XpRopeArgs* a, void* stream) {
  if (a->rows <= 0) return 0;
  const int heads_total = a->q_heads + 2 * a->kv_heads;
  dim3 grid(a->rows, (heads_total + 7) / 8);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->head_dim == 128)
    xpool::rope::rope_kv_kernel<128><<<grid, 256, 0, s>>>(*a);
  else if (a->head_dim == 64)
    xpool::rope::rope_kv_kernel<64><<<grid, 256, 0, s>>>(*a);
  else
    return -10;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
