// Paged decode attention for grouped-query heads with split-KV ("flash
// decoding"). One CTA handles every query head that shares one KV head over one
// slice of the sequence; a second small kernel merges the slices. The op is
// bound by reading the KV cache once, so the layout aims at wide coalesced
// loads: 8 lanes cooperate on one cached token (16 or 32 bytes each), 16 tokens
// are in flight per CTA iteration.
//
// The reference has no attention code of its own (SGLang/FlashInfer provide
// it, pyproject.toml:17-35); the oracle is a plain fp32 softmax(QK^T)V.
#include <math_constants.h>

#include "xpool/api.h"
#include "xpool/sm100.cuh"

namespace xpool {
namespace attn {

constexpr int kDecodeThreads = 128;

template <int E>
struct RawVec {
  uint4 v[E / 8];
};

template <int E>
__device__ __forceinline__ void load_raw(const __nv_bfloat16* p, RawVec<E>& r) {
  static_assert(E == 8 || E == 16, "E");
#pragma unroll
  for (int c = 0; c < E / 8; ++c) r.v[c] = __ldg(reinterpret_cast<const uint4*>(p) + c);
}

template <int E>
__device__ __forceinline__ void zero_raw(RawVec<E>& r) {
#pragma unroll
  for (int c = 0; c < E / 8; ++c) r.v[c] = make_uint4(0, 0, 0, 0);
}

template <int E>
__device__ __forceinline__ void unpack(const RawVec<E>& r, float* out) {
#pragma unroll
  for (int c = 0; c < E / 8; ++c) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.v[c]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(h[j]);
      out[c * 8 + 2 * j] = f.x;
      out[c * 8 + 2 * j + 1] = f.y;
    }
  }
}

// Partial result layout in the workspace: [batch, q_head, split, D + 2] floats:
// D un-normalised accumulators, running max (log2 domain), running sum.
template <int D, int GMAX>
__global__ void __launch_bounds__(kDecodeThreads)
decode_attn_kernel(XpDecodeAttnArgs a) {
  constexpr int E = D / 8;  // elements per lane
  __shared__ float q_s[GMAX][D];
  __shared__ float red[4][GMAX][D + 2];

  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = a.q_heads / a.kv_heads;
  const int len = a.seq_lens[b];
  const int nsplit = gridDim.x;
  // Fixed-size slices (chunk_tokens > 0) give every CTA the same amount of work whatever the
  // sequence length, so long and short sequences in one batch balance across the SMs; slices
  // past a sequence's end have nothing to do. Otherwise the sequence is cut into nsplit even parts.
  int chunk = a.chunk_tokens;
  if (chunk <= 0) {
    chunk = (len + nsplit - 1) / nsplit;
    chunk = (chunk + 15) & ~15;
  }
  const int t0 = split * chunk;
  const int t1 = min(len, t0 + chunk);
  if (a.chunk_tokens > 0 && nsplit > 1 && t0 >= len) return;  // the merge kernel skips this slice

  // q pre-scaled into the exp2 domain
  const float qscale = a.scale * 1.4426950408889634f;
  for (int i = threadIdx.x; i < GMAX * D; i += kDecodeThreads) {
    const int g = i / D, d = i % D;
    float v = 0.f;
    if (g < G)
      v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(
              a.q)[(static_cast<size_t>(b) * a.q_heads + hk * G + g) * D + d]) * qscale;
    q_s[g][d] = v;
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g4 = lane >> 3, gl = lane & 7;  // token within the warp's group of four, lane within the token
  // A lane owns E dims of every head: 16-byte chunk `gl` of the row, and for D = 128 also chunk
  // `gl + 8` (so that the eight lanes of a token read one contiguous 128-byte run per load).
  auto dim_of = [&](int e) { return e < 8 ? gl * 8 + e : D / 2 + gl * 8 + (e - 8); };
  // (for 8 heads per KV head the registers do not suffice; those read shared memory)
  constexpr bool kQInRegs = GMAX <= 4;
  float qr[kQInRegs ? GMAX : 1][E];
  if constexpr (kQInRegs) {
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
#pragma unroll
      for (int e = 0; e < E; ++e) qr[g][e] = q_s[g][dim_of(e)];
  }
  const int page_shift = 31 - __clz(a.page_size);  // page size is a power of two
  const int page_mask = a.page_size - 1;
  float m[GMAX], l[GMAX], acc[GMAX][E];
#pragma unroll
  for (int g = 0; g < GMAX; ++g) {
    m[g] = -CUDART_INF_F;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
  }
  const int* table = a.block_table + static_cast<size_t>(b) * a.max_blocks;
  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);

  // K/V rows stream through a per-warp ring in shared memory filled with cp.async, so the bytes an
  // SM keeps in flight are set by the ring depth, not by registers (the kernel is bound by HBM
  // latency x bandwidth: about 64 KB must be in flight per SM). Each iteration a warp consumes four
  // tokens; iteration i of warp w covers tokens t0 + (i * 4 + w) * 4 .. + 3. Trip counts are
  // uniform across the CTA because the dot-product shuffles name every lane.
  constexpr int kStages = 4;
  constexpr int kRow = D * 2;             // bytes of one K (or V) row of this head
  constexpr int kStageBytes = 8 * kRow;   // 4 tokens x (K + V)
  extern __shared__ __align__(16) uint8_t ring_raw[];
  uint8_t* ring = ring_raw + static_cast<size_t>(warp) * kStages * kStageBytes;
  constexpr int kChunksPerRow = kRow / 16;
  constexpr int kLoads = 8 * kChunksPerRow / 32;  // 16-byte copies per lane per stage (4 or 2)
  const int iters = (t1 - t0 + 15) / 16;
  auto issue = [&](int it) {
    if (it < iters) {
      uint8_t* st = ring + (it % kStages) * kStageBytes;
      const int tbase = t0 + (it * 4 + warp) * 4;
#pragma unroll
      for (int j = 0; j < kLoads; ++j) {
        const int c = lane + 32 * j;                 // chunk index within the stage
        const int row = c / kChunksPerRow;           // 0..3 K rows, 4..7 V rows
        const int part = c % kChunksPerRow;
        const int t = tbase + (row & 3);
        const bool ok = t < t1;
        const int tt = ok ? t : t0;
        const int page = table[tt >> page_shift];
        const size_t tok = (static_cast<size_t>(page) << page_shift) + (tt & page_mask);
        const __nv_bfloat16* src = (row < 4 ? kc : vc) + (tok * a.kv_heads + hk) * D + part * 8;
        const uint32_t dst = sm100::smem_u32(st + row * kRow + part * 16);
        const int sz = ok ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
      }
    }
    asm volatile("cp.async.commit_group;");
  };
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) issue(i);
  for (int it = 0; it < iters; ++it) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
    __syncwarp();
    issue(it + kStages - 1);  // refills the slot consumed in the previous iteration
    const uint8_t* st = ring + (it % kStages) * kStageBytes;
    const int t = t0 + (it * 4 + warp) * 4 + g4;
    const bool valid = t < t1;
    RawVec<E> kr, vr;
#pragma unroll
    for (int c = 0; c < E / 8; ++c) {
      kr.v[c] = *reinterpret_cast<const uint4*>(st + g4 * kRow + (gl + 8 * c) * 16);
      vr.v[c] = *reinterpret_cast<const uint4*>(st + (4 + g4) * kRow + (gl + 8 * c) * 16);
    }
    float kf[E], vf[E];
    unpack<E>(kr, kf);
    unpack<E>(vr, vf);
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      if (g >= G) break;  // G is uniform
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) s += (kQInRegs ? qr[kQInRegs ? g : 0][e] : q_s[g][dim_of(e)]) * kf[e];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (valid) {
        // rescale the running sums only when the maximum actually moves
        if (s > m[g]) {
          const float corr = exp2f(m[g] - s);
          m[g] = s;
          l[g] *= corr;
#pragma unroll
          for (int e = 0; e < E; ++e) acc[g][e] *= corr;
        }
        const float p = exp2f(s - m[g]);
        l[g] += p;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[g][e] += p * vf[e];
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // merge the four token groups of a warp (lanes differing in bits 3 and 4)
#pragma unroll
  for (int g = 0; g < GMAX; ++g) {
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo);
      const float c0 = (m[g] == -CUDART_INF_F) ? 0.f : exp2f(m[g] - mn);
      const float c1 = (mo == -CUDART_INF_F) ? 0.f : exp2f(mo - mn);
      l[g] = l[g] * c0 + lo * c1;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
        acc[g][e] = acc[g][e] * c0 + ao * c1;
      }
      m[g] = mn;
    }
  }
  if (lane < 8) {
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
#pragma unroll
      for (int e = 0; e < E; ++e) red[warp][g][dim_of(e)] = acc[g][e];
      if (lane == 0) {
        red[warp][g][D] = m[g];
        red[warp][g][D + 1] = l[g];
      }
    }
  }
  __syncthreads();
  // merge the four warps; thread -> (g, d)
  for (int i = threadIdx.x; i < G * D; i += kDecodeThreads) {
    const int g = i / D, d = i % D;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[w][g][D]);
    float ll = 0.f, av = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red[w][g][D];
      const float c = (mw == -CUDART_INF_F) ? 0.f : exp2f(mw - mm);
      ll += red[w][g][D + 1] * c;
      av += red[w][g][d] * c;
    }
    const int hq = hk * G + g;
    if (nsplit == 1) {
      const float o = ll > 0.f ? av / ll : 0.f;
      reinterpret_cast<__nv_bfloat16*>(a.out)[(static_cast<size_t>(b) * a.q_heads + hq) * D + d] =
          __float2bfloat16_rn(o);
    } else {
      float* ws = a.ws + ((static_cast<size_t>(b) * a.q_heads + hq) * nsplit + split) * (D + 2);
      ws[d] = av;
      if (d == 0) {
        ws[D] = mm;
        ws[D + 1] = ll;
      }
    }
  }
}

template <int D>
__global__ void decode_combine_kernel(XpDecodeAttnArgs a, int nsplit) {
  const int hq = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float* ws = a.ws + (static_cast<size_t>(b) * a.q_heads + hq) * nsplit * (D + 2);
  if (a.chunk_tokens > 0) {
    const int len = a.seq_lens[b];
    nsplit = min(nsplit, (len + a.chunk_tokens - 1) / a.chunk_tokens);  // slices that ran
  }
  float mm = -CUDART_INF_F;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, ws[s * (D + 2) + D]);
  float ll = 0.f, av = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = ws[s * (D + 2) + D];
    const float c = (ms == -CUDART_INF_F) ? 0.f : exp2f(ms - mm);
    ll += ws[s * (D + 2) + D + 1] * c;
    av += ws[s * (D + 2) + d] * c;
  }
  reinterpret_cast<__nv_bfloat16*>(a.out)[(static_cast<size_t>(b) * a.q_heads + hq) * D + d] =
      __float2bfloat16_rn(ll > 0.f ? av / ll : 0.f);
}

template <int D, int GMAX>
static int launch_decode(const XpDecodeAttnArgs& a, int nsplit, cudaStream_t s) {
  dim3 grid(nsplit, a.kv_heads, a.batch);
  constexpr int kRing = 4 /*warps*/ * 4 /*stages*/ * 8 * D * 2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(decode_attn_kernel<D, GMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing);
    attr_set = true;
  }
  decode_attn_kernel<D, GMAX><<<grid, kDecodeThreads, kRing, s>>>(a);
  if (nsplit > 1) decode_combine_kernel<D><<<dim3(a.q_heads, a.batch), D, 0, s>>>(a, nsplit);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

}  // namespace attn
}  // namespace xpool

extern "C" int xp_decode_attn_splits(int batch, int kv_heads, int max_len) {
  // enough CTAs to fill 148 SMs a few times over, at least 256 tokens per slice
  int want = (148 * 4 + batch * kv_heads - 1) / (batch * kv_heads);
  int cap = (max_len + 255) / 256;
  int n = want < cap ? want : cap;
  if (n < 1) n = 1;
  if (n > 64) n = 64;
  return n;
}

extern "C" int xp_decode_attn(const XpDecodeAttnArgs* a, void* stream) {
  using namespace xpool::attn;
  if (a->batch <= 0) return 0;
  if (a->q_heads % a->kv_heads != 0) return -10;
  const int G = a->q_heads / a->kv_heads;
  int nsplit = a->num_splits > 0 ? a->num_splits : 1;
  if (nsplit > 1 && a->ws == nullptr) return -11;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->head_dim == 128) {
    if (G <= 2) return launch_decode<128, 2>(*a, nsplit, s);
    if (G <= 4) return launch_decode<128, 4>(*a, nsplit, s);
    if (G <= 8) return launch_decode<128, 8>(*a, nsplit, s);
  } else if (a->head_dim == 64) {
    if (G <= 2) return launch_decode<64, 2>(*a, nsplit, s);
    if (G <= 4) return launch_decode<64, 4>(*a, nsplit, s);
    if (G <= 8) return launch_decode<64, 8>(*a, nsplit, s);
  }
  return -12;
}
