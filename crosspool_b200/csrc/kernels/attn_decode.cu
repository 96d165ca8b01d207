// Paged decode attention for grouped-query heads with optional split-KV ("flash decoding"). One CTA handles
// every query head that shares one KV head over one slice of the sequence; a second small kernel merges the
// slices. The op is bound by reading the KV cache once. Two kernels:
//   decode_attn_tc_kernel  TMA-fed 16-token tiles, ldmatrix + mma.m16n8k16 (default; see its comment below);
//   decode_attn_kernel     plain SIMT version: 8 lanes cooperate on one cached token, cp.async ring; kept for
//                          page sizes below 16 tokens and as the numerical cross-check.
//
// The reference has no attention code of its own (SGLang/FlashInfer provide
// it, pyproject.toml:17-35); the oracle is a plain fp32 softmax(QK^T)V.
#include <math_constants.h>

#include "xpool/api.h"
#include "xpool/sm100.cuh"
#include "xpool/tensormap.hpp"

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

// ---------------------------------------------------------------------------------------------
// Tensor-core variant. The SIMT kernel above spends its issue slots on bf16 unpacking, FMAs and
// shuffles (issue-bound at about half of the HBM bandwidth); here the two contractions run on the
// tensor cores and the KV tiles arrive through TMA, so the warp issues a few dozen instructions
// per 16 tokens and the kernel is bound by the KV read alone.
//
//   CTA = (slice, KV head, sequence), 4 warps; every warp streams its own 16-token tiles through a
//   ring of kTcStages stages filled by TMA (3-D map over [tokens, kv_heads, D], box 16 x 1 x 64,
//   128-byte swizzle) and tracked by one mbarrier per stage;
//   S = Q K^T : mma.m16n8k16, A = the query heads of this KV head (rows padded to 16), B = K tile
//               read with ldmatrix (a K row is k-contiguous, i.e. a column-major B operand);
//   O += P V  : P is the S fragment rounded to bf16, B = V tile read with ldmatrix.trans.
//
// mma.sync rather than tcgen05: the op moves 2 x D x 2 bytes per token for 4 x G x D flops, i.e.
// at most 16 flop/byte with 8 heads per group -- two orders below the tensor roofline -- and a
// UMMA tile needs 64 or 128 query rows where there are 16 at most.
constexpr int kTcStages = 3;

__device__ __forceinline__ void tma_load_kv(uint32_t dst, const CUtensorMap* m, uint32_t bar, int d0, int head, int token) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(d0), "r"(head), "r"(token)
      : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(kDecodeThreads, 2)
decode_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                      XpDecodeAttnArgs a) {
  constexpr int kHalves = D / 64;              // 64-dim boxes per row
  constexpr int kBox = 16 * 128;               // bytes of one box: 16 tokens x 64 dims
  constexpr int kStage = 2 * kHalves * kBox;   // K boxes then V boxes
  constexpr int kWarpRing = kTcStages * kStage;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t full[4][kTcStages];

  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = a.q_heads / a.kv_heads;
  const int len = a.seq_lens[b];
  const int nsplit = gridDim.x;
  int chunk = a.chunk_tokens;
  if (chunk <= 0) {
    chunk = (len + nsplit - 1) / nsplit;
    chunk = (chunk + 15) & ~15;
  }
  const int t0 = split * chunk;
  const int t1 = min(len, t0 + chunk);
  if (a.chunk_tokens > 0 && nsplit > 1 && t0 >= len) return;  // the merge kernel skips this slice

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q4 = lane & 3;
  const uint32_t ring_base = (sm100::smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t ring = ring_base + warp * kWarpRing;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kTcStages; ++s) sm100::mbar_init(&full[warp][s], 1);
    sm100::mbar_fence_init();
    sm100::fence_proxy_async_smem();
  }
  __syncwarp();

  // this warp's tiles: tile index i * 4 + warp of the slice
  const int tiles = t1 > t0 ? (t1 - t0 + 15) >> 4 : 0;
  const int n_it = tiles > warp ? (tiles - warp + 3) >> 2 : 0;
  const int page_shift = 31 - __clz(a.page_size);
  const int page_mask = a.page_size - 1;
  const int* table = a.block_table + static_cast<size_t>(b) * a.max_blocks;
  // lane i looks up the cache position of the tile of iteration (base + i)
  auto lookup = [&](int it) -> int {
    if (it >= n_it) return 0;
    const int ts = t0 + ((it * 4 + warp) << 4);
    return (table[ts >> page_shift] << page_shift) + (ts & page_mask);
  };
  int my_tok = lookup(lane);
  auto issue = [&](int it, int tok) {  // lane 0 only
    const int s = it % kTcStages;
    const uint32_t bar = sm100::smem_u32(&full[warp][s]);
    const uint32_t dst = ring + s * kStage;
    sm100::mbar_arrive_expect_tx(&full[warp][s], kStage);
#pragma unroll
    for (int h = 0; h < kHalves; ++h) {
      tma_load_kv(dst + h * kBox, &tmap_k, bar, h * 64, hk, tok);
      tma_load_kv(dst + (kHalves + h) * kBox, &tmap_v, bar, h * 64, hk, tok);
    }
  };
#pragma unroll
  for (int i = 0; i < kTcStages; ++i) {
    const int tok = __shfl_sync(0xffffffffu, my_tok, i);
    if (lane == 0 && i < n_it) issue(i, tok);
  }

  // Q fragments (A operand), unscaled; rows >= G are zero
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(a.q) + (static_cast<size_t>(b) * a.q_heads + hk * G) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c = ks * 16 + q4 * 2;
      qf[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * D + c) : 0u;
      qf[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * D + c) : 0u;
      qf[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * D + c + 8) : 0u;
      qf[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * D + c + 8) : 0u;
    }
  }
  const float sscale = a.scale * 1.4426950408889634f;  // scores in the exp2 domain
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  const int lr = lane & 7, lm = lane >> 3;  // ldmatrix: row within a matrix, matrix index
  bool timed_out = false;
  for (int it = 0; it < n_it; ++it) {
    const int s = it % kTcStages;
    const uint32_t st = ring + s * kStage;
    const bool landed = sm100::mbar_wait(&full[warp][s], (it / kTcStages) & 1, sm100::global_timer_ns() + sm100::kPipelineWaitNs);
    if (!__all_sync(0xffffffffu, landed)) {  // warp-uniform: the shuffles below name every lane
      timed_out = true;
      break;
    }
    const int tbase = t0 + ((it * 4 + warp) << 4);
    const int nvalid = min(16, t1 - tbase);
    if (nvalid < 16) {
      // cache slots past the sequence end hold whatever was there: zero those V rows so that a
      // probability of exactly zero cannot meet a NaN
      for (int i = lane; i < (16 - nvalid) * kHalves * 8; i += 32) {
        const int r = nvalid + i / (kHalves * 8), rest = i % (kHalves * 8);
        const uint32_t addr = st + (kHalves + rest / 8) * kBox + r * 128 + (rest % 8) * 16;
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
      }
      __syncwarp();
    }
    // ---- S = Q K^T for two 8-token column tiles
    float sc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[nt][e] = 0.f;
      const int r = nt * 8 + lr;
#pragma unroll
      for (int j = 0; j < D / 32; ++j) {
        const int cc = 4 * j + lm;  // 16-byte chunk of the row: dims cc * 8 .. + 7
        const uint32_t addr = st + (cc >> 3) * kBox + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
        uint32_t kb[4];
        ldsm_x4(addr, kb);
        mma_bf16_16816(sc[nt], qf[2 * j], kb[0], kb[1]);
        mma_bf16_16816(sc[nt], qf[2 * j + 1], kb[2], kb[3]);
      }
    }
    // ---- online softmax on rows g and g + 8
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = nt * 8 + q4 * 2 + (e & 1);
        const float v = col < nvalid ? sc[nt][e] * sscale : -CUDART_INF_F;
        sc[nt][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v);
        else mx1 = fmaxf(mx1, v);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);  // finite: every tile has a valid token
    if (__any_sync(0xffffffffu, n0 > m0 || n1 > m1)) {
      const float c0 = exp2f(m0 - n0), c1 = exp2f(m1 - n1);
      l0 *= c0;
      l1 *= c1;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        acc[j][0] *= c0;
        acc[j][1] *= c0;
        acc[j][2] *= c1;
        acc[j][3] *= c1;
      }
      m0 = n0;
      m1 = n1;
    }
    uint32_t pf[4];
    {
      const float p00 = exp2f(sc[0][0] - m0), p01 = exp2f(sc[0][1] - m0), p02 = exp2f(sc[0][2] - m1), p03 = exp2f(sc[0][3] - m1);
      const float p10 = exp2f(sc[1][0] - m0), p11 = exp2f(sc[1][1] - m0), p12 = exp2f(sc[1][2] - m1), p13 = exp2f(sc[1][3] - m1);
      l0 += p00 + p01 + p10 + p11;
      l1 += p02 + p03 + p12 + p13;
      pf[0] = pack_bf16(p00, p01);  // (row g,     tokens 2 q4 ..)
      pf[1] = pack_bf16(p02, p03);  // (row g + 8, tokens 2 q4 ..)
      pf[2] = pack_bf16(p10, p11);  // (row g,     tokens 8 + 2 q4 ..)
      pf[3] = pack_bf16(p12, p13);  // (row g + 8, tokens 8 + 2 q4 ..)
    }
    // ---- O += P V
#pragma unroll
    for (int jp = 0; jp < D / 16; ++jp) {
      const int r = (lm & 1) * 8 + lr;
      const int cc = 2 * jp + (lm >> 1);
      const uint32_t addr = st + (kHalves + (cc >> 3)) * kBox + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
      uint32_t vb[4];
      ldsm_x4_trans(addr, vb);
      mma_bf16_16816(acc[2 * jp], pf, vb[0], vb[1]);
      mma_bf16_16816(acc[2 * jp + 1], pf, vb[2], vb[3]);
    }
    __syncwarp();  // every lane has consumed the stage
    const int nxt = it + kTcStages;
    if ((nxt & 31) == 0) my_tok = lookup(nxt + lane);
    const int tok = __shfl_sync(0xffffffffu, my_tok, nxt & 31);
    if (lane == 0 && nxt < n_it) {
      sm100::fence_proxy_async_smem();
      issue(nxt, tok);
    }
  }
  if (timed_out) {
    if (lane == 0 && a.status != nullptr) atomicCAS(a.status, 0u, 5u);
    __nanosleep(1000000);  // copies still in flight get one more bounded chance to land before the CTA retires
  }
  // row sums across the quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();  // all warps are done with their rings: reuse the memory for the merge
  float* red = reinterpret_cast<float*>(smem_dyn + (ring_base - sm100::smem_u32(smem_dyn)));  // [4][16][D + 2]
  {
    float* r0 = red + (warp * 16 + g) * (D + 2);
    float* r1 = red + (warp * 16 + g + 8) * (D + 2);
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int c = j * 8 + q4 * 2;
      r0[c] = acc[j][0];
      r0[c + 1] = acc[j][1];
      r1[c] = acc[j][2];
      r1[c + 1] = acc[j][3];
    }
    if (q4 == 0) {
      r0[D] = m0;
      r0[D + 1] = l0;
      r1[D] = m1;
      r1[D + 1] = l1;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += kDecodeThreads) {
    const int gg = i / D, d = i % D;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * 16 + gg) * (D + 2) + D]);
    float ll = 0.f, av = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* rw = red + (w * 16 + gg) * (D + 2);
      const float c = (rw[D] == -CUDART_INF_F) ? 0.f : exp2f(rw[D] - mm);
      ll += rw[D + 1] * c;
      av += rw[d] * c;
    }
    const int hq = hk * G + gg;
    if (nsplit == 1) {
      reinterpret_cast<__nv_bfloat16*>(a.out)[(static_cast<size_t>(b) * a.q_heads + hq) * D + d] =
          __float2bfloat16_rn(ll > 0.f ? av / ll : 0.f);
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

template <int D>
static int launch_decode_tc(const XpDecodeAttnArgs& a, int nsplit, cudaStream_t s) {
  CUtensorMap mk, mv;
  const uint64_t tokens = static_cast<uint64_t>(a.num_pages) * a.page_size;
  if (tmap::cache().get_kv(&mk, a.k_cache, tokens, a.kv_heads, D) != 0) return -20;
  if (tmap::cache().get_kv(&mv, a.v_cache, tokens, a.kv_heads, D) != 0) return -20;
  constexpr int kStage = 2 * (D / 64) * 16 * 128;
  constexpr int kSmem = 4 * kTcStages * kStage + 1024;  // rings of four warps + alignment slack
  static_assert(4 * 16 * (D + 2) * 4 <= 4 * kTcStages * kStage, "merge scratch must fit in the rings");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(decode_attn_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -21;
    attr_set = true;
  }
  dim3 grid(nsplit, a.kv_heads, a.batch);
  decode_attn_tc_kernel<D><<<grid, kDecodeThreads, kSmem, s>>>(mk, mv, a);
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
  // tensor-core kernel: 16-token tiles must not straddle pages, slices must start on a tile
  const bool tc_ok = !a->force_simt && a->num_pages > 0 && a->page_size >= 16 && (a->page_size & (a->page_size - 1)) == 0 &&
                     G <= 16 && a->chunk_tokens % 16 == 0 && (reinterpret_cast<uintptr_t>(a->q) & 3) == 0;
  if (tc_ok && a->head_dim == 128) return launch_decode_tc<128>(*a, nsplit, s);
  if (tc_ok && a->head_dim == 64) return launch_decode_tc<64>(*a, nsplit, s);
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
