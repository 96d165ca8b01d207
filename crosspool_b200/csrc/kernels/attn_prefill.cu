// Chunked-prefill attention over the paged KV cache: causal, grouped-query,
// variable-length. The chunk's K and V have already been written to the cache,
// so every query row attends to cache positions [0, context + its index].
//
// Two kernels, both flash-style single pass with the softmax state in registers and the two matrix
// products on the warp-level tensor-core path (mma.sync m16n8k16, bf16 in / fp32 accumulate):
//   prefill_attn_kernel     one CTA = 64 query rows of one head, K/V tiles fetched with cp.async; handles any
//                           page size and head grouping (fallback);
//   prefill_attn_tc_kernel  one CTA = all query heads of a KV head, K/V tiles through a TMA ring (default).
// Measured on B200 (16 q / 8 kv heads, d 128): 121-142 TFLOP/s for the first, 145-172 TFLOP/s for the second.
// A tcgen05 version (S and O in TMEM, P fed back as a TMEM operand) is the known next step.
#include <math_constants.h>

#include "xpool/api.h"
#include "xpool/sm100.cuh"
#include "xpool/tensormap.hpp"

namespace xpool {
namespace attn {

constexpr int kBM = 64;  // query rows per CTA
constexpr int kBN = 64;  // cached tokens per tile
constexpr int kPrefillThreads = 128;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = sm100::smem_u32(smem);
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared tiles are [rows][D] bf16 with the 16-byte chunks of each row XOR-ed
// with (row & 7) so that ldmatrix reads are bank-conflict free.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return static_cast<uint32_t>(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(kPrefillThreads)
prefill_attn_kernel(XpPrefillAttnArgs a) {
  constexpr int CH = D / 8;    // 16-byte chunks per row
  constexpr int KS = D / 16;   // k-steps over the head dim
  constexpr int NB = kBN / 8;  // 8-token column blocks per tile
  constexpr int DB = D / 8;    // 8-wide output column blocks
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + kBM * D * 2;
  uint8_t* v_s = k_s + kBN * D * 2;

  const int seq = blockIdx.z, hq = blockIdx.y, qt = blockIdx.x;
  const int q_len = a.q_lens[seq];
  const int q0 = qt * kBM;
  if (q0 >= q_len) return;
  const int ctx = a.ctx_lens[seq];
  const int q_base = a.q_starts[seq];
  const int hk = hq / (a.q_heads / a.kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);

  // Q tile -> smem
  for (int i = threadIdx.x; i < kBM * CH; i += kPrefillThreads) {
    const int r = i / CH, c = i % CH;
    const bool ok = q0 + r < q_len;
    const __nv_bfloat16* src =
        qg + (static_cast<size_t>(q_base + (ok ? q0 + r : 0)) * a.q_heads + hq) * D + c * 8;
    cp_async16(q_s + tile_off<D>(r, c), src, ok);
  }
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();

  // Q fragments for this warp's 16 rows
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int r = warp * 16 + (lane & 15);
    const int c = ks * 2 + (lane >> 4);
    ldmatrix_x4(sm100::smem_u32(q_s + tile_off<D>(r, c)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  float o[DB][4];
#pragma unroll
  for (int i = 0; i < DB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  const float sc = a.scale * 1.4426950408889634f;
  const int row0 = q0 + warp * 16 + (lane >> 2);  // this thread's two rows: row0, row0 + 8
  const int kv_end = min(ctx + q_len, ctx + q0 + kBM);  // causal upper bound for the tile

  for (int t0 = 0; t0 < kv_end; t0 += kBN) {
    __syncthreads();  // previous tile fully consumed
    for (int i = threadIdx.x; i < kBN * CH; i += kPrefillThreads) {
      const int r = i / CH, c = i % CH;
      const int t = t0 + r;
      const bool ok = t < kv_end;
      size_t off = 0;
      if (ok) {
        const int page = table[t / a.page_size];
        off = ((static_cast<size_t>(page) * a.page_size + (t % a.page_size)) * a.kv_heads + hk) * D + c * 8;
      }
      cp_async16(k_s + tile_off<D>(r, c), kc + off, ok);
      cp_async16(v_s + tile_off<D>(r, c), vc + off, ok);
    }
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();

    // S = Q K^T for 16 rows x 64 tokens
    float s[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int nb2 = 0; nb2 < NB / 2; ++nb2) {
        // x4: tokens nb2*16 + {0..7, 8..15} x head-dim halves of this k-step
        const int r = nb2 * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int c = ks * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(sm100::smem_u32(k_s + tile_off<D>(r, c)), b0, b1, b2, b3);
        mma_bf16(s[nb2 * 2], qf[ks], b0, b1);
        mma_bf16(s[nb2 * 2 + 1], qf[ks], b2, b3);
      }
    }
    // scale, causal mask, online softmax
    float mx0 = m0, mx1 = m1;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = t0 + nb * 8 + (lane & 3) * 2 + (j & 1);
        const int r = row0 + ((j >> 1) << 3);
        const bool ok = t <= ctx + r && t < kv_end;
        s[nb][j] = ok ? s[nb][j] * sc : -CUDART_INF_F;
      }
      mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float c0 = (m0 == -CUDART_INF_F) ? 0.f : exp2f(m0 - mx0);
    const float c1 = (m1 == -CUDART_INF_F) ? 0.f : exp2f(m1 - mx1);
    const float e0 = (mx0 == -CUDART_INF_F) ? 0.f : mx0;  // rows with nothing visible yet
    const float e1 = (mx1 == -CUDART_INF_F) ? 0.f : mx1;
    m0 = mx0;
    m1 = mx1;
    float ps0 = 0.f, ps1 = 0.f;
    uint32_t pf[NB / 2][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const float p0 = exp2f(s[nb][0] - e0), p1 = exp2f(s[nb][1] - e0);
      const float p2 = exp2f(s[nb][2] - e1), p3 = exp2f(s[nb][3] - e1);
      ps0 += p0 + p1;
      ps1 += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l0 = l0 * c0 + ps0;
    l1 = l1 * c1 + ps1;
#pragma unroll
    for (int i = 0; i < DB; ++i) {
      o[i][0] *= c0;
      o[i][1] *= c0;
      o[i][2] *= c1;
      o[i][3] *= c1;
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < NB / 2; ++kk) {  // 16 tokens per step
#pragma unroll
      for (int db2 = 0; db2 < DB / 2; ++db2) {
        // x4.trans: tokens kk*16 + {0..7, 8..15} x dims db2*16 + {0..7, 8..15}
        const int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int c = db2 * 2 + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(sm100::smem_u32(v_s + tile_off<D>(r, c)), b0, b1, b2, b3);
        mma_bf16(o[db2 * 2], pf[kk], b0, b1);
        mma_bf16(o[db2 * 2 + 1], pf[kk], b2, b3);
      }
    }
  }
  // finish: row sums across the quad, normalise, store
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.out);
#pragma unroll
  for (int db = 0; db < DB; ++db) {
    const int d = db * 8 + (lane & 3) * 2;
    if (row0 < q_len)
      *reinterpret_cast<uint32_t*>(og + (static_cast<size_t>(q_base + row0) * a.q_heads + hq) * D + d) =
          pack_bf16(o[db][0] * i0, o[db][1] * i0);
    if (row0 + 8 < q_len)
      *reinterpret_cast<uint32_t*>(og + (static_cast<size_t>(q_base + row0 + 8) * a.q_heads + hq) * D + d) =
          pack_bf16(o[db][2] * i1, o[db][3] * i1);
  }
}


// ---------------------------------------------------------------------------------------------
// Pipelined variant. Differences from the kernel above:
//   * the K/V tiles (64 tokens) arrive through TMA (3-D map over [tokens, kv_heads, D], box 16 tokens x
//     64 dims, 128-byte swizzle) into a ring of kPfStages stages tracked by mbarriers, so loads of the
//     next tiles overlap the tensor-core work of the current one and no thread computes addresses;
//   * one CTA serves every query head of a KV head (8 warps = G heads x 8/G blocks of 16 query rows),
//     so a K/V tile is fetched once per group instead of once per query head;
//   * Q fragments come straight from global memory into registers;
//   * the causal mask is evaluated only on tiles that touch the diagonal.
constexpr int kPfStages = 3;
constexpr int kPfThreads = 256;

__device__ __forceinline__ void tma_load_kv3(uint32_t dst, const CUtensorMap* m, uint32_t bar, int d0, int head, int token) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(d0), "r"(head), "r"(token)
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       XpPrefillAttnArgs a, int G, int rows_per_cta) {
  constexpr int KS = D / 16;    // k-steps over the head dim
  constexpr int NB = kBN / 8;   // 8-token column blocks per tile
  constexpr int DB = D / 8;     // 8-wide output column blocks
  constexpr int kHalves = D / 64;
  constexpr int kBox = 16 * 128;                  // 16 tokens x 64 dims
  constexpr int kHalfBytes = (kBN / 16) * kBox;   // the 64 tokens of one 64-dim half
  constexpr int kTile = kHalves * kHalfBytes;     // K (or V) tile
  constexpr int kStage = 2 * kTile;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t full[kPfStages];

  // Query tiles are taken from the end of the sequence first: under the causal mask the last tile reads the
  // most K/V, and CTAs are dispatched in index order, so the longest ones start first and the short ones fill
  // the tail (longest-processing-time-first) instead of one 32-tile CTA running alone at the end.
  const int seq = blockIdx.z, hk = blockIdx.y, qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int q_len = a.q_lens[seq];
  const int q0 = qt * rows_per_cta;
  if (q0 >= q_len) return;
  const int ctx = a.ctx_lens[seq];
  const int q_base = a.q_starts[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = warp % G;                       // query head within the group
  const int hq = hk * G + g;
  const int wrow0 = q0 + (warp / G) * 16;       // first query row of this warp
  const uint32_t ring = (sm100::smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int page_shift = 31 - __clz(a.page_size);
  const int page_mask = a.page_size - 1;
  const int* table = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const int kv_end = ctx + min(q_len, q0 + rows_per_cta);   // causal bound of the CTA
  const int n_tiles = (kv_end + kBN - 1) / kBN;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < kPfStages; ++s) sm100::mbar_init(&full[s], 1);
    sm100::mbar_fence_init();
    sm100::fence_proxy_async_smem();
  }
  __syncthreads();
  auto issue = [&](int t) {  // thread 0: the four 16-token boxes of tile t, both halves, K and V
    const int s = t % kPfStages;
    const uint32_t bar = sm100::smem_u32(&full[s]);
    const uint32_t dst = ring + s * kStage;
    sm100::mbar_arrive_expect_tx(&full[s], kStage);
#pragma unroll
    for (int j = 0; j < kBN / 16; ++j) {
      int tk = t * kBN + j * 16;
      if (tk >= kv_end) tk = (kv_end - 1) & ~15;   // boxes past the end repeat the last valid one (masked below)
      const int tok = (table[tk >> page_shift] << page_shift) + (tk & page_mask);
#pragma unroll
      for (int h = 0; h < kHalves; ++h) {
        tma_load_kv3(dst + h * kHalfBytes + j * kBox, &tmap_k, bar, h * 64, hk, tok);
        tma_load_kv3(dst + kTile + h * kHalfBytes + j * kBox, &tmap_v, bar, h * 64, hk, tok);
      }
    }
  };
  if (threadIdx.x == 0) {
    for (int t = 0; t < kPfStages && t < n_tiles; ++t) issue(t);
  }

  // Q fragments of this warp's 16 rows (rows past the chunk read row 0 and are never stored)
  const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q);
  uint32_t qf[KS][4];
  {
    const int r0 = wrow0 + (lane >> 2), r1 = r0 + 8;
    const __nv_bfloat16* p0 = qg + (static_cast<size_t>(q_base + (r0 < q_len ? r0 : 0)) * a.q_heads + hq) * D;
    const __nv_bfloat16* p1 = qg + (static_cast<size_t>(q_base + (r1 < q_len ? r1 : 0)) * a.q_heads + hq) * D;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c = ks * 16 + (lane & 3) * 2;
      qf[ks][0] = *reinterpret_cast<const uint32_t*>(p0 + c);
      qf[ks][1] = *reinterpret_cast<const uint32_t*>(p1 + c);
      qf[ks][2] = *reinterpret_cast<const uint32_t*>(p0 + c + 8);
      qf[ks][3] = *reinterpret_cast<const uint32_t*>(p1 + c + 8);
    }
  }
  float o[DB][4];
#pragma unroll
  for (int i = 0; i < DB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  const float sc = a.scale * 1.4426950408889634f;
  const int row0 = wrow0 + (lane >> 2);          // this thread's two rows: row0, row0 + 8
  const int warp_kv_end = ctx + min(q_len, wrow0 + 16);   // tiles at or past this bound hold nothing for the warp
  // swizzled offset of (token row R of the tile, 16-byte chunk cc of the head dim)
  auto toff = [&](int R, int cc) -> uint32_t {
    return static_cast<uint32_t>((cc >> 3) * kHalfBytes + (R >> 4) * kBox + (R & 15) * 128 + (((cc & 7) ^ (R & 7)) << 4));
  };
  bool timed_out = false;
  for (int t = 0; t < n_tiles; ++t) {
    const int s = t % kPfStages;
    const uint32_t ks_base = ring + s * kStage, vs_base = ks_base + kTile;
    // No CTA barrier here: a warp starts on the tile as soon as it has seen it land. A wait that ran out is
    // reported at the barrier that ends the tile, which every thread reaches whatever it saw.
    const bool landed = sm100::mbar_wait(&full[s], (t / kPfStages) & 1, sm100::global_timer_ns() + sm100::kPipelineWaitNs);
    const int t0 = t * kBN;
    if (t0 + kBN > kv_end) {
      // cache slots past the sequence end may hold anything: zero those V rows (probability 0 x NaN)
      const int first = kv_end - t0;
      for (int i = threadIdx.x; i < (kBN - first) * (D / 8); i += kPfThreads) {
        const int R = first + i / (D / 8), cc = i % (D / 8);
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vs_base + toff(R, cc)), "r"(0u) : "memory");
      }
      __syncthreads();
    }
    if (landed && t0 < warp_kv_end) {
      // S = Q K^T for 16 rows x 64 tokens
      float sacc[NB][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int nb2 = 0; nb2 < NB / 2; ++nb2) {
          const int R = nb2 * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int cc = ks * 2 + ((lane >> 3) & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(ks_base + toff(R, cc), b0, b1, b2, b3);
          mma_bf16(sacc[nb2 * 2], qf[ks], b0, b1);
          mma_bf16(sacc[nb2 * 2 + 1], qf[ks], b2, b3);
        }
      }
      const bool diagonal = t0 + kBN > ctx + wrow0 + 1 || t0 + kBN > kv_end;   // some (row, token) pair is masked
      float mx0 = m0, mx1 = m1;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v = sacc[nb][j] * sc;
          if (diagonal) {
            const int tk = t0 + nb * 8 + (lane & 3) * 2 + (j & 1);
            const int r = row0 + ((j >> 1) << 3);
            if (!(tk <= ctx + r && tk < kv_end)) v = -CUDART_INF_F;
          }
          sacc[nb][j] = v;
        }
        mx0 = fmaxf(mx0, fmaxf(sacc[nb][0], sacc[nb][1]));
        mx1 = fmaxf(mx1, fmaxf(sacc[nb][2], sacc[nb][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float c0 = (m0 == -CUDART_INF_F) ? 0.f : exp2f(m0 - mx0);
      const float c1 = (m1 == -CUDART_INF_F) ? 0.f : exp2f(m1 - mx1);
      const float e0 = (mx0 == -CUDART_INF_F) ? 0.f : mx0;
      const float e1 = (mx1 == -CUDART_INF_F) ? 0.f : mx1;
      m0 = mx0;
      m1 = mx1;
      float ps0 = 0.f, ps1 = 0.f;
      uint32_t pf[NB / 2][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const float p0 = exp2f(sacc[nb][0] - e0), p1 = exp2f(sacc[nb][1] - e0);
        const float p2 = exp2f(sacc[nb][2] - e1), p3 = exp2f(sacc[nb][3] - e1);
        ps0 += p0 + p1;
        ps1 += p2 + p3;
        pf[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
        pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      l0 = l0 * c0 + ps0;
      l1 = l1 * c1 + ps1;
      if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {
#pragma unroll
        for (int i = 0; i < DB; ++i) {
          o[i][0] *= c0;
          o[i][1] *= c0;
          o[i][2] *= c1;
          o[i][3] *= c1;
        }
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < NB / 2; ++kk) {
#pragma unroll
        for (int db2 = 0; db2 < DB / 2; ++db2) {
          const int R = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int cc = db2 * 2 + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(vs_base + toff(R, cc), b0, b1, b2, b3);
          mma_bf16(o[db2 * 2], pf[kk], b0, b1);
          mma_bf16(o[db2 * 2 + 1], pf[kk], b2, b3);
        }
      }
    }
    if (__syncthreads_or(!landed)) {   // every warp is done with the stage; CTA-uniform outcome of the waits
      timed_out = true;
      break;
    }
    if (threadIdx.x == 0 && t + kPfStages < n_tiles) {
      sm100::fence_proxy_async_smem();
      issue(t + kPfStages);
    }
  }
  if (timed_out) {
    if (threadIdx.x == 0 && a.status != nullptr) atomicCAS(a.status, 0u, 6u);
    __nanosleep(1000000);   // copies still in flight get a bounded chance to land before the CTA retires
    return;
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.out);
#pragma unroll
  for (int db = 0; db < DB; ++db) {
    const int d = db * 8 + (lane & 3) * 2;
    if (row0 < q_len)
      *reinterpret_cast<uint32_t*>(og + (static_cast<size_t>(q_base + row0) * a.q_heads + hq) * D + d) =
          pack_bf16(o[db][0] * i0, o[db][1] * i0);
    if (row0 + 8 < q_len)
      *reinterpret_cast<uint32_t*>(og + (static_cast<size_t>(q_base + row0 + 8) * a.q_heads + hq) * D + d) =
          pack_bf16(o[db][2] * i1, o[db][3] * i1);
  }
}

template <int D>
static int launch_prefill_tc(const XpPrefillAttnArgs& a, int G, cudaStream_t s) {
  CUtensorMap mk, mv;
  const uint64_t tokens = static_cast<uint64_t>(a.num_pages) * a.page_size;
  if (tmap::cache().get_kv(&mk, a.k_cache, tokens, a.kv_heads, D) != 0) return -20;
  if (tmap::cache().get_kv(&mv, a.v_cache, tokens, a.kv_heads, D) != 0) return -20;
  constexpr int kStage = 2 * (D / 64) * (kBN / 16) * 16 * 128;
  constexpr int kSmem = kPfStages * kStage + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(prefill_attn_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -21;
    attr_set = true;
  }
  const int rows_per_cta = 16 * (8 / G);
  dim3 grid((a.max_q_len + rows_per_cta - 1) / rows_per_cta, a.kv_heads, a.num_seqs);
  prefill_attn_tc_kernel<D><<<grid, kPfThreads, kSmem, s>>>(mk, mv, a, G, rows_per_cta);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

}  // namespace attn
}  // namespace xpool

extern "C" int xp_prefill_attn(const XpPrefillAttnArgs* a, void* stream) {
  using namespace xpool::attn;
  if (a->num_seqs <= 0 || a->max_q_len <= 0) return 0;
  if (a->q_heads % a->kv_heads != 0) return -11;
  if ((a->force_simple & 0xff) == 0) {
    const int rc = xp_prefill_attn_umma(a, stream);
    if (rc <= 0) return rc;   // launched (0) or failed (< 0); 1: shape outside the tcgen05 kernel
  }
  {
    const int G = a->q_heads / a->kv_heads;
    const bool tc_ok = (a->force_simple & 0xff) != 1 && a->num_pages > 0 && a->page_size >= 16 && (a->page_size & (a->page_size - 1)) == 0 &&
                       (G == 1 || G == 2 || G == 4 || G == 8) && (reinterpret_cast<uintptr_t>(a->q) & 3) == 0;
    if (tc_ok && a->head_dim == 128) return launch_prefill_tc<128>(*a, G, reinterpret_cast<cudaStream_t>(stream));
    if (tc_ok && a->head_dim == 64) return launch_prefill_tc<64>(*a, G, reinterpret_cast<cudaStream_t>(stream));
  }
  dim3 grid((a->max_q_len + kBM - 1) / kBM, a->q_heads, a->num_seqs);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (a->head_dim == 128) {
    const int smem = (kBM + 2 * kBN) * 128 * 2;
    static bool set = false;
    if (!set) {
      cudaFuncSetAttribute(prefill_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      set = true;
    }
    prefill_attn_kernel<128><<<grid, kPrefillThreads, smem, s>>>(*a);
  } else if (a->head_dim == 64) {
    const int smem = (kBM + 2 * kBN) * 64 * 2;
    prefill_attn_kernel<64><<<grid, kPrefillThreads, smem, s>>>(*a);
  } else {
    return -10;
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
