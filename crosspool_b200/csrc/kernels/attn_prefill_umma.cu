// Chunked-prefill attention on the Blackwell tensor cores: S = Q K^T and O += P V as tcgen05.mma with the
// accumulators in tensor memory, K/V and Q tiles staged by TMA (no multicast), causal, grouped-query, paged KV.
//
// One CTA serves the G query heads that share one KV head for 2 x (128 / G) consecutive query positions: two
// query tiles of 128 rows each (row = position * G + head), both multiplied against the same 64-token K/V tiles,
// so a K/V tile is fetched once for all heads of the group and the tensor pipe works on one tile while the
// softmax of the other runs.
//
//   warps 0-3   softmax of tile A: thread = query row = TMEM lane. Reads its S row with tcgen05.ld, masks the
//               diagonal, keeps a running maximum and sum, writes P (bf16) into swizzled shared memory as the A
//               operand of the PV product, rescales O in tensor memory only when the maximum grew by more than
//               2^8 (the accumulated sum carries the same stale maximum, so the quotient is exact), and at the
//               end normalises O and stores it.
//   warps 4-7   the same for tile B.
//   warp 8      TMA producer: Q tiles once, then a 3-stage ring of K/V tiles through the page table (128-byte
//               swizzle). With pages of at least 64 tokens one 4-D copy brings a whole K (or V) tile; with smaller
//               pages every 16 tokens and 64 dims are one copy. The lanes of the warp issue a stage's copies side
//               by side: a single thread issuing sixteen small copies per stage was what bounded the kernel.
//   warp 9      allocates tensor memory and issues every tcgen05.mma from one thread. S is double-buffered per
//               tile and issued one K/V tile ahead, in the order S_A(t+1), PV_A(t), S_B(t+1), PV_B(t).
//
// V is used where it lands (token-major rows of 64 dims) through an MN-major operand descriptor; no transpose.
// Tensor memory: S buffers 4 x 64 columns, O 2 x D columns (512 columns with D = 128).
// Every wait is bounded; a wait that runs out sets the abort word, the status word (7) and ends the CTA after a
// common barrier that frees the tensor memory.
#include <math_constants.h>

#include "xpool/api.h"
#include "xpool/sm100.cuh"
#include "xpool/tensormap.hpp"

namespace xpool {
namespace attn5 {

constexpr int kRows = 128;       // rows of one query tile (UMMA M)
constexpr int kBN = 64;          // cached tokens per K/V tile
constexpr int kStages = 3;
constexpr int kThreads = 320;
constexpr float kRescaleStep = 8.0f;   // log2 units
constexpr int kDefaultTS = 1;          // P through tensor memory unless bit 8 of force_simple asks for shared memory

struct __align__(8) Bars {
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2][2];
  uint64_t s_empty[2][2];
  uint64_t p_full[2];
  uint64_t pv_done[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

// Bounded wait that also gives up when another role of the CTA has aborted.
// `site` (1..255) names the wait in the status detail word when it is the one that runs out.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, Bars* b, uint32_t site) {
  if (sm100::mbar_try_wait(bar, parity)) return true;
  const uint64_t deadline = sm100::global_timer_ns() + sm100::kPipelineWaitNs;
  uint32_t spins = 0;
  while (!sm100::mbar_try_wait(bar, parity)) {
    if ((++spins & 0xffu) == 0) {
      if (b->abort_flag != 0) return false;
      if (sm100::global_timer_ns() > deadline) {
        b->abort_flag = site;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, bool kTS>
__global__ void __launch_bounds__(kThreads, 1)
prefill_attn_umma_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_k3,
                         const __grid_constant__ CUtensorMap tmap_v3, XpPrefillAttnArgs a, int G, int g_shift,
                         int box_tokens) {
  constexpr int kHalves = D / 64;                 // 64-dim (128-byte) column blocks of a row
  constexpr int kQHalf = kRows * 128;             // one 64-dim block of a query tile
  constexpr int kQTile = kHalves * kQHalf;
  constexpr int kKVHalf = kBN * 128;              // one 64-dim block of a K (or V) tile
  constexpr int kKVTile = kHalves * kKVHalf;
  constexpr int kStage = 2 * kKVTile;             // K then V
  constexpr int kPTile = kRows * 128;             // P: 128 rows x 64 tokens bf16
  constexpr uint32_t kTmemCols = (4 * kBN + 2 * D) <= 256 ? 256 : 512;
  constexpr uint32_t kOCol = 4 * kBN;             // O_A at 256, O_B at 256 + D
  extern __shared__ uint8_t smem_dyn[];
  __shared__ Bars bars;

  const int np = kRows >> g_shift;                // query positions per tile
  // blocks are dispatched x-fastest: (head, sequence) vary fastest and the query tile slowest, so that the tiles with
  // the longest key range of every head and sequence start first and the short ones fill the tail
  const int hk = blockIdx.x, seq = blockIdx.y, qt = static_cast<int>(gridDim.z) - 1 - static_cast<int>(blockIdx.z);
  const int q_len = a.q_lens[seq];
  const int q0 = qt * 2 * np;                     // first position of the CTA (longest tiles are dispatched first)
  if (q0 >= q_len) return;
  const int ctx = a.ctx_lens[seq];
  const int q_base = a.q_starts[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (sm100::smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t q_s = base, kv_s = base + 2 * kQTile, p_s = kv_s + kStages * kStage;
  const bool act_b = q0 + np < q_len;             // tile B holds at least one real row
  const int kv_end = ctx + min(q_len, q0 + 2 * np);            // causal bound of the CTA
  const int n_tiles = (kv_end + kBN - 1) / kBN;
  const int n_a = min(n_tiles, (ctx + min(q_len, q0 + np) + kBN - 1) / kBN);   // tiles that tile A can see

  if (threadIdx.x == 0) {
    sm100::mbar_init(&bars.q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      sm100::mbar_init(&bars.kv_full[s], 1);
      sm100::mbar_init(&bars.kv_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      for (int bf = 0; bf < 2; ++bf) {
        sm100::mbar_init(&bars.s_full[x][bf], 1);
        sm100::mbar_init(&bars.s_empty[x][bf], 4);
      }
      sm100::mbar_init(&bars.p_full[x], 4);
      sm100::mbar_init(&bars.pv_done[x], 1);
    }
    bars.abort_flag = 0;
    sm100::mbar_fence_init();
    sm100::fence_proxy_async_smem();
  }
  if (warp == 9) {
    sm100::tmem_alloc(&bars.tmem_base, kTmemCols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::tc_fence_after_sync();
  const uint32_t tmem = bars.tmem_base;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    // One copy per (K or V, box of box_tokens tokens); the lanes of the warp issue a stage's copies side by side,
    // each after its own page-table lookup.
    if (lane == 0) {
      sm100::tma_prefetch_desc(&tmap_q);
      sm100::tma_prefetch_desc(&tmap_k);
      sm100::tma_prefetch_desc(&tmap_v);
      sm100::mbar_arrive_expect_tx(&bars.q_full, 2 * kQTile);
    }
    __syncwarp();
    if (lane < 2 * kHalves) {
      const int x = lane / kHalves, h = lane % kHalves;
      sm100::tma_load_3d_addr(q_s + x * kQTile + h * kQHalf, &tmap_q, sm100::smem_u32(&bars.q_full), h * 64, hk * G,
                              q_base + q0 + x * np);
    }
    const int page_shift = 31 - __clz(a.page_size);
    const int page_mask = a.page_size - 1;
    const int* table = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
    const int boxes = kBN / box_tokens;            // boxes per tile and tensor
    const int box_bytes = box_tokens * 128;        // one 64-dim block of a box
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kStages;
      if (t >= kStages && !__all_sync(0xffffffffu, wait_bar(&bars.kv_empty[s], ((t / kStages) - 1) & 1, &bars, 1))) break;
      if (lane == 0) sm100::mbar_arrive_expect_tx(&bars.kv_full[s], kStage);
      __syncwarp();
      if (boxes == 1) {
        if (lane < 2) {
          int tk = t * kBN;
          if (tk >= kv_end) tk = (kv_end - 1) & ~(kBN - 1);
          const int tok = (table[tk >> page_shift] << page_shift) + (tk & page_mask);
          sm100::tma_load_4d_addr(kv_s + s * kStage + lane * kKVTile, lane ? &tmap_v : &tmap_k,
                                  sm100::smem_u32(&bars.kv_full[s]), 0, tok, 0, hk);
        }
      } else if (lane < 2 * boxes * kHalves) {
        const int h = lane % kHalves, is_v = (lane / kHalves) & 1, j = lane / (2 * kHalves);
        int tk = t * kBN + j * box_tokens;
        if (tk >= kv_end) tk = (kv_end - 1) & ~(box_tokens - 1);   // boxes past the end repeat the last valid one (masked)
        const int tok = (table[tk >> page_shift] << page_shift) + (tk & page_mask);
        sm100::tma_load_3d_addr(kv_s + s * kStage + is_v * kKVTile + h * kKVHalf + j * box_bytes, is_v ? &tmap_v3 : &tmap_k3,
                                sm100::smem_u32(&bars.kv_full[s]), h * 64, hk, tok);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = sm100::umma_idesc_bf16(kRows, kBN);
      const uint32_t idesc_o = sm100::umma_idesc_bf16_bmn(kRows, D);
      auto issue_s = [&](int x, int t) {       // S_x(t) = Q_x K(t)^T into buffer t & 1
        const int s = t % kStages, bf = t & 1;
        const uint32_t d = tmem + static_cast<uint32_t>((x * 2 + bf) * kBN);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t da = sm100::umma_desc_sw128(q_s + x * kQTile + (ks >> 2) * kQHalf) + (ks & 3) * 2;
          const uint64_t db = sm100::umma_desc_sw128(kv_s + s * kStage + (ks >> 2) * kKVHalf) + (ks & 3) * 2;
          sm100::umma_bf16(d, da, db, idesc_s, ks > 0 ? 1u : 0u);
        }
        sm100::umma_commit(&bars.s_full[x][bf]);
      };
      auto issue_pv = [&](int x, int t) {      // O_x (+)= P_x V(t)
        const int s = t % kStages;
        const uint32_t d = tmem + kOCol + static_cast<uint32_t>(x * D);
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          const uint64_t da = sm100::umma_desc_sw128(p_s + x * kPTile) + kk * 2;
          const uint64_t db = sm100::umma_desc_mn_sw128(kv_s + s * kStage + kKVTile + kk * 2048, kKVHalf, 1024);
          if constexpr (kTS) {
            // P(t) sits in the first 32 columns of the S buffer it was computed from, 8 columns per K step
            sm100::umma_bf16_ts(d, tmem + static_cast<uint32_t>((x * 2 + (t & 1)) * kBN + kk * 8), db, idesc_o,
                                (t > 0 || kk > 0) ? 1u : 0u);
          } else {
            sm100::umma_bf16(d, da, db, idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
          }
        }
        sm100::umma_commit(&bars.pv_done[x]);
      };
      bool ok = wait_bar(&bars.q_full, 0, &bars, 2) && wait_bar(&bars.kv_full[0], 0, &bars, 3);
      if (ok) {
        sm100::tc_fence_after_sync();
        issue_s(0, 0);
        if (act_b) issue_s(1, 0);
      }
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int t1 = t + 1;
        const bool next = t1 < n_tiles;
        if (next) ok = wait_bar(&bars.kv_full[t1 % kStages], (t1 / kStages) & 1, &bars, 4);
        // tile A
        if (ok && next && t1 < n_a) {
          if (!kTS && t1 >= 2) ok = wait_bar(&bars.s_empty[0][t1 & 1], ((t1 >> 1) - 1) & 1, &bars, 5);
          if (ok) {
            sm100::tc_fence_after_sync();
            issue_s(0, t1);
          }
        }
        if (ok && t < n_a) {
          ok = wait_bar(&bars.p_full[0], t & 1, &bars, 6);
          if (ok) {
            sm100::tc_fence_after_sync();
            issue_pv(0, t);
          }
        }
        // tile B
        if (ok && act_b) {
          if (next) {
            if (!kTS && t1 >= 2) ok = wait_bar(&bars.s_empty[1][t1 & 1], ((t1 >> 1) - 1) & 1, &bars, 7);
            if (ok) {
              sm100::tc_fence_after_sync();
              issue_s(1, t1);
            }
          }
          if (ok) ok = wait_bar(&bars.p_full[1], t & 1, &bars, 8);
          if (ok) {
            sm100::tc_fence_after_sync();
            issue_pv(1, t);
          }
        }
        if (ok) sm100::umma_commit(&bars.kv_empty[t % kStages]);   // every MMA that reads the stage has been issued
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 0-7)
    const int x = warp >> 2;                          // tile
    const int row = (warp & 3) * 32 + lane;           // row of the tile = TMEM lane
    const int pos = q0 + x * np + (row >> g_shift);   // query position inside the chunk
    const int hq = hk * G + (row & (G - 1));
    const bool tile_on = x == 0 || act_b;
    const int my_tiles = x == 0 ? n_a : n_tiles;
    const int limit = min(ctx + pos, kv_end - 1);     // last visible cache position of this row
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t o_t = tmem + lane_off + kOCol + static_cast<uint32_t>(x * D);
    const uint32_t p_row = p_s + x * kPTile + row * 128;
    const float sc2 = a.scale * 1.4426950408889634f;
    float m_used = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    if (tile_on) {
      for (int t = 0; t < my_tiles; ++t) {
        const int bf = t & 1;
        ok = __all_sync(0xffffffffu, wait_bar(&bars.s_full[x][bf], (t >> 1) & 1, &bars, 9));
        if (!ok) break;
        sm100::tc_fence_after_sync();
        uint32_t sv[kBN];
        const uint32_t s_t = tmem + lane_off + static_cast<uint32_t>((x * 2 + bf) * kBN);
        sm100::tmem_ld32_issue(s_t, sv);
        sm100::tmem_ld32_issue(s_t + 32, sv + 32);
        sm100::tmem_ld_wait_all(sv);
        sm100::tmem_ld_wait_all(sv + 32);
        if constexpr (!kTS) {       // with P in tensor memory the buffer is free only after the PV product (issue order)
          sm100::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) sm100::mbar_arrive(&bars.s_empty[x][bf]);
        }

        const int nvis = min(kBN, max(0, limit - t * kBN + 1));   // visible tokens of this tile for this row
        if (nvis < kBN) {
#pragma unroll
          for (int j = 0; j < kBN; ++j)
            if (j >= nvis) sv[j] = 0xff800000u;       // -inf: selected, never computed with (the slot may hold NaN)
        }
        // four independent chains of three-input maxima: a serial chain over 64 values costs its latency 64 times
        float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int j = 0; j < kBN; j += 8) {
#pragma unroll
          for (int c = 0; c < 4; ++c) mx4[c] = max3(mx4[c], __uint_as_float(sv[j + 2 * c]), __uint_as_float(sv[j + 2 * c + 1]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_new = mx * sc2;
        float factor = 1.f;
        if (m_new > m_used + kRescaleStep || m_used == -CUDART_INF_F) {
          if (m_new != -CUDART_INF_F) {
            factor = m_used == -CUDART_INF_F ? 0.f : sm100::ex2_approx(m_used - m_new);
            m_used = m_new;
          }
        }
        const float m_sub = m_used == -CUDART_INF_F ? 0.f : m_used;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[kBN / 2];
#pragma unroll
        for (int j = 0; j < kBN; j += 2) {
          const float p0 = sm100::ex2_approx(fmaf(__uint_as_float(sv[j]), sc2, -m_sub));
          const float p1 = sm100::ex2_approx(fmaf(__uint_as_float(sv[j + 1]), sc2, -m_sub));
          sum4[(j >> 1) & 3] += p0 + p1;
          pk[j >> 1] = pack2(p0, p1);
        }
        l = l * factor + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        const bool rescale = __any_sync(0xffffffffu, factor != 1.f);
        if (t > 0 && (!kTS || rescale)) {
          // the previous PV product must have retired: it accumulates into O (and reads the shared-memory P buffer)
          ok = __all_sync(0xffffffffu, wait_bar(&bars.pv_done[x], (t - 1) & 1, &bars, 10));
          if (!ok) break;
          if (rescale) {
            sm100::tc_fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
              uint32_t ov[32];
              sm100::tmem_ld32_issue(o_t + c, ov);
              sm100::tmem_ld_wait_all(ov);
#pragma unroll
              for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * factor);
              sm100::tmem_st32(o_t + c, ov);
            }
            sm100::tmem_st_wait();
            sm100::tc_fence_before_sync();
          }
        }
        if constexpr (kTS) {
          // P row as the tensor core's A operand: 32 columns of two bf16 each, over the start of the S buffer
          sm100::tmem_st32(s_t, pk);
        }
        // P row: 8 chunks of 8 tokens, 16-byte chunks XOR-swizzled by the row like a TMA-written tile
#pragma unroll
        for (int c = 0; c < (kTS ? 0 : kBN / 8); ++c) {
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + (((c ^ (row & 7))) << 4)), "r"(pk[c * 4]),
                       "r"(pk[c * 4 + 1]), "r"(pk[c * 4 + 2]), "r"(pk[c * 4 + 3])
                       : "memory");
        }
        const bool v_tail = (x == 0 || t >= n_a) && t * kBN + kBN > kv_end;
        if (v_tail) {
          // cache slots past the sequence end may hold anything: zero those V rows (probability 0 x NaN).
          // Tile A's PV product is issued before tile B's and both read this stage, so tile A's threads do it
          // on the tiles that tile A visits, tile B's on the rest.
          const uint32_t v_s = kv_s + (t % kStages) * kStage + kKVTile;
          const int first = kv_end - t * kBN;
          for (int i = row; i < (kBN - first) * (D / 8); i += kRows) {
            const int R = first + i / (D / 8), cc = i % (D / 8);
            const uint32_t off = (cc >> 3) * kKVHalf + R * 128 + (((cc & 7) ^ (R & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(v_s + off), "r"(0u) : "memory");
          }
        }
        if (!kTS || v_tail) sm100::fence_proxy_async_smem();   // this thread's P (and V) stores, for the tensor core's reads
        if constexpr (kTS) {
          sm100::tmem_st_wait();
          sm100::tc_fence_before_sync();
          // Every phase of pv_done is consumed in order, also when no rescale needed it: a parity wait tells phase
          // t - 1 from phase t + 1 only if none is skipped. PV(t-1) was issued a whole tile ago, so this returns at
          // once; it must come before the arrive below, after which PV(t) may complete and flip the parity again.
          if (t > 0 && !rescale) {
            ok = __all_sync(0xffffffffu, wait_bar(&bars.pv_done[x], (t - 1) & 1, &bars, 12));
            if (!ok) break;
          }
        }
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&bars.p_full[x]);
      }
      if (ok && my_tiles > 0) ok = __all_sync(0xffffffffu, wait_bar(&bars.pv_done[x], (my_tiles - 1) & 1, &bars, 11));
      if (ok) {
        sm100::tc_fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.out) + (static_cast<size_t>(q_base + pos) * a.q_heads + hq) * D;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t ov[32];
          sm100::tmem_ld32_issue(o_t + c, ov);
          sm100::tmem_ld_wait_all(ov);
          if (pos < q_len) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              v.x = pack2(__uint_as_float(ov[j]) * inv, __uint_as_float(ov[j + 1]) * inv);
              v.y = pack2(__uint_as_float(ov[j + 2]) * inv, __uint_as_float(ov[j + 3]) * inv);
              v.z = pack2(__uint_as_float(ov[j + 4]) * inv, __uint_as_float(ov[j + 5]) * inv);
              v.w = pack2(__uint_as_float(ov[j + 6]) * inv, __uint_as_float(ov[j + 7]) * inv);
              *reinterpret_cast<uint4*>(og + c + j) = v;
            }
          }
        }
      }
    }
  }
  // ------------------------------------------------------------------ common exit
  sm100::tc_fence_before_sync();
  __syncthreads();
  if (bars.abort_flag != 0) {
    if (threadIdx.x == 0 && a.status != nullptr && atomicCAS(a.status, 0u, 7u) == 0u) {
      // detail words of the first CTA that gave up: the wait that ran out, and where the CTA was
      a.status[1] = bars.abort_flag;
      a.status[2] = (blockIdx.z << 20) | (blockIdx.y << 8) | blockIdx.x;
      a.status[3] = static_cast<uint32_t>(n_tiles);
    }
    __nanosleep(1000000);   // copies still in flight get a bounded chance to land before the CTA retires
  }
  if (warp == 9) {
    sm100::tc_fence_after_sync();
    sm100::tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, bool kTS>
static int launch(const XpPrefillAttnArgs& a, int G, cudaStream_t s) {
  CUtensorMap mq, mk, mv, mk3, mv3;
  const uint64_t tokens = static_cast<uint64_t>(a.num_pages) * a.page_size;
  int g_shift = 0;
  while ((1 << g_shift) < G) ++g_shift;
  const int np = kRows >> g_shift;
  // pages of 64 tokens or more: one copy brings a whole K (or V) tile; smaller pages: one copy per page and 64 dims
  const int box_tokens = a.page_size >= kBN ? kBN : 16;
  if (tmap::cache().get_kv4(&mk, a.k_cache, tokens, a.kv_heads, D, kBN) != 0) return -20;
  if (tmap::cache().get_kv4(&mv, a.v_cache, tokens, a.kv_heads, D, kBN) != 0) return -20;
  if (tmap::cache().get_kv(&mk3, a.k_cache, tokens, a.kv_heads, D) != 0) return -20;
  if (tmap::cache().get_kv(&mv3, a.v_cache, tokens, a.kv_heads, D) != 0) return -20;
  if (tmap::cache().get_q(&mq, a.q, static_cast<uint64_t>(a.total_q), a.q_heads, D, G, np) != 0) return -20;
  constexpr int kSmem = 2 * (D / 64) * kRows * 128 + kStages * 2 * (D / 64) * kBN * 128 + 2 * kRows * 128 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(prefill_attn_umma_kernel<D, kTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
      return -21;
    attr_set = true;
  }
  dim3 grid(a.kv_heads, a.num_seqs, (a.max_q_len + 2 * np - 1) / (2 * np));
  prefill_attn_umma_kernel<D, kTS><<<grid, kThreads, kSmem, s>>>(mq, mk, mv, mk3, mv3, a, G, g_shift, box_tokens);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

}  // namespace attn5
}  // namespace xpool

// Returns 1 when the arguments are outside what the tcgen05 kernel covers (the caller then takes another kernel),
// 0 when it was launched, a negative code on failure.
extern "C" int xp_prefill_attn_umma(const XpPrefillAttnArgs* a, void* stream) {
  using namespace xpool::attn5;
  if (a->num_seqs <= 0 || a->max_q_len <= 0) return 0;
  if (a->q_heads % a->kv_heads != 0) return -11;
  const int G = a->q_heads / a->kv_heads;
  const bool ok = a->num_pages > 0 && a->total_q > 0 && a->page_size >= 16 && (a->page_size & (a->page_size - 1)) == 0 &&
                  (G == 1 || G == 2 || G == 4 || G == 8 || G == 16) && (reinterpret_cast<uintptr_t>(a->q) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(a->out) & 15) == 0;
  if (!ok) return 1;
  // P (the probabilities) reaches the second product through tensor memory; bit 8 of force_simple selects the
  // form that stages P in shared memory instead
  const bool ts = ((a->force_simple >> 8) & 1) != kDefaultTS;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->head_dim == 128) return ts ? launch<128, true>(*a, G, s) : launch<128, false>(*a, G, s);
  if (a->head_dim == 64) return ts ? launch<64, true>(*a, G, s) : launch<64, false>(*a, G, s);
  return 1;
}
