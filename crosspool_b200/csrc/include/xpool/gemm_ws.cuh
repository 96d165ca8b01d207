// Weight-stationary tcgen05 GEMM tile engine for sm_100a.
//
// Computes Y[r, f] = sum_k X[r, k] * W[f, k]  (torch.nn.Linear layout) with the
// WEIGHT rows on the tensor core's M axis (always a full 128-row tile) and the
// activation rows on its N axis (16..256, chosen per call). Decode batches of a
// few rows and prefill chunks of thousands of rows go through the same code;
// the epilogue thread that owns TMEM lane `f` writes consecutive features, so
// global stores are coalesced without a shared-memory transpose.
//
// Roles inside one 192-thread CTA:
//   warp 0      TMA producer (one elected thread), non-multicast 2-D tile loads
//   warp 1      TMEM allocation + tcgen05.mma issue (one elected thread)
//   warps 2..5  epilogue: tcgen05.ld -> registers -> fused epilogue -> global
// Accumulators are double-buffered in TMEM when they fit, so the epilogue of one
// tile overlaps the main loop of the next (the CTA loops over tiles).
//
// The "dual" form multiplies one activation tile with a gate tile and an up
// tile of the same weight tensor and applies SwiGLU in the epilogue; this
// replaces the reference's matmul + activation kernels
// (src/xpool/runtime/ffnagent/operators/{linear,activation,dense}.py).
#pragma once

#include "xpool/sm100.cuh"

namespace xpool {
namespace gemm {

constexpr int kTileM = 128;    // weight rows per tile (UMMA M)
constexpr int kTileK = 64;     // bf16 elements per K block = one 128-byte swizzle row
constexpr int kMaxBnF8 = 64;   // widest activation tile of the block-scaled fp8 path (accumulators live in registers)
constexpr int kUmmaK = 16;     // K per tcgen05.mma for 16-bit inputs
constexpr int kMaxStages = 12;
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;

enum Epilogue : int {
  kEpiStore = 0,     // out = acc (+ bias)
  kEpiSwiglu = 1,    // dual: out = silu(round(g)) * round(u)
  kEpiResidual = 2,  // out = round(acc) + resid
  kEpiStoreF32 = 3,  // fp32 out = acc (+ bias)
};

enum Status : uint32_t {
  kOk = 0,
  kTimeoutProducer = 1,
  kTimeoutMma = 2,
  kTimeoutEpilogue = 3,
  kTimeoutFlag = 4,
  kBadArgument = 5,
};

// One GEMM problem. All pointers are device pointers valid on the executing GPU
// (out / resid may be peer memory; they are only touched with plain stores and
// loads, never by TMA).
struct Problem {
  const CUtensorMap* tmap_w;  // [n_rows_total, k], box {64, 128}
  const CUtensorMap* tmap_x;  // [rows, k], box {64, bn}
  void* out;                  // [rows, ld_out]
  const void* resid;          // [rows, ld_resid] bf16 or null
  const float* bias;          // [n_out] or null
  float* ws;                  // split-K workspace or null
  uint32_t* counters;         // one per (m, n) tile, zero between calls
  int n_out;                  // features produced (multiple of 128)
  int k;                      // multiple of 64
  int rows;                   // live activation rows
  int ld_out;
  int ld_resid;
  int bn;                     // activation rows per tile: 16, 32, 64, 128 or 256
  int splits;                 // split-K factor (>= 1)
  int epilogue;               // Epilogue
  int dual;                   // 1: gate rows [0, n_out), up rows [up_offset, up_offset + n_out)
  int up_offset;
  int w_evict_first;          // stream weights through L2
  int w_tiled;                // weights stored as contiguous 128x64 tiles (see tile_weight)
  float gate_limit;           // > 0: clamp gate from above and up to [-limit, limit]
  float up_add;               // added to up before the product (0 for plain SwiGLU)
  float act_alpha;            // 0: silu(g); else g * sigmoid(alpha * g)
  // Grouped (mixture-of-experts) form: tiles come from a device table of
  // {group, feature tile start, first row, row end}; group g uses weight rows
  // [g * w_rows_per_group, ...). Activation rows of a group are contiguous.
  const int4* tile_table;
  const int* n_tiles;
  int w_rows_per_group;
  // Block-scaled fp8 (e4m3) operands: a K block is 128 elements (still one 128-byte swizzle row);
  // weights carry one fp32 scale per 128 x 128 block ([rows / 128][k / 128]), activations one per
  // row and K block, stored transposed ([k / 128][ld_xscale]) so that a tile's scales are contiguous.
  int kblk;                // elements per K block: 64 (bf16) or 128 (fp8)
  int fp8;
  const float* w_scale;
  const float* x_scale;
  int ld_xscale;
};

struct SmemLayout {
  int stages;
  int a_bytes;      // per stage, all A tiles
  int b_bytes;      // per stage
  int stage_bytes;
  int total_bytes;  // including barriers and alignment slack
};

__host__ __device__ inline SmemLayout smem_layout(int bn, int dual, int budget_bytes) {
  SmemLayout s;
  s.a_bytes = kTileM * kTileK * 2 * (dual ? 2 : 1);
  s.b_bytes = bn * kTileK * 2;
  // B tiles start on 1024-byte boundaries (128-byte swizzle atoms).
  int b_pad = (s.b_bytes + 1023) / 1024 * 1024;
  s.stage_bytes = s.a_bytes + b_pad;
  int st = (budget_bytes - 2048) / s.stage_bytes;
  if (st > kMaxStages) st = kMaxStages;
  if (st < 2) st = 2;
  s.stages = st;
  s.total_bytes = st * s.stage_bytes + 1024 /*align slack*/ + 512 /*barriers*/;
  return s;
}

struct Barriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t bcast;
  uint32_t pad;
};

__device__ __forceinline__ void record_status(uint32_t* status, uint32_t code) {
  if (status != nullptr) atomicCAS(status, 0u, code);
}

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Pipeline position carried across tiles by each role.
struct PipeState {
  uint32_t stage = 0;
  uint32_t phase = 0;
  uint32_t acc = 0;
  uint32_t acc_phase = 0;
  __device__ __forceinline__ void advance(uint32_t stages) {
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
    }
  }
  __device__ __forceinline__ void advance_acc(uint32_t nacc) {
    if (++acc == nacc) {
      acc = 0;
      acc_phase ^= 1;
    }
  }
};

struct TileCoord {
  int m0;     // first weight row / feature
  int n0;     // first activation row
  int split;  // split-K index
  int mn;     // linear (m, n) tile index
  int kb0;    // first K block
  int kbn;    // number of K blocks
  int w_row0; // first weight row in the weight tensor (differs from m0 for grouped problems)
  int row_end;  // activation rows >= row_end are not stored
};

__device__ __forceinline__ int tiles_m(const Problem& p) { return p.n_out / kTileM; }
__device__ __forceinline__ int tiles_n(const Problem& p) { return (p.rows + p.bn - 1) / p.bn; }
__device__ __forceinline__ int tile_count(const Problem& p) {
  if (p.tile_table != nullptr) return *p.n_tiles;
  return tiles_m(p) * tiles_n(p) * p.splits;
}

__device__ __forceinline__ TileCoord tile_coord(const Problem& p, int t) {
  TileCoord c;
  if (p.tile_table != nullptr) {
    const int4 e = p.tile_table[t];
    c.m0 = e.y;
    c.n0 = e.z;
    c.row_end = e.w;
    c.w_row0 = e.x * p.w_rows_per_group + e.y;
    c.split = 0;
    c.mn = t;
    c.kb0 = 0;
    c.kbn = p.k / p.kblk;
    return c;
  }
  int tm = tiles_m(p);
  c.split = t % p.splits;
  int mn = t / p.splits;
  c.mn = mn;
  c.m0 = (mn % tm) * kTileM;
  c.n0 = (mn / tm) * p.bn;
  int kb_total = p.k / p.kblk;
  int per = (kb_total + p.splits - 1) / p.splits;
  c.kb0 = c.split * per;
  int end = c.kb0 + per;
  if (end > kb_total) end = kb_total;
  c.kbn = end > c.kb0 ? end - c.kb0 : 0;
  c.w_row0 = c.m0;
  c.row_end = p.rows;
  return c;
}

// ---------------------------------------------------------------- producer
//
// The producer and the MMA issuer are single threads; nothing hides the latency
// of their scalar instructions, so the per-K-block bookkeeping is kept to a few
// adds: shared-memory addresses, barrier addresses, TMA coordinates and UMMA
// descriptors all advance incrementally (a tcgen05.mma of N <= 32 retires in
// about 45 cycles, four of them per K block).

__device__ __forceinline__ bool produce_tile(const Problem& p, const TileCoord& c,
                                             const SmemLayout& L, uint8_t* tiles, Barriers* bar,
                                             PipeState& st, uint64_t deadline) {
  const uint64_t pol_w = p.w_evict_first ? sm100::l2_policy_evict_first() : sm100::l2_policy_evict_normal();
  const uint64_t pol_x = sm100::l2_policy_evict_last();
  const uint32_t tx = static_cast<uint32_t>(L.a_bytes + L.b_bytes);
  const uint32_t tiles_addr = sm100::smem_u32(tiles);
  const uint32_t full0 = sm100::smem_u32(&bar->full[0]);
  const uint32_t empty0 = sm100::smem_u32(&bar->empty[0]);
  const uint32_t stage_bytes = static_cast<uint32_t>(L.stage_bytes);
  const uint32_t a_bytes = static_cast<uint32_t>(L.a_bytes);
  const uint32_t stages = static_cast<uint32_t>(L.stages);
  const uint64_t tw = reinterpret_cast<uint64_t>(p.tmap_w);
  const uint64_t tx_map = reinterpret_cast<uint64_t>(p.tmap_x);
  // Row-major weights: box at (k, row). Tiled weights: every 128x64 tile is one
  // contiguous 16 KB run, tile index = m_tile * k_tiles + k_tile.
  const int kb_total = p.k / p.kblk;
  int wc0, wc1, uc1, dwc0, dwc1;
  if (p.w_tiled) {
    wc0 = 0;
    dwc0 = 0;
    wc1 = ((c.w_row0 / kTileM) * kb_total + c.kb0) * kTileM;
    uc1 = (((p.up_offset + c.w_row0) / kTileM) * kb_total + c.kb0) * kTileM;
    dwc1 = kTileM;
  } else {
    wc0 = c.kb0 * p.kblk;
    dwc0 = p.kblk;
    wc1 = c.w_row0;
    uc1 = p.up_offset + c.w_row0;
    dwc1 = 0;
  }
  int xc0 = c.kb0 * p.kblk;
  uint32_t stage = st.stage, phase = st.phase;
  uint32_t a_addr = tiles_addr + stage * stage_bytes;
  const bool dual = p.dual != 0;
  for (int i = 0; i < c.kbn; ++i) {
    const uint32_t full = full0 + stage * 8, empty = empty0 + stage * 8;
    if (!sm100::mbar_try_wait_addr(empty, phase ^ 1) &&
        !sm100::mbar_wait_addr(empty, phase ^ 1, deadline)) {
      st.stage = stage;
      st.phase = phase;
      return false;
    }
    sm100::mbar_arrive_expect_tx_addr(full, tx);
    sm100::tma_load_2d_addr(a_addr, tw, full, wc0, wc1, pol_w);
    if (dual) sm100::tma_load_2d_addr(a_addr + kTileM * kTileK * 2, tw, full, wc0, uc1, pol_w);
    sm100::tma_load_2d_addr(a_addr + a_bytes, tx_map, full, xc0, c.n0, pol_x);
    wc0 += dwc0;
    wc1 += dwc1;
    uc1 += dwc1;
    xc0 += p.kblk;
    a_addr += stage_bytes;
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
      a_addr = tiles_addr;
    }
  }
  st.stage = stage;
  st.phase = phase;
  return true;
}

// After a failed wait: give loads still in flight a bounded time to land so that
// nothing writes this CTA's shared memory after it has exited.
__device__ __forceinline__ void producer_drain(const SmemLayout& L, Barriers* bar,
                                               const PipeState& st) {
  uint64_t deadline = sm100::global_timer_ns() + 2000000ull;  // 2 ms
  for (uint32_t s = 0; s < static_cast<uint32_t>(L.stages); ++s) {
    // Stages below the cursor were armed in the current phase, the others in the
    // previous one (a never-armed barrier passes the previous-phase test at once).
    const uint32_t parity = s < st.stage ? st.phase : (st.phase ^ 1);
    if (!sm100::mbar_wait(&bar->full[s], parity, deadline)) break;
  }
}

// ---------------------------------------------------------------- MMA issuer

__device__ __forceinline__ bool mma_tile_f8(const Problem& p, const TileCoord& c, const SmemLayout& L, uint8_t* tiles,
                                            Barriers* bar, PipeState& st, int nacc, uint64_t deadline);

__device__ __forceinline__ bool mma_tile(const Problem& p, const TileCoord& c, const SmemLayout& L,
                                         uint8_t* tiles, Barriers* bar, PipeState& st, int nacc,
                                         uint64_t deadline) {
  if (p.fp8) return mma_tile_f8(p, c, L, tiles, bar, st, nacc, deadline);
  const uint32_t acc_w = static_cast<uint32_t>(p.bn * (p.dual ? 2 : 1));
  const uint32_t tmem_g = bar->tmem_base + st.acc * acc_w;
  const uint32_t tmem_u = tmem_g + p.bn;
  const uint32_t idesc = sm100::umma_idesc_bf16(kTileM, static_cast<uint32_t>(p.bn));
  if (!sm100::mbar_wait(&bar->acc_empty[st.acc], st.acc_phase ^ 1, deadline)) return false;
  sm100::tc_fence_after_sync();
  const uint32_t tiles_addr = sm100::smem_u32(tiles);
  const uint32_t full0 = sm100::smem_u32(&bar->full[0]);
  const uint32_t empty0 = sm100::smem_u32(&bar->empty[0]);
  const uint32_t stages = static_cast<uint32_t>(L.stages);
  // descriptors of stage 0; a stage further adds stage_bytes / 16 to the address field
  const uint64_t da0 = sm100::umma_desc_sw128(tiles_addr);
  const uint64_t du0 = sm100::umma_desc_sw128(tiles_addr + kTileM * kTileK * 2);
  const uint64_t db0 = sm100::umma_desc_sw128(tiles_addr + L.a_bytes);
  const uint64_t dstage = static_cast<uint64_t>(L.stage_bytes >> 4);
  uint32_t stage = st.stage, phase = st.phase;
  uint64_t da = da0 + stage * dstage, du = du0 + stage * dstage, db = db0 + stage * dstage;
  const bool dual = p.dual != 0;
  uint32_t accum = 0;
  for (int i = 0; i < c.kbn; ++i) {
    const uint32_t full = full0 + stage * 8;
    if (!sm100::mbar_try_wait_addr(full, phase) && !sm100::mbar_wait_addr(full, phase, deadline)) {
      st.stage = stage;
      st.phase = phase;
      return false;
    }
    sm100::tc_fence_after_sync();
    // 32 bytes (two 16-byte units) per UMMA K step inside the 128-byte swizzle row
    sm100::umma_bf16(tmem_g, da, db, idesc, accum);
    if (dual) sm100::umma_bf16(tmem_u, du, db, idesc, accum);
    sm100::umma_bf16(tmem_g, da + 2, db + 2, idesc, 1u);
    if (dual) sm100::umma_bf16(tmem_u, du + 2, db + 2, idesc, 1u);
    sm100::umma_bf16(tmem_g, da + 4, db + 4, idesc, 1u);
    if (dual) sm100::umma_bf16(tmem_u, du + 4, db + 4, idesc, 1u);
    sm100::umma_bf16(tmem_g, da + 6, db + 6, idesc, 1u);
    if (dual) sm100::umma_bf16(tmem_u, du + 6, db + 6, idesc, 1u);
    accum = 1;
    sm100::umma_commit_addr(empty0 + stage * 8);  // frees the stage when these MMAs retire
    da += dstage;
    du += dstage;
    db += dstage;
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
      da = da0;
      du = du0;
      db = db0;
    }
  }
  st.stage = stage;
  st.phase = phase;
  sm100::umma_commit(&bar->acc_full[st.acc]);
  st.advance_acc(nacc);
  return true;
}

// Block-scaled fp8: every K block (one scale block) is accumulated on its own into one of the two
// TMEM buffers and handed to the epilogue warps, which scale it and keep the running sum in
// registers; the buffers alternate per K block instead of per tile.
__device__ __forceinline__ bool mma_tile_f8(const Problem& p, const TileCoord& c, const SmemLayout& L,
                                            uint8_t* tiles, Barriers* bar, PipeState& st, int nacc,
                                            uint64_t deadline) {
  const uint32_t acc_w = static_cast<uint32_t>(p.bn);
  const uint32_t idesc = sm100::umma_idesc_e4m3(kTileM, static_cast<uint32_t>(p.bn));
  const uint32_t tiles_addr = sm100::smem_u32(tiles);
  const uint32_t full0 = sm100::smem_u32(&bar->full[0]);
  const uint32_t empty0 = sm100::smem_u32(&bar->empty[0]);
  const uint32_t stages = static_cast<uint32_t>(L.stages);
  const uint64_t da0 = sm100::umma_desc_sw128(tiles_addr);
  const uint64_t db0 = sm100::umma_desc_sw128(tiles_addr + L.a_bytes);
  const uint64_t dstage = static_cast<uint64_t>(L.stage_bytes >> 4);
  uint32_t stage = st.stage, phase = st.phase;
  uint64_t da = da0 + stage * dstage, db = db0 + stage * dstage;
  for (int i = 0; i < c.kbn; ++i) {
    if (!sm100::mbar_wait(&bar->acc_empty[st.acc], st.acc_phase ^ 1, deadline)) return false;
    const uint32_t full = full0 + stage * 8;
    if (!sm100::mbar_try_wait_addr(full, phase) && !sm100::mbar_wait_addr(full, phase, deadline)) {
      st.stage = stage;
      st.phase = phase;
      return false;
    }
    sm100::tc_fence_after_sync();
    const uint32_t tmem_d = bar->tmem_base + st.acc * acc_w;
    // 32 fp8 elements = 32 bytes per UMMA K step: the same descriptor stride as bf16
    sm100::umma_f8(tmem_d, da, db, idesc, 0u);
    sm100::umma_f8(tmem_d, da + 2, db + 2, idesc, 1u);
    sm100::umma_f8(tmem_d, da + 4, db + 4, idesc, 1u);
    sm100::umma_f8(tmem_d, da + 6, db + 6, idesc, 1u);
    sm100::umma_commit_addr(empty0 + stage * 8);
    sm100::umma_commit(&bar->acc_full[st.acc]);
    st.advance_acc(nacc);
    da += dstage;
    db += dstage;
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
      da = da0;
      db = db0;
    }
  }
  st.stage = stage;
  st.phase = phase;
  return true;
}

// ---------------------------------------------------------------- epilogue

__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Applies the fused epilogue to 16 accumulator columns (activation rows
// n .. n+15) of feature f and stores them. `fb` is the feature's weight row in
// the whole weight tensor, which indexes the bias: equal to f except for
// grouped problems, where every group (expert) has its own bias row.
//
// One warp per scheduler runs this, so nothing hides an instruction's latency
// but the warp's own independent work: the 16 values are computed as 16
// independent chains (fully unrolled, no early exit) and stored with
// predicates, the epilogue kind is tested once per call.
__device__ __forceinline__ void epilogue_store16(const Problem& p, int f, int fb, int n_first, int row_end,
                                                 const float* g, const float* u) {
  const float bias = p.bias != nullptr ? p.bias[fb] : 0.f;
  const int valid = row_end - n_first;  // > 0 by the callers' checks
  const size_t o0 = static_cast<size_t>(n_first) * p.ld_out + f;
  float v[16];
  if (p.epilogue == kEpiSwiglu) {
    const float bias_u = (p.bias != nullptr && p.dual) ? p.bias[p.up_offset + fb] : 0.f;
    const float lim = p.gate_limit > 0.f ? p.gate_limit : 3.0e38f;
    const float a = p.act_alpha == 0.f ? 1.f : p.act_alpha;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float gg = fminf(round_bf16(g[j] + bias), lim);
      const float uu = fminf(fmaxf(round_bf16(u[j] + bias_u), -lim), lim);
      v[j] = __fdividef(gg, 1.f + __expf(-a * gg)) * (uu + p.up_add);
    }
  } else if (p.epilogue == kEpiResidual) {
    const __nv_bfloat16* r = reinterpret_cast<const __nv_bfloat16*>(p.resid) + static_cast<size_t>(n_first) * p.ld_resid + f;
    float rr[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) rr[j] = j < valid ? __bfloat162float(r[static_cast<size_t>(j) * p.ld_resid]) : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = round_bf16(g[j] + bias) + rr[j];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = g[j] + bias;
  }
  if (p.epilogue == kEpiStoreF32) {
    float* o = reinterpret_cast<float*>(p.out) + o0;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (j < valid) o[static_cast<size_t>(j) * p.ld_out] = v[j];
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + o0;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (j < valid) o[static_cast<size_t>(j) * p.ld_out] = __float2bfloat16_rn(v[j]);
  }
}

// Runs on the 128 epilogue threads. `ew` is the warp's TMEM lane quarter.
__device__ __forceinline__ bool epilogue_tile(const Problem& p, const TileCoord& c, Barriers* bar,
                                              PipeState& st, int nacc, int ew, int lane,
                                              uint64_t deadline) {
  const uint32_t acc_cols = static_cast<uint32_t>(p.bn * (p.dual ? 2 : 1));
  const uint32_t tmem_acc =
      bar->tmem_base + st.acc * acc_cols + (static_cast<uint32_t>(ew * 32) << 16);
  const int lane_in_tile = ew * 32 + lane;
  const int f = c.m0 + lane_in_tile;
  const int fb = c.w_row0 + lane_in_tile;
  // all lanes agree on the outcome so that the aligned TMEM loads below stay convergent
  bool acc_ok = __all_sync(0xffffffffu, sm100::mbar_wait(&bar->acc_full[st.acc], st.acc_phase, deadline));
  if (p.splits > 1) {
    // Split-K tiles meet at named barriers further down: the four warps agree on the outcome first, so that a wait
    // that ran out in one warp cannot leave the others blocked at a barrier it never reaches.
    if (!acc_ok) *reinterpret_cast<volatile uint32_t*>(&bar->abort_flag) = 1u;
    epi_bar_sync();
    acc_ok = *reinterpret_cast<volatile uint32_t*>(&bar->abort_flag) == 0u;
  }
  if (!acc_ok) return false;
  sm100::tc_fence_after_sync();

  float g[16], u[16];
  if (p.fp8) {
    // scaled accumulation over the K blocks of this tile (bn <= 64: four chunks of 16 columns)
    float acc[kMaxBnF8];
#pragma unroll
    for (int j = 0; j < kMaxBnF8; ++j) acc[j] = 0.f;
    const int kb_total = p.k / p.kblk;
    const float* wsc = p.w_scale + static_cast<size_t>(c.w_row0 >> 7) * kb_total + c.kb0;
    for (int i = 0; i < c.kbn; ++i) {
      // The scales of this K block do not depend on its MMAs: their loads are issued before the wait
      // for the accumulator so that the L2 round trip overlaps it.
      const float sw = __ldg(wsc + i);
      const float4* xs = reinterpret_cast<const float4*>(p.x_scale + static_cast<size_t>(c.kb0 + i) * p.ld_xscale + c.n0);
      float4 sx[kMaxBnF8 / 4];
#pragma unroll
      for (int q = 0; q < kMaxBnF8 / 4; ++q) sx[q] = q * 4 < p.bn ? __ldg(xs + q) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (i > 0) {
        if (!__all_sync(0xffffffffu, sm100::mbar_wait(&bar->acc_full[st.acc], st.acc_phase, deadline))) return false;
        sm100::tc_fence_after_sync();
      }
      const uint32_t tacc = bar->tmem_base + st.acc * acc_cols + (static_cast<uint32_t>(ew * 32) << 16);
      // two halves of 32 columns: both TMEM reads of a half in flight, one wait
#pragma unroll
      for (int h = 0; h < kMaxBnF8 / 32; ++h) {
        if (h * 32 < p.bn) {
          uint32_t ra[16], rb[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) rb[j] = 0u;
          sm100::tmem_ld16_issue(tacc + h * 32, ra);
          if (h * 32 + 16 < p.bn) sm100::tmem_ld16_issue(tacc + h * 32 + 16, rb);
          sm100::tmem_ld_wait32(ra, rb);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 sa = sx[h * 8 + q], sb = sx[h * 8 + 4 + q];
            acc[h * 32 + q * 4 + 0] += __uint_as_float(ra[q * 4 + 0]) * (sw * sa.x);
            acc[h * 32 + q * 4 + 1] += __uint_as_float(ra[q * 4 + 1]) * (sw * sa.y);
            acc[h * 32 + q * 4 + 2] += __uint_as_float(ra[q * 4 + 2]) * (sw * sa.z);
            acc[h * 32 + q * 4 + 3] += __uint_as_float(ra[q * 4 + 3]) * (sw * sa.w);
            acc[h * 32 + 16 + q * 4 + 0] += __uint_as_float(rb[q * 4 + 0]) * (sw * sb.x);
            acc[h * 32 + 16 + q * 4 + 1] += __uint_as_float(rb[q * 4 + 1]) * (sw * sb.y);
            acc[h * 32 + 16 + q * 4 + 2] += __uint_as_float(rb[q * 4 + 2]) * (sw * sb.z);
            acc[h * 32 + 16 + q * 4 + 3] += __uint_as_float(rb[q * 4 + 3]) * (sw * sb.w);
          }
        }
      }
      sm100::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&bar->acc_empty[st.acc]);
      st.advance_acc(nacc);
    }
    if (p.splits == 1) {
#pragma unroll
      for (int cc = 0; cc < kMaxBnF8 / 16; ++cc)
        if (cc * 16 < p.bn && c.n0 + cc * 16 < c.row_end) epilogue_store16(p, f, fb, c.n0 + cc * 16, c.row_end, &acc[cc * 16], u);
    } else {
      float* ws = p.ws + (static_cast<size_t>(c.mn) * p.splits + c.split) * acc_cols * kTileM;
#pragma unroll
      for (int j = 0; j < kMaxBnF8; ++j)
        if (j < p.bn) ws[static_cast<size_t>(j) * kTileM + lane_in_tile] = acc[j];
    }
  } else if (p.splits == 1) {
    // Two register buffers: the TMEM read of the next 16 columns is in flight while the current
    // ones go through the epilogue math and their stores. All conditions are warp-uniform.
    const int ncol = min(p.bn, c.row_end - c.n0);  // columns that hold rows to store (> 0)
    const uint32_t up = tmem_acc + static_cast<uint32_t>(p.bn);
    uint32_t ga[16], ua[16], gb[16], ub[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) ua[j] = ub[j] = 0u;
    sm100::tmem_ld16_issue(tmem_acc, ga);
    if (p.dual) sm100::tmem_ld16_issue(up, ua);
    for (int col = 0; col < ncol; col += 32) {
      sm100::tmem_ld_wait32(ga, ua);
      const bool more = col + 16 < ncol;
      if (more) {
        sm100::tmem_ld16_issue(tmem_acc + col + 16, gb);
        if (p.dual) sm100::tmem_ld16_issue(up + col + 16, ub);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        g[j] = __uint_as_float(ga[j]);
        u[j] = __uint_as_float(ua[j]);
      }
      epilogue_store16(p, f, fb, c.n0 + col, c.row_end, g, u);
      if (more) {
        sm100::tmem_ld_wait32(gb, ub);
        if (col + 32 < ncol) {
          sm100::tmem_ld16_issue(tmem_acc + col + 32, ga);
          if (p.dual) sm100::tmem_ld16_issue(up + col + 32, ua);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          g[j] = __uint_as_float(gb[j]);
          u[j] = __uint_as_float(ub[j]);
        }
        epilogue_store16(p, f, fb, c.n0 + col + 16, c.row_end, g, u);
      }
    }
  } else {
    // Split-K: park raw partial sums, last-arriving CTA folds them in split order.
    float* ws = p.ws + (static_cast<size_t>(c.mn) * p.splits + c.split) * acc_cols * kTileM;
    for (uint32_t col = 0; col < acc_cols; col += 16) {
      sm100::tmem_ld16(tmem_acc + col, g);
#pragma unroll
      for (int j = 0; j < 16; ++j) ws[static_cast<size_t>(col + j) * kTileM + lane_in_tile] = g[j];
    }
  }
  if (!p.fp8) {
    // The accumulator buffer is free again once every epilogue warp has read it.
    sm100::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) sm100::mbar_arrive(&bar->acc_empty[st.acc]);
    st.advance_acc(nacc);
  }

  if (p.splits > 1) {
    __threadfence();
    epi_bar_sync();
    if (ew == 0 && lane == 0) bar->bcast = atomicAdd(&p.counters[c.mn], 1u);
    epi_bar_sync();
    const bool last = bar->bcast == static_cast<uint32_t>(p.splits - 1);
    epi_bar_sync();  // everyone has read bcast before a later tile overwrites it
    if (last) {
      __threadfence();
      const float* base = p.ws + static_cast<size_t>(c.mn) * p.splits * acc_cols * kTileM;
      for (int col = 0; col < p.bn; col += 16) {
        if (c.n0 + col >= c.row_end) break;
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.f;
        // Split order is the summation order (deterministic). The loads of four splits (two when
        // gate and up are both read) are issued together: 64 independent L2 reads in flight per
        // thread instead of 16, or this loop costs one L2 round trip per split and chunk.
        const int per = p.dual ? 2 : 4;
        for (int s0 = 0; s0 < p.splits; s0 += per) {
          float t[64];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int s = p.dual ? s0 + (q >> 1) : s0 + q;
            const int cb = (p.dual && (q & 1)) ? p.bn + col : col;
            const bool on = s < p.splits;
            const float* w = base + static_cast<size_t>(on ? s : 0) * acc_cols * kTileM + lane_in_tile;
#pragma unroll
            for (int j = 0; j < 16; ++j) t[q * 16 + j] = on ? __ldcg(&w[static_cast<size_t>(cb + j) * kTileM]) : 0.f;
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (p.dual && (q & 1)) u[j] += t[q * 16 + j];
              else g[j] += t[q * 16 + j];
            }
          }
        }
        epilogue_store16(p, f, fb, c.n0 + col, c.row_end, g, u);
      }
      if (ew == 0 && lane == 0) p.counters[c.mn] = 0;  // ready for the next call
    }
  }
  return true;
}

// ---------------------------------------------------------------- CTA set-up / tear-down

__device__ __forceinline__ uint32_t tmem_columns_needed(int bn, int dual, int nacc) {
  uint32_t need = static_cast<uint32_t>(bn * (dual ? 2 : 1) * nacc);
  uint32_t cols = 32;
  while (cols < need) cols <<= 1;
  return cols;
}

// Called by all threads of the CTA once. Returns the aligned tile area.
__device__ __forceinline__ uint8_t* cta_setup(uint8_t* smem_raw, const SmemLayout& L,
                                              Barriers** bar_out, uint32_t tmem_cols, int warp,
                                              int lane) {
  uint8_t* tiles = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Barriers* bar = reinterpret_cast<Barriers*>(tiles + static_cast<size_t>(L.stages) * L.stage_bytes);
  *bar_out = bar;
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      sm100::mbar_init(&bar->full[s], 1);
      sm100::mbar_init(&bar->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&bar->acc_full[a], 1);
      sm100::mbar_init(&bar->acc_empty[a], 4);
    }
    bar->abort_flag = 0;
    sm100::mbar_fence_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(&bar->tmem_base, tmem_cols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::tc_fence_after_sync();
  return tiles;
}

__device__ __forceinline__ void cta_teardown(Barriers* bar, uint32_t tmem_cols, int warp) {
  sm100::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after_sync();
    sm100::tmem_dealloc(bar->tmem_base, tmem_cols);
  }
}

}  // namespace gemm
}  // namespace xpool
