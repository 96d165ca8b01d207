// Stream-launched entry points of the weight-stationary tcgen05 GEMM
// (see xpool/gemm_ws.cuh). Exported with C linkage and loaded through ctypes.
#include <algorithm>

#include "xpool/api.h"
#include "xpool/gemm_ws.cuh"
#include "xpool/lane.cuh"
#include "xpool/tensormap.hpp"

namespace xpool {
namespace gemm {

// Body shared by the stream-launched kernel and the Lane kernel: every CTA loops
// over the tiles assigned to it.
__device__ __forceinline__ void run_tiles(const Problem& p, int nacc, int smem_budget, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const SmemLayout L = smem_layout(p.bn, p.dual, smem_budget);
  const uint32_t tmem_cols = tmem_columns_needed(p.bn, p.dual, nacc);
  Barriers* bar;
  uint8_t* tiles = cta_setup(smem_raw, L, &bar, tmem_cols, warp, lane);
  const int ntiles = tile_count(p);

  if (warp == 0) {
    if (lane == 0) {
      sm100::tma_prefetch_desc(p.tmap_w);
      sm100::tma_prefetch_desc(p.tmap_x);
      PipeState st;
      for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const uint64_t deadline = sm100::global_timer_ns() + sm100::kPipelineWaitNs;
        if (!produce_tile(p, tile_coord(p, t), L, tiles, bar, st, deadline)) {
          record_status(status, kTimeoutProducer);
          producer_drain(L, bar, st);
          break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      PipeState st;
      for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const uint64_t deadline = sm100::global_timer_ns() + sm100::kPipelineWaitNs;
        if (!mma_tile(p, tile_coord(p, t), L, tiles, bar, st, nacc, deadline)) {
          record_status(status, kTimeoutMma);
          break;
        }
      }
    }
    __syncwarp();
  } else {
    PipeState st;
    const int ew = warp & 3;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
      const uint64_t deadline = sm100::global_timer_ns() + sm100::kPipelineWaitNs;
      if (!epilogue_tile(p, tile_coord(p, t), bar, st, nacc, ew, lane, deadline)) {
        record_status(status, kTimeoutEpilogue);
        break;
      }
    }
  }
  cta_teardown(bar, tmem_cols, warp);
}

// At most 208 registers: 192 threads x 208 leave room on the SM for one decode-attention CTA of another
// stream (128 threads x 192 registers), which is how decode GEMMs hide behind the co-located Instance's
// attention.
__global__ void __maxnreg__(208)
gemm_ws_kernel(const __grid_constant__ CUtensorMap tmap_w,
               const __grid_constant__ CUtensorMap tmap_x, Problem p, int nacc, int smem_budget,
               uint32_t* status) {
  p.tmap_w = &tmap_w;
  p.tmap_x = &tmap_x;
  run_tiles(p, nacc, smem_budget, status);
}

// Lane form: the problem is assembled on the device from the descriptor table
// entry of the invocation the Lane was given (phase 0: gate/up projection with
// the activation epilogue into local scratch; phase 1: down projection whose
// epilogue stores into the attention device's partial buffer for this TP rank).
__global__ void __launch_bounds__(kThreads, 1)
gemm_lane_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, int phase, float* ws,
                 uint32_t* counters, int smem_budget, uint32_t* status, const lane::MoeLaneWs* mws,
                 const lane::MoeLaneMaps* mmaps) {
  if (cur->valid == 0 || cur->rows == 0) return;  // idle replay: uniform exit
  const lane::InstanceSlot& s = slots[cur->instance];
  const lane::LayerEntry& le = s.layers[cur->layer];
  const lane::MoeLayer* moe = le.moe;
  if (phase == 2 && (moe == nullptr || moe->router_precision != 0)) return;  // payload-precision router projection only
  if (phase >= 3 && (moe == nullptr || le.shared_inter_local == 0)) return;  // shared experts of a MoE layer
  const int rows = static_cast<int>(cur->rows);
  int bucket = 0;
  while ((1 << bucket) < rows && bucket < lane::kRowBuckets - 1) ++bucket;
  Problem p{};
  p.kblk = kTileK;
  p.rows = rows;
  p.ws = ws;
  p.counters = counters;
  p.w_tiled = le.w_tiled;
  p.w_evict_first = rows <= 64;
  if (phase == 3) {
    // shared experts, gate/up + SwiGLU into the slot's activation scratch
    p.bn = le.bn_sh_gateup[bucket] == 255 ? 256 : le.bn_sh_gateup[bucket];
    p.splits = le.splits_sh_gateup[bucket];
    p.tmap_w = &le.tmap_shared_gateup;
    p.tmap_x = &s.tmap_x[lane::bn_index(p.bn)];
    p.out = s.act;
    p.n_out = le.shared_inter_local;
    p.k = s.hidden;
    p.ld_out = s.act_ld;
    p.dual = 1;
    p.up_offset = le.shared_inter_local;
    p.epilogue = kEpiSwiglu;
    p.w_tiled = 0;
  } else if (phase == 4) {
    // shared experts, down projection added to the routed result, stored to the attention device
    p.bn = le.bn_sh_down[bucket] == 255 ? 256 : le.bn_sh_down[bucket];
    p.splits = le.splits_sh_down[bucket];
    p.tmap_w = &le.tmap_shared_down;
    p.tmap_x = &s.tmap_act[lane::bn_index(p.bn)];
    p.out = s.out_peer;
    p.resid = mws->comb;
    p.n_out = s.hidden;
    p.k = le.shared_inter_local;
    p.ld_out = s.hidden;
    p.epilogue = kEpiResidual;
    p.w_tiled = 0;
  } else if (phase == 2) {
    p.bn = moe->bn_router[bucket] == 255 ? 256 : moe->bn_router[bucket];
    p.splits = moe->splits_router[bucket];
    p.tmap_w = &moe->tmap_router;
    p.tmap_x = &s.tmap_x[lane::bn_index(p.bn)];
    p.out = mws->logits;
    p.n_out = moe->e_pad;
    p.k = s.hidden;
    p.ld_out = moe->e_pad;
    p.epilogue = kEpiStore;
    p.w_tiled = 0;
  } else if (moe != nullptr) {
    // grouped projections over the routes ordered by expert; tile tables come from moe_lane_route
    const lane::MoeLaneMaps& mm = mmaps[cur->instance];
    p.bn = lane::moe_tile_width(rows, moe->top_k, moe->expert_hi - moe->expert_lo);
    p.splits = 1;
    p.rows = rows * moe->top_k;
    p.w_tiled = 0;
    p.w_evict_first = 0;
    if (phase == 0) {
      p.tmap_w = &le.tmap_gateup;
      p.tmap_x = &mm.tmap_xp[lane::bn_index(p.bn)];
      p.out = mws->act;
      p.n_out = le.inter_local;
      p.k = s.hidden;
      p.ld_out = le.inter_local;
      p.dual = 1;
      p.up_offset = le.inter_local;
      p.epilogue = kEpiSwiglu;
      p.gate_limit = le.gate_limit;
      p.up_add = le.up_add;
      p.act_alpha = le.act_alpha;
      p.bias = le.bias_gateup;   // [local experts, 2 * inter]: the epilogue indexes it by stacked weight row
      p.tile_table = mws->tiles_gateup;
      p.n_tiles = mws->n_tiles;
      p.w_rows_per_group = 2 * le.inter_local;
    } else {
      p.tmap_w = &le.tmap_down;
      p.tmap_x = &mm.tmap_act[lane::bn_index(p.bn)];
      p.out = mws->yp;
      p.n_out = s.hidden;
      p.k = le.inter_local;
      p.ld_out = s.hidden;
      p.epilogue = kEpiStore;
      p.bias = le.bias_down;     // [local experts, hidden]
      p.tile_table = mws->tiles_down;
      p.n_tiles = mws->n_tiles + 1;
      p.w_rows_per_group = s.hidden;
    }
  } else if (phase == 0) {
    p.bn = le.bn_gateup[bucket] == 255 ? 256 : le.bn_gateup[bucket];
    p.splits = le.splits_gateup[bucket];
    p.tmap_w = &le.tmap_gateup;
    p.tmap_x = &s.tmap_x[lane::bn_index(p.bn)];
    p.out = s.act;
    p.bias = le.bias_gateup;
    p.n_out = le.inter_local;
    p.k = s.hidden;
    p.ld_out = s.act_ld;
    p.dual = le.gated;
    p.up_offset = le.inter_local;
    p.epilogue = le.gated ? kEpiSwiglu : kEpiStore;
    p.gate_limit = le.gate_limit;
    p.up_add = le.up_add;
    p.act_alpha = le.act_alpha;
  } else {
    p.bn = le.bn_down[bucket] == 255 ? 256 : le.bn_down[bucket];
    p.splits = le.splits_down[bucket];
    p.tmap_w = &le.tmap_down;
    p.tmap_x = &s.tmap_act[lane::bn_index(p.bn)];
    p.out = s.out_peer;
    p.bias = le.bias_down;
    p.n_out = s.hidden;
    p.k = le.inter_local;
    p.ld_out = s.hidden;
    p.epilogue = kEpiStore;
  }
  p.ld_resid = p.ld_out;
  const int nacc = p.bn * (p.dual ? 2 : 1) * 2 <= 512 ? 2 : 1;
  if (threadIdx.x == 0 && (phase == 0 || phase == 2 || phase == 3)) sm100::fence_proxy_async();  // payload arrived through peer stores
  run_tiles(p, nacc, smem_budget, status);
}

// Estimated duration (microseconds) of one launch for a tile width and split-K factor, fitted to
// measurements on B200 (python -m crosspool_b200.bench.kernels gemm ...): a CTA streams its stages at
// about 45 GB/s whatever the source (a 48-64 KB stage takes 1.0-1.4 us), HBM delivers about 6 TB/s in
// total, a tcgen05.mma of M=128 retires in max(45, N/2) cycles, a launch costs about 3 us of set-up and
// pipeline fill, and split-K pays for parking and re-reading fp32 partials (about 3 TB/s through L2:
// two splits of a 4096 x 12288 gate/up projection at 256 rows cost +45 us). Only relative order matters.
static double estimate_us(int tm, int rows, int kb, int dual, int bn, int splits, int sms) {
  const int tn = (rows + bn - 1) / bn;
  const int ctas = tm * tn * splits;
  const int waves = (ctas + sms - 1) / sms;
  const int kb_per = (kb + splits - 1) / splits;
  const double stage_kb = (kTileM * kTileK * 2 * (dual ? 2 : 1) + bn * kTileK * 2) / 1000.0;
  const int active = std::min(ctas, sms);
  const double bw = std::min(45.0, 6000.0 / active);  // KB per us per SM
  const double t_mem = stage_kb / bw;
  const double t_mma = (dual ? 8 : 4) * std::max(45.0, bn / 2.0) / 1900.0;
  const int acc_cols = bn * (dual ? 2 : 1);
  double t = waves * (3.0 + kb_per * std::max(t_mem, t_mma) + (acc_cols / 16) * 0.12);
  if (splits > 1) {
    const double ws_mb = static_cast<double>(tm) * tn * splits * acc_cols * kTileM * 4 / 1e6;
    t += 2.0 + ws_mb * 2.0 / 3.0 + splits * acc_cols * 0.512 / 55.0;
  }
  return t;
}

struct TileChoice {
  int bn, splits;
};

static TileChoice choose_tiles(int tm, int rows, int kb, int dual, int sms, int fixed_bn, int fixed_splits,
                               size_t ws_bytes_available, int max_bn = 256) {
  // 256-wide dual tiles use all 512 TMEM columns (one accumulator buffer, no epilogue overlap): worth it
  // only when they make the activation a single tile, so that every weight byte is fetched once
  const int cap = std::min((dual && fixed_bn != 256 && !(rows > 128 && rows <= 256)) ? 128 : 256, max_bn);
  int top = 16;
  while (top < rows && top < cap) top <<= 1;
  TileChoice best{top, 1};
  double best_t = 1e30;
  static const int kSplits[] = {1, 2, 3, 4, 6, 8, 12, 16};
  for (int bn = 16; bn <= top; bn <<= 1) {
    if (fixed_bn > 0 && bn != fixed_bn) continue;
    if (fixed_bn <= 0 && bn * 4 < top && bn < 64) continue;  // no forests of tiny tiles
    const int tn = (rows + bn - 1) / bn;
    for (int s : kSplits) {
      if (fixed_splits > 0 && s != fixed_splits) continue;
      if (s > kb) continue;
      if (s > 1 && (s - 1) * ((kb + s - 1) / s) >= kb) continue;  // every split owns a K block
      const size_t ws = s > 1 ? static_cast<size_t>(tm) * tn * s * bn * (dual ? 2 : 1) * kTileM * 4 : 0;
      if (ws > ws_bytes_available) continue;
      const double t = estimate_us(tm, rows, kb, dual, bn, s, sms);
      if (t < best_t) {
        best_t = t;
        best = TileChoice{bn, s};
      }
    }
  }
  return best;
}

TileChoice choose_tiles_host(int tm, int rows, int kb, int dual, int sms, size_t ws_bytes_available) {
  return choose_tiles(tm, rows, kb, dual, sms, 0, 0, ws_bytes_available);
}

}  // namespace gemm
}  // namespace xpool

using namespace xpool;

static inline int kblk_of(const XpGemmArgs* a) { return a->fp8 ? 128 : gemm::kTileK; }

extern "C" int xp_gemm_plan(const XpGemmArgs* a, XpGemmPlan* plan) {
  const int kblk = a->fp8 ? 128 : gemm::kTileK;
  if (a->n_out <= 0 || a->n_out % gemm::kTileM != 0 || a->k <= 0 || a->k % kblk != 0 || a->rows <= 0) return -10;
  if (a->fp8 && (a->dual || a->w_tiled || a->tile_table != nullptr || a->w_scale == nullptr || a->x_scale == nullptr ||
                 a->ld_xscale % 4 != 0 || a->bn > gemm::kMaxBnF8))
    return -14;
  int dev = 0;
  cudaGetDevice(&dev);
  static int sm_count_cache[64] = {0};
  if (dev < 64 && sm_count_cache[dev] == 0)
    cudaDeviceGetAttribute(&sm_count_cache[dev], cudaDevAttrMultiProcessorCount, dev);
  int sms = a->num_sms > 0 ? a->num_sms : (dev < 64 ? sm_count_cache[dev] : 148);
  if (sms <= 0) sms = 148;
  const int tm = a->n_out / gemm::kTileM;
  const int kb = a->k / kblk;
  if (a->bn > 0 && a->bn != 16 && a->bn != 32 && a->bn != 64 && a->bn != 128 && a->bn != 256) return -11;
  int fixed_splits = a->splits;
  if (fixed_splits > kb) fixed_splits = kb;
  while (fixed_splits > 1 && (fixed_splits - 1) * ((kb + fixed_splits - 1) / fixed_splits) >= kb) --fixed_splits;
  const size_t ws_avail = (a->ws != nullptr && a->counters != nullptr) ? a->ws_bytes : 0;
  const gemm::TileChoice ch = gemm::choose_tiles(tm, a->rows, kb, a->dual, sms, a->bn, fixed_splits, ws_avail,
                                                 a->fp8 ? gemm::kMaxBnF8 : 256);
  const int bn = a->bn > 0 ? a->bn : ch.bn;
  int splits = fixed_splits > 0 ? fixed_splits : ch.splits;
  const int acc_cols = bn * (a->dual ? 2 : 1);
  const int nacc = acc_cols * 2 <= 512 ? 2 : 1;
  const int tn = (a->rows + bn - 1) / bn;
  plan->bn = bn;
  plan->nacc = nacc;
  plan->splits = splits;
  plan->tiles = tm * tn * splits;
  plan->grid = std::min(plan->tiles, sms);
  plan->ws_bytes = splits > 1 ? static_cast<size_t>(tm) * tn * splits * acc_cols * gemm::kTileM * 4 : 0;
  plan->counter_bytes = splits > 1 ? static_cast<size_t>(tm) * tn * 4 : 0;
  plan->smem_budget = 220 * 1024;
  if (a->smem_limit > 0 && a->smem_limit < plan->smem_budget) plan->smem_budget = std::max(a->smem_limit, 48 * 1024);
  gemm::SmemLayout L = gemm::smem_layout(bn, a->dual, plan->smem_budget);
  plan->smem_bytes = L.total_bytes;
  plan->stages = L.stages;
  return 0;
}

extern "C" int xp_gemm(const XpGemmArgs* a) {
  XpGemmPlan plan;
  int rc = xp_gemm_plan(a, &plan);
  if (rc != 0) return rc;
  if (plan.splits > 1) {
    if (a->ws == nullptr || a->counters == nullptr || a->ws_bytes < plan.ws_bytes ||
        a->counter_bytes < plan.counter_bytes) {
      // fall back to no split-K rather than touching memory we do not own
      XpGemmArgs b = *a;
      b.splits = 1;
      b.bn = plan.bn;
      return xp_gemm(&b);
    }
  }
  CUtensorMap tw, tx;
  const int w_rows = a->w_rows_total > 0 ? a->w_rows_total : (a->dual ? a->up_offset + a->n_out : a->n_out);
  if (a->w_tiled) {
    if (w_rows % gemm::kTileM != 0 || (a->dual && a->up_offset % gemm::kTileM != 0)) return -22;
    rc = tmap::cache().get(&tw, a->w, static_cast<uint64_t>(w_rows) * (a->k / gemm::kTileK), gemm::kTileK,
                           gemm::kTileK * 2, gemm::kTileM, 2);
  } else {
    const int eb = a->fp8 ? 1 : 2;
    rc = tmap::cache().get(&tw, a->w, w_rows, a->k, static_cast<uint64_t>(a->ldw > 0 ? a->ldw : a->k) * eb,
                           gemm::kTileM, eb);
  }
  if (rc != 0) return -20;
  {
    const int eb = a->fp8 ? 1 : 2;
    rc = tmap::cache().get(&tx, a->x, a->rows, a->k, static_cast<uint64_t>(a->ldx > 0 ? a->ldx : a->k) * eb, plan.bn, eb);
  }
  if (rc != 0) return -21;
  if (a->fp8 && a->ld_xscale < (a->rows + plan.bn - 1) / plan.bn * plan.bn) return -15;  // scales padded to whole tiles

  gemm::Problem p{};
  p.out = a->out;
  p.resid = a->resid;
  p.bias = a->bias;
  p.ws = a->ws;
  p.counters = a->counters;
  p.n_out = a->n_out;
  p.k = a->k;
  p.rows = a->rows;
  p.ld_out = a->ld_out > 0 ? a->ld_out : a->n_out;
  p.ld_resid = a->ld_resid > 0 ? a->ld_resid : p.ld_out;
  p.bn = plan.bn;
  p.splits = plan.splits;
  p.epilogue = a->epilogue;
  p.dual = a->dual;
  p.up_offset = a->up_offset;
  p.w_evict_first = a->w_evict_first;
  p.w_tiled = a->w_tiled;
  p.gate_limit = a->gate_limit;
  p.up_add = a->up_add;
  p.act_alpha = a->act_alpha;
  p.tile_table = reinterpret_cast<const int4*>(a->tile_table);
  p.n_tiles = a->n_tiles;
  p.w_rows_per_group = a->w_rows_per_group;
  p.kblk = kblk_of(a);
  p.fp8 = a->fp8;
  p.w_scale = a->w_scale;
  p.x_scale = a->x_scale;
  p.ld_xscale = a->ld_xscale;
  if (a->tile_table != nullptr) {
    if (plan.splits != 1) return -13;
    plan.grid = plan.smem_bytes > 0 ? 148 : 148;
    int dev2 = 0, sms2 = 148;
    cudaGetDevice(&dev2);
    cudaDeviceGetAttribute(&sms2, cudaDevAttrMultiProcessorCount, dev2);
    plan.grid = a->num_sms > 0 ? a->num_sms : sms2;
  }

  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm::gemm_ws_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return -30;
    attr_set[dev] = true;
  }
  gemm::gemm_ws_kernel<<<plan.grid, gemm::kThreads, plan.smem_bytes,
                         reinterpret_cast<cudaStream_t>(a->stream)>>>(
      tw, tx, p, plan.nacc, plan.smem_budget, a->status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" int xp_encode_tmap_2d(void* out128, const void* base, uint64_t rows, uint64_t cols,
                                 uint64_t pitch_bytes, uint32_t box_rows, uint32_t elem_bytes) {
  return tmap::encode_2d(reinterpret_cast<CUtensorMap*>(out128), base, rows, cols, pitch_bytes,
                         box_rows, 128 / elem_bytes, elem_bytes);
}
