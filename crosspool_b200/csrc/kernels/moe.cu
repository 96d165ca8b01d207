// Mixture-of-experts plumbing around the grouped tcgen05 GEMM: router top-k,
// route ordering, tile table, row gather and the weighted combine.
//
// Router semantics are the reference's (src/xpool/runtime/ffnagent/operators/
// routing.py:21-190): fp32 scores from softmax or sigmoid; selection on score plus
// optional correction bias; ties go to the lower expert id for softmax and the
// higher id for sigmoid; the weights are the original scores of the selected
// experts, normalised (a zero sum stays zero), then scaled.
//
// Expert parallelism needs no second code path: a rank owning experts [lo, hi)
// orders only the routes that name its experts, and the combine kernel leaves
// the other contributions out, producing this rank's partial sum. Partials of all
// ranks are folded in rank order by the attention side, exactly like TP partials.
#include <math_constants.h>

#include "xpool/api.h"
#include "xpool/lane.cuh"
#include "xpool/sm100.cuh"

namespace xpool {
namespace moe {

constexpr int kMaxPerLane = 8;  // up to 256 experts

// One warp per token.
__device__ __forceinline__ void router_topk_row(const XpRouterArgs& a, int row, int lane) {
  const int E = a.num_experts;
  float score[kMaxPerLane], sel[kMaxPerLane];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    float v = -CUDART_INF_F;
    if (e < E) {
      v = a.logits_fp32 ? reinterpret_cast<const float*>(a.logits)[static_cast<size_t>(row) * a.ld_logits + e]
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.logits)[static_cast<size_t>(row) * a.ld_logits + e]);
      if (a.logit_bias != nullptr) v += a.logit_bias[e];
    }
    score[j] = v;
    mx = fmaxf(mx, v);
  }
  if (a.sigmoid) {
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) score[j] = (lane + 32 * j < E) ? 1.f / (1.f + __expf(-score[j])) : -CUDART_INF_F;
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      score[j] = (lane + 32 * j < E) ? __expf(score[j] - mx) : 0.f;
      sum += score[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) score[j] = (lane + 32 * j < E) ? score[j] * inv : -CUDART_INF_F;
  }
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    sel[j] = (e < E) ? score[j] + (a.correction_bias != nullptr ? a.correction_bias[e] : 0.f) : -CUDART_INF_F;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = -1;
  for (int k = 0; k < a.top_k; ++k) {
    // lane-local best, then warp argmax with the tie rule
    float bv = -CUDART_INF_F, bs = 0.f;
    int be = -1;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      const bool better = sel[j] > bv || (sel[j] == bv && be >= 0 && (a.sigmoid ? e > be : e < be));
      if (e < E && better) {
        bv = sel[j];
        be = e;
        bs = score[j];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      const bool better = oe >= 0 && (be < 0 || ov > bv || (ov == bv && (a.sigmoid ? oe > be : oe < be)));
      if (better) {
        bv = ov;
        be = oe;
        bs = os;
      }
    }
    // remove the winner from further rounds
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (lane + 32 * j == be) sel[j] = -CUDART_INF_F;
    wsum += bs;
    if (lane == k) {
      my_w = bs;
      my_id = be;
    }
  }
  if (lane < a.top_k) {
    float w = my_w;
    if (a.renormalize && wsum > 0.f) w = w / wsum;
    w *= a.scale;
    if (a.round_weights_bf16) w = __bfloat162float(__float2bfloat16_rn(w));
    a.topk_ids[static_cast<size_t>(row) * a.top_k + lane] = my_id;
    a.topk_weights[static_cast<size_t>(row) * a.top_k + lane] = w;
  }
}

__global__ void __launch_bounds__(128)
router_topk_kernel(XpRouterArgs a) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  router_topk_row(a, row, threadIdx.x & 31);
}

// counts[e - lo] = routes naming expert e; one CTA per local expert.
__global__ void __launch_bounds__(256)
route_count_kernel(const int* __restrict__ ids, int n_routes, int lo, int* __restrict__ counts) {
  __shared__ int red[8];
  const int e = lo + blockIdx.x;
  int c = 0;
  for (int i = threadIdx.x; i < n_routes; i += 256) c += ids[i] == e;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < 8; ++w) t += red[w];
    counts[blockIdx.x] = t;
  }
}

// offsets = exclusive prefix of counts; also builds the grouped-GEMM tile tables for
// both projections: entry = {expert (local), feature tile start, first row, row end}.
__global__ void __launch_bounds__(1024)
route_offsets_tiles_kernel(const int* __restrict__ counts, int n_experts, int* __restrict__ offsets,
                           int tm_gateup, int bn_gateup, int4* __restrict__ tiles_gateup, int* __restrict__ n_tiles_gateup,
                           int tm_down, int bn_down, int4* __restrict__ tiles_down, int* __restrict__ n_tiles_down) {
  __shared__ int s_off[1025], s_t0[1025], s_t1[1025];
  const int e = threadIdx.x;
  const int c = e < n_experts ? counts[e] : 0;
  s_off[e] = c;
  s_t0[e] = tm_gateup * ((c + bn_gateup - 1) / bn_gateup);
  s_t1[e] = tm_down * ((c + bn_down - 1) / bn_down);
  __syncthreads();
  if (threadIdx.x == 0) {
    int a0 = 0, a1 = 0, a2 = 0;
    for (int i = 0; i <= n_experts; ++i) {
      const int v0 = s_off[i], v1 = s_t0[i], v2 = s_t1[i];
      s_off[i] = a0;
      s_t0[i] = a1;
      s_t1[i] = a2;
      a0 += v0;
      a1 += v1;
      a2 += v2;
    }
    *n_tiles_gateup = s_t0[n_experts];
    *n_tiles_down = s_t1[n_experts];
  }
  __syncthreads();
  if (e <= n_experts) offsets[e] = s_off[e];
  if (e < n_experts) {
    const int row0 = s_off[e], row1 = s_off[e] + c;
    int idx = s_t0[e];
    for (int m = 0; m < tm_gateup; ++m)
      for (int r = row0; r < row1; r += bn_gateup) tiles_gateup[idx++] = make_int4(e, m * 128, r, row1);
    idx = s_t1[e];
    for (int m = 0; m < tm_down; ++m)
      for (int r = row0; r < row1; r += bn_down) tiles_down[idx++] = make_int4(e, m * 128, r, row1);
  }
}

// Stable placement: routes of an expert keep their (token, k) order.
__global__ void __launch_bounds__(256)
route_place_kernel(const int* __restrict__ ids, int n_routes, int top_k, int lo, const int* __restrict__ offsets,
                   int* __restrict__ perm_token, int* __restrict__ route_pos) {
  __shared__ int warp_tot[8];
  __shared__ int base;
  const int e = lo + blockIdx.x;
  if (threadIdx.x == 0) base = offsets[blockIdx.x];
  __syncthreads();
  for (int start = 0; start < n_routes; start += 256) {
    const int i = start + threadIdx.x;
    const int hit = (i < n_routes && ids[i] == e) ? 1 : 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) warp_tot[w] = __popc(ballot);
    __syncthreads();
    int before = __popc(ballot & ((1u << lane) - 1));
    for (int j = 0; j < w; ++j) before += warp_tot[j];
    if (hit) {
      const int pos = base + before;
      perm_token[pos] = i / top_k;
      route_pos[i] = pos;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int j = 0; j < 8; ++j) t += warp_tot[j];
      base += t;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(128)
gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ perm_token, const int* __restrict__ n_rows_ptr,
                   uint4* __restrict__ out, int hidden8, int ldx8) {
  const int pos = blockIdx.x;
  if (pos >= *n_rows_ptr) return;
  const uint4* src = x + static_cast<size_t>(perm_token[pos]) * ldx8;
  uint4* dst = out + static_cast<size_t>(pos) * hidden8;
  for (int i = threadIdx.x; i < hidden8; i += 128) dst[i] = src[i];
}

// out[token] = sum over k (in order) of w[token, k] * y[route_pos[token, k]]; routes with
// position < 0 (experts of other ranks, padding) contribute nothing.
__device__ __forceinline__ void combine_token(const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_pos,
                                              const float* __restrict__ weights, __nv_bfloat16* __restrict__ out, int top_k,
                                              int hidden, int ld_out, int token) {
  for (int c = threadIdx.x * 8; c < hidden; c += 128 * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < top_k; ++k) {
      const int pos = route_pos[token * top_k + k];
      if (pos < 0) continue;
      const float w = weights[token * top_k + k];
      const uint4 raw = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(pos) * hidden + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += w * f.x;
        acc[2 * j + 1] += w * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(token) * ld_out + c) = o;
  }
}

__global__ void __launch_bounds__(128)
combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_pos, const float* __restrict__ weights,
               __nv_bfloat16* __restrict__ out, int top_k, int hidden, int ld_out) {
  combine_token(y, route_pos, weights, out, top_k, hidden, ld_out, blockIdx.x);
}

// ---------------------------------------------------------------------------------------------
// Lane forms: the same steps with every parameter read from the Lane's current invocation, so
// that one captured graph serves dense and MoE layers of every model. Each is a no-op unless the
// invocation's layer is a mixture-of-experts layer.

__device__ __forceinline__ const lane::MoeLayer* lane_moe_layer(const lane::InstanceSlot* slots, const lane::LaneCur* cur) {
  if (cur->valid == 0 || cur->rows == 0) return nullptr;
  return slots[cur->instance].layers[cur->layer].moe;
}

__global__ void __launch_bounds__(128)
moe_lane_topk_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws) {
  const lane::MoeLayer* m = lane_moe_layer(slots, cur);
  if (m == nullptr) return;
  XpRouterArgs a;
  a.logits = m->router_precision != 0 ? static_cast<const void*>(ws->logits32) : static_cast<const void*>(ws->logits);
  a.logit_bias = m->router_bias;
  a.correction_bias = m->correction_bias;
  a.topk_ids = ws->ids;
  a.topk_weights = ws->weights;
  a.rows = static_cast<int>(cur->rows);
  a.num_experts = m->num_experts;
  a.top_k = m->top_k;
  a.ld_logits = m->e_pad;
  a.logits_fp32 = m->router_precision != 0;
  a.sigmoid = m->sigmoid;
  a.renormalize = m->renormalize;
  a.round_weights_bf16 = 0;
  a.scale = m->scale;
  for (int row = blockIdx.x * 4 + (threadIdx.x >> 5); row < a.rows; row += gridDim.x * 4) router_topk_row(a, row, threadIdx.x & 31);
}

// Exclusive scan of one int per thread across a 1024-thread CTA; returns the prefix, *total the sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_sums[w] = inc;
  __syncthreads();
  if (w == 0) {
    int ws = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, ws, o);
      if (lane >= o) ws += t;
    }
    warp_sums[lane] = ws;
  }
  __syncthreads();
  const int base = w > 0 ? warp_sums[w - 1] : 0;
  *total = warp_sums[31];
  __syncthreads();
  return base + inc - v;
}

// One CTA orders the routes of this rank's experts and writes both tile tables. Positions inside
// an expert's segment are handed out by an atomic cursor; expert outputs do not depend on the
// position of a row, and the combine step sums a token's routes in top-k order, so results are
// reproducible although the placement is not.
__global__ void __launch_bounds__(1024)
moe_lane_route_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws) {
  const lane::MoeLayer* m = lane_moe_layer(slots, cur);
  if (m == nullptr) return;
  __shared__ int hist[1024], cursor[1024], warp_sums[32];
  const lane::InstanceSlot& s = slots[cur->instance];
  const lane::LayerEntry& le = s.layers[cur->layer];
  const int lo = m->expert_lo, n_local = m->expert_hi - m->expert_lo;
  const int n_routes = static_cast<int>(cur->rows) * m->top_k;
  const int bn = lane::moe_tile_width(static_cast<int>(cur->rows), m->top_k, n_local);
  const int tm_gu = le.inter_local / 128, tm_dn = s.hidden / 128;
  const int e = threadIdx.x;
  hist[e] = 0;
  __syncthreads();
  for (int i = e; i < n_routes; i += 1024) {
    const int x = ws->ids[i] - lo;
    if (x >= 0 && x < n_local) atomicAdd(&hist[x], 1);
    else ws->route_pos[i] = -1;
  }
  __syncthreads();
  const int c = e < n_local ? hist[e] : 0;
  const int nb = (c + bn - 1) / bn;
  int total_rows, total_gu, total_dn;
  const int off = block_exclusive_scan(c, warp_sums, &total_rows);
  const int t_gu = block_exclusive_scan(tm_gu * nb, warp_sums, &total_gu);
  const int t_dn = block_exclusive_scan(tm_dn * nb, warp_sums, &total_dn);
  cursor[e] = off;
  if (e <= n_local) ws->offsets[e] = off;  // thread n_local sees the sum of all counts
  if (e == 0) {
    ws->n_tiles[0] = total_gu;
    ws->n_tiles[1] = total_dn;
    if (n_local == 1024) ws->offsets[1024] = total_rows;
  }
  __syncthreads();
  for (int i = e; i < n_routes; i += 1024) {
    const int x = ws->ids[i] - lo;
    if (x >= 0 && x < n_local) {
      const int pos = atomicAdd(&cursor[x], 1);
      ws->perm_token[pos] = i / m->top_k;
      ws->route_pos[i] = pos;
    }
  }
  if (e < n_local) {
    const int row0 = off, row1 = off + c;
    int idx = t_gu;
    for (int t = 0; t < tm_gu; ++t)
      for (int r = row0; r < row1; r += bn) ws->tiles_gateup[idx++] = make_int4(e, t * 128, r, row1);
    idx = t_dn;
    for (int t = 0; t < tm_dn; ++t)
      for (int r = row0; r < row1; r += bn) ws->tiles_down[idx++] = make_int4(e, t * 128, r, row1);
  }
}

__global__ void __launch_bounds__(128)
moe_lane_gather_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws) {
  const lane::MoeLayer* m = lane_moe_layer(slots, cur);
  if (m == nullptr) return;
  const lane::InstanceSlot& s = slots[cur->instance];
  const int n = ws->offsets[m->expert_hi - m->expert_lo];
  const int hidden8 = s.hidden / 8;
  const uint4* x = reinterpret_cast<const uint4*>(s.input);
  uint4* out = reinterpret_cast<uint4*>(ws->xp);
  for (int pos = blockIdx.x; pos < n; pos += gridDim.x) {
    const uint4* src = x + static_cast<size_t>(ws->perm_token[pos]) * hidden8;
    uint4* dst = out + static_cast<size_t>(pos) * hidden8;
    for (int i = threadIdx.x; i < hidden8; i += 128) dst[i] = src[i];
  }
}

__global__ void __launch_bounds__(128)
moe_lane_combine_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws) {
  const lane::MoeLayer* m = lane_moe_layer(slots, cur);
  if (m == nullptr) return;
  const lane::InstanceSlot& s = slots[cur->instance];
  // with shared experts the routed sum stays local: their down projection adds it and stores the total
  void* dst = s.layers[cur->layer].shared_inter_local > 0 ? ws->comb : s.out_peer;
  for (int token = blockIdx.x; token < static_cast<int>(cur->rows); token += gridDim.x)
    combine_token(reinterpret_cast<const __nv_bfloat16*>(ws->yp), ws->route_pos, ws->weights,
                  reinterpret_cast<__nv_bfloat16*>(dst), m->top_k, s.hidden, s.hidden, token);
}

// Router projection with IEEE fp32 accumulation: logits[r, e] = sum_k x[r, k] * w[e, k] in fp32, the products
// summed per lane in index order and the lanes folded by a fixed butterfly, so results are reproducible. The
// reference keeps two router precisions beside the payload one (docs/designs/ffn-execution.md:165-173): fp32 weights
// and fp32 inputs (GLM, sigmoid routers) and payload-dtype weights with fp32 accumulate and fp32 logits
// (DeepSeek-V2); both run on its SIMT fp32 GEMMs (operators/simt.py:80-240), never on TF32. The tensor cores
// accumulate bf16 products in fp32 too, but round the logits to bf16 on the way out and sum in hardware order;
// a router is a few hundred MFLOP at most, so the exact form costs microseconds.
template <typename WT>
__device__ __forceinline__ void router_fp32_rows(const __nv_bfloat16* __restrict__ x, int ldx, const WT* __restrict__ w,
                                                 float* __restrict__ logits, int ld_logits, int rows, int hidden, int E,
                                                 float* xs) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __syncthreads();
    for (int k = threadIdx.x; k < hidden; k += blockDim.x) xs[k] = __bfloat162float(x[static_cast<size_t>(row) * ldx + k]);
    __syncthreads();
    for (int e = warp; e < E; e += nwarps) {
      const WT* wr = w + static_cast<size_t>(e) * hidden;
      float acc = 0.f;
      for (int k = lane; k < hidden; k += 32) {
        float wv;
        if constexpr (sizeof(WT) == 4) wv = wr[k];
        else wv = __bfloat162float(wr[k]);
        acc = fmaf(xs[k], wv, acc);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) logits[static_cast<size_t>(row) * ld_logits + e] = acc;
    }
  }
}

__global__ void __launch_bounds__(256)
router_fp32_kernel(const __nv_bfloat16* x, int ldx, const void* w, int w_fp32, float* logits, int ld_logits, int rows, int hidden, int E) {
  extern __shared__ float xs_dyn[];
  if (w_fp32) router_fp32_rows(x, ldx, static_cast<const float*>(w), logits, ld_logits, rows, hidden, E, xs_dyn);
  else router_fp32_rows(x, ldx, static_cast<const __nv_bfloat16*>(w), logits, ld_logits, rows, hidden, E, xs_dyn);
}

// Lane node: the same projection for the invocation the Lane holds; returns at once unless the layer's router asks
// for fp32 logits (the payload-precision router runs as a tensor-core GEMM node instead).
__global__ void __launch_bounds__(256)
moe_lane_router_fp32_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws) {
  extern __shared__ float xs_dyn[];
  const lane::MoeLayer* m = lane_moe_layer(slots, cur);
  if (m == nullptr || m->router_precision == 0) return;
  const lane::InstanceSlot& s = slots[cur->instance];
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(s.input);
  if (m->router_precision == 2)
    router_fp32_rows(x, s.hidden, static_cast<const float*>(m->router_raw), ws->logits32, m->e_pad, static_cast<int>(cur->rows), s.hidden,
                     m->num_experts, xs_dyn);
  else
    router_fp32_rows(x, s.hidden, static_cast<const __nv_bfloat16*>(m->router_raw), ws->logits32, m->e_pad, static_cast<int>(cur->rows),
                     s.hidden, m->num_experts, xs_dyn);
}

}  // namespace moe
}  // namespace xpool

using namespace xpool::moe;

static int last_error() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" int xp_router_fp32(const void* x, int ldx, const void* w, int w_fp32, float* logits, int ld_logits, int rows, int hidden,
                              int num_experts, void* stream) {
  if (rows <= 0) return 0;
  if (hidden <= 0 || hidden > 16384 || num_experts <= 0) return -10;
  const int grid = rows < 148 * 4 ? rows : 148 * 4;
  router_fp32_kernel<<<grid, 256, hidden * sizeof(float), reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, w, w_fp32, logits, ld_logits, rows, hidden, num_experts);
  return last_error();
}

extern "C" int xp_router_topk(const XpRouterArgs* a, void* stream) {
  if (a->rows <= 0) return 0;
  if (a->num_experts > 32 * kMaxPerLane || a->top_k > 32 || a->top_k > a->num_experts) return -10;
  router_topk_kernel<<<(a->rows + 3) / 4, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  return last_error();
}

extern "C" int xp_moe_route(const XpRouteArgs* a, void* stream) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int n_local = a->expert_hi - a->expert_lo;
  if (n_local < 1 || n_local > 1023) return -10;
  const int n_routes = a->rows * a->top_k;
  cudaMemsetAsync(a->route_pos, 0xff, sizeof(int) * n_routes, s);  // -1: not handled by this rank
  route_count_kernel<<<n_local, 256, 0, s>>>(a->topk_ids, n_routes, a->expert_lo, a->counts);
  route_offsets_tiles_kernel<<<1, 1024, 0, s>>>(a->counts, n_local, a->offsets, a->tm_gateup, a->bn_gateup,
                                                reinterpret_cast<int4*>(a->tiles_gateup), a->n_tiles_gateup, a->tm_down,
                                                a->bn_down, reinterpret_cast<int4*>(a->tiles_down), a->n_tiles_down);
  route_place_kernel<<<n_local, 256, 0, s>>>(a->topk_ids, n_routes, a->top_k, a->expert_lo, a->offsets, a->perm_token,
                                             a->route_pos);
  return last_error();
}

extern "C" int xp_moe_gather(const void* x, const int* perm_token, const int* n_rows_ptr, void* out, int max_rows,
                             int hidden, int ldx, void* stream) {
  if (hidden % 8 || ldx % 8) return -10;
  gather_rows_kernel<<<max_rows, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), perm_token, n_rows_ptr, reinterpret_cast<uint4*>(out), hidden / 8, ldx / 8);
  return last_error();
}

extern "C" int xp_moe_combine(const void* y, const int* route_pos, const float* weights, void* out, int rows, int top_k,
                              int hidden, int ld_out, void* stream) {
  if (rows <= 0) return 0;
  if (hidden % 8) return -10;
  combine_kernel<<<rows, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(y), route_pos, weights, reinterpret_cast<__nv_bfloat16*>(out), top_k, hidden,
      ld_out);
  return last_error();
}
