// Device-resident state of an FFN device's Executor Lanes.
//
// An FFN device serves many Instances (models) with a few Lanes. A Lane is a
// CUDA stream that keeps replaying one generic graph:
//
//   lane_wait      scans the Instances' invocation slots, lets the device-side
//                  Scheduler pick one for this Lane (FIFO / Random / SLO), and
//                  publishes the choice in LaneCur        (reference K3 + K5)
//   gate/up GEMM   tcgen05 GEMM whose Problem is read from the descriptor table
//                  entry of (instance, layer): weights are bound per call by
//                  table lookup, not by patching graph nodes     (K6 + K18/K19)
//   down GEMM      same, epilogue stores straight into the attention device's
//                  partial buffer for this TP rank                   (K18 + K11)
//   lane_complete  releases the completion word on the attention device and
//                  returns the Lane to the Scheduler                      (K10)
//
// One graph therefore serves every layer signature of every model (the
// reference captures one child graph per Signature x Capacity and switches
// between them with conditional nodes, src/cext/ffnagent/runtime.cu:701-1006).
// No Lane ever waits on another FFN device: TP partials are pushed to the
// attention device and folded there in rank order.
#pragma once

#include "xpool/gemm_ws.cuh"
#include "xpool/protocol.hpp"
#include "xpool/scheduler.hpp"
#include "xpool/hooks.cuh"
#include "xpool/trace.cuh"

namespace xpool {
namespace lane {

constexpr int kMaxInstances = 32;
constexpr int kMaxLanes = 8;
constexpr int kBnVariants = 5;  // 16, 32, 64, 128, 256
constexpr int kRowBuckets = 16; // row-count buckets 2^0 .. 2^15 (the reference's Capacities)

// Router and expert bookkeeping of a mixture-of-experts layer. The expert weights themselves are
// bound through LayerEntry::tmap_gateup / tmap_down (all local experts stacked along the rows).
struct alignas(128) MoeLayer {
  CUtensorMap tmap_router;      // [e_pad, hidden] box {64, 128}; rows past num_experts are zero
  const float* correction_bias; // optional, added to the scores for selection only
  const float* router_bias;     // optional, added to the logits
  int num_experts, top_k;
  int expert_lo, expert_hi;     // experts this rank owns (expert parallelism); all of them under TP
  int sigmoid, renormalize;
  float scale;
  int e_pad;
  uint8_t bn_router[kRowBuckets], splits_router[kRowBuckets];
  int router_precision;         // 0 payload (tensor-core GEMM, bf16 logits), 1 fp32 logits from payload weights, 2 fp32 weights
  int reserved;
  const void* router_raw;       // [num_experts, hidden] router weights for the fp32 projection (bf16, or fp32 for precision 2)
};

// Per (instance, layer): weight tensor maps and epilogue parameters.
struct alignas(128) LayerEntry {
  CUtensorMap tmap_gateup;  // [2 * inter_local (or inter_local), hidden] box {64, 128}
  CUtensorMap tmap_down;    // [hidden, inter_local]
  const float* bias_gateup;
  const float* bias_down;
  int inter_local;
  int gated;                // 1: SwiGLU-style dual projection
  int w_tiled;
  int kind;                 // LayerKind
  float gate_limit, up_add, act_alpha;
  int reserved;
  const MoeLayer* moe;      // null for a dense layer
  // shared experts of a MoE layer (one dense gated FFN added to the routed output); 0: none
  int shared_inter_local;
  int reserved2;
  CUtensorMap tmap_shared_gateup;  // [2 * shared_inter_local, hidden]
  CUtensorMap tmap_shared_down;    // [hidden, shared_inter_local]
  uint8_t bn_sh_gateup[kRowBuckets], splits_sh_gateup[kRowBuckets];
  uint8_t bn_sh_down[kRowBuckets], splits_sh_down[kRowBuckets];
  // tile width and split-K factor per row bucket, chosen on the host at install time
  uint8_t bn_gateup[kRowBuckets], splits_gateup[kRowBuckets];
  uint8_t bn_down[kRowBuckets], splits_down[kRowBuckets];
};

// Per instance slot on this FFN rank.
struct alignas(128) InstanceSlot {
  CUtensorMap tmap_x[kBnVariants];    // input payload [capacity, hidden]
  CUtensorMap tmap_act[kBnVariants];  // activation scratch [capacity, max inter_local]
  const void* input;                  // the payload buffer tmap_x covers (plain loads by the MoE row gather)
  const uint32_t* in_flag;            // local word the attention side releases (sequence)
  const InvocationRecord* record;     // local record written before the flag
  void* act;                          // local scratch between the two GEMMs
  void* out_peer;                     // attention device: partial buffer of this TP rank
  uint32_t* done_flag_peer;           // attention device: completion sequence word
  FailureSlot* failure_local;         // this slot's failure word (the attention side writes it when its wait ran out)
  FailureSlot* failure_peer;          // attention device: the Instance's canonical failure slot
  const LayerEntry* layers;           // this instance's layer table
  int capacity_rows;
  int hidden;
  int num_layers;
  int act_ld;                         // leading dimension of the scratch (max inter_local)
};

// Scratch of one Lane for mixture-of-experts layers (sized for the largest MoE instance).
struct MoeLaneWs {
  __nv_bfloat16* logits;  // [capacity_rows, e_pad of the layer]
  float* logits32;        // the same in fp32, for routers that ask for fp32 logits
  int* ids;               // [capacity_rows, top_k]
  float* weights;         // [capacity_rows, top_k]
  int* offsets;           // [n_local + 1] first route position of every local expert
  int* perm_token;        // [routes] token of the route at a position
  int* route_pos;         // [capacity_rows, top_k] position of a route, -1 if another rank owns the expert
  int4* tiles_gateup;     // grouped-GEMM tile tables
  int4* tiles_down;
  int* n_tiles;           // [2]
  void* xp;               // [routes, hidden] gathered rows
  void* act;              // [routes, inter_local]
  void* yp;               // [routes, hidden] expert outputs
  void* comb;             // [capacity_rows, hidden] routed result when shared experts still have to be added
  int cap_routes;
  int reserved;
};

// Tensor maps over a Lane's MoE scratch, laid out for one instance's hidden / inter sizes.
struct alignas(64) MoeLaneMaps {
  CUtensorMap tmap_xp[kBnVariants];
  CUtensorMap tmap_act[kBnVariants];
};

// Tile width of the grouped GEMMs: the power of two covering the mean routes per expert.
__host__ __device__ inline int moe_tile_width(int rows, int top_k, int n_local) {
  int avg = rows * top_k / (n_local > 0 ? n_local : 1);
  if (avg < 1) avg = 1;
  int bn = 16;
  while (bn < avg && bn < 128) bn <<= 1;
  return bn;
}

struct alignas(128) LaneCtl {
  uint32_t lock;
  uint32_t shutdown;       // host-written: Lanes stop waiting and report idle
  uint32_t n_instances;
  uint32_t n_lanes;
  uint32_t policy;         // SchedulerPolicyKind
  uint32_t reserved;
  uint64_t seed;
  uint64_t next_ticket;
  uint64_t served[kMaxInstances];  // invocations completed per instance (statistics)
  trace::BufferView trace;         // fabric observer (null events pointer: off)
  FailureSlot failure;             // first failure met on this device (canonical for the generation once reported)
  uint32_t pe;                     // this device's PE number (origin of the failures it claims)
  SchedulerEntry entries[kMaxInstances];
  LaneState lanes[kMaxLanes];
};

// What a Lane is currently executing; written by lane_wait, read by the GEMMs.
struct alignas(64) LaneCur {
  uint32_t valid;     // 0: idle replay (lease ran out, shutdown or error)
  uint32_t instance;
  uint32_t layer;
  uint32_t rows;
  uint32_t sequence;  // invocation sequence being served
  uint32_t mode;
  uint64_t lease;     // scheduler lease
  uint64_t t_start_ns;
  uint32_t idle_replays;
  uint32_t result_code;
};

__device__ __forceinline__ bool lock_acquire(uint32_t* lock, uint64_t deadline_ns) {
  uint32_t spins = 0;
  while (atomicCAS(lock, 0u, 1u) != 0u) {
    if ((++spins & 0xffu) == 0 && sm100::global_timer_ns() > deadline_ns) return false;
    __nanosleep(50);
  }
  __threadfence();
  return true;
}
__device__ __forceinline__ void lock_release(uint32_t* lock) {
  __threadfence();
  atomicExch(lock, 0u);
}

__host__ __device__ inline int bn_index(int bn) {
  return bn <= 16 ? 0 : bn <= 32 ? 1 : bn <= 64 ? 2 : bn <= 128 ? 3 : 4;
}

}  // namespace lane
}  // namespace xpool
