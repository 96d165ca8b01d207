// Executor-Lane kernels and the host object that owns an FFN device's Lane state
// (see xpool/lane.cuh for the design), plus the attention-side flag wait.
#include <string.h>

#include <algorithm>
#include <atomic>
#include <deque>
#include <string>
#include <thread>
#include <vector>

#include "xpool/api.h"
#include "xpool/lane.cuh"
#include "xpool/tensormap.hpp"

namespace xpool {
namespace gemm {
// defined in gemm.cu
struct TileChoice {
  int bn, splits;
};
TileChoice choose_tiles_host(int tm, int rows, int kb, int dual, int sms, size_t ws_bytes_available);
__global__ void gemm_lane_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, int phase, float* ws,
                                 uint32_t* counters, int smem_budget, uint32_t* status, const lane::MoeLaneWs* mws,
                                 const lane::MoeLaneMaps* mmaps);
}  // namespace gemm
namespace moe {
// defined in moe.cu
__global__ void moe_lane_topk_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws);
__global__ void moe_lane_route_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws);
__global__ void moe_lane_gather_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws);
__global__ void moe_lane_combine_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws);
__global__ void moe_lane_router_fp32_kernel(const lane::InstanceSlot* slots, const lane::LaneCur* cur, const lane::MoeLaneWs* ws);
}  // namespace moe

namespace lane {

// First failure wins on this device; the winner copies it into the failure slot of every Instance's attention
// rank (first wins there as well), so that every kernel waiting for this device leaves with the same payload
// (the reference's converge_failure + publish_to_all, src/cext/fabric/atnagent.cu:101-119, coordinator.cu:403-410).
__device__ void converge_failure(LaneCtl* ctl, const InstanceSlot* slots, uint32_t result_code, uint32_t instance,
                                 uint32_t sequence, uint32_t layer) {
  if (!failure::claim(&ctl->failure, result_code, ctl->pe, instance, sequence, layer)) return;
  hooks::Point<hooks::LaneFailureClaimed>::hooks({ctl->trace, instance, result_code});
  for (uint32_t i = 0; i < ctl->n_instances; ++i)
    failure::claim(slots[i].failure_peer, result_code, ctl->pe, instance, sequence, layer);
}

// One thread: find work for this Lane or give up when the lease runs out.
__global__ void lane_wait_kernel(LaneCtl* ctl, const InstanceSlot* slots, LaneCur* cur, uint32_t lane_index,
                                 uint64_t lease_ns) {
  cur->valid = 0;
  cur->rows = 0;
  cur->result_code = 0;
  const uint64_t t0 = sm100::global_timer_ns();
  const uint64_t deadline = t0 + lease_ns;
  const uint32_t n = ctl->n_instances;
  uint32_t spins = 0;
  while (true) {
    if (sm100::ld_relaxed_sys(&ctl->shutdown) != 0) {
      cur->result_code = static_cast<uint32_t>(ResultCode::Shutdown);
      hooks::Point<hooks::LaneShutdown>::hooks({ctl->trace, lane_index});
      return;
    }
    // A failed generation serves nothing more: a failure claimed on this device, or one that an attention rank
    // wrote into the slot of one of its Instances, ends the iteration (the slot's failure becomes this device's).
    if (failure::claimed(&ctl->failure)) {
      cur->result_code = static_cast<uint32_t>(ResultCode::Shutdown);
      hooks::Point<hooks::LaneFailureObserved>::hooks({ctl->trace, lane_index, ctl->failure.origin});
      return;
    }
    for (uint32_t i = 0; i < n; ++i) {
      const FailureSlot* f = slots[i].failure_local;
      if (f != nullptr && sm100::ld_acquire_sys(&f->claim) == kFailureClaimed)
        failure::claim(&ctl->failure, f->result_code, f->origin, i, f->invocation_sequence, f->layer_ordinal);
    }
    // cheap look before taking the lock: is any slot ahead of its completed sequence?
    bool any = false;
    for (uint32_t i = 0; i < n; ++i) {
      const uint32_t seq = sm100::ld_acquire_sys(slots[i].in_flag);
      const uint32_t done = static_cast<uint32_t>(ctl->entries[i].completed_sequence);
      if (static_cast<int32_t>(seq - done) > 0 && ctl->entries[i].state != static_cast<uint32_t>(EntryState::Running))
        any = true;
    }
    if (any && lock_acquire(&ctl->lock, sm100::global_timer_ns() + 1000000ull)) {
      Scheduler sched(ctl->entries, n, ctl->lanes, ctl->n_lanes,
                      SchedulerPolicy{static_cast<SchedulerPolicyKind>(ctl->policy), ctl->seed}, &ctl->next_ticket);
      for (uint32_t i = 0; i < n; ++i) {
        SchedulerEntry& e = ctl->entries[i];
        if (e.state != static_cast<uint32_t>(EntryState::Idle)) continue;
        const uint32_t seq = sm100::ld_acquire_sys(slots[i].in_flag);
        const uint32_t done = static_cast<uint32_t>(e.completed_sequence);
        const int32_t ahead = static_cast<int32_t>(seq - done);
        if (ahead > 0) {
          sched.enqueue(i, e.completed_sequence + static_cast<uint64_t>(ahead), slots[i].record->deadline_us);
          hooks::Point<hooks::LaneDiscovered>::hooks({ctl->trace, i, seq});
        }
      }
      const Decision d = sched.try_schedule_on(lane_index);
      lock_release(&ctl->lock);
      if (d.scheduled) {
        const InstanceSlot& s = slots[d.instance];
        const InvocationRecord* rec = s.record;
        uint32_t rows = rec->rows, layer = rec->layer_ordinal;
        uint32_t rc = 0;
        if (rows > static_cast<uint32_t>(s.capacity_rows) || layer >= static_cast<uint32_t>(s.num_layers) ||
            s.layers[layer < static_cast<uint32_t>(s.num_layers) ? layer : 0].inter_local == 0) {  // not held here
          rc = static_cast<uint32_t>(ResultCode::ProtocolMismatch);
          rows = 0;
          layer = 0;
        }
        if (rec->forward_mode == static_cast<uint32_t>(ForwardMode::Idle)) rows = 0;
        cur->instance = d.instance;
        cur->layer = layer;
        cur->rows = rows;
        cur->sequence = static_cast<uint32_t>(ctl->entries[d.instance].invocation_sequence);
        cur->mode = rec->forward_mode;
        cur->lease = d.lease_sequence;
        cur->t_start_ns = sm100::global_timer_ns();
        cur->result_code = rc;
        __threadfence();
        cur->valid = 1;
        if (rc != 0) {
          hooks::Point<hooks::LaneRejected>::hooks({ctl->trace, d.instance, rc});
          converge_failure(ctl, slots, rc, d.instance, cur->sequence, rec->layer_ordinal);
        }
        hooks::Point<hooks::LaneAdmitted>::hooks({ctl->trace, d.instance, layer, rows});
        return;
      }
    }
    if ((++spins & 0xfu) == 0 && sm100::global_timer_ns() > deadline) {
      cur->idle_replays += 1;
      hooks::Point<hooks::LaneIdle>::hooks({ctl->trace, lane_index, cur->idle_replays});
      return;
    }
    __nanosleep(200);
  }
}

// One thread: publish the completion on the attention device, free the Lane.
__global__ void lane_complete_kernel(LaneCtl* ctl, const InstanceSlot* slots, LaneCur* cur, uint32_t lane_index,
                                     const uint32_t* status) {
  if (cur->valid == 0) return;
  const InstanceSlot& s = slots[cur->instance];
  // a bounded wait inside the Lane's GEMMs ran out: the output is not trustworthy
  if (cur->result_code == 0 && status != nullptr && *status != 0) {
    cur->result_code = static_cast<uint32_t>(ResultCode::Timeout);
    converge_failure(ctl, slots, cur->result_code, cur->instance, cur->sequence, cur->layer);
  }
  CompletionRecord* done = reinterpret_cast<CompletionRecord*>(s.done_flag_peer);
  done->result_code = cur->result_code;
  done->rows = cur->rows;
  __threadfence_system();
  sm100::st_release_sys(&done->sequence, cur->sequence);
  // The Lane must go back to the scheduler or the Instance stays Running for ever: keep trying for the
  // data-plane limit, and make a failure of it if even that runs out.
  bool released = false;
  for (int attempt = 0; attempt < 5000 && !released; ++attempt) {
    if (lock_acquire(&ctl->lock, sm100::global_timer_ns() + 1000000ull)) {
      Scheduler sched(ctl->entries, ctl->n_instances, ctl->lanes, ctl->n_lanes,
                      SchedulerPolicy{static_cast<SchedulerPolicyKind>(ctl->policy), ctl->seed}, &ctl->next_ticket);
      sched.release(cur->instance, cur->lease);
      ctl->served[cur->instance] += 1;
      lock_release(&ctl->lock);
      released = true;
    }
  }
  if (!released) {
    hooks::Point<hooks::LaneLockTimeout>::hooks({ctl->trace, lane_index, 1});
    converge_failure(ctl, slots, static_cast<uint32_t>(ResultCode::Timeout), cur->instance, cur->sequence, cur->layer);
  }
  hooks::Point<hooks::LaneCompleted>::hooks({ctl->trace, cur->instance, cur->sequence});
  cur->valid = 0;
}

// Attention side: up to 8 threads each wait until their flag reaches *want.
__global__ void wait_flags_kernel(XpWaitArgs a) {
  const int i = threadIdx.x;
  if (i >= a.n) return;
  const trace::BufferView tv{static_cast<trace::Event*>(a.trace_events), static_cast<trace::BufferState*>(a.trace_state),
                             a.trace_capacity, 0};
  const uint32_t want = a.want_ptr != nullptr ? *a.want_ptr : a.want;
  hooks::Point<hooks::AtnWaitBegin>::hooks({tv, static_cast<uint32_t>(i), want});
  const uint64_t deadline = sm100::global_timer_ns() + a.wait_ns;
  const int rc = sm100::wait_flag_ge(a.flags[i], want, deadline, a.cancel);
  hooks::Point<hooks::AtnWaitEnd>::hooks({tv, static_cast<uint32_t>(i), want, static_cast<uint32_t>(rc)});
  if (rc == 0) return;
  if (a.status != nullptr) atomicCAS(a.status, 0u, rc == 2 ? 5u /*cancelled by a failure elsewhere*/ : 4u /*timed out*/);
  if (rc == 1) {
    // our own wait ran out and nobody reported a failure: this rank claims it and tells the FFN ranks
    FailureSlot* f = static_cast<FailureSlot*>(a.failure);
    if (failure::claim(f, static_cast<uint32_t>(ResultCode::Timeout), a.origin_pe, a.instance, want, 0xffffffffu)) {
      for (int d = 0; d < a.n_peer_failures && d < 8; ++d)
        failure::claim(static_cast<FailureSlot*>(a.peer_failures[d]), static_cast<uint32_t>(ResultCode::Timeout), a.origin_pe,
                       a.instance, want, 0xffffffffu);
    }
  }
}

// Bumps a device-resident sequence counter and releases the new value into up to 8 flag words
// (typically one per peer GPU): the producer half of a flag handshake whose consumer half is
// wait_flags_kernel with want_ptr on a counter that advances in step.
__global__ void signal_flags_kernel(XpSignalArgs a) {
  const uint32_t seq = *a.seq_counter + 1;
  __threadfence_system();  // everything this stream wrote before is visible before the flags move
  if (threadIdx.x < static_cast<unsigned>(a.n)) sm100::st_release_sys(a.flags[threadIdx.x], seq);
  __syncthreads();
  if (threadIdx.x == 0) *a.seq_counter = seq;
}

struct Runtime {
  int n_instances = 0, n_lanes = 0, sms = 148;
  size_t ws_bytes_per_lane = 0;
  std::vector<InstanceSlot> slots_h;
  std::vector<std::vector<LayerEntry>> layers_h;
  std::vector<LayerEntry*> layers_d;
  LaneCtl* ctl_d = nullptr;
  InstanceSlot* slots_d = nullptr;
  LaneCur* cur_d = nullptr;
  float* ws_d = nullptr;
  uint32_t* counters_d = nullptr;
  uint32_t* status_d = nullptr;
  trace::Event* trace_events_d = nullptr;
  trace::BufferState* trace_state_d = nullptr;
  uint32_t trace_capacity = 0;
  bool committed = false;
  // mixture of experts (only when some installed layer has experts)
  std::vector<std::vector<MoeLayer>> moe_h;   // per instance, one entry per MoE layer (dense layers keep a blank)
  std::vector<MoeLayer*> moe_d;
  std::vector<int> moe_top_k, moe_inter, moe_n_local, moe_e_pad;  // per instance maxima (0: dense instance)
  MoeLaneWs* mws_d = nullptr;      // [n_lanes]
  MoeLaneMaps* mmaps_d = nullptr;  // [n_lanes][n_instances]
  std::vector<void*> moe_allocs;
  bool has_moe = false;
  bool has_fp32_router = false;
  int max_hidden = 0;
  int pe = 0;
  // replay threads (xp_lane_threads_start): one host thread, stream and instantiated graph per Lane
  int device = 0;
  std::vector<std::thread> threads;
  std::vector<cudaStream_t> lane_streams;
  std::vector<cudaGraph_t> lane_graphs;
  std::vector<cudaGraphExec_t> lane_execs;
  std::atomic<bool> stop_threads{false};
  std::atomic<int> thread_error{0};      // first CUDA error code a replay thread met (0: none)
  std::atomic<uint64_t> replays{0};
};

constexpr size_t kCounterWords = 1 << 14;

}  // namespace lane
}  // namespace xpool

using namespace xpool;
using lane::Runtime;

extern "C" void* xp_lane_create(int n_instances, int n_lanes, int policy, uint64_t seed, size_t ws_bytes_per_lane) {
  if (n_instances < 1 || n_instances > lane::kMaxInstances || n_lanes < 1 || n_lanes > lane::kMaxLanes) return nullptr;
  auto* rt = new Runtime();
  rt->n_instances = n_instances;
  rt->n_lanes = n_lanes;
  rt->ws_bytes_per_lane = ws_bytes_per_lane;
  int dev = 0;
  cudaGetDevice(&dev);
  rt->device = dev;
  cudaDeviceGetAttribute(&rt->sms, cudaDevAttrMultiProcessorCount, dev);
  rt->slots_h.resize(n_instances);
  rt->layers_h.resize(n_instances);
  rt->layers_d.assign(n_instances, nullptr);
  rt->moe_h.resize(n_instances);
  rt->moe_d.assign(n_instances, nullptr);
  rt->moe_top_k.assign(n_instances, 0);
  rt->moe_inter.assign(n_instances, 0);
  rt->moe_n_local.assign(n_instances, 0);
  rt->moe_e_pad.assign(n_instances, 0);
  for (auto& s : rt->slots_h) memset(&s, 0, sizeof(s));
  lane::LaneCtl ctl;
  memset(&ctl, 0, sizeof(ctl));
  ctl.n_instances = n_instances;
  ctl.n_lanes = n_lanes;
  ctl.policy = policy;
  ctl.seed = seed;
  ctl.next_ticket = 1;
  for (int i = 0; i < lane::kMaxInstances; ++i) ctl.entries[i].lane = kNoLane;
  bool ok = cudaMalloc(&rt->ctl_d, sizeof(lane::LaneCtl)) == cudaSuccess &&
            cudaMalloc(&rt->slots_d, sizeof(lane::InstanceSlot) * n_instances) == cudaSuccess &&
            cudaMalloc(&rt->cur_d, sizeof(lane::LaneCur) * n_lanes) == cudaSuccess &&
            cudaMalloc(&rt->ws_d, ws_bytes_per_lane * n_lanes) == cudaSuccess &&
            cudaMalloc(&rt->counters_d, lane::kCounterWords * 4 * n_lanes) == cudaSuccess &&
            cudaMalloc(&rt->status_d, 64) == cudaSuccess;
  if (ok) {
    cudaMemcpy(rt->ctl_d, &ctl, sizeof(ctl), cudaMemcpyHostToDevice);
    cudaMemset(rt->cur_d, 0, sizeof(lane::LaneCur) * n_lanes);
    cudaMemset(rt->counters_d, 0, lane::kCounterWords * 4 * n_lanes);
    cudaMemset(rt->status_d, 0, 64);
  } else {
    delete rt;
    return nullptr;
  }
  return rt;
}

extern "C" int xp_lane_set_instance(void* h, int idx, const XpLaneInstanceDesc* d) {
  auto* rt = static_cast<Runtime*>(h);
  if (idx < 0 || idx >= rt->n_instances || d->num_layers < 1) return -1;
  lane::InstanceSlot& s = rt->slots_h[idx];
  static const int kBn[lane::kBnVariants] = {16, 32, 64, 128, 256};
  for (int v = 0; v < lane::kBnVariants; ++v) {
    if (tmap::encode_2d(&s.tmap_x[v], d->input, d->capacity_rows, d->hidden, static_cast<uint64_t>(d->hidden) * 2,
                        kBn[v], 64, 2) != 0)
      return -2;
    if (tmap::encode_2d(&s.tmap_act[v], d->act, d->capacity_rows, d->act_ld, static_cast<uint64_t>(d->act_ld) * 2,
                        kBn[v], 64, 2) != 0)
      return -3;
  }
  s.input = d->input;
  s.in_flag = reinterpret_cast<const uint32_t*>(d->in_flag);
  s.record = reinterpret_cast<const InvocationRecord*>(d->record);
  s.act = d->act;
  s.out_peer = d->out_peer;
  s.done_flag_peer = reinterpret_cast<uint32_t*>(d->done_record_peer);
  s.failure_local = reinterpret_cast<FailureSlot*>(reinterpret_cast<uint8_t*>(const_cast<void*>(d->record)) + kFailureSlotOffset);
  s.failure_peer = reinterpret_cast<FailureSlot*>(d->failure_peer);
  rt->pe = d->pe;
  s.capacity_rows = d->capacity_rows;
  s.hidden = d->hidden;
  s.num_layers = d->num_layers;
  s.act_ld = d->act_ld;
  rt->layers_h[idx].assign(d->num_layers, lane::LayerEntry{});
  rt->moe_h[idx].assign(d->num_layers, lane::MoeLayer{});
  return 0;
}

extern "C" int xp_lane_set_layer(void* h, int inst, int layer, const XpLaneLayerDesc* d) {
  auto* rt = static_cast<Runtime*>(h);
  if (inst < 0 || inst >= rt->n_instances) return -1;
  auto& layers = rt->layers_h[inst];
  if (layer < 0 || layer >= static_cast<int>(layers.size())) return -1;
  const lane::InstanceSlot& s = rt->slots_h[inst];
  const bool is_moe = d->num_experts > 0;
  if (d->inter_local % 128 != 0 || s.hidden % 128 != 0 || (!is_moe && d->inter_local > s.act_ld)) return -2;
  lane::LayerEntry& e = layers[layer];
  memset(&e, 0, sizeof(e));
  const int n_local = is_moe ? d->expert_hi - d->expert_lo : 1;
  if (is_moe && (d->w_tiled || !d->gated || n_local < 1 || n_local > 1024 || d->expert_lo < 0 ||
                 d->expert_hi > d->num_experts || d->num_experts > 256 || d->top_k < 1 || d->top_k > 32 ||
                 d->top_k > d->num_experts || d->router == nullptr))
    return -4;
  const int gu_rows = d->inter_local * (d->gated ? 2 : 1) * n_local;
  const uint64_t down_rows = static_cast<uint64_t>(s.hidden) * n_local;
  int rc;
  if (is_moe) {
    rc = tmap::encode_2d(&e.tmap_gateup, d->w_gateup, gu_rows, s.hidden, static_cast<uint64_t>(s.hidden) * 2, 128, 64, 2);
    if (rc == 0)
      rc = tmap::encode_2d(&e.tmap_down, d->w_down, down_rows, d->inter_local, static_cast<uint64_t>(d->inter_local) * 2, 128, 64, 2);
    lane::MoeLayer& m = rt->moe_h[inst][layer];
    memset(&m, 0, sizeof(m));
    m.e_pad = (d->num_experts + 127) / 128 * 128;
    if (rc == 0)
      rc = tmap::encode_2d(&m.tmap_router, d->router, m.e_pad, s.hidden, static_cast<uint64_t>(s.hidden) * 2, 128, 64, 2);
    m.correction_bias = d->correction_bias;
    m.router_bias = d->router_bias;
    m.router_precision = d->router_precision;
    m.router_raw = d->router_raw;
    if (d->router_precision != 0 && d->router_raw == nullptr) return -5;
    if (d->router_precision != 0) rt->has_fp32_router = true;
    rt->max_hidden = std::max(rt->max_hidden, s.hidden);
    m.num_experts = d->num_experts;
    m.top_k = d->top_k;
    m.expert_lo = d->expert_lo;
    m.expert_hi = d->expert_hi;
    m.sigmoid = d->sigmoid;
    m.renormalize = d->renormalize;
    m.scale = d->scale;
    for (int b = 0; b < lane::kRowBuckets; ++b) {
      const int rows = std::min(1 << b, s.capacity_rows);
      gemm::TileChoice r = gemm::choose_tiles_host(m.e_pad / 128, rows, s.hidden / 64, 0, rt->sms, rt->ws_bytes_per_lane);
      m.bn_router[b] = static_cast<uint8_t>(r.bn == 256 ? 255 : r.bn);
      m.splits_router[b] = static_cast<uint8_t>(r.splits);
    }
    rt->has_moe = true;
    rt->moe_top_k[inst] = std::max(rt->moe_top_k[inst], d->top_k);
    rt->moe_inter[inst] = std::max(rt->moe_inter[inst], d->inter_local);
    rt->moe_n_local[inst] = std::max(rt->moe_n_local[inst], n_local);
    rt->moe_e_pad[inst] = std::max(rt->moe_e_pad[inst], m.e_pad);
    e.kind = 2;
    if (d->shared_inter_local > 0) {
      if (d->shared_inter_local % 128 != 0 || d->shared_inter_local > s.act_ld || d->w_shared_gateup == nullptr ||
          d->w_shared_down == nullptr)
        return -5;
      if (rc == 0)
        rc = tmap::encode_2d(&e.tmap_shared_gateup, d->w_shared_gateup, 2 * d->shared_inter_local, s.hidden,
                             static_cast<uint64_t>(s.hidden) * 2, 128, 64, 2);
      if (rc == 0)
        rc = tmap::encode_2d(&e.tmap_shared_down, d->w_shared_down, s.hidden, d->shared_inter_local,
                             static_cast<uint64_t>(d->shared_inter_local) * 2, 128, 64, 2);
      e.shared_inter_local = d->shared_inter_local;
      for (int b = 0; b < lane::kRowBuckets; ++b) {
        const int rows = std::min(1 << b, s.capacity_rows);
        gemm::TileChoice g = gemm::choose_tiles_host(d->shared_inter_local / 128, rows, s.hidden / 64, 1, rt->sms, rt->ws_bytes_per_lane);
        gemm::TileChoice w = gemm::choose_tiles_host(s.hidden / 128, rows, d->shared_inter_local / 64, 0, rt->sms, rt->ws_bytes_per_lane);
        e.bn_sh_gateup[b] = static_cast<uint8_t>(g.bn == 256 ? 255 : g.bn);
        e.splits_sh_gateup[b] = static_cast<uint8_t>(g.splits);
        e.bn_sh_down[b] = static_cast<uint8_t>(w.bn == 256 ? 255 : w.bn);
        e.splits_sh_down[b] = static_cast<uint8_t>(w.splits);
      }
    }
  } else if (d->w_tiled) {
    rc = tmap::encode_2d(&e.tmap_gateup, d->w_gateup, static_cast<uint64_t>(gu_rows) * (s.hidden / 64), 64, 128, 128, 64, 2);
    if (rc == 0)
      rc = tmap::encode_2d(&e.tmap_down, d->w_down, static_cast<uint64_t>(s.hidden) * (d->inter_local / 64), 64, 128, 128, 64, 2);
  } else {
    rc = tmap::encode_2d(&e.tmap_gateup, d->w_gateup, gu_rows, s.hidden, static_cast<uint64_t>(s.hidden) * 2, 128, 64, 2);
    if (rc == 0)
      rc = tmap::encode_2d(&e.tmap_down, d->w_down, s.hidden, d->inter_local, static_cast<uint64_t>(d->inter_local) * 2, 128, 64, 2);
  }
  if (rc != 0) return -3;
  e.bias_gateup = d->bias_gateup;
  e.bias_down = d->bias_down;
  e.inter_local = d->inter_local;
  e.gated = d->gated;
  e.w_tiled = d->w_tiled;
  if (!is_moe) e.kind = 1;
  e.gate_limit = d->gate_limit;
  e.up_add = d->up_add;
  e.act_alpha = d->act_alpha;
  for (int b = 0; b < lane::kRowBuckets; ++b) {
    const int rows = std::min(1 << b, s.capacity_rows);
    gemm::TileChoice g = gemm::choose_tiles_host(d->inter_local / 128, rows, s.hidden / 64, d->gated, rt->sms, rt->ws_bytes_per_lane);
    gemm::TileChoice w = gemm::choose_tiles_host(s.hidden / 128, rows, d->inter_local / 64, 0, rt->sms, rt->ws_bytes_per_lane);
    e.bn_gateup[b] = static_cast<uint8_t>(g.bn == 256 ? 255 : g.bn);
    e.splits_gateup[b] = static_cast<uint8_t>(g.splits);
    e.bn_down[b] = static_cast<uint8_t>(w.bn == 256 ? 255 : w.bn);
    e.splits_down[b] = static_cast<uint8_t>(w.splits);
  }
  return 0;
}

// Allocates the per-Lane MoE scratch (sized for the largest MoE instance) and the tensor maps
// over it for every MoE instance.
static int commit_moe(Runtime* rt) {
  size_t routes = 0, rows = 0, hidden = 0, inter = 0, e_pad = 0, n_local = 0, tm = 0;
  for (int i = 0; i < rt->n_instances; ++i) {
    if (rt->moe_top_k[i] == 0) continue;
    const lane::InstanceSlot& s = rt->slots_h[i];
    routes = std::max<size_t>(routes, static_cast<size_t>(s.capacity_rows) * rt->moe_top_k[i]);
    rows = std::max<size_t>(rows, s.capacity_rows);
    hidden = std::max<size_t>(hidden, s.hidden);
    inter = std::max<size_t>(inter, rt->moe_inter[i]);
    e_pad = std::max<size_t>(e_pad, rt->moe_e_pad[i]);
    n_local = std::max<size_t>(n_local, rt->moe_n_local[i]);
    tm = std::max<size_t>(tm, std::max<size_t>(s.hidden / 128, rt->moe_inter[i] / 128));
  }
  const size_t max_tiles = tm * (routes / 16 + n_local) + 8;
  std::vector<lane::MoeLaneWs> ws(rt->n_lanes);
  std::vector<lane::MoeLaneMaps> maps(static_cast<size_t>(rt->n_lanes) * rt->n_instances);
  auto alloc = [&](size_t bytes) -> void* {
    void* p = nullptr;
    if (cudaMalloc(&p, std::max<size_t>(bytes, 256)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, std::max<size_t>(bytes, 256));
    rt->moe_allocs.push_back(p);
    return p;
  };
  static const int kBn[lane::kBnVariants] = {16, 32, 64, 128, 256};
  for (int l = 0; l < rt->n_lanes; ++l) {
    lane::MoeLaneWs& w = ws[l];
    w.logits = static_cast<__nv_bfloat16*>(alloc(rows * e_pad * 2));
    w.logits32 = rt->has_fp32_router ? static_cast<float*>(alloc(rows * e_pad * 4)) : nullptr;
    w.ids = static_cast<int*>(alloc(routes * 4));
    w.weights = static_cast<float*>(alloc(routes * 4));
    w.offsets = static_cast<int*>(alloc((n_local + 1) * 4));
    w.perm_token = static_cast<int*>(alloc(routes * 4));
    w.route_pos = static_cast<int*>(alloc(routes * 4));
    w.tiles_gateup = static_cast<int4*>(alloc(max_tiles * 16));
    w.tiles_down = static_cast<int4*>(alloc(max_tiles * 16));
    w.n_tiles = static_cast<int*>(alloc(8));
    w.xp = alloc(routes * hidden * 2);
    w.act = alloc(routes * inter * 2);
    w.yp = alloc(routes * hidden * 2);
    w.comb = alloc(rows * hidden * 2);
    w.cap_routes = static_cast<int>(routes);
    if (!w.logits || !w.ids || !w.weights || !w.offsets || !w.perm_token || !w.route_pos || !w.tiles_gateup || !w.tiles_down ||
        !w.n_tiles || !w.xp || !w.act || !w.yp || !w.comb)
      return -5;
    for (int i = 0; i < rt->n_instances; ++i) {
      if (rt->moe_top_k[i] == 0) continue;
      const lane::InstanceSlot& s = rt->slots_h[i];
      const uint64_t r = static_cast<uint64_t>(s.capacity_rows) * rt->moe_top_k[i];
      lane::MoeLaneMaps& m = maps[static_cast<size_t>(l) * rt->n_instances + i];
      for (int v = 0; v < lane::kBnVariants; ++v) {
        if (tmap::encode_2d(&m.tmap_xp[v], w.xp, r, s.hidden, static_cast<uint64_t>(s.hidden) * 2, kBn[v], 64, 2) != 0) return -6;
        if (tmap::encode_2d(&m.tmap_act[v], w.act, r, rt->moe_inter[i], static_cast<uint64_t>(rt->moe_inter[i]) * 2, kBn[v], 64, 2) != 0)
          return -6;
      }
    }
  }
  if (cudaMalloc(&rt->mws_d, sizeof(lane::MoeLaneWs) * rt->n_lanes) != cudaSuccess) return -5;
  if (cudaMalloc(&rt->mmaps_d, sizeof(lane::MoeLaneMaps) * maps.size()) != cudaSuccess) return -5;
  cudaMemcpy(rt->mws_d, ws.data(), sizeof(lane::MoeLaneWs) * rt->n_lanes, cudaMemcpyHostToDevice);
  cudaMemcpy(rt->mmaps_d, maps.data(), sizeof(lane::MoeLaneMaps) * maps.size(), cudaMemcpyHostToDevice);
  return 0;
}

extern "C" int xp_lane_commit(void* h) {
  auto* rt = static_cast<Runtime*>(h);
  if (rt->has_moe && rt->mws_d == nullptr) {
    const int rc = commit_moe(rt);
    if (rc != 0) return rc;
  }
  for (int i = 0; i < rt->n_instances; ++i) {
    auto& L = rt->layers_h[i];
    if (L.empty()) return -1;
    if (rt->moe_top_k[i] > 0) {
      // every MoE layer of one instance must share the inter size the scratch maps were built for
      for (size_t l = 0; l < L.size(); ++l)
        if (L[l].kind == 2 && L[l].inter_local != rt->moe_inter[i]) return -7;
      if (rt->moe_d[i] == nullptr && cudaMalloc(&rt->moe_d[i], sizeof(lane::MoeLayer) * L.size()) != cudaSuccess) return -2;
      cudaMemcpy(rt->moe_d[i], rt->moe_h[i].data(), sizeof(lane::MoeLayer) * L.size(), cudaMemcpyHostToDevice);
      for (size_t l = 0; l < L.size(); ++l) L[l].moe = L[l].kind == 2 ? rt->moe_d[i] + l : nullptr;
    }
    if (rt->layers_d[i] == nullptr && cudaMalloc(&rt->layers_d[i], sizeof(lane::LayerEntry) * L.size()) != cudaSuccess) return -2;
    cudaMemcpy(rt->layers_d[i], L.data(), sizeof(lane::LayerEntry) * L.size(), cudaMemcpyHostToDevice);
    rt->slots_h[i].layers = rt->layers_d[i];
  }
  cudaMemcpy(rt->slots_d, rt->slots_h.data(), sizeof(lane::InstanceSlot) * rt->n_instances, cudaMemcpyHostToDevice);
  const uint32_t pe = static_cast<uint32_t>(rt->pe);
  cudaMemcpy(&rt->ctl_d->pe, &pe, sizeof(pe), cudaMemcpyHostToDevice);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm::gemm_lane_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  rt->committed = cudaDeviceSynchronize() == cudaSuccess;
  return rt->committed ? 0 : -4;
}

// Enqueues one Lane iteration (wait, gate/up, down, complete) on `stream`; the
// caller may capture this into a CUDA graph and replay it.
extern "C" int xp_lane_launch(void* h, int lane_index, uint64_t lease_ns, void* stream) {
  auto* rt = static_cast<Runtime*>(h);
  if (!rt->committed || lane_index < 0 || lane_index >= rt->n_lanes) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  lane::LaneCur* cur = rt->cur_d + lane_index;
  float* ws = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(rt->ws_d) + rt->ws_bytes_per_lane * lane_index);
  uint32_t* counters = rt->counters_d + lane::kCounterWords * lane_index;
  const int smem_budget = 220 * 1024;
  const int smem = smem_budget + 2048;
  const lane::MoeLaneWs* mws = rt->has_moe ? rt->mws_d + lane_index : nullptr;
  const lane::MoeLaneMaps* mmaps = rt->has_moe ? rt->mmaps_d + static_cast<size_t>(lane_index) * rt->n_instances : nullptr;
  lane::lane_wait_kernel<<<1, 1, 0, s>>>(rt->ctl_d, rt->slots_d, cur, lane_index, lease_ns);
  if (rt->has_moe) {
    // MoE prologue; every kernel returns at once when the invocation's layer is dense
    gemm::gemm_lane_kernel<<<rt->sms, gemm::kThreads, smem, s>>>(rt->slots_d, cur, 2, ws, counters, smem_budget, rt->status_d,
                                                                 mws, mmaps);
    if (rt->has_fp32_router)   // routers that ask for fp32 logits: exact SIMT projection (a no-op for the other layers)
      moe::moe_lane_router_fp32_kernel<<<rt->sms * 2, 256, rt->max_hidden * sizeof(float), s>>>(rt->slots_d, cur, mws);
    moe::moe_lane_topk_kernel<<<rt->sms, 128, 0, s>>>(rt->slots_d, cur, mws);
    moe::moe_lane_route_kernel<<<1, 1024, 0, s>>>(rt->slots_d, cur, mws);
    moe::moe_lane_gather_kernel<<<rt->sms * 4, 128, 0, s>>>(rt->slots_d, cur, mws);
  }
  gemm::gemm_lane_kernel<<<rt->sms, gemm::kThreads, smem, s>>>(rt->slots_d, cur, 0, ws, counters, smem_budget, rt->status_d, mws,
                                                               mmaps);
  gemm::gemm_lane_kernel<<<rt->sms, gemm::kThreads, smem, s>>>(rt->slots_d, cur, 1, ws, counters, smem_budget, rt->status_d, mws,
                                                               mmaps);
  if (rt->has_moe) {
    moe::moe_lane_combine_kernel<<<rt->sms * 4, 128, 0, s>>>(rt->slots_d, cur, mws);
    // shared experts (no-ops unless the layer has them)
    gemm::gemm_lane_kernel<<<rt->sms, gemm::kThreads, smem, s>>>(rt->slots_d, cur, 3, ws, counters, smem_budget, rt->status_d,
                                                                 mws, mmaps);
    gemm::gemm_lane_kernel<<<rt->sms, gemm::kThreads, smem, s>>>(rt->slots_d, cur, 4, ws, counters, smem_budget, rt->status_d,
                                                                 mws, mmaps);
  }
  lane::lane_complete_kernel<<<1, 1, 0, s>>>(rt->ctl_d, rt->slots_d, cur, lane_index, rt->status_d);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

// Replays every Lane's graph from a host thread of this library, so that no interpreter lock and no other host
// work of the process sits between two Lane iterations. The reference launches each Lane's persistent graph once
// and lets it loop on the device (src/cext/ffnagent/runtime.cu:1041-1047); here a Lane iteration is a short graph
// with a lease, and `depth` replays are kept enqueued so the device never waits for the host.
// Captures happen on the calling thread, one Lane after the other; the threads only replay.
extern "C" int xp_lane_threads_start(void* h, uint64_t lease_ns, int depth) {
  auto* rt = static_cast<Runtime*>(h);
  if (!rt->committed || !rt->threads.empty() || depth < 1 || depth > 16) return -1;
  cudaSetDevice(rt->device);
  rt->stop_threads.store(false);
  rt->thread_error.store(0);
  for (int lane = 0; lane < rt->n_lanes; ++lane) {
    cudaStream_t s = nullptr;
    cudaGraph_t g = nullptr;
    cudaGraphExec_t x = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) return -2;
    // one eager iteration with a short lease: first-use set-up stays outside the capture
    if (xp_lane_launch(h, lane, 1000000ull, s) != 0 || cudaStreamSynchronize(s) != cudaSuccess) return -3;
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return -4;
    const int rc = xp_lane_launch(h, lane, lease_ns, s);
    if (cudaStreamEndCapture(s, &g) != cudaSuccess || rc != 0) return -5;
    if (cudaGraphInstantiate(&x, g, 0) != cudaSuccess) return -6;
    rt->lane_streams.push_back(s);
    rt->lane_graphs.push_back(g);
    rt->lane_execs.push_back(x);
  }
  for (int lane = 0; lane < rt->n_lanes; ++lane) {
    rt->threads.emplace_back([rt, lane, depth]() {
      cudaSetDevice(rt->device);
      cudaStream_t s = rt->lane_streams[lane];
      std::vector<cudaEvent_t> ev(depth);
      for (auto& e : ev) cudaEventCreateWithFlags(&e, cudaEventDisableTiming | cudaEventBlockingSync);
      std::deque<int> pending;
      int next = 0;
      while (!rt->stop_threads.load(std::memory_order_acquire)) {
        cudaError_t e = cudaGraphLaunch(rt->lane_execs[lane], s);
        if (e == cudaSuccess) e = cudaEventRecord(ev[next], s);
        if (e != cudaSuccess) {
          int zero = 0;
          rt->thread_error.compare_exchange_strong(zero, static_cast<int>(e));
          break;
        }
        rt->replays.fetch_add(1, std::memory_order_relaxed);
        pending.push_back(next);
        next = (next + 1) % depth;
        if (static_cast<int>(pending.size()) >= depth) {
          e = cudaEventSynchronize(ev[pending.front()]);
          pending.pop_front();
          if (e != cudaSuccess) {
            int zero = 0;
            rt->thread_error.compare_exchange_strong(zero, static_cast<int>(e));
            break;
          }
        }
      }
      cudaStreamSynchronize(s);
      for (auto& e : ev) cudaEventDestroy(e);
    });
  }
  return 0;
}

// Ends the replay threads: the caller first sets the device-side shutdown word (xp_lane_shutdown) so that leases in
// flight end at once. Returns the first CUDA error a thread met, as -100 - code, or 0.
extern "C" int xp_lane_threads_stop(void* h) {
  auto* rt = static_cast<Runtime*>(h);
  rt->stop_threads.store(true, std::memory_order_release);
  for (auto& t : rt->threads)
    if (t.joinable()) t.join();
  rt->threads.clear();
  for (auto x : rt->lane_execs) cudaGraphExecDestroy(x);
  for (auto g : rt->lane_graphs) cudaGraphDestroy(g);
  for (auto s : rt->lane_streams) cudaStreamDestroy(s);
  rt->lane_execs.clear();
  rt->lane_graphs.clear();
  rt->lane_streams.clear();
  const int e = rt->thread_error.load();
  return e == 0 ? 0 : -100 - e;
}

// (replays issued so far, first error code of a replay thread or 0)
extern "C" int xp_lane_threads_state(void* h, uint64_t* replays) {
  auto* rt = static_cast<Runtime*>(h);
  if (replays != nullptr) *replays = rt->replays.load();
  return rt->thread_error.load();
}

extern "C" int xp_lane_shutdown(void* h, void* stream) {
  auto* rt = static_cast<Runtime*>(h);
  static const uint32_t one = 1;
  return cudaMemcpyAsync(&rt->ctl_d->shutdown, &one, 4, cudaMemcpyHostToDevice, reinterpret_cast<cudaStream_t>(stream)) ==
                 cudaSuccess
             ? 0
             : -1;
}

// The first failure this device met, as {claim, result code, origin PE, instance, sequence, layer}; claim 0: none.
extern "C" int xp_lane_failure(void* h, uint32_t out6[6], void* stream) {
  auto* rt = static_cast<Runtime*>(h);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FailureSlot f;
  if (cudaMemcpyAsync(&f, &rt->ctl_d->failure, sizeof(f), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -2;
  out6[0] = f.claim;
  out6[1] = f.result_code;
  out6[2] = f.origin;
  out6[3] = f.instance_index;
  out6[4] = f.invocation_sequence;
  out6[5] = f.layer_ordinal;
  return 0;
}

extern "C" int xp_trace_create(uint32_t capacity, void** events, void** state) {
  if (capacity == 0 || events == nullptr || state == nullptr) return -1;
  if (cudaMalloc(events, sizeof(trace::Event) * capacity) != cudaSuccess) return -2;
  if (cudaMalloc(state, sizeof(trace::BufferState)) != cudaSuccess) return -2;
  return cudaMemset(*state, 0, sizeof(trace::BufferState)) == cudaSuccess ? 0 : -3;
}

extern "C" int64_t xp_trace_read(void* events, void* state, uint32_t capacity, uint64_t* out, uint64_t max_events,
                                 uint64_t* dropped, void* stream) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  trace::BufferState st;
  if (cudaMemcpyAsync(&st, state, sizeof(st), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -2;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -2;
  const uint64_t n = std::min<uint64_t>(std::min<uint64_t>(st.sequence, capacity), max_events);
  std::vector<trace::Event> ev(n);
  if (n > 0) {
    cudaMemcpyAsync(ev.data(), events, sizeof(trace::Event) * n, cudaMemcpyDeviceToHost, s);
    if (cudaStreamSynchronize(s) != cudaSuccess) return -2;
  }
  for (uint64_t i = 0; i < n; ++i) {
    out[3 * i] = (static_cast<uint64_t>(ev[i].kind) << 32) | ev[i].a;
    out[3 * i + 1] = ev[i].b;
    out[3 * i + 2] = ev[i].timestamp_ns;
  }
  if (dropped != nullptr) *dropped = st.dropped;
  return static_cast<int64_t>(n);
}

extern "C" void xp_trace_destroy(void* events, void* state) {
  if (events != nullptr) cudaFree(events);
  if (state != nullptr) cudaFree(state);
}

// served[n_instances], idle[n_lanes], status[1]; synchronous copies on `stream`.
extern "C" int xp_lane_stats(void* h, uint64_t* served, uint32_t* idle, uint32_t* status, void* stream) {
  auto* rt = static_cast<Runtime*>(h);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  lane::LaneCtl ctl;
  std::vector<lane::LaneCur> cur(rt->n_lanes);
  if (cudaMemcpyAsync(&ctl, rt->ctl_d, sizeof(ctl), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
  cudaMemcpyAsync(cur.data(), rt->cur_d, sizeof(lane::LaneCur) * rt->n_lanes, cudaMemcpyDeviceToHost, s);
  cudaMemcpyAsync(status, rt->status_d, 4, cudaMemcpyDeviceToHost, s);
  if (cudaStreamSynchronize(s) != cudaSuccess) return -2;
  for (int i = 0; i < rt->n_instances; ++i) served[i] = ctl.served[i];
  for (int l = 0; l < rt->n_lanes; ++l) idle[l] = cur[l].idle_replays;
  return 0;
}

// Fabric observer: allocates an event buffer and points the Lane kernels at it. Call before the
// first launch; events are read back with xp_lane_trace_read while the Lanes are stopped or running.
extern "C" int xp_lane_trace_enable(void* h, uint32_t capacity) {
  auto* rt = static_cast<Runtime*>(h);
  if (rt->trace_events_d != nullptr || capacity == 0) return -1;
  if (cudaMalloc(&rt->trace_events_d, sizeof(trace::Event) * capacity) != cudaSuccess) return -2;
  if (cudaMalloc(&rt->trace_state_d, sizeof(trace::BufferState)) != cudaSuccess) return -2;
  cudaMemset(rt->trace_state_d, 0, sizeof(trace::BufferState));
  rt->trace_capacity = capacity;
  trace::BufferView v{rt->trace_events_d, rt->trace_state_d, capacity, 0};
  return cudaMemcpy(&rt->ctl_d->trace, &v, sizeof(v), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -3;
}

// Copies up to max_events events as (kind << 32 | a, b, timestamp_ns) triples; returns the count,
// *dropped receives the number of events that did not fit.
extern "C" int64_t xp_lane_trace_read(void* h, uint64_t* out, uint64_t max_events, uint64_t* dropped, void* stream) {
  auto* rt = static_cast<Runtime*>(h);
  if (rt->trace_events_d == nullptr) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  trace::BufferState st;
  if (cudaMemcpyAsync(&st, rt->trace_state_d, sizeof(st), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -2;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -2;
  uint64_t n = std::min<uint64_t>(std::min<uint64_t>(st.sequence, rt->trace_capacity), max_events);
  std::vector<trace::Event> ev(n);
  if (n > 0) {
    cudaMemcpyAsync(ev.data(), rt->trace_events_d, sizeof(trace::Event) * n, cudaMemcpyDeviceToHost, s);
    if (cudaStreamSynchronize(s) != cudaSuccess) return -2;
  }
  for (uint64_t i = 0; i < n; ++i) {
    out[3 * i] = (static_cast<uint64_t>(ev[i].kind) << 32) | ev[i].a;
    out[3 * i + 1] = ev[i].b;
    out[3 * i + 2] = ev[i].timestamp_ns;
  }
  *dropped = st.dropped;
  return static_cast<int64_t>(n);
}

extern "C" void xp_lane_destroy(void* h) {
  auto* rt = static_cast<Runtime*>(h);
  if (rt == nullptr) return;
  if (!rt->threads.empty()) xp_lane_threads_stop(h);
  if (rt->trace_events_d != nullptr) cudaFree(rt->trace_events_d);
  if (rt->trace_state_d != nullptr) cudaFree(rt->trace_state_d);
  for (auto* p : rt->layers_d)
    if (p != nullptr) cudaFree(p);
  for (auto* p : rt->moe_d)
    if (p != nullptr) cudaFree(p);
  for (void* p : rt->moe_allocs) cudaFree(p);
  if (rt->mws_d != nullptr) cudaFree(rt->mws_d);
  if (rt->mmaps_d != nullptr) cudaFree(rt->mmaps_d);
  cudaFree(rt->ctl_d);
  cudaFree(rt->slots_d);
  cudaFree(rt->cur_d);
  cudaFree(rt->ws_d);
  cudaFree(rt->counters_d);
  cudaFree(rt->status_d);
  delete rt;
}

extern "C" int xp_signal_flags(const XpSignalArgs* a, void* stream) {
  if (a->n < 0 || a->n > 8 || a->seq_counter == nullptr) return -1;  // n == 0: advance the counter only
  lane::signal_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" int xp_wait_flags(const XpWaitArgs* a, void* stream) {
  if (a->n < 1 || a->n > 8) return -1;
  lane::wait_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
