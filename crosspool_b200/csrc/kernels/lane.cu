// Executor-Lane kernels and the host object that owns an FFN device's Lane state
// (see xpool/lane.cuh for the design), plus the attention-side flag wait.
#include <string.h>

#include <algorithm>
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
                                 uint32_t* counters, int smem_budget, uint32_t* status);
}  // namespace gemm

namespace lane {

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
      trace::record(ctl->trace, trace::kLaneShutdown, lane_index, 0);
      return;
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
        if (ahead > 0) sched.enqueue(i, e.completed_sequence + static_cast<uint64_t>(ahead), slots[i].record->deadline_us);
      }
      const Decision d = sched.try_schedule_on(lane_index);
      lock_release(&ctl->lock);
      if (d.scheduled) {
        const InstanceSlot& s = slots[d.instance];
        const InvocationRecord* rec = s.record;
        uint32_t rows = rec->rows, layer = rec->layer_ordinal;
        uint32_t rc = 0;
        if (rows > static_cast<uint32_t>(s.capacity_rows) || layer >= static_cast<uint32_t>(s.num_layers)) {
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
        if (rc != 0) trace::record(ctl->trace, trace::kLaneRejected, d.instance, rc);
        trace::record(ctl->trace, trace::kLaneAdmitted, d.instance, (layer << 16) | (rows > 0xffffu ? 0xffffu : rows));
        return;
      }
    }
    if ((++spins & 0xfu) == 0 && sm100::global_timer_ns() > deadline) {
      cur->idle_replays += 1;
      trace::record(ctl->trace, trace::kLaneIdle, lane_index, cur->idle_replays);
      return;
    }
    __nanosleep(200);
  }
}

// One thread: publish the completion on the attention device, free the Lane.
__global__ void lane_complete_kernel(LaneCtl* ctl, const InstanceSlot* slots, LaneCur* cur, uint32_t lane_index) {
  if (cur->valid == 0) return;
  const InstanceSlot& s = slots[cur->instance];
  CompletionRecord* done = reinterpret_cast<CompletionRecord*>(s.done_flag_peer);
  done->result_code = cur->result_code;
  done->rows = cur->rows;
  __threadfence_system();
  sm100::st_release_sys(&done->sequence, cur->sequence);
  if (lock_acquire(&ctl->lock, sm100::global_timer_ns() + 1000000ull)) {
    Scheduler sched(ctl->entries, ctl->n_instances, ctl->lanes, ctl->n_lanes,
                    SchedulerPolicy{static_cast<SchedulerPolicyKind>(ctl->policy), ctl->seed}, &ctl->next_ticket);
    sched.release(cur->instance, cur->lease);
    ctl->served[cur->instance] += 1;
    lock_release(&ctl->lock);
  }
  trace::record(ctl->trace, trace::kLaneCompleted, cur->instance, cur->sequence);
  cur->valid = 0;
  (void)lane_index;
}

// Attention side: up to 8 threads each wait until their flag reaches *want.
__global__ void wait_flags_kernel(XpWaitArgs a) {
  const int i = threadIdx.x;
  if (i >= a.n) return;
  const uint32_t want = a.want_ptr != nullptr ? *a.want_ptr : a.want;
  const uint64_t deadline = sm100::global_timer_ns() + a.wait_ns;
  const int rc = sm100::wait_flag_ge(a.flags[i], want, deadline, a.cancel);
  if (rc != 0 && a.status != nullptr) atomicCAS(a.status, 0u, 4u);
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
  cudaDeviceGetAttribute(&rt->sms, cudaDevAttrMultiProcessorCount, dev);
  rt->slots_h.resize(n_instances);
  rt->layers_h.resize(n_instances);
  rt->layers_d.assign(n_instances, nullptr);
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
  s.in_flag = reinterpret_cast<const uint32_t*>(d->in_flag);
  s.record = reinterpret_cast<const InvocationRecord*>(d->record);
  s.act = d->act;
  s.out_peer = d->out_peer;
  s.done_flag_peer = reinterpret_cast<uint32_t*>(d->done_record_peer);
  s.capacity_rows = d->capacity_rows;
  s.hidden = d->hidden;
  s.num_layers = d->num_layers;
  s.act_ld = d->act_ld;
  rt->layers_h[idx].assign(d->num_layers, lane::LayerEntry{});
  return 0;
}

extern "C" int xp_lane_set_layer(void* h, int inst, int layer, const XpLaneLayerDesc* d) {
  auto* rt = static_cast<Runtime*>(h);
  if (inst < 0 || inst >= rt->n_instances) return -1;
  auto& layers = rt->layers_h[inst];
  if (layer < 0 || layer >= static_cast<int>(layers.size())) return -1;
  const lane::InstanceSlot& s = rt->slots_h[inst];
  if (d->inter_local % 128 != 0 || s.hidden % 128 != 0 || d->inter_local > s.act_ld) return -2;
  lane::LayerEntry& e = layers[layer];
  memset(&e, 0, sizeof(e));
  const int gu_rows = d->inter_local * (d->gated ? 2 : 1);
  int rc;
  if (d->w_tiled) {
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
  e.kind = 1;
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

extern "C" int xp_lane_commit(void* h) {
  auto* rt = static_cast<Runtime*>(h);
  for (int i = 0; i < rt->n_instances; ++i) {
    auto& L = rt->layers_h[i];
    if (L.empty()) return -1;
    if (rt->layers_d[i] == nullptr && cudaMalloc(&rt->layers_d[i], sizeof(lane::LayerEntry) * L.size()) != cudaSuccess) return -2;
    cudaMemcpy(rt->layers_d[i], L.data(), sizeof(lane::LayerEntry) * L.size(), cudaMemcpyHostToDevice);
    rt->slots_h[i].layers = rt->layers_d[i];
  }
  cudaMemcpy(rt->slots_d, rt->slots_h.data(), sizeof(lane::InstanceSlot) * rt->n_instances, cudaMemcpyHostToDevice);
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
  const int smem_budget = 200 * 1024;
  const int smem = smem_budget + 2048;
  lane::lane_wait_kernel<<<1, 1, 0, s>>>(rt->ctl_d, rt->slots_d, cur, lane_index, lease_ns);
  gemm::gemm_lane_kernel<<<rt->sms, gemm::kThreads, smem, s>>>(rt->slots_d, cur, 0, ws, counters, smem_budget, rt->status_d);
  gemm::gemm_lane_kernel<<<rt->sms, gemm::kThreads, smem, s>>>(rt->slots_d, cur, 1, ws, counters, smem_budget, rt->status_d);
  lane::lane_complete_kernel<<<1, 1, 0, s>>>(rt->ctl_d, rt->slots_d, cur, lane_index);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" int xp_lane_shutdown(void* h, void* stream) {
  auto* rt = static_cast<Runtime*>(h);
  static const uint32_t one = 1;
  return cudaMemcpyAsync(&rt->ctl_d->shutdown, &one, 4, cudaMemcpyHostToDevice, reinterpret_cast<cudaStream_t>(stream)) ==
                 cudaSuccess
             ? 0
             : -1;
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
  if (rt->trace_events_d != nullptr) cudaFree(rt->trace_events_d);
  if (rt->trace_state_d != nullptr) cudaFree(rt->trace_state_d);
  for (auto* p : rt->layers_d)
    if (p != nullptr) cudaFree(p);
  cudaFree(rt->ctl_d);
  cudaFree(rt->slots_d);
  cudaFree(rt->cur_d);
  cudaFree(rt->ws_d);
  cudaFree(rt->counters_d);
  cudaFree(rt->status_d);
  delete rt;
}

extern "C" int xp_wait_flags(const XpWaitArgs* a, void* stream) {
  if (a->n < 1 || a->n > 8) return -1;
  lane::wait_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
