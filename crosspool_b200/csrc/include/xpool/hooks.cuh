// Hook points of the data plane: every protocol transition calls Point<Context>::hooks(ctx), which fans the
// typed context out to the adapters registered at compile time. The registry is a type list, so a build without
// observers (-DXPOOL_NO_OBSERVERS) compiles every hook call to nothing; the default registry holds the trace
// adapter, whose cost without an attached buffer is one predictable branch on a null pointer.
// (Reference: typed zero-cost registries in src/cext-include/xpool/hooks.hpp and hooks/registry.cuh, with the
// protocol event kinds of transport/hooks.hpp and fabric/hooks.hpp.)
#pragma once

#include "xpool/protocol.hpp"
#include "xpool/trace.cuh"

namespace xpool {
namespace hooks {

// Event kinds as they appear in trace buffers. 1..5 keep the values the Lane kernels have always written.
enum Kind : uint32_t {
  // FfnAgent Lane (coordinator + execution + delivery)
  kLaneAdmitted = 1,         // a = instance, b = layer << 16 | rows (saturated)
  kLaneCompleted = 2,        // a = instance, b = invocation sequence
  kLaneIdle = 3,             // a = lane, b = idle replays so far
  kLaneShutdown = 4,         // a = lane
  kLaneRejected = 5,         // a = instance, b = result code
  kLaneDiscovered = 6,       // a = instance, b = invocation sequence seen in the slot
  kLaneLockTimeout = 7,      // a = lane, b = 0 wait / 1 complete
  kLaneFailureClaimed = 8,   // a = instance, b = result code (this rank claimed the generation failure)
  kLaneFailureObserved = 9,  // a = lane, b = origin PE
  // attention side (transport producer, completion wait)
  kAtnPublished = 16,        // a = layer << 16 | rows (saturated), b = invocation sequence
  kAtnFoldWaitTimedOut = 17, // a = row, b = sequence waited for
  kAtnWaitBegin = 18,        // a = flag index, b = sequence waited for
  kAtnWaitEnd = 19,          // a = flag index, b = sequence
  kAtnWaitTimedOut = 20,     // a = flag index, b = sequence
  kAtnWaitCancelled = 21,    // a = flag index, b = sequence (the generation failed elsewhere)
};

// ---------------------------------------------------------------- contexts
struct LaneAdmitted { const trace::BufferView& buf; uint32_t instance, layer, rows; };
struct LaneCompleted { const trace::BufferView& buf; uint32_t instance, sequence; };
struct LaneIdle { const trace::BufferView& buf; uint32_t lane, idle_replays; };
struct LaneShutdown { const trace::BufferView& buf; uint32_t lane; };
struct LaneRejected { const trace::BufferView& buf; uint32_t instance, result_code; };
struct LaneDiscovered { const trace::BufferView& buf; uint32_t instance, sequence; };
struct LaneLockTimeout { const trace::BufferView& buf; uint32_t lane, where; };
struct LaneFailureClaimed { const trace::BufferView& buf; uint32_t instance, result_code; };
struct LaneFailureObserved { const trace::BufferView& buf; uint32_t lane, origin_pe; };
struct AtnPublished { const trace::BufferView& buf; uint32_t layer, rows, sequence; };
struct AtnFoldWaitTimedOut { const trace::BufferView& buf; uint32_t row, sequence; };
struct AtnWaitBegin { const trace::BufferView& buf; uint32_t flag, sequence; };
struct AtnWaitEnd { const trace::BufferView& buf; uint32_t flag, sequence, status; };   // status: 0 ready, 1 timed out, 2 cancelled

// ---------------------------------------------------------------- adapters
__device__ __forceinline__ uint32_t sat16(uint32_t v) { return v > 0xffffu ? 0xffffu : v; }

struct TraceAdapter {
  __device__ static void on(const LaneAdmitted& c) { trace::record(c.buf, kLaneAdmitted, c.instance, (c.layer << 16) | sat16(c.rows)); }
  __device__ static void on(const LaneCompleted& c) { trace::record(c.buf, kLaneCompleted, c.instance, c.sequence); }
  __device__ static void on(const LaneIdle& c) { trace::record(c.buf, kLaneIdle, c.lane, c.idle_replays); }
  __device__ static void on(const LaneShutdown& c) { trace::record(c.buf, kLaneShutdown, c.lane, 0); }
  __device__ static void on(const LaneRejected& c) { trace::record(c.buf, kLaneRejected, c.instance, c.result_code); }
  __device__ static void on(const LaneDiscovered& c) { trace::record(c.buf, kLaneDiscovered, c.instance, c.sequence); }
  __device__ static void on(const LaneLockTimeout& c) { trace::record(c.buf, kLaneLockTimeout, c.lane, c.where); }
  __device__ static void on(const LaneFailureClaimed& c) { trace::record(c.buf, kLaneFailureClaimed, c.instance, c.result_code); }
  __device__ static void on(const LaneFailureObserved& c) { trace::record(c.buf, kLaneFailureObserved, c.lane, c.origin_pe); }
  __device__ static void on(const AtnPublished& c) { trace::record(c.buf, kAtnPublished, (c.layer << 16) | sat16(c.rows), c.sequence); }
  __device__ static void on(const AtnFoldWaitTimedOut& c) { trace::record(c.buf, kAtnFoldWaitTimedOut, c.row, c.sequence); }
  __device__ static void on(const AtnWaitBegin& c) { trace::record(c.buf, kAtnWaitBegin, c.flag, c.sequence); }
  __device__ static void on(const AtnWaitEnd& c) {
    trace::record(c.buf, c.status == 0 ? kAtnWaitEnd : c.status == 1 ? kAtnWaitTimedOut : kAtnWaitCancelled, c.flag, c.sequence);
  }
};

// ---------------------------------------------------------------- registry
template <class... Adapters>
struct DeviceRegistry {
  template <class Context>
  __device__ __forceinline__ static void fire(const Context& c) {
    (Adapters::on(c), ...);
  }
};

#ifdef XPOOL_NO_OBSERVERS
using Registry = DeviceRegistry<>;
#else
using Registry = DeviceRegistry<TraceAdapter>;
#endif

template <class Context>
struct Point {
  __device__ __forceinline__ static void hooks(const Context& c) { Registry::fire(c); }
};

}  // namespace hooks

// ---------------------------------------------------------------- canonical failure
namespace failure {

// Tries to claim `slot` (local or in a peer GPU's memory) for this failure. Returns true when this call won.
__device__ __forceinline__ bool claim(FailureSlot* slot, uint32_t result_code, uint32_t origin, uint32_t instance,
                                      uint32_t sequence, uint32_t layer) {
  if (slot == nullptr) return false;
  if (atomicCAS_system(&slot->claim, 0u, kFailureWriting) != 0u) return false;
  slot->result_code = result_code;
  slot->origin = origin;
  slot->instance_index = instance;
  slot->invocation_sequence = sequence;
  slot->layer_ordinal = layer;
  __threadfence_system();
  sm100::st_release_sys(&slot->claim, kFailureClaimed);
  return true;
}

__device__ __forceinline__ bool claimed(const FailureSlot* slot) {
  return slot != nullptr && sm100::ld_relaxed_sys(&slot->claim) != 0u;
}

}  // namespace failure
}  // namespace xpool
