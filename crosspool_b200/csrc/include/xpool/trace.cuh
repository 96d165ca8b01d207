// Device-side writers for the observers' event buffers (host layout in xpool/trace.hpp).
// A writer reserves a slot with a relaxed atomic add, stamps the event with %globaltimer and
// counts it as dropped when the buffer is full; the buffer never wraps
// (reference: src/cext-include/xpool/utils/trace.cuh, utils/time.cuh).
// A null view makes record() a single predictable branch, so un-observed runs pay nothing else.
#pragma once

#include "xpool/sm100.cuh"
#include "xpool/trace.hpp"

namespace xpool {
namespace trace {

struct BufferView {
  Event* events;
  BufferState* state;
  uint32_t capacity;
  uint32_t reserved;
};

// Event kinds are listed in xpool/hooks.cuh (hooks::Kind), beside the hook points that write them.

__device__ __forceinline__ void record(const BufferView& v, uint32_t kind, uint32_t a, uint32_t b) {
  if (v.events == nullptr) return;
  const unsigned long long slot = atomicAdd(reinterpret_cast<unsigned long long*>(&v.state->sequence), 1ull);
  if (slot >= v.capacity) {
    atomicAdd(reinterpret_cast<unsigned long long*>(&v.state->dropped), 1ull);
    return;
  }
  Event e;
  e.kind = kind;
  e.a = a;
  e.b = b;
  e.reserved = 0;
  e.timestamp_ns = sm100::global_timer_ns();
  v.events[slot] = e;
}

}  // namespace trace
}  // namespace xpool
