// Lock-free event buffers for the devkit observers: writers reserve a slot with
// a relaxed fetch_add, events that do not fit are counted as dropped, and the
// buffer never wraps (reference: src/cext-include/xpool/utils/trace.hpp).
// The same Event/BufferState structs are written by device code in
// xpool/trace.cuh; HostBuffer is the host-side owner used by CPU roles.
#pragma once

#include <stdint.h>

#include <atomic>
#include <vector>

namespace xpool {
namespace trace {

struct Event {
  uint32_t kind;
  uint32_t a;
  uint32_t b;
  uint32_t reserved;
  uint64_t timestamp_ns;
};

struct BufferState {
  uint64_t sequence;  // slots reserved so far (may exceed capacity)
  uint64_t dropped;
};

class HostBuffer {
 public:
  explicit HostBuffer(uint32_t capacity) : events_(capacity) {}

  bool record(uint32_t kind, uint32_t a, uint32_t b, uint64_t ts) {
    const uint64_t slot = sequence_.fetch_add(1, std::memory_order_relaxed);
    if (slot >= events_.size()) {
      dropped_.fetch_add(1, std::memory_order_relaxed);
      return false;
    }
    events_[slot] = Event{kind, a, b, 0, ts};
    committed_.fetch_add(1, std::memory_order_release);
    return true;
  }
  uint64_t size() const {
    const uint64_t s = sequence_.load(std::memory_order_acquire);
    return s < events_.size() ? s : events_.size();
  }
  uint64_t dropped() const { return dropped_.load(std::memory_order_acquire); }
  uint64_t read(uint64_t first, uint64_t count, uint64_t* out) const {
    const uint64_t n = size();
    uint64_t k = 0;
    for (uint64_t i = first; i < n && k < count; ++i, ++k) {
      out[3 * k] = (static_cast<uint64_t>(events_[i].kind) << 32) | events_[i].a;
      out[3 * k + 1] = events_[i].b;
      out[3 * k + 2] = events_[i].timestamp_ns;
    }
    return k;
  }

 private:
  std::vector<Event> events_;
  std::atomic<uint64_t> sequence_{0};
  std::atomic<uint64_t> dropped_{0};
  std::atomic<uint64_t> committed_{0};
};

}  // namespace trace
}  // namespace xpool
