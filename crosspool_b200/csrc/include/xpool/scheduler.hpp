// Executor-Lane scheduler, compilable for host and device.
//
// Each Instance has one SchedulerEntry. `enqueue` stamps a FIFO ticket (and the
// invocation's SLO deadline); when a Lane is idle `try_schedule` picks among the
// queued entries by policy:
//   Fifo    smallest ticket                       (reference scheduler.cuh)
//   Random  smallest SplitMix64(seed ^ ticket)    (reference utils/random.hpp)
//   Slo     earliest deadline first, ticket breaks ties (not in the reference;
//           the reference only carries scheduler.slo values to the KV policy)
// `release` returns the Lane and bumps the entry's completed sequence so that a
// stale lease can be recognised (reference fabric/scheduler.hpp:1-170).
#pragma once

#include <stdint.h>

#include "xpool/protocol.hpp"

namespace xpool {

enum class SchedulerPolicyKind : uint32_t { Fifo = 0, Random = 1, Slo = 2 };

struct SchedulerPolicy {
  SchedulerPolicyKind kind;
  uint64_t seed;
  static XP_HD SchedulerPolicy fifo() { return {SchedulerPolicyKind::Fifo, 0}; }
  static XP_HD SchedulerPolicy random(uint64_t seed) { return {SchedulerPolicyKind::Random, seed}; }
  static XP_HD SchedulerPolicy slo() { return {SchedulerPolicyKind::Slo, 0}; }
};

XP_HD inline uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

enum class EntryState : uint32_t { Idle = 0, Queued = 1, Running = 2 };

struct SchedulerEntry {
  uint32_t state;
  uint32_t lane;                // valid while Running
  uint64_t ticket;              // FIFO order
  uint64_t deadline;            // SLO deadline (any monotonic unit)
  uint64_t invocation_sequence; // the queued / running invocation
  uint64_t completed_sequence;  // last released invocation
  uint64_t lease_sequence;      // bumped at every admission
};

struct LaneState {
  uint32_t busy;
  uint32_t instance;
  uint64_t lease_sequence;
};

struct Decision {
  bool scheduled;
  uint32_t instance;
  uint32_t lane;
  uint64_t lease_sequence;
};

constexpr uint32_t kNoLane = 0xffffffffu;

class Scheduler {
 public:
  XP_HD Scheduler(SchedulerEntry* entries, uint32_t n_instances, LaneState* lanes, uint32_t n_lanes,
                  SchedulerPolicy policy, uint64_t* next_ticket)
      : entries_(entries), n_(n_instances), lanes_(lanes), nl_(n_lanes), policy_(policy),
        next_ticket_(next_ticket) {}

  // Returns false if the instance already has a queued or running invocation
  // (one active FFN invocation per Instance) or the sequence does not advance.
  XP_HD bool enqueue(uint32_t instance, uint64_t invocation_sequence, uint64_t deadline) {
    if (instance >= n_) return false;
    SchedulerEntry& e = entries_[instance];
    if (e.state != static_cast<uint32_t>(EntryState::Idle)) return false;
    if (invocation_sequence <= e.completed_sequence) return false;
    e.state = static_cast<uint32_t>(EntryState::Queued);
    e.ticket = (*next_ticket_)++;
    e.deadline = deadline;
    e.invocation_sequence = invocation_sequence;
    return true;
  }

  XP_HD uint32_t find_idle_lane() const {
    for (uint32_t l = 0; l < nl_; ++l)
      if (!lanes_[l].busy) return l;
    return kNoLane;
  }

  XP_HD Decision try_schedule() { return try_schedule_on(find_idle_lane()); }

  // Schedules onto a specific idle Lane (a Lane that polls for its own work).
  XP_HD Decision try_schedule_on(uint32_t lane) {
    Decision d{false, 0, kNoLane, 0};
    if (lane == kNoLane || lane >= nl_ || lanes_[lane].busy) return d;
    bool found = false;
    uint32_t best = 0;
    uint64_t best_key = 0, best_ticket = 0;
    // Deadlines arrive as 32-bit microsecond stamps that wrap; they are ordered relative to the first
    // queued entry (valid while all queued deadlines lie within 35 minutes of one another). A zero
    // deadline means "none" and sorts last.
    bool have_ref = false;
    uint32_t ref = 0;
    for (uint32_t i = 0; i < n_; ++i) {
      const SchedulerEntry& e = entries_[i];
      if (e.state != static_cast<uint32_t>(EntryState::Queued)) continue;
      uint64_t key;
      switch (policy_.kind) {
        case SchedulerPolicyKind::Random: key = splitmix64(policy_.seed ^ e.ticket); break;
        case SchedulerPolicyKind::Slo: {
          const uint32_t dl = static_cast<uint32_t>(e.deadline);
          if (dl == 0) {
            key = ~0ull;
          } else {
            if (!have_ref) {
              have_ref = true;
              ref = dl;
            }
            key = static_cast<uint64_t>(static_cast<int64_t>(static_cast<int32_t>(dl - ref)) + (1ll << 32));
          }
          break;
        }
        default: key = e.ticket; break;
      }
      if (!found || key < best_key || (key == best_key && e.ticket < best_ticket)) {
        found = true;
        best = i;
        best_key = key;
        best_ticket = e.ticket;
      }
    }
    if (!found) return d;
    SchedulerEntry& e = entries_[best];
    e.state = static_cast<uint32_t>(EntryState::Running);
    e.lane = lane;
    e.lease_sequence += 1;
    lanes_[lane].busy = 1;
    lanes_[lane].instance = best;
    lanes_[lane].lease_sequence = e.lease_sequence;
    d.scheduled = true;
    d.instance = best;
    d.lane = lane;
    d.lease_sequence = e.lease_sequence;
    return d;
  }

  // The running decision of an instance, if any.
  XP_HD Decision active_decision(uint32_t instance) const {
    Decision d{false, instance, kNoLane, 0};
    if (instance >= n_) return d;
    const SchedulerEntry& e = entries_[instance];
    if (e.state != static_cast<uint32_t>(EntryState::Running)) return d;
    d.scheduled = true;
    d.lane = e.lane;
    d.lease_sequence = e.lease_sequence;
    return d;
  }

  // Releases the lane held under `lease_sequence`; a stale lease is refused.
  XP_HD bool release(uint32_t instance, uint64_t lease_sequence) {
    if (instance >= n_) return false;
    SchedulerEntry& e = entries_[instance];
    if (e.state != static_cast<uint32_t>(EntryState::Running)) return false;
    if (e.lease_sequence != lease_sequence) return false;
    if (e.lane >= nl_ || lanes_[e.lane].lease_sequence != lease_sequence) return false;
    lanes_[e.lane].busy = 0;
    e.completed_sequence = e.invocation_sequence;
    e.state = static_cast<uint32_t>(EntryState::Idle);
    e.lane = kNoLane;
    return true;
  }

 private:
  SchedulerEntry* entries_;
  uint32_t n_;
  LaneState* lanes_;
  uint32_t nl_;
  SchedulerPolicy policy_;
  uint64_t* next_ticket_;
};

}  // namespace xpool
