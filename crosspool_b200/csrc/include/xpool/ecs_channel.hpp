// Elastic Context State control channel: one POSIX-shm block shared by the
// daemon (capacity policy), the AtnAgents (device memory reports) and the
// Instance ranks (demand / completion), with one seqlock per published record.
//
// Down:  QuotaCommand{sequence, target_bytes}            daemon   -> instance
// Up:    QuotaDemand{evaluated_sequence, required_bytes,
//                    deadline_monotonic_ns}              instance -> daemon
//        QuotaCompletion{sequence, mapped_bytes}         instance -> daemon
//        DeviceMemoryReport{free, total}                 atnagent -> daemon
// (Reference: src/cext-include/xpool/ecs/{layout,channel}.hpp,
// src/cext/ecs/channel.cpp:28-35 for the odd/even revision protocol.)
#pragma once

#include <stdint.h>

#include <atomic>
#include <thread>

namespace xpool {
namespace ecs {

constexpr uint64_t kChannelMagic = 0x5850423230304b56ull;  // "XPB200KV"

struct QuotaCommand {
  uint64_t sequence;
  uint64_t target_bytes;
};
struct QuotaDemand {
  uint64_t evaluated_sequence;
  uint64_t required_bytes;
  uint64_t deadline_monotonic_ns;
  uint64_t mapped_bytes;
};
struct QuotaCompletion {
  uint64_t sequence;
  uint64_t mapped_bytes;
};
struct DeviceMemoryReport {
  uint64_t free_bytes;
  uint64_t total_bytes;
  uint64_t report_sequence;
};

template <typename T>
struct alignas(64) SeqRecord {
  std::atomic<uint64_t> revision;  // odd while a writer is inside
  T value;
};

struct alignas(64) ChannelHeader {
  uint64_t magic;
  uint32_t abi_version;
  uint32_t device_count;
  uint32_t partition_count;
  uint32_t generation;
  uint64_t total_bytes;
};

struct alignas(64) DeviceEntry {
  uint32_t device;
  uint32_t reserved;
  SeqRecord<DeviceMemoryReport> report;
};

// One Instance rank's KV partition on one attention device.
struct alignas(64) PartitionEntry {
  uint32_t device;
  uint32_t group;  // attention TP group the rank belongs to
  uint32_t rank;
  uint32_t reserved;
  uint64_t floor_bytes;
  uint64_t reservation_bytes;
  SeqRecord<QuotaCommand> command;
  SeqRecord<QuotaDemand> demand;
  SeqRecord<QuotaCompletion> completion;
};

inline uint64_t channel_bytes(uint32_t devices, uint32_t partitions) {
  return sizeof(ChannelHeader) + static_cast<uint64_t>(devices) * sizeof(DeviceEntry) +
         static_cast<uint64_t>(partitions) * sizeof(PartitionEntry);
}

// The payload is copied word by word with relaxed atomic accesses: a reader that races with a writer may
// see a mix of old and new words, which the revision check then discards -- without the plain-access data
// race a textbook seqlock has (found by running the channel under ThreadSanitizer).
template <typename T>
inline void seq_copy_in(T* dst, const T& src) {
  static_assert(sizeof(T) % 8 == 0 && alignof(T) >= 8, "seqlock payloads are made of 64-bit words");
  const uint64_t* s = reinterpret_cast<const uint64_t*>(&src);
  uint64_t* d = reinterpret_cast<uint64_t*>(dst);
  for (size_t i = 0; i < sizeof(T) / 8; ++i) std::atomic_ref<uint64_t>(d[i]).store(s[i], std::memory_order_relaxed);
}
template <typename T>
inline void seq_copy_out(T* dst, const T* src) {
  uint64_t* d = reinterpret_cast<uint64_t*>(dst);
  uint64_t* s = const_cast<uint64_t*>(reinterpret_cast<const uint64_t*>(src));
  for (size_t i = 0; i < sizeof(T) / 8; ++i) d[i] = std::atomic_ref<uint64_t>(s[i]).load(std::memory_order_relaxed);
}

template <typename T>
inline void seq_publish(SeqRecord<T>* r, const T& v) {
  uint64_t rev = r->revision.load(std::memory_order_relaxed);
  r->revision.store(rev + 1, std::memory_order_seq_cst);  // odd: write in progress
  std::atomic_thread_fence(std::memory_order_seq_cst);
  seq_copy_in(&r->value, v);
  r->revision.store(rev + 2, std::memory_order_seq_cst);
}

// Returns false if no stable snapshot could be taken within `attempts`. A reader that keeps colliding with the
// writer gives its time slice away every 64 tries, so a writer that was descheduled in the middle of a publication
// (odd revision) gets to finish it even on a loaded host.
template <typename T>
inline bool seq_read(const SeqRecord<T>* r, T* out, uint64_t* revision, int attempts = 20000) {
  for (int i = 0; i < attempts; ++i) {
    if ((i & 63) == 63) std::this_thread::yield();
    uint64_t a = r->revision.load(std::memory_order_seq_cst);
    if (a & 1) continue;
    T v;
    seq_copy_out(&v, &r->value);
    std::atomic_thread_fence(std::memory_order_seq_cst);
    uint64_t b = r->revision.load(std::memory_order_seq_cst);
    if (a == b) {
      *out = v;
      if (revision != nullptr) *revision = a;
      return true;
    }
  }
  return false;
}

}  // namespace ecs
}  // namespace xpool
