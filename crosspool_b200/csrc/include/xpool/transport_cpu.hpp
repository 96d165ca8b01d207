// Transport arena in host shared memory and the two halves of the mailbox
// protocol on CPU threads. This is the loopback data plane used when attention
// and FFN roles run as separate CPU processes; it executes the same state
// machine as the GPU mailbox (xpool/protocol.hpp) with std::atomic_ref in place
// of system-scope PTX accesses.
//
// Arena: LayoutHeader | ArenaState | Mailbox | input payload | output payload
// (reference layout: src/cext-include/xpool/transport/layout.hpp,
// src/cext/transport/layout.cpp).
#pragma once

#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>

#include "xpool/protocol.hpp"

namespace xpool {
namespace cpu {

struct ArenaState {
  uint32_t shutdown;
  uint32_t generation_failure_code;
  uint32_t drain_requested;
  uint32_t reserved;
};

struct ArenaLayout {
  uint64_t state_offset, mailbox_offset, input_offset, output_offset, total_bytes;
  uint64_t max_rows, row_bytes;
};

inline bool plan_arena(uint64_t max_rows, uint64_t row_bytes, ArenaLayout* L) {
  Checked pay = checked_mul(max_rows, row_bytes);
  if (!pay.ok || row_bytes % kPayloadAlignment != 0) return false;
  uint64_t off = sizeof(LayoutHeader);
  L->state_offset = checked_align_up(off, kAllocationAlignment).value;
  L->mailbox_offset = checked_align_up(L->state_offset + sizeof(ArenaState), kAllocationAlignment).value;
  L->input_offset = checked_align_up(L->mailbox_offset + sizeof(Mailbox), kAllocationAlignment).value;
  Checked out = checked_align_up(L->input_offset + pay.value, kAllocationAlignment);
  if (!out.ok) return false;
  L->output_offset = out.value;
  Checked tot = checked_align_up(out.value + pay.value, kAllocationAlignment);
  if (!tot.ok) return false;
  L->total_bytes = tot.value;
  L->max_rows = max_rows;
  L->row_bytes = row_bytes;
  return true;
}

enum class WaitStatus : int { Ready = 0, TimedOut = 1, Cancelled = 2 };

class ArenaView {
 public:
  ArenaView(void* base, const ArenaLayout& L) : base_(static_cast<uint8_t*>(base)), L_(L) {}

  void format() {
    std::memset(base_, 0, L_.input_offset);
    LayoutHeader* h = header();
    h->magic = kTransportMagic;
    h->abi_version = kAbiVersion;
    h->layout_size = sizeof(ArenaLayout);
    h->total_bytes = L_.total_bytes;
    h->state_offset = L_.state_offset;
  }
  bool valid() const {
    const LayoutHeader* h = reinterpret_cast<const LayoutHeader*>(base_);
    return h->magic == kTransportMagic && h->abi_version == kAbiVersion && h->total_bytes == L_.total_bytes;
  }
  LayoutHeader* header() { return reinterpret_cast<LayoutHeader*>(base_); }
  ArenaState* state() { return reinterpret_cast<ArenaState*>(base_ + L_.state_offset); }
  Mailbox* mailbox() { return reinterpret_cast<Mailbox*>(base_ + L_.mailbox_offset); }
  uint8_t* input() { return base_ + L_.input_offset; }
  uint8_t* output() { return base_ + L_.output_offset; }
  const ArenaLayout& layout() const { return L_; }

  std::atomic_ref<uint32_t> status() { return std::atomic_ref<uint32_t>(mailbox()->status); }
  std::atomic_ref<uint32_t> shutdown() { return std::atomic_ref<uint32_t>(state()->shutdown); }
  std::atomic_ref<uint32_t> failure() { return std::atomic_ref<uint32_t>(state()->generation_failure_code); }

  // Compare-and-swap guarded by the transition table.
  bool transition(MailboxStatus from, MailboxStatus to) {
    if (!mailbox_transition_allowed(from, to)) return false;
    uint32_t expect = static_cast<uint32_t>(from);
    return status().compare_exchange_strong(expect, static_cast<uint32_t>(to), std::memory_order_acq_rel);
  }

  WaitStatus wait_status(MailboxStatus want, uint64_t timeout_ns) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(timeout_ns);
    uint32_t spins = 0;
    while (true) {
      uint32_t s = status().load(std::memory_order_acquire);
      if (s == static_cast<uint32_t>(want)) return WaitStatus::Ready;
      if (s == static_cast<uint32_t>(MailboxStatus::Closed)) return WaitStatus::Cancelled;
      if (shutdown().load(std::memory_order_acquire) != 0) return WaitStatus::Cancelled;
      if ((++spins & 0xff) == 0) {
        if (std::chrono::steady_clock::now() > deadline) return WaitStatus::TimedOut;
        std::this_thread::sleep_for(std::chrono::microseconds(20));
      }
    }
  }

  // First failure wins.
  bool claim_failure(ResultCode code) {
    uint32_t expect = 0;
    return failure().compare_exchange_strong(expect, static_cast<uint32_t>(code), std::memory_order_acq_rel);
  }

  // Producer half: claim, stage, publish, wait for evaluation, copy back, acknowledge.
  ResultCode submit(const void* in, void* out, uint32_t rows, const RequestMetadata& meta, uint64_t timeout_ns) {
    if (rows > L_.max_rows) return ResultCode::ProtocolMismatch;
    if (!transition(MailboxStatus::Idle, MailboxStatus::Staging)) return ResultCode::ProtocolMismatch;
    Mailbox* m = mailbox();
    m->payload_rows = rows;
    m->request = meta;
    m->sequence += 1;
    std::memcpy(input(), in, static_cast<size_t>(rows) * L_.row_bytes);
    if (!transition(MailboxStatus::Staging, MailboxStatus::Published)) return ResultCode::ProtocolMismatch;
    WaitStatus w = wait_status(MailboxStatus::Evaluated, timeout_ns);
    if (w != WaitStatus::Ready) {
      // never trap: report the failure and leave the mailbox closed
      ResultCode rc = w == WaitStatus::TimedOut ? ResultCode::Timeout : ResultCode::Shutdown;
      claim_failure(rc);
      status().store(static_cast<uint32_t>(MailboxStatus::Closed), std::memory_order_release);
      return rc;
    }
    ResultCode rc = static_cast<ResultCode>(m->result_code);
    if (rc == ResultCode::Ok) std::memcpy(out, output(), static_cast<size_t>(rows) * L_.row_bytes);
    transition(MailboxStatus::Evaluated, MailboxStatus::Idle);
    return rc;
  }

 private:
  uint8_t* base_;
  ArenaLayout L_;
};

}  // namespace cpu
}  // namespace xpool
