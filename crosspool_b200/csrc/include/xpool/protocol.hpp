// Host- and device-compilable protocol core: enums of the FFN ABI, the
// Transport mailbox state machine, invocation records and the arena layout
// planner. Everything here is plain C++ with no CUDA dependency so that the
// same structures are exercised by CPU tests, used by the CPU loopback fabric,
// and placed in GPU peer memory by the CUDA data plane.
//
// Semantics follow the reference's ABI (src/cext-include/xpool/ffn.hpp:1-87,
// transport/protocol.hpp:33-46, fabric/protocol.hpp:72-234) but the record set
// is collapsed: the producer of the hidden states writes the payload and one
// invocation record straight into the FFN rank's memory, and each FFN rank
// answers with its partial and one sequence word; there is no coordinator hop
// on the payload path.
#pragma once

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define XP_HD __host__ __device__
#else
#define XP_HD
#endif

namespace xpool {

constexpr uint32_t kAbiVersion = 21;
constexpr uint64_t kAllocationAlignment = 256;  // every arena region
constexpr uint64_t kPayloadAlignment = 16;      // every payload row

enum class RuntimeRole : uint32_t { None = 0, Daemon = 1, Instance = 2, AtnAgent = 3, FfnAgent = 4 };
enum class ForwardMode : uint32_t { Prefill = 1, Decode = 2, Idle = 4 };
enum class OutputRequirement : uint32_t { PerRankComplete = 1, GroupSumComplete = 2 };
enum class DpRowLayout : uint32_t { None = 0, UniformByRank = 1, PackedByRank = 2 };
enum class ResultCode : uint32_t { Ok = 0, Shutdown = 1, ProtocolMismatch = 2, Timeout = 3 };
enum class LayerKind : uint32_t { Dense = 1, Moe = 2 };
enum class PayloadDtype : uint32_t { BF16 = 1, FP16 = 2 };

// ---------------------------------------------------------------- mailbox

// Single-producer single-consumer mailbox between an Instance rank and the
// transport consumer. Transitions:
//   Dormant -> Idle (consumer activates) ; Idle -> Staging (producer claims) ;
//   Staging -> Published ; Published -> Evaluated (consumer) ; Evaluated -> Idle
//   (producer acknowledges) ; any -> Closed.
enum class MailboxStatus : uint32_t {
  Dormant = 0, Idle = 1, Staging = 2, Published = 3, Evaluated = 4, Closed = 5
};

struct RequestMetadata {
  uint32_t layer_ordinal;
  uint32_t forward_mode;
  uint32_t output_requirement;
  uint32_t dp_row_layout;
};

struct alignas(8) Mailbox {
  uint32_t status;
  uint32_t result_code;
  uint32_t payload_rows;
  uint32_t sequence;
  RequestMetadata request;
};

XP_HD inline bool mailbox_transition_allowed(MailboxStatus from, MailboxStatus to) {
  if (to == MailboxStatus::Closed) return true;
  switch (from) {
    case MailboxStatus::Dormant: return to == MailboxStatus::Idle;
    case MailboxStatus::Idle: return to == MailboxStatus::Staging;
    case MailboxStatus::Staging: return to == MailboxStatus::Published;
    case MailboxStatus::Published: return to == MailboxStatus::Evaluated;
    case MailboxStatus::Evaluated: return to == MailboxStatus::Idle;
    default: return false;
  }
}

// ---------------------------------------------------------------- invocation record

// Written by the attention side into an FFN rank's memory before the sequence
// word of the slot is released (256-byte aligned like the reference's
// Publication<>, fabric/protocol.hpp:24-31).
struct alignas(256) InvocationRecord {
  uint32_t rows;            // live payload rows
  uint32_t layer_ordinal;   // index into the instance's layer table
  uint32_t forward_mode;    // ForwardMode
  uint32_t deadline_us;     // SLO deadline: microseconds of the host's monotonic clock mod 2^32; 0 = none
  uint32_t output_requirement;
  uint32_t dp_row_layout;
  uint32_t reserved[2];
  uint32_t sequence;        // released last; monotonic per slot, starts at 1
};

struct alignas(256) CompletionRecord {
  uint32_t result_code;
  uint32_t rows;
  uint32_t reserved[2];
  uint32_t sequence;
};

// First failure wins (the reference's canonical generation failure,
// fabric/protocol.hpp:236-270): whoever moves `claim` from 0 owns the slot, fills the payload and
// releases claim = kFailureClaimed; everybody else only reads. Waiting kernels poll `claim` as their
// cancel word, so one failure ends every wait of the generation within microseconds.
struct alignas(64) FailureSlot {
  uint32_t claim;  // 0 free, kFailureWriting while the owner fills the payload, kFailureClaimed after
  uint32_t result_code;
  uint32_t origin;  // PE that met the failure
  uint32_t instance_index;
  uint32_t invocation_sequence;
  uint32_t layer_ordinal;
};
constexpr uint32_t kFailureWriting = 2;
constexpr uint32_t kFailureClaimed = 1;
// Both 256-byte record blocks have room behind their fields: the failure slot of an FFN-side Instance slot
// sits this many bytes into its InvocationRecord block, the failure slot of an attention-side slot this many
// bytes into the block of its first CompletionRecord.
constexpr uint64_t kFailureSlotOffset = 64;

// ---------------------------------------------------------------- checked arithmetic

struct Checked {
  uint64_t value;
  bool ok;
};
XP_HD inline Checked checked_add(uint64_t a, uint64_t b) {
  uint64_t r = a + b;
  return {r, r >= a};
}
XP_HD inline Checked checked_mul(uint64_t a, uint64_t b) {
  if (a == 0 || b == 0) return {0, true};
  uint64_t r = a * b;
  return {r, r / a == b};
}
XP_HD inline Checked checked_align_up(uint64_t v, uint64_t a) {
  if (a == 0 || (a & (a - 1)) != 0) return {0, false};
  Checked s = checked_add(v, a - 1);
  return {s.value & ~(a - 1), s.ok};
}

// ---------------------------------------------------------------- arena layouts

constexpr uint64_t kTransportMagic = 0x5850423230305452ull;  // "XPB200TR"
constexpr uint64_t kFabricMagic = 0x5850423230304642ull;     // "XPB200FB"

struct LayoutHeader {
  uint64_t magic;
  uint32_t abi_version;
  uint32_t reserved;
  uint64_t layout_size;
  uint64_t total_bytes;
  uint64_t state_offset;
};

// FFN-rank side slot of one (instance, attention rank): payload in, record, flag.
struct FfnSlotLayout {
  uint64_t record_offset;   // InvocationRecord
  uint64_t input_offset;    // [capacity_rows, hidden] payload
  uint64_t act_offset;      // [capacity_rows, local_intermediate] scratch between the two GEMMs
  uint64_t total_bytes;
};

// Attention-rank side slot of one instance: tp partial outputs + completion words.
struct AtnSlotLayout {
  uint64_t completion_offset;  // tp * CompletionRecord
  uint64_t output_offset;      // [tp, capacity_rows, hidden]
  uint64_t output_stride;      // bytes between tp partials
  uint64_t total_bytes;
};

inline bool plan_ffn_slot(uint64_t capacity_rows, uint64_t hidden, uint64_t local_inter,
                          uint64_t elem_bytes, FfnSlotLayout* out) {
  uint64_t off = 0;
  out->record_offset = off;
  off += sizeof(InvocationRecord);
  Checked a = checked_align_up(off, kAllocationAlignment);
  if (!a.ok) return false;
  out->input_offset = a.value;
  Checked in = checked_mul(checked_mul(capacity_rows, hidden).value, elem_bytes);
  if (!checked_mul(capacity_rows, hidden).ok || !in.ok) return false;
  a = checked_align_up(a.value + in.value, kAllocationAlignment);
  if (!a.ok) return false;
  out->act_offset = a.value;
  Checked act = checked_mul(checked_mul(capacity_rows, local_inter).value, elem_bytes);
  if (!checked_mul(capacity_rows, local_inter).ok || !act.ok) return false;
  a = checked_align_up(a.value + act.value, kAllocationAlignment);
  if (!a.ok) return false;
  out->total_bytes = a.value;
  return true;
}

inline bool plan_atn_slot(uint64_t capacity_rows, uint64_t hidden, uint64_t tp, uint64_t elem_bytes,
                          AtnSlotLayout* out) {
  out->completion_offset = 0;
  Checked c = checked_mul(tp, sizeof(CompletionRecord));
  if (!c.ok) return false;
  Checked a = checked_align_up(c.value, kAllocationAlignment);
  out->output_offset = a.value;
  Checked one = checked_mul(checked_mul(capacity_rows, hidden).value, elem_bytes);
  if (!checked_mul(capacity_rows, hidden).ok || !one.ok) return false;
  Checked st = checked_align_up(one.value, kAllocationAlignment);
  if (!st.ok) return false;
  out->output_stride = st.value;
  Checked all = checked_mul(st.value, tp);
  if (!all.ok) return false;
  Checked tot = checked_add(a.value, all.value);
  if (!tot.ok) return false;
  out->total_bytes = tot.value;
  return true;
}

}  // namespace xpool
