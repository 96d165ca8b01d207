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

// ---------------------------------------------------------------- runtime state and debug options
//
// One per process: which role the process plays, on which device, and which observers are switched on
// (the reference's RuntimeState and debug Options, runtime.hpp:17-22 and debug/options.hpp). The options are
// mirrored into constant memory of the kernel library (`xp_debug_options_set`) so that device code can read them.
struct DebugOptions {
  uint32_t transport_observer;
  uint32_t fabric_observer;
  uint32_t graph_observer;
  uint32_t ffn_routing_observer;
};

struct RuntimeState {
  uint32_t initialized;
  uint32_t role;     // RuntimeRole
  int32_t device;    // -1: none (the daemon)
  DebugOptions options;
};

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

// ---------------------------------------------------------------- record expectations
//
// What a consumer checks before it acts on a record (the reference validates every publication against the
// expected key and bounds, fabric/protocol.hpp `validate_expected`). Each returns ResultCode::Ok or
// ProtocolMismatch; nothing traps.

XP_HD inline bool valid_forward_mode(uint32_t m) {
  return m == static_cast<uint32_t>(ForwardMode::Prefill) || m == static_cast<uint32_t>(ForwardMode::Decode) ||
         m == static_cast<uint32_t>(ForwardMode::Idle);
}

// An invocation read from a slot whose previous completed sequence is `completed`: the next sequence, a layer the
// Instance has, a known mode and requirement, rows within capacity (0 rows only for an idle step).
XP_HD inline ResultCode validate_expected(const InvocationRecord& r, uint32_t completed, uint32_t capacity_rows,
                                          uint32_t num_layers) {
  const bool ok = r.sequence == completed + 1u && r.layer_ordinal < num_layers && valid_forward_mode(r.forward_mode) &&
                  r.rows <= capacity_rows &&
                  (r.rows > 0u || r.forward_mode == static_cast<uint32_t>(ForwardMode::Idle)) &&
                  (r.output_requirement == 0u ||   // 0: the publisher predates the field (treated as per-rank complete)
                   r.output_requirement == static_cast<uint32_t>(OutputRequirement::PerRankComplete) ||
                   r.output_requirement == static_cast<uint32_t>(OutputRequirement::GroupSumComplete)) &&
                  r.dp_row_layout <= static_cast<uint32_t>(DpRowLayout::PackedByRank);
  return ok ? ResultCode::Ok : ResultCode::ProtocolMismatch;
}

// A completion read by the attention side for the invocation (`sequence`, `rows`) it published.
XP_HD inline ResultCode validate_expected(const CompletionRecord& c, uint32_t sequence, uint32_t rows) {
  if (c.sequence != sequence) return ResultCode::ProtocolMismatch;
  if (c.result_code != static_cast<uint32_t>(ResultCode::Ok)) return static_cast<ResultCode>(c.result_code);
  return c.rows == rows ? ResultCode::Ok : ResultCode::ProtocolMismatch;
}

// ---------------------------------------------------------------- attention-DP row tables
//
// The rows that the data-parallel attention ranks of one Instance contribute to one merged invocation
// (the reference's Coordinator checks the same before it admits a rendezvous, fabric/coordinator.cu:55-117).
//   None:          one rank (dp_size 1); its rows are the payload.
//   UniformByRank: every rank holds the same number of (padded) rows; payload = dp_size x that number.
//   PackedByRank:  ranks hold their own counts back to back; an idle rank holds none; the counts sum to the payload.
// `modes[r]` / `rank_rows[r]` are rank r's forward mode and row count. Returns the merged forward mode (Prefill if
// any rank prefills, else Decode) or 0 when the table is inconsistent.
XP_HD inline uint32_t dp_inspect_rows(DpRowLayout layout, uint32_t dp_size, uint32_t payload_rows, const uint32_t* modes,
                                      const uint32_t* rank_rows) {
  if (dp_size == 0 || (dp_size == 1) != (layout == DpRowLayout::None)) return 0;
  const uint32_t idle = static_cast<uint32_t>(ForwardMode::Idle);
  bool any_prefill = false, any_non_idle = false;
  uint64_t packed = 0;
  uint32_t uniform = 0;
  for (uint32_t r = 0; r < dp_size; ++r) {
    const uint32_t mode = modes[r], rows = rank_rows[r];
    if (!valid_forward_mode(mode)) return 0;
    if (layout == DpRowLayout::None && (mode == idle || rows != payload_rows)) return 0;
    if (layout == DpRowLayout::PackedByRank && ((mode == idle) != (rows == 0))) return 0;
    if (layout == DpRowLayout::UniformByRank && (rows == 0 || (r != 0 && rows != uniform))) return 0;
    any_prefill = any_prefill || mode == static_cast<uint32_t>(ForwardMode::Prefill);
    any_non_idle = any_non_idle || mode != idle;
    if (layout == DpRowLayout::PackedByRank) {
      if (rows > payload_rows - packed) return 0;
      packed += rows;
    } else if (layout == DpRowLayout::UniformByRank && r == 0) {
      uniform = rows;
    }
  }
  if (!any_non_idle) return 0;
  if (layout == DpRowLayout::PackedByRank && packed != payload_rows) return 0;
  if (layout == DpRowLayout::UniformByRank && (payload_rows % dp_size != 0 || payload_rows / dp_size != uniform)) return 0;
  return static_cast<uint32_t>(any_prefill ? ForwardMode::Prefill : ForwardMode::Decode);
}

// First payload row of rank `r` in the merged invocation (valid tables only).
XP_HD inline uint32_t dp_row_offset(DpRowLayout layout, uint32_t r, const uint32_t* rank_rows) {
  if (layout == DpRowLayout::UniformByRank) return r * rank_rows[0];
  uint32_t off = 0;
  if (layout == DpRowLayout::PackedByRank)
    for (uint32_t i = 0; i < r; ++i) off += rank_rows[i];
  return off;
}

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
