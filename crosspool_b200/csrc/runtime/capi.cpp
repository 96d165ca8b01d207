// C ABI of libxpool_runtime.so (host-only): layouts, Lane scheduler, shared
// memory, the ECS control channel, the CPU transport mailbox and trace buffers.
// Loaded with ctypes from crosspool_b200/native/runtime.py.
#include <mutex>
#include <string.h>

#include <memory>
#include <new>
#include <vector>

#include "xpool/ecs_channel.hpp"
#include "xpool/protocol.hpp"
#include "xpool/scheduler.hpp"
#include "xpool/shmem.hpp"
#include "xpool/trace.hpp"
#include "xpool/transport_cpu.hpp"

using namespace xpool;

extern "C" {

int xr_abi_version(void) { return static_cast<int>(kAbiVersion); }

// ---------------------------------------------------------------- layouts

int xr_plan_ffn_slot(uint64_t capacity_rows, uint64_t hidden, uint64_t local_inter, uint64_t elem_bytes,
                     uint64_t* out4) {
  FfnSlotLayout L;
  if (!plan_ffn_slot(capacity_rows, hidden, local_inter, elem_bytes, &L)) return -1;
  out4[0] = L.record_offset;
  out4[1] = L.input_offset;
  out4[2] = L.act_offset;
  out4[3] = L.total_bytes;
  return 0;
}

int xr_plan_atn_slot(uint64_t capacity_rows, uint64_t hidden, uint64_t tp, uint64_t elem_bytes, uint64_t* out4) {
  AtnSlotLayout L;
  if (!plan_atn_slot(capacity_rows, hidden, tp, elem_bytes, &L)) return -1;
  out4[0] = L.completion_offset;
  out4[1] = L.output_offset;
  out4[2] = L.output_stride;
  out4[3] = L.total_bytes;
  return 0;
}

// 0 when the table is inconsistent, else the merged forward mode; offsets_out (may be null) receives every rank's
// first row in the merged payload.
uint32_t xr_dp_inspect_rows(uint32_t layout, uint32_t dp_size, uint32_t payload_rows, const uint32_t* modes,
                            const uint32_t* rank_rows, uint32_t* offsets_out) {
  if (layout > static_cast<uint32_t>(DpRowLayout::PackedByRank)) return 0;
  const DpRowLayout l = static_cast<DpRowLayout>(layout);
  const uint32_t merged = dp_inspect_rows(l, dp_size, payload_rows, modes, rank_rows);
  if (merged != 0 && offsets_out != nullptr)
    for (uint32_t r = 0; r < dp_size; ++r) offsets_out[r] = dp_row_offset(l, r, rank_rows);
  return merged;
}

// Invocation record fields -> ResultCode of validate_expected.
uint32_t xr_validate_invocation(uint32_t rows, uint32_t layer, uint32_t mode, uint32_t requirement, uint32_t dp_layout,
                                uint32_t sequence, uint32_t completed, uint32_t capacity_rows, uint32_t num_layers) {
  InvocationRecord r{};
  r.rows = rows, r.layer_ordinal = layer, r.forward_mode = mode, r.output_requirement = requirement;
  r.dp_row_layout = dp_layout, r.sequence = sequence;
  return static_cast<uint32_t>(validate_expected(r, completed, capacity_rows, num_layers));
}

uint32_t xr_validate_completion(uint32_t result_code, uint32_t rows, uint32_t sequence, uint32_t want_sequence,
                                uint32_t want_rows) {
  CompletionRecord c{};
  c.result_code = result_code, c.rows = rows, c.sequence = sequence;
  return static_cast<uint32_t>(validate_expected(c, want_sequence, want_rows));
}

// Process-wide runtime state. Initialising twice with the same role and device is a no-op (options are replaced);
// a different role or device is refused (-1); an unknown role is -2.
static RuntimeState g_runtime_state{0u, 0u, -1, DebugOptions{}};
static std::mutex g_runtime_mu;

int xr_runtime_initialize(uint32_t role, int32_t device, const uint32_t* options4) {
  if (role < static_cast<uint32_t>(RuntimeRole::Daemon) || role > static_cast<uint32_t>(RuntimeRole::FfnAgent)) return -2;
  std::lock_guard<std::mutex> g(g_runtime_mu);
  if (g_runtime_state.initialized != 0 && (g_runtime_state.role != role || g_runtime_state.device != device)) return -1;
  g_runtime_state.initialized = 1;
  g_runtime_state.role = role;
  g_runtime_state.device = device;
  if (options4 != nullptr)
    g_runtime_state.options = DebugOptions{options4[0], options4[1], options4[2], options4[3]};
  return 0;
}

// out7: initialized, role, device (as two's complement), four option words
void xr_runtime_state(uint32_t* out7) {
  std::lock_guard<std::mutex> g(g_runtime_mu);
  out7[0] = g_runtime_state.initialized;
  out7[1] = g_runtime_state.role;
  out7[2] = static_cast<uint32_t>(g_runtime_state.device);
  out7[3] = g_runtime_state.options.transport_observer;
  out7[4] = g_runtime_state.options.fabric_observer;
  out7[5] = g_runtime_state.options.graph_observer;
  out7[6] = g_runtime_state.options.ffn_routing_observer;
}

void xr_runtime_reset_for_tests(void) {
  std::lock_guard<std::mutex> g(g_runtime_mu);
  g_runtime_state = RuntimeState{0u, 0u, -1, DebugOptions{}};
}

uint64_t xr_record_bytes(int which) {
  switch (which) {
    case 0: return sizeof(InvocationRecord);
    case 1: return sizeof(CompletionRecord);
    case 2: return sizeof(FailureSlot);
    case 3: return sizeof(Mailbox);
    default: return 0;
  }
}

int xr_mailbox_transition_allowed(uint32_t from, uint32_t to) {
  return mailbox_transition_allowed(static_cast<MailboxStatus>(from), static_cast<MailboxStatus>(to)) ? 1 : 0;
}

// ---------------------------------------------------------------- scheduler

struct SchedHandle {
  std::vector<SchedulerEntry> entries;
  std::vector<LaneState> lanes;
  uint64_t next_ticket = 1;
  SchedulerPolicy policy;
  Scheduler view() {
    return Scheduler(entries.data(), static_cast<uint32_t>(entries.size()), lanes.data(),
                     static_cast<uint32_t>(lanes.size()), policy, &next_ticket);
  }
};

void* xr_sched_create(uint32_t instances, uint32_t lanes, uint32_t policy, uint64_t seed) {
  auto* h = new (std::nothrow) SchedHandle();
  if (h == nullptr) return nullptr;
  h->entries.assign(instances, SchedulerEntry{0, kNoLane, 0, 0, 0, 0, 0});
  h->lanes.assign(lanes, LaneState{0, 0, 0});
  h->policy = SchedulerPolicy{static_cast<SchedulerPolicyKind>(policy), seed};
  return h;
}
void xr_sched_destroy(void* p) { delete static_cast<SchedHandle*>(p); }
int xr_sched_enqueue(void* p, uint32_t instance, uint64_t sequence, uint64_t deadline) {
  return static_cast<SchedHandle*>(p)->view().enqueue(instance, sequence, deadline) ? 1 : 0;
}
int xr_sched_try(void* p, uint32_t* instance, uint32_t* lane, uint64_t* lease) {
  Decision d = static_cast<SchedHandle*>(p)->view().try_schedule();
  if (!d.scheduled) return 0;
  *instance = d.instance;
  *lane = d.lane;
  *lease = d.lease_sequence;
  return 1;
}
int xr_sched_active(void* p, uint32_t instance, uint32_t* lane, uint64_t* lease) {
  Decision d = static_cast<SchedHandle*>(p)->view().active_decision(instance);
  if (!d.scheduled) return 0;
  *lane = d.lane;
  *lease = d.lease_sequence;
  return 1;
}
int xr_sched_release(void* p, uint32_t instance, uint64_t lease) {
  return static_cast<SchedHandle*>(p)->view().release(instance, lease) ? 1 : 0;
}
uint64_t xr_splitmix64(uint64_t x) { return splitmix64(x); }

// ---------------------------------------------------------------- shared memory

void* xr_shm_create(const char* name, uint64_t bytes, int* err) {
  auto* s = new (std::nothrow) SharedMemory();
  if (s == nullptr) return nullptr;
  int rc = s->create(name, bytes);
  if (err != nullptr) *err = rc;
  if (rc != 0) {
    delete s;
    return nullptr;
  }
  return s;
}
void* xr_shm_attach(const char* name, int* err) {
  auto* s = new (std::nothrow) SharedMemory();
  if (s == nullptr) return nullptr;
  int rc = s->attach(name);
  if (err != nullptr) *err = rc;
  if (rc != 0) {
    delete s;
    return nullptr;
  }
  return s;
}
void* xr_shm_data(void* h) { return static_cast<SharedMemory*>(h)->data(); }
uint64_t xr_shm_size(void* h) { return static_cast<SharedMemory*>(h)->size(); }
void xr_shm_close(void* h) { delete static_cast<SharedMemory*>(h); }

// ---------------------------------------------------------------- ECS channel

struct EcsHandle {
  SharedMemory shm;
  ecs::ChannelHeader* header = nullptr;
  ecs::DeviceEntry* devices = nullptr;
  ecs::PartitionEntry* partitions = nullptr;
  void bind() {
    uint8_t* b = static_cast<uint8_t*>(shm.data());
    header = reinterpret_cast<ecs::ChannelHeader*>(b);
    devices = reinterpret_cast<ecs::DeviceEntry*>(b + sizeof(ecs::ChannelHeader));
    partitions = reinterpret_cast<ecs::PartitionEntry*>(b + sizeof(ecs::ChannelHeader) +
                                                        sizeof(ecs::DeviceEntry) * header->device_count);
  }
};

void* xr_ecs_create(const char* name, uint32_t devices, uint32_t partitions, uint32_t generation, int* err) {
  auto* h = new (std::nothrow) EcsHandle();
  if (h == nullptr) return nullptr;
  const uint64_t bytes = ecs::channel_bytes(devices, partitions);
  int rc = h->shm.create(name, bytes);
  if (err != nullptr) *err = rc;
  if (rc != 0) {
    delete h;
    return nullptr;
  }
  memset(h->shm.data(), 0, bytes);
  auto* hd = static_cast<ecs::ChannelHeader*>(h->shm.data());
  hd->abi_version = kAbiVersion;
  hd->device_count = devices;
  hd->partition_count = partitions;
  hd->generation = generation;
  hd->total_bytes = bytes;
  hd->magic = ecs::kChannelMagic;
  h->bind();
  return h;
}
void* xr_ecs_attach(const char* name, int* err) {
  auto* h = new (std::nothrow) EcsHandle();
  if (h == nullptr) return nullptr;
  int rc = h->shm.attach(name);
  if (rc == 0) {
    auto* hd = static_cast<ecs::ChannelHeader*>(h->shm.data());
    if (h->shm.size() < sizeof(ecs::ChannelHeader) || hd->magic != ecs::kChannelMagic ||
        hd->abi_version != kAbiVersion || hd->total_bytes > h->shm.size())
      rc = -71;  // EPROTO
  }
  if (err != nullptr) *err = rc;
  if (rc != 0) {
    delete h;
    return nullptr;
  }
  h->bind();
  return h;
}
void xr_ecs_close(void* p) { delete static_cast<EcsHandle*>(p); }
uint32_t xr_ecs_counts(void* p, uint32_t* devices, uint32_t* partitions) {
  auto* h = static_cast<EcsHandle*>(p);
  *devices = h->header->device_count;
  *partitions = h->header->partition_count;
  return h->header->generation;
}
int xr_ecs_set_device(void* p, uint32_t idx, uint32_t device) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->device_count) return -1;
  h->devices[idx].device = device;
  return 0;
}
int xr_ecs_set_partition(void* p, uint32_t idx, uint32_t device, uint32_t group, uint32_t rank, uint64_t floor_bytes,
                         uint64_t reservation_bytes) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  ecs::PartitionEntry& e = h->partitions[idx];
  e.device = device;
  e.group = group;
  e.rank = rank;
  e.floor_bytes = floor_bytes;
  e.reservation_bytes = reservation_bytes;
  return 0;
}
int xr_ecs_get_partition(void* p, uint32_t idx, uint64_t* out5) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  const ecs::PartitionEntry& e = h->partitions[idx];
  out5[0] = e.device;
  out5[1] = e.group;
  out5[2] = e.rank;
  out5[3] = e.floor_bytes;
  out5[4] = e.reservation_bytes;
  return 0;
}
int xr_ecs_publish_report(void* p, uint32_t idx, uint64_t free_bytes, uint64_t total_bytes, uint64_t seq) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->device_count) return -1;
  ecs::seq_publish(&h->devices[idx].report, ecs::DeviceMemoryReport{free_bytes, total_bytes, seq});
  return 0;
}
int xr_ecs_read_report(void* p, uint32_t idx, uint64_t* out3) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->device_count) return -1;
  ecs::DeviceMemoryReport r;
  if (!ecs::seq_read(&h->devices[idx].report, &r, nullptr)) return -2;
  out3[0] = r.free_bytes;
  out3[1] = r.total_bytes;
  out3[2] = r.report_sequence;
  return 0;
}
int xr_ecs_publish_command(void* p, uint32_t idx, uint64_t sequence, uint64_t target_bytes) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  ecs::seq_publish(&h->partitions[idx].command, ecs::QuotaCommand{sequence, target_bytes});
  return 0;
}
int xr_ecs_read_command(void* p, uint32_t idx, uint64_t* out2) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  ecs::QuotaCommand c;
  if (!ecs::seq_read(&h->partitions[idx].command, &c, nullptr)) return -2;
  out2[0] = c.sequence;
  out2[1] = c.target_bytes;
  return 0;
}
int xr_ecs_publish_demand(void* p, uint32_t idx, uint64_t evaluated_sequence, uint64_t required_bytes,
                          uint64_t deadline_ns, uint64_t mapped_bytes) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  ecs::seq_publish(&h->partitions[idx].demand,
                   ecs::QuotaDemand{evaluated_sequence, required_bytes, deadline_ns, mapped_bytes});
  return 0;
}
int xr_ecs_read_demand(void* p, uint32_t idx, uint64_t* out4) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  ecs::QuotaDemand d;
  if (!ecs::seq_read(&h->partitions[idx].demand, &d, nullptr)) return -2;
  out4[0] = d.evaluated_sequence;
  out4[1] = d.required_bytes;
  out4[2] = d.deadline_monotonic_ns;
  out4[3] = d.mapped_bytes;
  return 0;
}
int xr_ecs_publish_completion(void* p, uint32_t idx, uint64_t sequence, uint64_t mapped_bytes) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  ecs::seq_publish(&h->partitions[idx].completion, ecs::QuotaCompletion{sequence, mapped_bytes});
  return 0;
}
int xr_ecs_read_completion(void* p, uint32_t idx, uint64_t* out2) {
  auto* h = static_cast<EcsHandle*>(p);
  if (idx >= h->header->partition_count) return -1;
  ecs::QuotaCompletion c;
  if (!ecs::seq_read(&h->partitions[idx].completion, &c, nullptr)) return -2;
  out2[0] = c.sequence;
  out2[1] = c.mapped_bytes;
  return 0;
}

// ---------------------------------------------------------------- CPU transport mailbox

struct MboxHandle {
  SharedMemory shm;
  cpu::ArenaLayout layout;
  std::unique_ptr<cpu::ArenaView> view;
};

uint64_t xr_mbox_bytes(uint64_t max_rows, uint64_t row_bytes) {
  cpu::ArenaLayout L;
  return cpu::plan_arena(max_rows, row_bytes, &L) ? L.total_bytes : 0;
}

void* xr_mbox_create(const char* name, uint64_t max_rows, uint64_t row_bytes, int* err) {
  auto* h = new (std::nothrow) MboxHandle();
  if (h == nullptr) return nullptr;
  int rc = cpu::plan_arena(max_rows, row_bytes, &h->layout) ? 0 : -22;
  if (rc == 0) rc = h->shm.create(name, h->layout.total_bytes);
  if (err != nullptr) *err = rc;
  if (rc != 0) {
    delete h;
    return nullptr;
  }
  h->view = std::make_unique<cpu::ArenaView>(h->shm.data(), h->layout);
  h->view->format();
  return h;
}
void* xr_mbox_attach(const char* name, uint64_t max_rows, uint64_t row_bytes, int* err) {
  auto* h = new (std::nothrow) MboxHandle();
  if (h == nullptr) return nullptr;
  int rc = cpu::plan_arena(max_rows, row_bytes, &h->layout) ? 0 : -22;
  if (rc == 0) rc = h->shm.attach(name);
  if (rc == 0) {
    h->view = std::make_unique<cpu::ArenaView>(h->shm.data(), h->layout);
    if (h->shm.size() < h->layout.total_bytes || !h->view->valid()) rc = -71;
  }
  if (err != nullptr) *err = rc;
  if (rc != 0) {
    delete h;
    return nullptr;
  }
  return h;
}
void xr_mbox_close(void* p) { delete static_cast<MboxHandle*>(p); }
uint32_t xr_mbox_status(void* p) {
  return static_cast<MboxHandle*>(p)->view->status().load(std::memory_order_acquire);
}
uint32_t xr_mbox_failure(void* p) {
  return static_cast<MboxHandle*>(p)->view->failure().load(std::memory_order_acquire);
}
// consumer: Dormant -> Idle
int xr_mbox_activate(void* p) {
  return static_cast<MboxHandle*>(p)->view->transition(MailboxStatus::Dormant, MailboxStatus::Idle) ? 0 : -1;
}
void xr_mbox_shutdown(void* p) {
  static_cast<MboxHandle*>(p)->view->shutdown().store(1, std::memory_order_release);
}
int xr_mbox_wait_status(void* p, uint32_t want, uint64_t timeout_ns) {
  return static_cast<int>(static_cast<MboxHandle*>(p)->view->wait_status(static_cast<MailboxStatus>(want), timeout_ns));
}
// producer: blocking submit; returns a ResultCode.
uint32_t xr_mbox_submit(void* p, const void* in, void* out, uint32_t rows, uint32_t layer, uint32_t mode,
                        uint32_t requirement, uint32_t dp_layout, uint64_t timeout_ns) {
  RequestMetadata m{layer, mode, requirement, dp_layout};
  return static_cast<uint32_t>(static_cast<MboxHandle*>(p)->view->submit(in, out, rows, m, timeout_ns));
}
// consumer: waits for Published; fills rows/layer/mode/sequence. Returns WaitStatus.
int xr_mbox_take(void* p, uint64_t timeout_ns, uint32_t* out4) {
  auto* h = static_cast<MboxHandle*>(p);
  cpu::WaitStatus w = h->view->wait_status(MailboxStatus::Published, timeout_ns);
  if (w != cpu::WaitStatus::Ready) return static_cast<int>(w);
  const Mailbox* m = h->view->mailbox();
  out4[0] = m->payload_rows;
  out4[1] = m->request.layer_ordinal;
  out4[2] = m->request.forward_mode;
  out4[3] = m->sequence;
  return 0;
}
void* xr_mbox_input(void* p) { return static_cast<MboxHandle*>(p)->view->input(); }
void* xr_mbox_output(void* p) { return static_cast<MboxHandle*>(p)->view->output(); }
int xr_mbox_complete(void* p, uint32_t result_code) {
  auto* h = static_cast<MboxHandle*>(p);
  h->view->mailbox()->result_code = result_code;
  if (result_code != 0) h->view->claim_failure(static_cast<ResultCode>(result_code));
  return h->view->transition(MailboxStatus::Published, MailboxStatus::Evaluated) ? 0 : -1;
}

// ---------------------------------------------------------------- trace buffers

void* xr_trace_create(uint32_t capacity) {
  auto* t = new (std::nothrow) trace::HostBuffer(capacity);
  return t;
}
void xr_trace_destroy(void* p) { delete static_cast<trace::HostBuffer*>(p); }
int xr_trace_record(void* p, uint32_t kind, uint32_t a, uint32_t b, uint64_t timestamp_ns) {
  return static_cast<trace::HostBuffer*>(p)->record(kind, a, b, timestamp_ns) ? 1 : 0;
}
uint64_t xr_trace_counts(void* p, uint64_t* dropped) {
  auto* t = static_cast<trace::HostBuffer*>(p);
  *dropped = t->dropped();
  return t->size();
}
uint64_t xr_trace_read(void* p, uint64_t first, uint64_t count, uint64_t* out /* 3 words per event */) {
  return static_cast<trace::HostBuffer*>(p)->read(first, count, out);
}

}  // extern "C"
