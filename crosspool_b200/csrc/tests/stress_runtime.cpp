// Concurrency stress of the host runtime (mailbox hand-off, ECS seqlock channel, trace buffer), meant to be
// built with -fsanitize=thread or -fsanitize=address,undefined: the reference has no sanitizer targets
// (its CMake has none); here the pure C++ protocol code is exercised under both.
//
//   mailbox : a producer thread submits 2000 requests, a consumer thread takes, transforms and completes them;
//             every reply must be the transform of its request (no torn payloads, no lost hand-offs).
//   seqlock : one writer publishes (sequence, 3 * sequence) pairs into a channel slot while readers poll;
//             a reader must never observe a pair that was not published together.
//   trace   : four writers race for slots of a small buffer; size + dropped must equal the attempts.
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <thread>
#include <vector>

extern "C" {
void* xr_mbox_create(const char* name, uint64_t max_rows, uint64_t row_bytes, int* err);
void* xr_mbox_attach(const char* name, uint64_t max_rows, uint64_t row_bytes, int* err);
void xr_mbox_close(void* p);
int xr_mbox_activate(void* p);
void xr_mbox_shutdown(void* p);
uint32_t xr_mbox_submit(void* p, const void* in, void* out, uint32_t rows, uint32_t layer, uint32_t mode, uint32_t requirement,
                        uint32_t dp_layout, uint64_t timeout_ns);
int xr_mbox_take(void* p, uint64_t timeout_ns, uint32_t* out4);
void* xr_mbox_input(void* p);
void* xr_mbox_output(void* p);
int xr_mbox_complete(void* p, uint32_t result_code);
void* xr_ecs_create(const char* name, uint32_t devices, uint32_t partitions, uint32_t generation, int* err);
void xr_ecs_close(void* p);
int xr_ecs_publish_demand(void* p, uint32_t idx, uint64_t evaluated_sequence, uint64_t required_bytes, uint64_t deadline_ns,
                          uint64_t mapped_bytes);
int xr_ecs_read_demand(void* p, uint32_t idx, uint64_t* out4);
void* xr_trace_create(uint32_t capacity);
void xr_trace_destroy(void* p);
int xr_trace_record(void* p, uint32_t kind, uint32_t a, uint32_t b, uint64_t timestamp_ns);
uint64_t xr_trace_counts(void* p, uint64_t* dropped);
}

static int fail(const char* what) {
  fprintf(stderr, "stress_runtime: %s\n", what);
  return 1;
}

static int stress_mailbox() {
  char name[64];
  snprintf(name, sizeof(name), "/xp-stress-mbox-%d", static_cast<int>(getpid()));
  int err = 0;
  const uint32_t rows = 4, row_bytes = 64, n = 2000;
  void* prod = xr_mbox_create(name, rows, row_bytes, &err);
  if (prod == nullptr) return fail("mailbox create");
  void* cons = xr_mbox_attach(name, rows, row_bytes, &err);
  if (cons == nullptr) return fail("mailbox attach");
  std::atomic<int> bad{0};
  std::atomic<bool> active{false};
  std::thread consumer([&] {
    if (xr_mbox_activate(cons) != 0) bad++;
    active.store(true, std::memory_order_release);
    for (uint32_t i = 0; i < n; ++i) {
      uint32_t meta[4];
      if (xr_mbox_take(cons, 5000000000ull, meta) != 0) {
        bad++;
        return;
      }
      const uint8_t* in = static_cast<const uint8_t*>(xr_mbox_input(cons));
      uint8_t* out = static_cast<uint8_t*>(xr_mbox_output(cons));
      for (uint32_t b = 0; b < meta[0] * row_bytes; ++b) out[b] = static_cast<uint8_t>(in[b] ^ 0x5a);
      if (xr_mbox_complete(cons, 0) != 0) bad++;
    }
  });
  std::vector<uint8_t> in(rows * row_bytes), out(rows * row_bytes);
  while (!active.load(std::memory_order_acquire)) std::this_thread::yield();  // a Dormant mailbox accepts nothing
  for (uint32_t i = 0; i < n; ++i) {
    for (size_t b = 0; b < in.size(); ++b) in[b] = static_cast<uint8_t>(i + b);
    if (xr_mbox_submit(prod, in.data(), out.data(), rows, i % 7, 2, 1, 0, 5000000000ull) != 0) {
      bad++;
      break;
    }
    for (size_t b = 0; b < in.size(); ++b)
      if (out[b] != static_cast<uint8_t>(in[b] ^ 0x5a)) bad++;
  }
  consumer.join();
  xr_mbox_close(cons);
  xr_mbox_close(prod);
  return bad.load() == 0 ? 0 : fail("mailbox hand-off corrupted or lost");
}

static int stress_seqlock() {
  char name[64];
  snprintf(name, sizeof(name), "/xp-stress-ecs-%d", static_cast<int>(getpid()));
  int err = 0;
  void* ch = xr_ecs_create(name, 1, 1, 1, &err);
  if (ch == nullptr) return fail("ecs create");
  std::atomic<bool> stop{false};
  std::atomic<int> torn{0};
  std::vector<std::thread> readers;
  for (int r = 0; r < 3; ++r)
    readers.emplace_back([&] {
      uint64_t v[4];
      while (!stop.load(std::memory_order_acquire)) {
        if (xr_ecs_read_demand(ch, 0, v) != 0) continue;
        if (v[0] == 0) continue;  // nothing published yet
        if (v[1] != 3 * v[0] || v[2] != v[0] + 7 || v[3] != 2 * v[0]) torn++;
      }
    });
  for (uint64_t s = 1; s <= 200000; ++s) xr_ecs_publish_demand(ch, 0, s, 3 * s, s + 7, 2 * s);
  stop.store(true, std::memory_order_release);
  for (auto& t : readers) t.join();
  xr_ecs_close(ch);
  return torn.load() == 0 ? 0 : fail("seqlock reader saw a torn record");
}

static int stress_trace() {
  void* t = xr_trace_create(1000);
  std::vector<std::thread> ws;
  for (int w = 0; w < 4; ++w)
    ws.emplace_back([&, w] {
      for (uint32_t i = 0; i < 1000; ++i) xr_trace_record(t, 1 + w, i, w, i);
    });
  for (auto& th : ws) th.join();
  uint64_t dropped = 0;
  const uint64_t n = xr_trace_counts(t, &dropped);
  xr_trace_destroy(t);
  return (n == 1000 && dropped == 3000) ? 0 : fail("trace buffer lost or duplicated events");
}

int main() {
  int rc = stress_mailbox();
  rc |= stress_seqlock();
  rc |= stress_trace();
  if (rc == 0) printf("stress_runtime ok\n");
  return rc;
}
