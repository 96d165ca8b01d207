// Elastic physical backing of a paged KV cache on CUDA virtual memory management.
//
// Every KV buffer (one K and one V per layer) is a fixed range of one reserved
// virtual address span, so tensors over it keep their addresses for the life of
// the process and captured CUDA graphs stay valid. Physical memory is attached
// and detached in *bundles*: bundle b backs the same page range of every buffer
// (one allocation of `chunk_bytes` per buffer). Mapping charges a MemoryQuota
// shared by the co-located Instances of a device; an out-of-memory answer from
// the driver (or a quota refusal) rolls back everything the call had mapped.
//
// The reference implements this in Python over cuda-bindings
// (src/xpool/integrations/sglang/ecs/vmm.py:25-351); here it is native, with the
// driver entry points injected through a table so that the ledger and rollback
// logic are testable on a machine without a GPU.
#pragma once

#include <stddef.h>
#include <stdint.h>

#include <mutex>
#include <vector>

namespace xpool {
namespace vmm {

// Subset of the CUDA driver VMM API, C-callable. Return 0 on success, 2 for
// out-of-memory (CUDA_ERROR_OUT_OF_MEMORY), anything else for other failures.
struct DriverApi {
  void* ctx;
  int (*granularity)(void* ctx, int device, uint64_t* out);
  int (*reserve)(void* ctx, uint64_t bytes, uint64_t alignment, uint64_t* va);
  int (*release_va)(void* ctx, uint64_t va, uint64_t bytes);
  int (*create)(void* ctx, int device, uint64_t bytes, uint64_t* handle);
  int (*release)(void* ctx, uint64_t handle);
  int (*map)(void* ctx, uint64_t va, uint64_t bytes, uint64_t handle);
  int (*unmap)(void* ctx, uint64_t va, uint64_t bytes);
  int (*set_access)(void* ctx, uint64_t va, uint64_t bytes, int device);
};

constexpr int kOutOfMemory = 2;
constexpr int kQuotaExceeded = -2;

// Byte ledger shared by the Instances that borrow from one another.
class MemoryQuota {
 public:
  explicit MemoryQuota(uint64_t limit) : limit_(limit) {}
  bool charge(uint64_t bytes) {
    std::lock_guard<std::mutex> g(mu_);
    if (charged_ + bytes > limit_) return false;
    charged_ += bytes;
    return true;
  }
  void refund(uint64_t bytes) {
    std::lock_guard<std::mutex> g(mu_);
    charged_ = bytes > charged_ ? 0 : charged_ - bytes;
  }
  void set_limit(uint64_t limit) {
    std::lock_guard<std::mutex> g(mu_);
    limit_ = limit;
  }
  uint64_t limit() const { return limit_; }
  uint64_t charged() const { return charged_; }

 private:
  mutable std::mutex mu_;
  uint64_t limit_;
  uint64_t charged_ = 0;
};

class KvBacking {
 public:
  KvBacking(const DriverApi& api, int device, uint32_t n_buffers, uint64_t buffer_bytes, uint64_t chunk_bytes,
            MemoryQuota* quota);
  ~KvBacking();
  KvBacking(const KvBacking&) = delete;
  KvBacking& operator=(const KvBacking&) = delete;

  int reserve();  // 0 or a driver error
  uint64_t base() const { return va_; }
  uint64_t buffer_address(uint32_t buffer) const { return va_ + static_cast<uint64_t>(buffer) * buffer_bytes_; }
  uint32_t bundle_count() const { return n_bundles_; }
  uint64_t bundle_bytes() const { return static_cast<uint64_t>(n_buffers_) * chunk_bytes_; }
  uint64_t mapped_bytes() const { return mapped_ * bundle_bytes(); }
  bool is_mapped(uint32_t bundle) const { return bundle < n_bundles_ && !handles_[bundle].empty(); }

  // Maps the given bundles. On failure nothing of this call stays mapped; returns
  // 0, kOutOfMemory, kQuotaExceeded or another driver code.
  int try_map(const uint32_t* bundles, uint32_t n);
  // Unmaps and releases; unknown or unmapped ids are ignored. Returns bundles unmapped.
  uint32_t unmap(const uint32_t* bundles, uint32_t n);

 private:
  int map_one(uint32_t bundle);
  void unmap_one(uint32_t bundle);

  DriverApi api_;
  int device_;
  uint32_t n_buffers_;
  uint64_t buffer_bytes_, chunk_bytes_;
  uint32_t n_bundles_;
  MemoryQuota* quota_;
  uint64_t va_ = 0;
  uint64_t mapped_ = 0;
  std::vector<std::vector<uint64_t>> handles_;  // per bundle: one handle per buffer
};

// A driver that only keeps books: a byte budget, call counters, optional failure
// injection. Used by CPU tests; never touches a GPU.
struct FakeDriver {
  uint64_t budget_bytes = 0;
  uint64_t allocated_bytes = 0;
  uint64_t next_handle = 1;
  uint64_t next_va = 0x100000000ull;
  uint64_t granularity_bytes = 2ull << 20;
  int fail_create_after = -1;  // >= 0: the (n+1)-th create from now fails with out-of-memory
  int fail_map_after = -1;
  uint64_t creates = 0, releases = 0, maps = 0, unmaps = 0, reserves = 0;
  std::vector<std::pair<uint64_t, uint64_t>> live;  // handle, bytes
  DriverApi api();
};

}  // namespace vmm
}  // namespace xpool
