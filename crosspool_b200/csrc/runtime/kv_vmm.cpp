#include "xpool/kv_vmm.hpp"

#include <algorithm>
#include <new>

namespace xpool {
namespace vmm {

KvBacking::KvBacking(const DriverApi& api, int device, uint32_t n_buffers, uint64_t buffer_bytes, uint64_t chunk_bytes,
                     MemoryQuota* quota)
    : api_(api), device_(device), n_buffers_(n_buffers), buffer_bytes_(buffer_bytes), chunk_bytes_(chunk_bytes),
      n_bundles_(chunk_bytes ? static_cast<uint32_t>(buffer_bytes / chunk_bytes) : 0), quota_(quota),
      handles_(n_bundles_) {}

KvBacking::~KvBacking() {
  for (uint32_t b = 0; b < n_bundles_; ++b)
    if (!handles_[b].empty()) unmap_one(b);
  if (va_ != 0) api_.release_va(api_.ctx, va_, static_cast<uint64_t>(n_buffers_) * buffer_bytes_);
}

int KvBacking::reserve() {
  if (va_ != 0) return 0;
  uint64_t gran = 0;
  int rc = api_.granularity(api_.ctx, device_, &gran);
  if (rc != 0) return rc;
  if (gran == 0 || chunk_bytes_ % gran != 0 || buffer_bytes_ % chunk_bytes_ != 0) return -22;
  return api_.reserve(api_.ctx, static_cast<uint64_t>(n_buffers_) * buffer_bytes_, gran, &va_);
}

int KvBacking::map_one(uint32_t bundle) {
  std::vector<uint64_t> hs;
  hs.reserve(n_buffers_);
  int rc = 0;
  uint32_t mapped = 0;
  for (uint32_t buf = 0; buf < n_buffers_; ++buf) {
    uint64_t h = 0;
    rc = api_.create(api_.ctx, device_, chunk_bytes_, &h);
    if (rc != 0) break;
    hs.push_back(h);
    const uint64_t va = buffer_address(buf) + static_cast<uint64_t>(bundle) * chunk_bytes_;
    rc = api_.map(api_.ctx, va, chunk_bytes_, h);
    if (rc != 0) break;
    ++mapped;
    rc = api_.set_access(api_.ctx, va, chunk_bytes_, device_);
    if (rc != 0) break;
  }
  if (rc != 0) {
    for (uint32_t buf = 0; buf < mapped; ++buf)
      api_.unmap(api_.ctx, buffer_address(buf) + static_cast<uint64_t>(bundle) * chunk_bytes_, chunk_bytes_);
    for (uint64_t h : hs) api_.release(api_.ctx, h);
    return rc;
  }
  handles_[bundle] = std::move(hs);
  ++mapped_;
  return 0;
}

void KvBacking::unmap_one(uint32_t bundle) {
  for (uint32_t buf = 0; buf < n_buffers_; ++buf) {
    api_.unmap(api_.ctx, buffer_address(buf) + static_cast<uint64_t>(bundle) * chunk_bytes_, chunk_bytes_);
    api_.release(api_.ctx, handles_[bundle][buf]);
  }
  handles_[bundle].clear();
  --mapped_;
}

int KvBacking::try_map(const uint32_t* bundles, uint32_t n) {
  if (va_ == 0) return -1;
  std::vector<uint32_t> done;
  int rc = 0;
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t b = bundles[i];
    if (b >= n_bundles_) {
      rc = -22;
      break;
    }
    if (!handles_[b].empty()) continue;  // already mapped
    if (quota_ != nullptr && !quota_->charge(bundle_bytes())) {
      rc = kQuotaExceeded;
      break;
    }
    rc = map_one(b);
    if (rc != 0) {
      if (quota_ != nullptr) quota_->refund(bundle_bytes());
      break;
    }
    done.push_back(b);
  }
  if (rc != 0) {
    for (uint32_t b : done) {
      unmap_one(b);
      if (quota_ != nullptr) quota_->refund(bundle_bytes());
    }
  }
  return rc;
}

uint32_t KvBacking::unmap(const uint32_t* bundles, uint32_t n) {
  uint32_t k = 0;
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t b = bundles[i];
    if (b >= n_bundles_ || handles_[b].empty()) continue;
    unmap_one(b);
    if (quota_ != nullptr) quota_->refund(bundle_bytes());
    ++k;
  }
  return k;
}

// ---------------------------------------------------------------- fake driver

namespace {
FakeDriver* F(void* c) { return static_cast<FakeDriver*>(c); }
int f_gran(void* c, int, uint64_t* out) {
  *out = F(c)->granularity_bytes;
  return 0;
}
int f_reserve(void* c, uint64_t bytes, uint64_t, uint64_t* va) {
  *va = F(c)->next_va;
  F(c)->next_va += bytes + (1ull << 30);
  F(c)->reserves++;
  return 0;
}
int f_release_va(void*, uint64_t, uint64_t) { return 0; }
int f_create(void* c, int, uint64_t bytes, uint64_t* h) {
  FakeDriver* f = F(c);
  if (f->fail_create_after == 0) {
    f->fail_create_after = -1;
    return kOutOfMemory;
  }
  if (f->fail_create_after > 0) f->fail_create_after--;
  if (f->allocated_bytes + bytes > f->budget_bytes) return kOutOfMemory;
  f->allocated_bytes += bytes;
  *h = f->next_handle++;
  f->live.emplace_back(*h, bytes);
  f->creates++;
  return 0;
}
int f_release(void* c, uint64_t h) {
  FakeDriver* f = F(c);
  auto it = std::find_if(f->live.begin(), f->live.end(), [&](auto& p) { return p.first == h; });
  if (it == f->live.end()) return 1;
  f->allocated_bytes -= it->second;
  f->live.erase(it);
  f->releases++;
  return 0;
}
int f_map(void* c, uint64_t, uint64_t, uint64_t) {
  FakeDriver* f = F(c);
  if (f->fail_map_after == 0) {
    f->fail_map_after = -1;
    return 999;
  }
  if (f->fail_map_after > 0) f->fail_map_after--;
  f->maps++;
  return 0;
}
int f_unmap(void* c, uint64_t, uint64_t) {
  F(c)->unmaps++;
  return 0;
}
int f_access(void*, uint64_t, uint64_t, int) { return 0; }
}  // namespace

DriverApi FakeDriver::api() {
  return DriverApi{this, f_gran, f_reserve, f_release_va, f_create, f_release, f_map, f_unmap, f_access};
}

}  // namespace vmm
}  // namespace xpool

using namespace xpool::vmm;

extern "C" {

void* xr_vmm_fake_driver_create(uint64_t budget_bytes, uint64_t granularity) {
  auto* f = new (std::nothrow) FakeDriver();
  if (f == nullptr) return nullptr;
  f->budget_bytes = budget_bytes;
  if (granularity) f->granularity_bytes = granularity;
  return f;
}
void xr_vmm_fake_driver_destroy(void* f) { delete static_cast<FakeDriver*>(f); }
void xr_vmm_fake_driver_inject(void* f, int fail_create_after, int fail_map_after) {
  static_cast<FakeDriver*>(f)->fail_create_after = fail_create_after;
  static_cast<FakeDriver*>(f)->fail_map_after = fail_map_after;
}
void xr_vmm_fake_driver_counts(void* p, uint64_t* out6) {
  auto* f = static_cast<FakeDriver*>(p);
  out6[0] = f->creates;
  out6[1] = f->releases;
  out6[2] = f->maps;
  out6[3] = f->unmaps;
  out6[4] = f->allocated_bytes;
  out6[5] = f->live.size();
}
// Copies the fake's function table into `out` (sizeof(DriverApi) bytes).
void xr_vmm_fake_driver_api(void* f, void* out) {
  DriverApi a = static_cast<FakeDriver*>(f)->api();
  *static_cast<DriverApi*>(out) = a;
}
uint64_t xr_vmm_driver_api_bytes(void) { return sizeof(DriverApi); }

void* xr_vmm_quota_create(uint64_t limit) { return new (std::nothrow) MemoryQuota(limit); }
void xr_vmm_quota_destroy(void* q) { delete static_cast<MemoryQuota*>(q); }
void xr_vmm_quota_set_limit(void* q, uint64_t limit) { static_cast<MemoryQuota*>(q)->set_limit(limit); }
void xr_vmm_quota_get(void* q, uint64_t* out2) {
  out2[0] = static_cast<MemoryQuota*>(q)->limit();
  out2[1] = static_cast<MemoryQuota*>(q)->charged();
}

void* xr_vmm_backing_create(const void* driver_api, int device, uint32_t n_buffers, uint64_t buffer_bytes,
                            uint64_t chunk_bytes, void* quota) {
  if (driver_api == nullptr || n_buffers == 0 || buffer_bytes == 0 || chunk_bytes == 0) return nullptr;
  return new (std::nothrow) KvBacking(*static_cast<const DriverApi*>(driver_api), device, n_buffers, buffer_bytes,
                                      chunk_bytes, static_cast<MemoryQuota*>(quota));
}
void xr_vmm_backing_destroy(void* b) { delete static_cast<KvBacking*>(b); }
int xr_vmm_backing_reserve(void* b) { return static_cast<KvBacking*>(b)->reserve(); }
uint64_t xr_vmm_backing_address(void* b, uint32_t buffer) { return static_cast<KvBacking*>(b)->buffer_address(buffer); }
void xr_vmm_backing_info(void* p, uint64_t* out3) {
  auto* b = static_cast<KvBacking*>(p);
  out3[0] = b->bundle_count();
  out3[1] = b->bundle_bytes();
  out3[2] = b->mapped_bytes();
}
int xr_vmm_backing_is_mapped(void* b, uint32_t bundle) { return static_cast<KvBacking*>(b)->is_mapped(bundle) ? 1 : 0; }
int xr_vmm_backing_try_map(void* b, const uint32_t* bundles, uint32_t n) {
  return static_cast<KvBacking*>(b)->try_map(bundles, n);
}
uint32_t xr_vmm_backing_unmap(void* b, const uint32_t* bundles, uint32_t n) {
  return static_cast<KvBacking*>(b)->unmap(bundles, n);
}

}  // extern "C"
