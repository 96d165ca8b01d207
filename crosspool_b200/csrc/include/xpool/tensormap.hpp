// Host-side helper that encodes 2-D TMA tensor maps without linking libcuda:
// the driver entry point is looked up through the CUDA runtime.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <tuple>
#include <map>

namespace xpool {
namespace tmap {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static EncodeFn fn = []() -> EncodeFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// Row-major matrix [rows, cols] of `elem_bytes`-byte elements with a row pitch of
// `pitch_bytes`; box = {box_cols, box_rows}; 128-byte swizzle (box_cols *
// elem_bytes must be 128). Out-of-range reads return zero. Returns 0 on success.
inline int encode_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                     uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                     uint32_t elem_bytes) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch_bytes & 15) != 0) return -2;
  if (box_cols * elem_bytes != 128 || box_rows == 0 || box_rows > 256) return -3;
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// Paged KV cache [tokens, kv_heads, head_dim] (bf16) as a 3-D map whose box is 16 tokens of one
// head by 64 dims (128 bytes, 128-byte swizzle): one box is what a warp's ldmatrix/mma tile needs.
inline int encode_kv_3d(CUtensorMap* out, const void* base, uint64_t tokens, uint32_t kv_heads, uint32_t head_dim) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || head_dim % 64 != 0) return -2;
  cuuint64_t dims[3] = {head_dim, kv_heads, tokens};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(head_dim) * 2 * kv_heads};
  cuuint32_t box[3] = {64, 1, 16};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// Paged KV cache [tokens, kv_heads, head_dim] (bf16) as a 4-D map (64 dims, tokens, 64-dim blocks of the head, heads)
// whose box is `box_tokens` tokens of one head over the whole head dim: it lands in shared memory as one
// [box_tokens][128 bytes] block per 64 dims, the blocks one after the other -- the operand layout of the tensor
// cores -- with one copy instead of one per 64-dim block. box_tokens must not cross a page.
inline int encode_kv_4d(CUtensorMap* out, const void* base, uint64_t tokens, uint32_t kv_heads, uint32_t head_dim,
                        uint32_t box_tokens) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || head_dim % 64 != 0 || box_tokens == 0 || box_tokens > 256) return -2;
  cuuint64_t dims[4] = {64, tokens, head_dim / 64, kv_heads};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_dim) * 2 * kv_heads, 128, static_cast<cuuint64_t>(head_dim) * 2};
  cuuint32_t box[4] = {64, box_tokens, head_dim / 64, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// Packed queries [rows, q_heads, head_dim] (bf16) as a 3-D map whose box is 64 dims x `heads` heads x
// `positions` rows (128-byte swizzle): the box lands in shared memory as heads * positions rows of 128 bytes,
// row index = position * heads + head. Out-of-range rows read as zero.
inline int encode_q_3d(CUtensorMap* out, const void* base, uint64_t rows, uint32_t q_heads, uint32_t head_dim,
                       uint32_t heads, uint32_t positions) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || head_dim % 64 != 0) return -2;
  if (heads == 0 || positions == 0 || heads > 256 || positions > 256) return -3;
  cuuint64_t dims[3] = {head_dim, q_heads, rows};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(head_dim) * 2 * q_heads};
  cuuint32_t box[3] = {64, heads, positions};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// Small cache: encoding costs a few microseconds and serving reuses the same
// (pointer, shape) pairs on every step.
class Cache {
 public:
  using Key = std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t>;
  int get(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
          uint32_t box_rows, uint32_t elem_bytes) {
    Key k{base, rows, cols, pitch_bytes, box_rows, elem_bytes};
    std::lock_guard<std::mutex> g(mu_);
    auto it = map_.find(k);
    if (it != map_.end()) {
      *out = it->second;
      return 0;
    }
    CUtensorMap m;
    int rc = encode_2d(&m, base, rows, cols, pitch_bytes, box_rows, 128 / elem_bytes, elem_bytes);
    if (rc != 0) return rc;
    if (map_.size() > 8192) map_.clear();
    map_.emplace(k, m);
    *out = m;
    return 0;
  }

  int get_kv(CUtensorMap* out, const void* base, uint64_t tokens, uint32_t kv_heads, uint32_t head_dim) {
    Key k{base, tokens, kv_heads, head_dim, 0xffffffffu, 3};
    std::lock_guard<std::mutex> g(mu_);
    auto it = map_.find(k);
    if (it != map_.end()) {
      *out = it->second;
      return 0;
    }
    CUtensorMap m;
    int rc = encode_kv_3d(&m, base, tokens, kv_heads, head_dim);
    if (rc != 0) return rc;
    if (map_.size() > 8192) map_.clear();
    map_.emplace(k, m);
    *out = m;
    return 0;
  }

  int get_kv4(CUtensorMap* out, const void* base, uint64_t tokens, uint32_t kv_heads, uint32_t head_dim, uint32_t box_tokens) {
    Key k{base, tokens, kv_heads, head_dim, box_tokens, 5};
    std::lock_guard<std::mutex> g(mu_);
    auto it = map_.find(k);
    if (it != map_.end()) {
      *out = it->second;
      return 0;
    }
    CUtensorMap m;
    int rc = encode_kv_4d(&m, base, tokens, kv_heads, head_dim, box_tokens);
    if (rc != 0) return rc;
    if (map_.size() > 8192) map_.clear();
    map_.emplace(k, m);
    *out = m;
    return 0;
  }

  int get_q(CUtensorMap* out, const void* base, uint64_t rows, uint32_t q_heads, uint32_t head_dim, uint32_t heads,
            uint32_t positions) {
    Key k{base, rows, (static_cast<uint64_t>(q_heads) << 32) | head_dim, heads, positions, 4};
    std::lock_guard<std::mutex> g(mu_);
    auto it = map_.find(k);
    if (it != map_.end()) {
      *out = it->second;
      return 0;
    }
    CUtensorMap m;
    int rc = encode_q_3d(&m, base, rows, q_heads, head_dim, heads, positions);
    if (rc != 0) return rc;
    if (map_.size() > 8192) map_.clear();
    map_.emplace(k, m);
    *out = m;
    return 0;
  }

 private:
  std::mutex mu_;
  std::map<Key, CUtensorMap> map_;
};

inline Cache& cache() {
  static Cache c;
  return c;
}

}  // namespace tmap
}  // namespace xpool
