// Embedding gather and greedy sampling (row-wise argmax; ties go to the lower id,
// which is what torch.argmax returns for the first maximal element).
#include <math_constants.h>

#include "xpool/api.h"
#include "xpool/sm100.cuh"

namespace {

__global__ void __launch_bounds__(128)
embedding_kernel(const int* __restrict__ ids, const uint4* __restrict__ table, uint4* __restrict__ out,
                 int hidden8, int vocab) {
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = table + static_cast<size_t>(id) * hidden8;
  uint4* dst = out + static_cast<size_t>(row) * hidden8;
  for (int i = threadIdx.x; i < hidden8; i += 128) dst[i] = __ldg(&src[i]);
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(1024)
argmax_kernel(const T* __restrict__ logits, int* __restrict__ out, int vocab, int ld) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += 1024) {
    const float v = to_f<T>(row[i]);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = sv[threadIdx.x];
    bi = si[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
  }
}

// Temperature sampling by the Gumbel-max trick: argmax_i (logit_i / T + g_i) with g_i = -log(-log u_i) draws
// from softmax(logits / T) exactly, in one pass and without normalising. u_i comes from a counter-based hash
// of (row seed, token index), so a (seed, step) pair always yields the same token. T <= 0 is greedy.
__device__ __forceinline__ uint32_t hash3(uint32_t a, uint32_t b, uint32_t c) {
  uint64_t x = (static_cast<uint64_t>(a) << 32) ^ (static_cast<uint64_t>(b) * 0x9E3779B97F4A7C15ull) ^ c;
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return static_cast<uint32_t>(x >> 16);
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, const float* __restrict__ temps, const uint32_t* __restrict__ seeds,
              int* __restrict__ out, int vocab, int ld) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  const float temp = temps[blockIdx.x];
  const float inv_t = temp > 0.f ? 1.f / temp : 1.f;
  const uint32_t seed = seeds[2 * blockIdx.x], step = seeds[2 * blockIdx.x + 1];
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += 1024) {
    float v = to_f<T>(row[i]) * inv_t;
    if (temp > 0.f) {
      const float u = (static_cast<float>(hash3(seed, step, static_cast<uint32_t>(i)) >> 8) + 0.5f) * (1.f / 16777216.f);
      v -= __logf(-__logf(u));
    }
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = sv[threadIdx.x];
    bi = si[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
  }
}

}  // namespace

// temps [rows] fp32, seeds [rows, 2] u32 (request seed, step counter), all device memory.
extern "C" int xp_sample(const void* logits, int is_fp32, const float* temps, const uint32_t* seeds, int* out, int rows,
                         int vocab, int ld, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_fp32)
    sample_kernel<float><<<rows, 1024, 0, s>>>(reinterpret_cast<const float*>(logits), temps, seeds, out, vocab, ld);
  else
    sample_kernel<__nv_bfloat16><<<rows, 1024, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), temps, seeds, out, vocab, ld);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" int xp_embedding(const int* ids, const void* table, void* out, int rows, int hidden,
                            int vocab, void* stream) {
  if (rows <= 0) return 0;
  if (hidden % 8 != 0) return -10;
  embedding_kernel<<<rows, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids, reinterpret_cast<const uint4*>(table), reinterpret_cast<uint4*>(out), hidden / 8, vocab);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

extern "C" int xp_argmax(const void* logits, int is_fp32, int* out, int rows, int vocab, int ld,
                         void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_fp32)
    argmax_kernel<float><<<rows, 1024, 0, s>>>(reinterpret_cast<const float*>(logits), out, vocab, ld);
  else
    argmax_kernel<__nv_bfloat16><<<rows, 1024, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits), out, vocab, ld);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
