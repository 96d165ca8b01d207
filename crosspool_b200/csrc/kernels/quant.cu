// Activation quantisation for the block-scaled fp8 GEMM: bf16 rows -> e4m3 with one fp32 scale per
// row and 128-element K block ("1 x 128" scaling). Scales are written transposed, [k / 128][ld],
// so that the GEMM epilogue reads the scales of a tile's rows as one contiguous run.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "xpool/api.h"

namespace {

// One warp per (row, K block); a lane owns four consecutive elements.
__global__ void __launch_bounds__(256)
quant_act_fp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ xq, float* __restrict__ scales, int rows,
                     int kblocks, int ldx, int ldq, int ld_scale) {
  const int warp = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows * kblocks) return;
  const int row = warp / kblocks, kb = warp % kblocks;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(row) * ldx + kb * 128 + lane * 4);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(row) * ldq + kb * 128 + lane * 4) =
      static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  if (lane == 0) scales[static_cast<size_t>(kb) * ld_scale + row] = scale;
}

}  // namespace

extern "C" int xp_quant_act_fp8(const void* x, void* xq, float* scales, int rows, int k, int ldx, int ldq, int ld_scale,
                                void* stream) {
  if (rows <= 0) return 0;
  if (k % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0 || ld_scale < rows) return -10;
  const int warps = rows * (k / 128);
  quant_act_fp8_kernel<<<(warps + 7) / 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(xq), scales, rows, k / 128, ldx, ldq, ld_scale);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
