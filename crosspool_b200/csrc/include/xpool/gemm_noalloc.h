/* Split-K linear layer for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference.
 *
 * Who needs it: an FfnAgent after memory admission (the daemon accepted its byte
 * estimate and the device budget is frozen, so a late cudaMalloc could fail or
 * steal memory lent to a co-located model's KV cache), and plain C hosts that
 * load libxpool_kernels.so without PyTorch's caching allocator. The ordinary
 * entry point (xp_gemm) takes its split-K workspace and tile counters from the
 * caller; this one keeps them in a fixed array inside the library image.
 *
 * What it computes: out[rows, n_out] = x[rows, k] * w[n_out, k]^T, bf16 in,
 * fp32 accumulate, bf16 out — the same kernel and the same numerics as xp_gemm
 * with epilogue 0 and the given split-K factor.
 *
 * Limits and sharp edges:
 *  - The scratch is XP_NOALLOC_WS_BYTES of workspace plus XP_NOALLOC_COUNTER_BYTES
 *    of counters (plus one 256-byte block for a status word) per GPU; every GPU that loads the library holds that memory
 *    until the process exits. A problem whose plan needs more is refused with
 *    XP_NOALLOC_E_TOO_LARGE (see xp_gemm_noalloc_strerror); nothing is launched.
 *  - The first call on a device looks up the device address of the array
 *    (cudaGetSymbolAddress, with that device current). Make that first call
 *    before starting any stream capture. Two host threads may make it at the
 *    same time: both find the same address.
 *  - All calls on a device share the one array, and it keeps the previous
 *    call's contents. The counters are cleared on the caller's stream before
 *    each launch; the workspace needs no clearing (every word read was written
 *    by the same launch). Two calls that overlap on the GPU (different streams
 *    without ordering) race on the array: order them.
 *  - No cudaMalloc, cudaFree or allocating library routine is called.
 */
#ifndef XPOOL_GEMM_NOALLOC_H_
#define XPOOL_GEMM_NOALLOC_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XP_NOALLOC_WS_BYTES (8u << 20)
#define XP_NOALLOC_COUNTER_BYTES (16u << 10)

/* Codes of this entry point sit below -1000: xp_gemm reports a CUDA launch error e as -100 - e, and those must
 * not be mistaken for these. */
#define XP_NOALLOC_E_TOO_LARGE (-1000)  /* plan needs more scratch than the fixed array holds */
#define XP_NOALLOC_E_SYMBOL (-1001)     /* the array's device address could not be obtained */
#define XP_NOALLOC_E_ARGUMENT (-1002)   /* null pointer or unsupported shape */
#define XP_NOALLOC_E_CLEAR (-1003)      /* clearing or reading the counters / status word failed */

/* w [n_out, k] and x [rows, k] are dense row-major bf16 device pointers, out is [rows, n_out] bf16.
 * n_out % 128 == 0, k % 64 == 0, splits >= 1 (1 = no split-K, the scratch is then unused).
 * Returns 0, one of the codes above, or a negative xp_gemm code. */
int xp_gemm_noalloc(const void* w, const void* x, void* out, int n_out, int k, int rows, int splits, void* stream);

/* Bytes of workspace the given problem would need (0 for splits == 1), or a negative code. */
long long xp_gemm_noalloc_required_bytes(int n_out, int k, int rows, int splits);

/* The kernel's bounded waits report through a status word that lives in the same fixed array and is cleared with
 * the counters before every launch: 0 = the last call on this device ran to completion, non-zero = one of its
 * pipeline waits gave up (the output is then not valid). Synchronises `stream`. Returns 0 or a code above. */
int xp_gemm_noalloc_status(unsigned int* out, void* stream);

const char* xp_gemm_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* XPOOL_GEMM_NOALLOC_H_ */
