/* terra_groupnorm_silu_noalloc: GroupNorm + SiLU forward for callers that are not allowed to allocate.
 *
 * This entry point has no counterpart in the reference; it exists for embedders of this library whose host code
 * runs where device allocation is off limits - a plugin inside another framework's allocator-owned region, a
 * real-time inference loop that forbids cudaMalloc after start-up, code running under a memory-pool policy that
 * rejects foreign allocations. The regular path (groupnorm_stats + groupnorm_silu_apply) needs a small scratch
 * tensor for the per-(sample, group) statistics that its caller allocates; here that scratch is a fixed
 * file-scope device array inside the library, so the call allocates nothing: no cudaMalloc / cudaFree, no
 * allocating library routine.
 *
 *   x, y   bf16 NHWC-flattened [B, HW, C] (caller-owned device memory, y may not alias x)
 *   gamma, beta  bf16 [C]
 *   y = silu((x - mean_g) * rstd_g * gamma + beta), statistics per (sample, group) over HW x (C / groups)
 *
 * Limits: B * groups <= TERRA_NOALLOC_GN_MAX_CELLS (4096), C % 8 == 0, C % groups == 0. Larger problems are
 * rejected with TERRA_NOALLOC_ERR_TOO_LARGE and nothing is launched.
 *
 * The scratch (4 floats per cell, 64 KiB) is held by every GPU that loads the library until the process exits.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call outside of any stream capture. All calls on a device share the one array and
 * it keeps the previous call's contents, so each call clears the cells it uses first; two calls whose kernels
 * may overlap on the GPU (different streams without ordering) race on it and must be serialised by the caller.
 *
 * Returns 0 on success, a negative TERRA_NOALLOC_ERR_* code otherwise. Work is queued on `stream`.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TERRA_NOALLOC_GN_MAX_CELLS 4096
#define TERRA_NOALLOC_ERR_BAD_ARG (-1)
#define TERRA_NOALLOC_ERR_TOO_LARGE (-2)
#define TERRA_NOALLOC_ERR_SYMBOL (-3)
#define TERRA_NOALLOC_ERR_LAUNCH (-4)

int terra_groupnorm_silu_noalloc(const void* x, const void* gamma, const void* beta, void* y, int B, long long HW,
                                 int C, int groups, float eps, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
