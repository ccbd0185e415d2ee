// GroupNorm + SiLU forward that allocates nothing (see terra_noalloc.h for the contract).
// The statistics scratch is a file-scope device array; its device address is resolved once per device.
#include "terra_noalloc.h"

#include <atomic>

#include "common.cuh"
#include "host_api.h"

namespace {

// {sum, sum of squares, mean, rstd} per (sample, group) cell.
static __device__ __align__(256) float g_gn_scratch[TERRA_NOALLOC_GN_MAX_CELLS * 4];

constexpr int kMaxDevices = 64;
// Device address of the array per device ordinal. Host threads may race on a device's first call: each resolves the
// same address, and the atomic slot makes the publication well defined.
std::atomic<float*> g_scratch_addr[kMaxDevices];

__global__ void gn_clear_kernel(float* scratch, int cells) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cells * 4) scratch[i] = 0.f;
}

// sums live interleaved as {sum, sumsq} pairs in the first 2 * cells floats; stats as {mean, rstd} after them
__global__ void gn_finalize_kernel(const float* sums, float* stats, int cells, float inv_count, float eps) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cells) {
    const float mean = sums[2 * i] * inv_count;
    const float var = fmaxf(sums[2 * i + 1] * inv_count - mean * mean, 0.f);
    stats[2 * i] = mean;
    stats[2 * i + 1] = rsqrtf(var + eps);
  }
}

// In host code the array's name is only a handle; kernels need its device address.
int scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TERRA_NOALLOC_ERR_SYMBOL;
  float* addr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_gn_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return TERRA_NOALLOC_ERR_SYMBOL;
    }
    addr = static_cast<float*>(p);
    g_scratch_addr[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return 0;
}

}  // namespace

extern "C" int terra_groupnorm_silu_noalloc(const void* x, const void* gamma, const void* beta, void* y, int B,
                                            long long HW, int C, int groups, float eps, cudaStream_t stream) {
  if (x == nullptr || y == nullptr || gamma == nullptr || beta == nullptr || B <= 0 || HW <= 0 || C <= 0 ||
      groups <= 0 || C % 8 != 0 || C % groups != 0)
    return TERRA_NOALLOC_ERR_BAD_ARG;
  const long long cells = static_cast<long long>(B) * groups;
  if (cells > TERRA_NOALLOC_GN_MAX_CELLS) return TERRA_NOALLOC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  float* sums = scratch;                      // [cells][2]
  float* stats = scratch + 2 * cells;         // [cells][2]
  const int n = static_cast<int>(cells);
  gn_clear_kernel<<<(n * 4 + 255) / 256, 256, 0, stream>>>(scratch, n);
  if (cudaGetLastError() != cudaSuccess) return TERRA_NOALLOC_ERR_LAUNCH;   // nothing else is queued after a failed clear
  if (tb::groupnorm_stats(x, sums, B, HW, C, groups, stream) != 0) return TERRA_NOALLOC_ERR_LAUNCH;
  const float inv_count = 1.0f / (static_cast<float>(HW) * static_cast<float>(C / groups));
  gn_finalize_kernel<<<(n + 255) / 256, 256, 0, stream>>>(sums, stats, n, inv_count, eps);
  if (cudaGetLastError() != cudaSuccess) return TERRA_NOALLOC_ERR_LAUNCH;
  if (tb::groupnorm_silu_apply(x, stats, gamma, beta, nullptr, y, B, HW, C, groups, stream) != 0)
    return TERRA_NOALLOC_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? 0 : TERRA_NOALLOC_ERR_LAUNCH;
}
