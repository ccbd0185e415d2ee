// Stream memory operations and a copy-engine row gather: the pieces of the all-gather that run beside a persistent
// GEMM without needing an SM. A kernel that waited on a flag could not be scheduled while the GEMM's CTAs (one per
// SM, all of its shared memory) are resident, so the waiting and the signalling are stream memory operations and the
// transfer is a cudaMemcpyAsync on the copy engines.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "comm_api.h"

namespace tb {
namespace {

using WaitFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
using WriteFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

void* entry(const char* name) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return ptr;
}

}  // namespace

// stream waits until *addr >= value (32-bit, wrap-safe comparison is the caller's business: epochs stay small)
int stream_wait_geq32(cudaStream_t stream, const void* addr, unsigned int value) {
  static WaitFn fn = reinterpret_cast<WaitFn>(entry("cuStreamWaitValue32"));
  if (fn == nullptr) return -1;
  return fn(stream, reinterpret_cast<CUdeviceptr>(addr), value, CU_STREAM_WAIT_VALUE_GEQ) == CUDA_SUCCESS ? 0 : -2;
}

// stream writes value to *addr after everything queued before it
int stream_write32(cudaStream_t stream, void* addr, unsigned int value) {
  static WriteFn fn = reinterpret_cast<WriteFn>(entry("cuStreamWriteValue32"));
  if (fn == nullptr) return -1;
  return fn(stream, reinterpret_cast<CUdeviceptr>(addr), value, CU_STREAM_WRITE_VALUE_DEFAULT) == CUDA_SUCCESS ? 0 : -2;
}

// For every peer p != my_rank, nearest first: wait for signals[p] >= epoch, then copy its shard (rows x row_bytes at
// src[p], peer memory) to dst + p * rows * row_bytes with the copy engine in `chunks` pieces of chunk_rows rows and
// publish ready[p * chunks + c] = epoch after piece c. Everything on `stream`. With include_self the own shard is
// copied into its place too (no wait, no ready word), so that dst ends up holding the whole gathered operand.
int gather_shards_async(cudaStream_t stream, void* dst, const void* const* src, int num_peers, int my_rank,
                        long long rows, size_t row_bytes, int chunks, long long chunk_rows, const unsigned int* signals,
                        unsigned int* ready, unsigned int epoch, int include_self) {
  if (num_peers < 1 || num_peers > COMM_MAX_PEERS || chunks < 1 || chunks > 4) return -1;
  const size_t shard = static_cast<size_t>(rows) * row_bytes;
  if (include_self && shard > 0 &&
      cudaMemcpyAsync(static_cast<char*>(dst) + my_rank * shard, src[my_rank], shard, cudaMemcpyDeviceToDevice, stream) !=
          cudaSuccess)
    return -21;
  for (int i = 1; i < num_peers; ++i) {
    const int p = (my_rank + i) % num_peers;
    int rc = stream_wait_geq32(stream, signals + p, epoch);
    if (rc != 0) return rc - 10;
    for (int c = 0; c < chunks; ++c) {
      const long long r0 = c * chunk_rows;
      const long long r1 = (c == chunks - 1) ? rows : (r0 + chunk_rows < rows ? r0 + chunk_rows : rows);
      if (r1 > r0) {
        const size_t off = static_cast<size_t>(r0) * row_bytes;
        if (cudaMemcpyAsync(static_cast<char*>(dst) + p * shard + off, static_cast<const char*>(src[p]) + off,
                            static_cast<size_t>(r1 - r0) * row_bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
          return -20;
      }
      rc = stream_write32(stream, ready + p * chunks + c, epoch);
      if (rc != 0) return rc - 30;
    }
  }
  return 0;
}

}  // namespace tb
