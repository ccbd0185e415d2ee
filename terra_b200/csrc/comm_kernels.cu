// Kernels that read and write other GPUs' memory directly (plain loads / stores over NVLink through NVSwitch).
#include "comm_api.h"
#include "common.cuh"

namespace tb {
namespace {

__global__ void __launch_bounds__(256) dist_adamw_kernel(const __grid_constant__ DistAdamWArgs a) {
  const long long nvec = a.n / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = a.lo + i * 4;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int p = 0; p < a.num_peers; ++p) {
      const float4 v = *reinterpret_cast<const float4*>(a.grad[p] + e);
      g.x += v.x; g.y += v.y; g.z += v.z; g.w += v.w;
    }
    float gv[4] = {g.x * a.grad_scale, g.y * a.grad_scale, g.z * a.grad_scale, g.w * a.grad_scale};
    float4 pm = *reinterpret_cast<const float4*>(a.master + e);
    float4 m4 = *reinterpret_cast<const float4*>(a.exp_avg + i * 4);
    float4 v4 = *reinterpret_cast<const float4*>(a.exp_avg_sq + i * 4);
    float pv[4] = {pm.x, pm.y, pm.z, pm.w}, mv[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      pv[k] *= 1.f - a.lr * a.weight_decay;
      mv[k] = a.beta1 * mv[k] + (1.f - a.beta1) * gv[k];
      vv[k] = a.beta2 * vv[k] + (1.f - a.beta2) * gv[k] * gv[k];
      const float denom = sqrtf(vv[k]) / a.bias_corr2_sqrt + a.eps;
      pv[k] -= (a.lr / a.bias_corr1) * (mv[k] / denom);
    }
    *reinterpret_cast<float4*>(a.master + e) = make_float4(pv[0], pv[1], pv[2], pv[3]);
    *reinterpret_cast<float4*>(a.exp_avg + i * 4) = make_float4(mv[0], mv[1], mv[2], mv[3]);
    *reinterpret_cast<float4*>(a.exp_avg_sq + i * 4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    const uint2 packed = make_uint2(pack_bf16x2(pv[0], pv[1]), pack_bf16x2(pv[2], pv[3]));
#pragma unroll 4
    for (int p = 0; p < a.num_peers; ++p)
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.param_bf16[p]) + e) = packed;
  }
}

__global__ void __launch_bounds__(256) peer_copy_rows_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                                                             long long rows, long long vec_per_row,
                                                             long long dst_stride, long long src_stride) {
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row, v = i % vec_per_row;
    *reinterpret_cast<uint4*>(dst + r * dst_stride + v * 16) = *reinterpret_cast<const uint4*>(src + r * src_stride + v * 16);
  }
}

struct PeerPtrs {
  const float* p[COMM_MAX_PEERS];
};
struct GatherPeers {
  const uint4* p[COMM_MAX_PEERS];
};
__global__ void peer_sum_small_kernel(float* dst, const __grid_constant__ PeerPtrs srcs, int num_peers, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    float s = 0.f;
    for (int p = 0; p < num_peers; ++p) s += srcs.p[p][i];
    dst[i] = s;
  }
}

struct PadPtrs {
  uint32_t* p[COMM_MAX_PEERS];
};
// One block. Thread t < num_peers signals peer t, then everyone waits on the local pad. The wait is bounded in time
// (`budget_ns` of the global timer): when a peer never signals, the kernel records {site, peer, expected epoch} in the
// status word and returns, so the context stays usable and the host can raise.
__global__ void peer_barrier_kernel(const __grid_constant__ PadPtrs pads, int my_rank, int num_peers, uint32_t epoch,
                                    KernelStatus* status, unsigned long long budget_ns) {
  const int t = threadIdx.x;
  if (t < num_peers) {
    __threadfence_system();
    // slot [my_rank] on peer t
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(pads.p[t] + my_rank) : "memory");
  }
  if (t < num_peers) {
    const volatile uint32_t* mine = pads.p[my_rank] + t;
    const unsigned long long t0 = global_timer_ns();
    uint32_t seen;
    unsigned int polls = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int32_t>(seen - epoch) >= 0) break;
      if ((++polls & 63u) == 0u && global_timer_ns() - t0 > budget_ns) {
        report_error(status, TB_ERR_PEER_TIMEOUT, 0x900u, static_cast<unsigned int>(t), epoch);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
}

// One-way signal: adds 1 to word [slot_base + my_rank] of every peer's pad after making this GPU's earlier writes
// visible system-wide. The consumers (for example the TMA thread of a GEMM that reads this GPU's shard) wait for the
// count to reach their epoch.
__global__ void peer_signal_kernel(const __grid_constant__ PadPtrs pads, int my_rank, int num_peers, int slot_base) {
  const int t = threadIdx.x;
  if (t < num_peers) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(pads.p[t] + slot_base + my_rank) : "memory");
  }
}

// Row gather over peer memory: dst row i = row src_row[i] of the buffer of GPU src_slot[i] (this GPU's own buffer
// included). One 16-byte vector per thread and step; a row's vectors are handled by neighbouring threads. The general
// form of the stripe <-> window relayout (an all-to-all-v in which every token has exactly one source).
__global__ void __launch_bounds__(256) peer_gather_indexed_kernel(uint4* __restrict__ dst, const __grid_constant__ GatherPeers peers,
                                                                  const int* __restrict__ src_slot,
                                                                  const int* __restrict__ src_row, long long rows,
                                                                  int vec_per_row, int num_peers, long long src_rows,
                                                                  KernelStatus* status) {
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    const int slot = src_slot[r], row = src_row[r];
    // debug build: a route must name a GPU of the group and a row of its staged buffer (src_rows < 0: unknown extent)
    if (!tb_index_ok(slot >= 0 && slot < num_peers && row >= 0 && (src_rows < 0 || row < src_rows), status, 0xA00u,
                     static_cast<unsigned int>(slot), static_cast<unsigned int>(row))) {
      dst[i] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* src = peers.p[slot] + static_cast<long long>(row) * vec_per_row + v;
    dst[i] = *src;
  }
}

// Halo exchange between row-stripe neighbours, push style: every block copies a share of this GPU's two boundary
// rows straight into the neighbours' receive buffers (16-byte stores over NVLink); the block that finishes last
// publishes "rows of epoch e written" to each neighbour with a release at system scope and then waits (bounded by the
// global timer) until the neighbours' rows for the same epoch have landed here. After the kernel the local receive
// buffers hold the halo rows, so the convolution that follows reads local memory only.
__global__ void __launch_bounds__(256) halo_push_kernel(const __grid_constant__ HaloPushArgs a) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (a.dst_prev != nullptr)
    for (long long i = t0; i < a.nvec; i += stride) a.dst_prev[i] = a.send_prev[i];
  if (a.dst_next != nullptr)
    for (long long i = t0; i < a.nvec; i += stride) a.dst_next[i] = a.send_next[i];
  __threadfence_system();
  __shared__ unsigned int last;
  __syncthreads();
  if (threadIdx.x == 0) last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (last == 0u) return;
  if (threadIdx.x == 0) *a.ticket = 0u;     // ready for the next exchange (stream order)
  if (threadIdx.x < 2) {
    uint32_t* peer_flag = threadIdx.x == 0 ? a.flag_at_prev : a.flag_at_next;
    const uint32_t* my_flag = threadIdx.x == 0 ? a.my_flag_from_prev : a.my_flag_from_next;
    if (peer_flag != nullptr) {
      __threadfence_system();
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(peer_flag) : "memory");
    }
    if (my_flag != nullptr) {
      const unsigned long long w0 = global_timer_ns();
      uint32_t seen;
      unsigned int polls = 0;
      while (true) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(my_flag) : "memory");
        if (static_cast<int32_t>(seen - a.epoch) >= 0) break;
        if ((++polls & 63u) == 0u && global_timer_ns() - w0 > a.budget_ns) {
          report_error(a.status, TB_ERR_PEER_TIMEOUT, 0xa00u + threadIdx.x, seen, a.epoch);
          break;
        }
        __nanosleep(100);
      }
    }
  }
}

// All-reduce (sum) of a small fp32 vector over the GPUs of a group in one single-block kernel: push this GPU's values
// into its slot on every peer, publish, wait (bounded) for everybody's slot here, add the slots up. The slots are
// double buffered by call parity: a peer can be at most one call ahead, because it needs this GPU's signal of call k + 1
// to get past it, and that signal is sent only after call k has been summed here (stream order).
__global__ void __launch_bounds__(512) peer_allreduce_small_kernel(const __grid_constant__ SmallReduceArgs a) {
  const int t = threadIdx.x;
  for (int p = 0; p < a.num_peers; ++p) {
    float* dst = a.slots[p] + (static_cast<size_t>(a.parity) * a.num_peers + a.my_rank) * a.capacity;
    for (int i = t; i < a.n; i += blockDim.x) dst[i] = a.in[i];
  }
  __threadfence_system();
  __syncthreads();
  if (t < a.num_peers) {
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(a.flags[t] + a.my_rank) : "memory");
    const volatile uint32_t* mine = a.flags[a.my_rank] + t;
    const unsigned long long w0 = global_timer_ns();
    uint32_t seen;
    unsigned int polls = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int32_t>(seen - a.epoch) >= 0) break;
      if ((++polls & 63u) == 0u && global_timer_ns() - w0 > a.budget_ns) {
        report_error(a.status, TB_ERR_PEER_TIMEOUT, 0xb00u, static_cast<unsigned int>(t), a.epoch);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  const float* base = a.slots[a.my_rank] + static_cast<size_t>(a.parity) * a.num_peers * a.capacity;
  for (int i = t; i < a.n; i += blockDim.x) {
    float acc = 0.f;
    for (int p = 0; p < a.num_peers; ++p) acc += base[static_cast<size_t>(p) * a.capacity + i];
    a.out[i] = acc;
  }
}

}  // namespace

int peer_gather_indexed(void* dst, const void* const* src_peers, int num_peers, const int* src_slot, const int* src_row,
                        long long rows, long long row_bytes, cudaStream_t stream, long long src_rows, void* status) {
  if (num_peers < 1 || num_peers > COMM_MAX_PEERS || row_bytes % 16 != 0) return -1;
  if (rows <= 0) return 0;
  GatherPeers gp;
  for (int i = 0; i < num_peers; ++i) gp.p[i] = static_cast<const uint4*>(src_peers[i]);
  const long long total = rows * (row_bytes / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  peer_gather_indexed_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<uint4*>(dst), gp, src_slot, src_row, rows,
                                                                          static_cast<int>(row_bytes / 16), num_peers, src_rows,
                                                                          static_cast<KernelStatus*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int halo_push(const HaloPushArgs& a, cudaStream_t stream) {
  if (a.nvec <= 0 || a.ticket == nullptr) return -1;
  long long blocks = (a.nvec + 255) / 256;
  if (blocks > 64) blocks = 64;
  halo_push_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int peer_allreduce_small(const SmallReduceArgs& a, cudaStream_t stream) {
  if (a.num_peers < 1 || a.num_peers > COMM_MAX_PEERS || a.n <= 0 || a.n > a.capacity) return -1;
  peer_allreduce_small_kernel<<<1, 512, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int peer_signal(uint32_t* const* signal_pads, int my_rank, int num_peers, int slot_base, cudaStream_t stream) {
  if (num_peers < 1 || num_peers > COMM_MAX_PEERS || slot_base < 0) return -1;
  PadPtrs pp;
  for (int i = 0; i < num_peers; ++i) pp.p[i] = signal_pads[i];
  peer_signal_kernel<<<1, 32, 0, stream>>>(pp, my_rank, num_peers, slot_base);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int dist_adamw_step(const DistAdamWArgs& a, cudaStream_t stream) {
  if (a.num_peers < 1 || a.num_peers > COMM_MAX_PEERS || a.n % 4 != 0 || a.lo % 4 != 0) return -1;
  if (a.n == 0) return 0;
  long long blocks = (a.n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  dist_adamw_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int peer_copy_rows(void* dst, const void* src_peer, long long rows, long long row_bytes, long long dst_stride_bytes,
                   long long src_stride_bytes, cudaStream_t stream) {
  if (row_bytes % 16 != 0 || dst_stride_bytes % 16 != 0 || src_stride_bytes % 16 != 0) return -1;
  if (rows <= 0 || row_bytes <= 0) return 0;
  const long long total = rows * (row_bytes / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  peer_copy_rows_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<uint8_t*>(dst),
                                                                      static_cast<const uint8_t*>(src_peer), rows,
                                                                      row_bytes / 16, dst_stride_bytes, src_stride_bytes);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int peer_sum_small(float* dst, const float* const* src_peers, int num_peers, int n, cudaStream_t stream) {
  if (num_peers < 1 || num_peers > COMM_MAX_PEERS || n <= 0) return -1;
  PeerPtrs pp;
  for (int i = 0; i < num_peers; ++i) pp.p[i] = src_peers[i];
  peer_sum_small_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dst, pp, num_peers, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int peer_barrier(uint32_t* const* signal_pads, int my_rank, int num_peers, uint32_t epoch, void* status,
                 unsigned long long budget_ns, cudaStream_t stream) {
  if (num_peers < 1 || num_peers > COMM_MAX_PEERS) return -1;
  PadPtrs pp;
  for (int i = 0; i < num_peers; ++i) pp.p[i] = signal_pads[i];
  peer_barrier_kernel<<<1, 32, 0, stream>>>(pp, my_rank, num_peers, epoch, static_cast<KernelStatus*>(status), budget_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace tb
