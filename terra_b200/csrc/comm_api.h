// Peer-memory (NVLink / NVSwitch) communication kernels. Buffers live in symmetric memory: every rank of a group
// allocated the same layout, so a kernel addresses a peer's copy as peer_base + the same offset.
#pragma once
#include <cstddef>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

struct KernelStatus;

constexpr int COMM_MAX_PEERS = 16;

// Sharded AdamW over replicas: this rank owns `n` elements starting at element `lo` of every replica's flat
// gradient / working-copy arena. For the owned range the kernel sums the fp32 gradients of all replicas (P2P
// loads), applies AdamW to the local fp32 master and moments, and stores the new bf16 values into every
// replica's working copy (P2P stores). Group barriers before and after are the caller's.
struct DistAdamWArgs {
  const float* grad[COMM_MAX_PEERS];   // base of each replica's fp32 gradient arena
  void* param_bf16[COMM_MAX_PEERS];    // base of each replica's bf16 working copy
  int num_peers;
  float* master;        // local fp32 master arena (base)
  float* exp_avg;       // local moments of the owned range (n elements)
  float* exp_avg_sq;
  long long lo, n;
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2_sqrt, grad_scale;
};
int dist_adamw_step(const DistAdamWArgs& a, cudaStream_t stream);

// Rows [row0, row0 + rows) x row_bytes copied from a peer buffer into a local one (halo rows, relayout pulls).
int peer_copy_rows(void* dst, const void* src_peer, long long rows, long long row_bytes, long long dst_stride_bytes,
                   long long src_stride_bytes, cudaStream_t stream);

// Sum of `num_peers` small fp32 vectors that live at the same offset on every peer (GroupNorm statistics).
int peer_sum_small(float* dst, const float* const* src_peers, int num_peers, int n, cudaStream_t stream);

// Group barrier on a symmetric signal pad: every rank adds 1 to its slot on all peers, then waits (bounded) until
// its own pad shows `epoch` from everyone. `status` receives TB_ERR_PEER_TIMEOUT when the wait runs out.
// stream_ops.cpp: SM-free pieces of the all-gather that overlaps a persistent GEMM (stream memory operations + copy engine)
int stream_wait_geq32(cudaStream_t stream, const void* addr, unsigned int value);
int stream_write32(cudaStream_t stream, void* addr, unsigned int value);
int gather_shards_async(cudaStream_t stream, void* dst, const void* const* src, int num_peers, int my_rank, long long rows,
                        size_t row_bytes, int chunks, long long chunk_rows, const unsigned int* signals, unsigned int* ready,
                        unsigned int epoch, int include_self = 0);
// dst[i] = row src_row[i] of src_peers[src_slot[i]] (rows of row_bytes, a multiple of 16; index arrays on the device).
// src_rows / status: extent of every source buffer and the KernelStatus word, used by the bounds-checked debug build.
int peer_gather_indexed(void* dst, const void* const* src_peers, int num_peers, const int* src_slot, const int* src_row,
                        long long rows, long long row_bytes, cudaStream_t stream, long long src_rows = -1,
                        void* status = nullptr);

// Halo exchange of two boundary rows with the row-stripe neighbours (see comm_kernels.cu). Null pointers: no neighbour
// on that side. Buffers and flag words live in symmetric memory; `epoch` counts the exchanges of the group.
struct HaloPushArgs {
  const uint4* send_prev;          // this GPU's first row (goes to the previous rank's "row below" buffer)
  const uint4* send_next;          // this GPU's last row (goes to the next rank's "row above" buffer)
  uint4* dst_prev;                 // peer address of the previous rank's receive buffer, or null
  uint4* dst_next;
  long long nvec;                  // 16-byte vectors per row
  uint32_t* flag_at_prev;          // peer address of the previous rank's "from next" counter, or null
  uint32_t* flag_at_next;          // peer address of the next rank's "from prev" counter, or null
  const uint32_t* my_flag_from_prev;   // local counters (null: no neighbour on that side)
  const uint32_t* my_flag_from_next;
  uint32_t epoch;
  unsigned int* ticket;            // local word, zero between exchanges
  unsigned long long budget_ns;
  KernelStatus* status;
};
int halo_push(const HaloPushArgs& a, cudaStream_t stream);

// Sum of an fp32 vector of at most `capacity` elements over the GPUs of a group, one single-block kernel.
struct SmallReduceArgs {
  float* slots[COMM_MAX_PEERS];    // every GPU's [2][num_peers][capacity] staging (symmetric)
  uint32_t* flags[COMM_MAX_PEERS]; // every GPU's [num_peers] arrival counters (symmetric)
  const float* in;
  float* out;
  int num_peers, my_rank, n, capacity, parity;
  uint32_t epoch;
  unsigned long long budget_ns;
  KernelStatus* status;
};
int peer_allreduce_small(const SmallReduceArgs& a, cudaStream_t stream);

// One-way "my earlier writes are visible" signal into word [slot_base + my_rank] of every peer's pad.
int peer_signal(uint32_t* const* signal_pads, int my_rank, int num_peers, int slot_base, cudaStream_t stream);
int peer_barrier(uint32_t* const* signal_pads, int my_rank, int num_peers, uint32_t epoch, void* status,
                 unsigned long long budget_ns, cudaStream_t stream);

}  // namespace tb
