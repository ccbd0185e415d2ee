// Host <-> device copy engine for activation offload and input staging: a pool of pinned host slabs
// (allocated once, reused), one D2H and one H2D stream per device, event fencing against the compute
// stream. One cudaMemcpyAsync per copy.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>
#include <vector>

namespace tb {

struct CopyStats {
  uint64_t d2h_bytes = 0, h2d_bytes = 0;
  uint64_t d2h_copies = 0, h2d_copies = 0;
  uint64_t pool_bytes = 0, pool_slabs = 0, slab_reuses = 0;
  uint64_t live_tickets = 0;
};

class CopyEngine {
 public:
  explicit CopyEngine(int device);
  ~CopyEngine();
  CopyEngine(const CopyEngine&) = delete;
  CopyEngine& operator=(const CopyEngine&) = delete;

  // Copy `bytes` from device memory to a pinned slab, ordered after everything queued so far on
  // `compute_stream`. Returns a ticket (> 0) or a negative error code.
  int64_t offload(const void* dev_src, size_t bytes, cudaStream_t compute_stream);
  // Queue the copy back into `dev_dst` on the H2D stream (after the ticket's D2H finished).
  // With make_compute_wait the compute stream is made to wait for it; otherwise call wait() later.
  int restore(int64_t ticket, void* dev_dst, cudaStream_t compute_stream, bool make_compute_wait);
  int wait(int64_t ticket, cudaStream_t compute_stream);
  // Drop a ticket; its slab returns to the pool (the next writer waits for the last reader).
  int release(int64_t ticket);
  // Plain staged upload from caller-owned pinned memory (input pipeline). Returns a fence id (>= 0) that
  // wait_upload() makes a stream wait for, or a negative error code.
  int upload(const void* host_src, void* dev_dst, size_t bytes, cudaStream_t compute_stream, bool make_compute_wait);
  int wait_upload(int fence, cudaStream_t compute_stream);
  int wait_uploads(cudaStream_t compute_stream);   // the most recent upload
  // Pinned host buffers for callers (inputs, checkpoint staging).
  void* alloc_pinned(size_t bytes);
  void free_pinned(void* p);

  cudaStream_t d2h_stream() const { return d2h_; }
  cudaStream_t h2d_stream() const { return h2d_; }
  CopyStats stats();
  void trim();   // free all idle slabs
  void* host_ptr(int64_t ticket);

 private:
  struct Slab {
    void* host = nullptr;
    size_t bytes = 0;
    bool busy = false;
    cudaEvent_t last_read = nullptr;   // recorded after the latest H2D that read this slab
    bool has_read = false;
  };
  struct Ticket {
    int slab = -1;
    size_t bytes = 0;
    cudaEvent_t d2h_done = nullptr;
    cudaEvent_t h2d_done = nullptr;
    bool restored = false;
  };
  int acquire_slab(size_t bytes);

  int device_;
  cudaStream_t d2h_ = nullptr, h2d_ = nullptr;
  static constexpr int kUploadFences = 16;
  cudaEvent_t upload_fence_[kUploadFences] = {nullptr};
  int next_fence_ = 0;
  int last_fence_ = -1;
  std::mutex mu_;
  std::vector<Slab> slabs_;
  std::unordered_map<int64_t, Ticket> tickets_;
  int64_t next_ticket_ = 1;
  CopyStats stats_;
};

}  // namespace tb
