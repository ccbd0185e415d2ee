#include "copy_engine.h"

#include <algorithm>

namespace tb {

namespace {
constexpr size_t kSlabGranule = size_t(2) << 20;
size_t round_up(size_t v, size_t g) { return (v + g - 1) / g * g; }
}  // namespace

CopyEngine::CopyEngine(int device) : device_(device) {
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  cudaStreamCreateWithFlags(&d2h_, cudaStreamNonBlocking);
  cudaStreamCreateWithFlags(&h2d_, cudaStreamNonBlocking);
  for (auto& e : upload_fence_) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
  cudaSetDevice(prev);
}

CopyEngine::~CopyEngine() {
  // Process teardown may already have destroyed the context; errors are ignored on purpose.
  if (d2h_) cudaStreamSynchronize(d2h_);
  if (h2d_) cudaStreamSynchronize(h2d_);
  for (auto& kv : tickets_) {
    if (kv.second.d2h_done) cudaEventDestroy(kv.second.d2h_done);
    if (kv.second.h2d_done) cudaEventDestroy(kv.second.h2d_done);
  }
  for (auto& s : slabs_) {
    if (s.last_read) cudaEventDestroy(s.last_read);
    if (s.host) cudaFreeHost(s.host);
  }
  for (auto& e : upload_fence_)
    if (e) cudaEventDestroy(e);
  if (d2h_) cudaStreamDestroy(d2h_);
  if (h2d_) cudaStreamDestroy(h2d_);
}

int CopyEngine::acquire_slab(size_t bytes) {
  int best = -1;
  for (size_t i = 0; i < slabs_.size(); ++i) {
    const Slab& s = slabs_[i];
    if (!s.busy && s.bytes >= bytes && (best < 0 || s.bytes < slabs_[best].bytes)) best = static_cast<int>(i);
  }
  if (best >= 0) {
    slabs_[best].busy = true;
    stats_.slab_reuses++;
    return best;
  }
  Slab s;
  s.bytes = round_up(bytes, kSlabGranule);
  if (cudaHostAlloc(&s.host, s.bytes, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  cudaEventCreateWithFlags(&s.last_read, cudaEventDisableTiming);
  s.busy = true;
  slabs_.push_back(s);
  stats_.pool_bytes += s.bytes;
  stats_.pool_slabs++;
  return static_cast<int>(slabs_.size()) - 1;
}

int64_t CopyEngine::offload(const void* dev_src, size_t bytes, cudaStream_t compute_stream) {
  std::lock_guard<std::mutex> lock(mu_);
  const int si = acquire_slab(bytes);
  if (si < 0) return -1;
  Slab& s = slabs_[si];
  Ticket t;
  t.slab = si;
  t.bytes = bytes;
  cudaEventCreateWithFlags(&t.d2h_done, cudaEventDisableTiming);
  cudaEventCreateWithFlags(&t.h2d_done, cudaEventDisableTiming);
  // order: producer kernels on the compute stream -> D2H; previous reader of the slab -> D2H
  cudaEvent_t ready;
  cudaEventCreateWithFlags(&ready, cudaEventDisableTiming);
  cudaEventRecord(ready, compute_stream);
  cudaStreamWaitEvent(d2h_, ready, 0);
  cudaEventDestroy(ready);
  if (s.has_read) cudaStreamWaitEvent(d2h_, s.last_read, 0);
  if (cudaMemcpyAsync(s.host, dev_src, bytes, cudaMemcpyDeviceToHost, d2h_) != cudaSuccess) {
    cudaGetLastError();
    s.busy = false;
    cudaEventDestroy(t.d2h_done);
    cudaEventDestroy(t.h2d_done);
    return -2;
  }
  cudaEventRecord(t.d2h_done, d2h_);
  const int64_t id = next_ticket_++;
  tickets_[id] = t;
  stats_.d2h_bytes += bytes;
  stats_.d2h_copies++;
  stats_.live_tickets = tickets_.size();
  return id;
}

int CopyEngine::restore(int64_t ticket, void* dev_dst, cudaStream_t compute_stream, bool make_compute_wait) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = tickets_.find(ticket);
  if (it == tickets_.end()) return -1;
  Ticket& t = it->second;
  Slab& s = slabs_[t.slab];
  cudaStreamWaitEvent(h2d_, t.d2h_done, 0);
  // the destination was allocated on the compute stream: do not write before that stream reaches here
  cudaEvent_t alloc_point;
  cudaEventCreateWithFlags(&alloc_point, cudaEventDisableTiming);
  cudaEventRecord(alloc_point, compute_stream);
  cudaStreamWaitEvent(h2d_, alloc_point, 0);
  cudaEventDestroy(alloc_point);
  if (cudaMemcpyAsync(dev_dst, s.host, t.bytes, cudaMemcpyHostToDevice, h2d_) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  cudaEventRecord(t.h2d_done, h2d_);
  cudaEventRecord(s.last_read, h2d_);
  s.has_read = true;
  t.restored = true;
  if (make_compute_wait) cudaStreamWaitEvent(compute_stream, t.h2d_done, 0);
  stats_.h2d_bytes += t.bytes;
  stats_.h2d_copies++;
  return 0;
}

int CopyEngine::wait(int64_t ticket, cudaStream_t compute_stream) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = tickets_.find(ticket);
  if (it == tickets_.end()) return -1;
  if (!it->second.restored) return -2;
  cudaStreamWaitEvent(compute_stream, it->second.h2d_done, 0);
  return 0;
}

int CopyEngine::release(int64_t ticket) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = tickets_.find(ticket);
  if (it == tickets_.end()) return -1;
  Ticket& t = it->second;
  Slab& s = slabs_[t.slab];
  if (!t.restored) {
    // never read back: the slab may be rewritten only after its D2H finished
    cudaEventRecord(s.last_read, d2h_);
    s.has_read = true;
  }
  s.busy = false;
  cudaEventDestroy(t.d2h_done);
  cudaEventDestroy(t.h2d_done);
  tickets_.erase(it);
  stats_.live_tickets = tickets_.size();
  return 0;
}

int CopyEngine::upload(const void* host_src, void* dev_dst, size_t bytes, cudaStream_t compute_stream,
                       bool make_compute_wait) {
  std::lock_guard<std::mutex> lock(mu_);
  cudaEvent_t point;
  cudaEventCreateWithFlags(&point, cudaEventDisableTiming);
  cudaEventRecord(point, compute_stream);
  cudaStreamWaitEvent(h2d_, point, 0);
  cudaEventDestroy(point);
  if (cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, h2d_) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  const int fence = next_fence_;
  next_fence_ = (next_fence_ + 1) % kUploadFences;
  cudaEventRecord(upload_fence_[fence], h2d_);
  last_fence_ = fence;
  if (make_compute_wait) cudaStreamWaitEvent(compute_stream, upload_fence_[fence], 0);
  stats_.h2d_bytes += bytes;
  stats_.h2d_copies++;
  return fence;
}

int CopyEngine::wait_upload(int fence, cudaStream_t compute_stream) {
  std::lock_guard<std::mutex> lock(mu_);
  if (fence < 0 || fence >= kUploadFences) return -1;
  cudaStreamWaitEvent(compute_stream, upload_fence_[fence], 0);
  return 0;
}

int CopyEngine::wait_uploads(cudaStream_t compute_stream) {
  std::lock_guard<std::mutex> lock(mu_);
  if (last_fence_ >= 0) cudaStreamWaitEvent(compute_stream, upload_fence_[last_fence_], 0);
  return 0;
}

void* CopyEngine::alloc_pinned(size_t bytes) {
  void* p = nullptr;
  if (cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

void CopyEngine::free_pinned(void* p) {
  if (p) cudaFreeHost(p);
}

CopyStats CopyEngine::stats() {
  std::lock_guard<std::mutex> lock(mu_);
  return stats_;
}

void CopyEngine::trim() {
  std::lock_guard<std::mutex> lock(mu_);
  cudaStreamSynchronize(d2h_);
  cudaStreamSynchronize(h2d_);
  for (auto& s : slabs_) {
    if (!s.busy && s.host) {
      cudaFreeHost(s.host);
      stats_.pool_bytes -= s.bytes;
      stats_.pool_slabs--;
      s.host = nullptr;
      s.bytes = 0;
    }
  }
}

void* CopyEngine::host_ptr(int64_t ticket) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = tickets_.find(ticket);
  return it == tickets_.end() ? nullptr : slabs_[it->second.slab].host;
}

}  // namespace tb
