// Bindings for the host copy engine and the peer-memory communication kernels.
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>

#include <memory>

#include "copy_engine.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

class PyCopyEngine {
 public:
  explicit PyCopyEngine(int64_t device) : eng_(new tb::CopyEngine(static_cast<int>(device))) {}
  int64_t offload(const torch::Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "offload: contiguous CUDA tensor");
    const int64_t id = eng_->offload(t.data_ptr(), t.nbytes(), cur_stream());
    TORCH_CHECK(id > 0, "copy engine offload failed: ", id);
    return id;
  }
  void restore(int64_t ticket, torch::Tensor& dst, bool wait) {
    TORCH_CHECK(dst.is_cuda() && dst.is_contiguous(), "restore: contiguous CUDA tensor");
    TORCH_CHECK(eng_->restore(ticket, dst.data_ptr(), cur_stream(), wait) == 0, "copy engine restore failed");
  }
  void wait(int64_t ticket) { TORCH_CHECK(eng_->wait(ticket, cur_stream()) == 0, "copy engine wait failed"); }
  void release(int64_t ticket) { eng_->release(ticket); }
  int64_t upload(const torch::Tensor& host, torch::Tensor& dst, bool wait) {
    TORCH_CHECK(!host.is_cuda() && host.is_pinned() && host.is_contiguous(), "upload: pinned contiguous host tensor");
    TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.nbytes() == host.nbytes(), "upload: matching CUDA tensor");
    const int fence = eng_->upload(host.data_ptr(), dst.data_ptr(), host.nbytes(), cur_stream(), wait);
    TORCH_CHECK(fence >= 0, "copy engine upload failed");
    return fence;
  }
  void wait_upload(int64_t fence) { TORCH_CHECK(eng_->wait_upload(static_cast<int>(fence), cur_stream()) == 0, "bad fence"); }
  void wait_uploads() { eng_->wait_uploads(cur_stream()); }
  int64_t d2h_stream() const { return reinterpret_cast<int64_t>(eng_->d2h_stream()); }
  int64_t h2d_stream() const { return reinterpret_cast<int64_t>(eng_->h2d_stream()); }
  void trim() { eng_->trim(); }
  py::dict stats() {
    const tb::CopyStats s = eng_->stats();
    py::dict d;
    d["d2h_bytes"] = s.d2h_bytes;
    d["h2d_bytes"] = s.h2d_bytes;
    d["d2h_copies"] = s.d2h_copies;
    d["h2d_copies"] = s.h2d_copies;
    d["pool_bytes"] = s.pool_bytes;
    d["pool_slabs"] = s.pool_slabs;
    d["slab_reuses"] = s.slab_reuses;
    d["live_tickets"] = s.live_tickets;
    return d;
  }

 private:
  std::unique_ptr<tb::CopyEngine> eng_;
};

}  // namespace

void bind_copy_engine(pybind11::module_& m) {
  py::class_<PyCopyEngine>(m, "CopyEngine")
      .def(py::init<int64_t>())
      .def("offload", &PyCopyEngine::offload)
      .def("restore", &PyCopyEngine::restore)
      .def("wait", &PyCopyEngine::wait)
      .def("release", &PyCopyEngine::release)
      .def("upload", &PyCopyEngine::upload)
      .def("wait_upload", &PyCopyEngine::wait_upload)
      .def("wait_uploads", &PyCopyEngine::wait_uploads)
      .def("d2h_stream", &PyCopyEngine::d2h_stream)
      .def("h2d_stream", &PyCopyEngine::h2d_stream)
      .def("trim", &PyCopyEngine::trim)
      .def("stats", &PyCopyEngine::stats);
}

void bind_comm(pybind11::module_& m);
