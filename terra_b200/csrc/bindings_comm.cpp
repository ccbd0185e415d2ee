// Bindings of the peer-memory (NVLink) communication kernels. Peer buffers are passed as raw device addresses.
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include <cmath>

#include "comm_api.h"
#include "launch_count.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void dist_adamw_step(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& bf16_ptrs, torch::Tensor& master,
                     torch::Tensor& exp_avg, torch::Tensor& exp_avg_sq, int64_t lo, int64_t n, double lr, double b1,
                     double b2, double eps, double wd, int64_t step, double grad_scale) {
  TORCH_CHECK(grad_ptrs.size() == bf16_ptrs.size() && !grad_ptrs.empty() && grad_ptrs.size() <= tb::COMM_MAX_PEERS,
              "dist_adamw_step: one gradient and one working-copy base per replica");
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == torch::kFloat32 && exp_avg.numel() >= n, "dist_adamw_step: bad state");
  const c10::cuda::CUDAGuard guard(master.device());
  tb::DistAdamWArgs a{};
  a.num_peers = static_cast<int>(grad_ptrs.size());
  for (int i = 0; i < a.num_peers; ++i) {
    a.grad[i] = reinterpret_cast<const float*>(grad_ptrs[i]);
    a.param_bf16[i] = reinterpret_cast<void*>(bf16_ptrs[i]);
  }
  a.master = master.data_ptr<float>();
  a.exp_avg = exp_avg.data_ptr<float>();
  a.exp_avg_sq = exp_avg_sq.data_ptr<float>();
  a.lo = lo;
  a.n = n;
  a.lr = static_cast<float>(lr);
  a.beta1 = static_cast<float>(b1);
  a.beta2 = static_cast<float>(b2);
  a.eps = static_cast<float>(eps);
  a.weight_decay = static_cast<float>(wd);
  a.bias_corr1 = static_cast<float>(1.0 - std::pow(b1, static_cast<double>(step)));
  a.bias_corr2_sqrt = static_cast<float>(std::sqrt(1.0 - std::pow(b2, static_cast<double>(step))));
  a.grad_scale = static_cast<float>(grad_scale);
  tb::note_launch();
  TORCH_CHECK(tb::dist_adamw_step(a, cur_stream()) == 0, "dist_adamw_step launch failed");
}

void peer_copy_rows(int64_t dst, int64_t src, int64_t rows, int64_t row_bytes, int64_t dst_stride, int64_t src_stride) {
  tb::note_launch();
  TORCH_CHECK(tb::peer_copy_rows(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), rows, row_bytes,
                                 dst_stride, src_stride, cur_stream()) == 0,
              "peer_copy_rows launch failed");
}

void peer_sum_small(torch::Tensor& dst, const std::vector<int64_t>& src_ptrs) {
  std::vector<const float*> p;
  for (auto v : src_ptrs) p.push_back(reinterpret_cast<const float*>(v));
  tb::note_launch();
  TORCH_CHECK(tb::peer_sum_small(dst.data_ptr<float>(), p.data(), static_cast<int>(p.size()), dst.numel(), cur_stream()) == 0,
              "peer_sum_small launch failed");
}

void peer_barrier(const std::vector<int64_t>& pads, int64_t my_rank, int64_t epoch, const c10::optional<torch::Tensor>& status,
                  int64_t budget_ns) {
  std::vector<uint32_t*> p;
  for (auto v : pads) p.push_back(reinterpret_cast<uint32_t*>(v));
  tb::note_launch();
  TORCH_CHECK(tb::peer_barrier(p.data(), static_cast<int>(my_rank), static_cast<int>(p.size()), static_cast<uint32_t>(epoch),
                               status.has_value() ? status->data_ptr() : nullptr,
                               static_cast<unsigned long long>(budget_ns), cur_stream()) == 0,
              "peer_barrier launch failed");
}

void peer_signal(const std::vector<int64_t>& pad_ptrs, int64_t my_rank, int64_t slot_base) {
  std::vector<uint32_t*> p;
  for (auto v : pad_ptrs) p.push_back(reinterpret_cast<uint32_t*>(v));
  tb::note_launch();
  TORCH_CHECK(tb::peer_signal(p.data(), static_cast<int>(my_rank), static_cast<int>(p.size()), static_cast<int>(slot_base),
                              cur_stream()) == 0,
              "peer_signal launch failed");
}

// stream: a cudaStream_t as an integer (torch.cuda.Stream.cuda_stream)
void gather_shards_async(int64_t stream, int64_t dst, const std::vector<int64_t>& src_ptrs, int64_t my_rank, int64_t rows,
                         int64_t row_bytes, int64_t chunks, int64_t chunk_rows, int64_t signals_ptr, int64_t ready_ptr,
                         int64_t epoch, bool include_self) {
  std::vector<const void*> p;
  for (auto v : src_ptrs) p.push_back(reinterpret_cast<const void*>(v));
  const int rc = tb::gather_shards_async(reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<void*>(dst), p.data(),
                                         static_cast<int>(p.size()), static_cast<int>(my_rank), rows,
                                         static_cast<size_t>(row_bytes), static_cast<int>(chunks), chunk_rows,
                                         reinterpret_cast<const unsigned int*>(signals_ptr),
                                         reinterpret_cast<unsigned int*>(ready_ptr), static_cast<unsigned int>(epoch),
                                         include_self ? 1 : 0);
  TORCH_CHECK(rc == 0, "gather_shards_async failed with code ", rc);
}

void peer_gather_indexed(torch::Tensor& dst, const std::vector<int64_t>& src_ptrs, const torch::Tensor& src_slot,
                         const torch::Tensor& src_row, int64_t src_rows, const c10::optional<torch::Tensor>& status) {
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.dim() == 2, "peer_gather_indexed: dst [rows, cols] contiguous");
  TORCH_CHECK(src_slot.scalar_type() == torch::kInt32 && src_row.scalar_type() == torch::kInt32 && src_slot.is_cuda() &&
                  src_row.is_cuda() && src_slot.numel() == dst.size(0) && src_row.numel() == dst.size(0),
              "peer_gather_indexed: int32 device index arrays, one entry per destination row");
  const c10::cuda::CUDAGuard guard(dst.device());
  std::vector<const void*> p;
  for (auto v : src_ptrs) p.push_back(reinterpret_cast<const void*>(v));
  tb::note_launch();
  TORCH_CHECK(tb::peer_gather_indexed(dst.data_ptr(), p.data(), static_cast<int>(p.size()), src_slot.data_ptr<int>(),
                                      src_row.data_ptr<int>(), dst.size(0), dst.size(1) * dst.element_size(),
                                      cur_stream(), src_rows, status.has_value() ? status->data_ptr() : nullptr) == 0,
              "peer_gather_indexed launch failed");
}

// All addresses are raw device addresses (0: absent).
void halo_push(int64_t send_prev, int64_t send_next, int64_t dst_prev, int64_t dst_next, int64_t nbytes, int64_t flag_at_prev,
               int64_t flag_at_next, int64_t my_flag_from_prev, int64_t my_flag_from_next, int64_t epoch, int64_t ticket,
               const c10::optional<torch::Tensor>& status, int64_t budget_ns) {
  TORCH_CHECK(nbytes % 16 == 0, "halo_push: rows must be a multiple of 16 bytes");
  tb::HaloPushArgs a{};
  a.send_prev = reinterpret_cast<const uint4*>(send_prev);
  a.send_next = reinterpret_cast<const uint4*>(send_next);
  a.dst_prev = reinterpret_cast<uint4*>(dst_prev);
  a.dst_next = reinterpret_cast<uint4*>(dst_next);
  a.nvec = nbytes / 16;
  a.flag_at_prev = reinterpret_cast<uint32_t*>(flag_at_prev);
  a.flag_at_next = reinterpret_cast<uint32_t*>(flag_at_next);
  a.my_flag_from_prev = reinterpret_cast<const uint32_t*>(my_flag_from_prev);
  a.my_flag_from_next = reinterpret_cast<const uint32_t*>(my_flag_from_next);
  a.epoch = static_cast<uint32_t>(epoch);
  a.ticket = reinterpret_cast<unsigned int*>(ticket);
  a.status = status.has_value() ? reinterpret_cast<tb::KernelStatus*>(status->data_ptr()) : nullptr;
  a.budget_ns = static_cast<unsigned long long>(budget_ns);
  tb::note_launch();
  TORCH_CHECK(tb::halo_push(a, cur_stream()) == 0, "halo_push launch failed");
}

void peer_allreduce_small(const std::vector<int64_t>& slot_ptrs, const std::vector<int64_t>& flag_ptrs, const torch::Tensor& in,
                          torch::Tensor& out, int64_t my_rank, int64_t capacity, int64_t epoch,
                          const c10::optional<torch::Tensor>& status, int64_t budget_ns) {
  TORCH_CHECK(slot_ptrs.size() == flag_ptrs.size() && !slot_ptrs.empty() && slot_ptrs.size() <= tb::COMM_MAX_PEERS,
              "peer_allreduce_small: one staging and one flag array per GPU");
  TORCH_CHECK(in.is_cuda() && in.is_contiguous() && out.is_contiguous() && in.scalar_type() == torch::kFloat32 &&
                  out.scalar_type() == torch::kFloat32 && in.numel() == out.numel() && in.numel() <= capacity,
              "peer_allreduce_small: fp32 contiguous vectors of at most `capacity` elements");
  const c10::cuda::CUDAGuard guard(in.device());
  tb::SmallReduceArgs a{};
  a.num_peers = static_cast<int>(slot_ptrs.size());
  for (int i = 0; i < a.num_peers; ++i) {
    a.slots[i] = reinterpret_cast<float*>(slot_ptrs[i]);
    a.flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  }
  a.in = in.data_ptr<float>();
  a.out = out.data_ptr<float>();
  a.my_rank = static_cast<int>(my_rank);
  a.n = static_cast<int>(in.numel());
  a.capacity = static_cast<int>(capacity);
  a.parity = static_cast<int>(epoch & 1);
  a.epoch = static_cast<uint32_t>(epoch);
  a.status = status.has_value() ? reinterpret_cast<tb::KernelStatus*>(status->data_ptr()) : nullptr;
  a.budget_ns = static_cast<unsigned long long>(budget_ns);
  tb::note_launch();
  TORCH_CHECK(tb::peer_allreduce_small(a, cur_stream()) == 0, "peer_allreduce_small launch failed");
}

// Stream memory operations on a stream given as an integer (torch.cuda.Stream.cuda_stream): the stream waits until the
// 32-bit word at `addr` is >= value / writes value to it, without occupying an SM.
void stream_wait_value(int64_t stream, int64_t addr, int64_t value) {
  TORCH_CHECK(tb::stream_wait_geq32(reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const void*>(addr),
                                    static_cast<unsigned int>(value)) == 0,
              "stream_wait_value failed");
}
void stream_write_value(int64_t stream, int64_t addr, int64_t value) {
  TORCH_CHECK(tb::stream_write32(reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<void*>(addr),
                                 static_cast<unsigned int>(value)) == 0,
              "stream_write_value failed");
}

}  // namespace

void bind_comm(pybind11::module_& m) {
  m.def("peer_gather_indexed", &peer_gather_indexed, pybind11::arg("dst"), pybind11::arg("src_ptrs"), pybind11::arg("src_slot"),
        pybind11::arg("src_row"), pybind11::arg("src_rows") = -1, pybind11::arg("status") = pybind11::none());
  m.def("halo_push", &halo_push);
  m.def("peer_allreduce_small", &peer_allreduce_small);
  m.def("stream_wait_value", &stream_wait_value);
  m.def("stream_write_value", &stream_write_value);
  m.def("dist_adamw_step", &dist_adamw_step);
  m.def("peer_copy_rows", &peer_copy_rows);
  m.def("peer_sum_small", &peer_sum_small);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_signal", &peer_signal);
  m.def("gather_shards_async", &gather_shards_async);
}
