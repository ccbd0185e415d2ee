// Python bindings (torch tensors -> raw-pointer host API). Only this file sees torch headers.
#include <cstring>
#include <vector>
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include "host_api.h"
#include "launch_count.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

const void* opt_ptr(const c10::optional<torch::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

void check_bf16_2d(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with unit inner stride");
}

// C = epilogue(A_op * B_op^T). a: [M,K] (or [K,M] when a_mn), b: [N,K] (or [K,N] when b_mn).
void gemm(const torch::Tensor& a, bool a_mn, const torch::Tensor& b, bool b_mn, torch::Tensor& c, int64_t flags,
          const c10::optional<torch::Tensor>& bias, const c10::optional<torch::Tensor>& residual,
          const c10::optional<torch::Tensor>& aux, const c10::optional<torch::Tensor>& c2, double alpha,
          int64_t split_k, int64_t bn, const c10::optional<torch::Tensor>& status, int64_t shuffle_cout,
          int64_t out_w, int64_t out_h, int64_t sms, const std::vector<int64_t>& a_peer_ptrs, int64_t rank,
          const std::vector<int64_t>& c_peer_ptrs, int64_t a_flags_ptr, int64_t a_epoch, int64_t a_budget_ns,
          int64_t a_interleave, int64_t a_chunks, const c10::optional<torch::Tensor>& colsum) {
  check_bf16_2d(a, "a");
  check_bf16_2d(b, "b");
  const c10::cuda::CUDAGuard guard(a.device());
  // a_peer_ptrs: `a` is this GPU's shard and the operand is the concatenation of all GPUs' shards (all-gather fused
  // into the loads). c_peer_ptrs: fp32 accumulation buffers of the row blocks' owners (reduce-scatter fused into the
  // stores); `c` is then this GPU's own buffer and only gives the leading dimension.
  const int64_t gather = a_peer_ptrs.size() > 1 ? static_cast<int64_t>(a_peer_ptrs.size()) : 1;
  TORCH_CHECK(gather == 1 || !a_mn, "gemm: gathered A must be K-major");
  const int64_t M = (a_mn ? a.size(1) : a.size(0)) * gather;
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: contraction mismatch ", K, " vs ", Kb);
  tb::GemmOperand A{a.data_ptr(), a.stride(0), a_mn ? 1 : 0};
  tb::GemmOperand B{b.data_ptr(), b.stride(0), b_mn ? 1 : 0};
  tb::GemmEpilogue e{};
  e.flags = static_cast<int>(flags);
  e.C = c.data_ptr();
  e.ldc = c.dim() >= 2 ? c.stride(c.dim() - 2) : c.size(-1);
  if (shuffle_cout > 0) e.ldc = shuffle_cout;
  e.C2 = c2.has_value() ? c2->data_ptr() : nullptr;
  e.ldc2 = c2.has_value() ? c2->stride(0) : 0;
  e.bias = opt_ptr(bias);
  e.residual = opt_ptr(residual);
  e.ldr = residual.has_value() ? residual->stride(residual->dim() - 2) : 0;
  e.aux = opt_ptr(aux);
  e.ldaux = aux.has_value() ? aux->stride(0) : 0;
  e.alpha = static_cast<float>(alpha);
  e.status = status.has_value() ? status->data_ptr() : nullptr;
  e.shuffle_cout = static_cast<int>(shuffle_cout);
  e.out_w = static_cast<int>(out_w);
  e.out_h = static_cast<int>(out_h);
  if (colsum.has_value()) {
    TORCH_CHECK(colsum->scalar_type() == torch::kFloat32 && colsum->is_contiguous() && colsum->numel() == M,
                "gemm: colsum must be contiguous fp32 with one entry per output row");
    e.colsum = colsum->data_ptr<float>();
  }
  tb::note_launch();
  tb::GemmPeers peers;
  std::memset(&peers, 0, sizeof(peers));
  TORCH_CHECK(a_peer_ptrs.size() <= 8 && c_peer_ptrs.size() <= 8, "gemm: at most 8 peers");
  if (gather > 1) {
    peers.a_peers = static_cast<int>(gather);
    peers.a_rows = a.size(0);
    for (size_t i = 0; i < a_peer_ptrs.size(); ++i) peers.a_ptr[i] = reinterpret_cast<const void*>(a_peer_ptrs[i]);
  }
  peers.rank = static_cast<int>(rank);
  peers.a_flags = reinterpret_cast<const void*>(a_flags_ptr);
  peers.a_epoch = static_cast<unsigned int>(a_epoch);
  peers.a_budget_ns = static_cast<unsigned long long>(a_budget_ns);
  peers.a_interleave = static_cast<int>(a_interleave);
  peers.a_chunks = static_cast<int>(a_chunks);
  if (c_peer_ptrs.size() > 1) {
    peers.c_peers = static_cast<int>(c_peer_ptrs.size());
    TORCH_CHECK(M % peers.c_peers == 0, "gemm: rows not divisible by the number of owners");
    peers.c_rows = M / peers.c_peers;
    for (size_t i = 0; i < c_peer_ptrs.size(); ++i) peers.c_ptr[i] = reinterpret_cast<void*>(c_peer_ptrs[i]);
  }
  const int rc = tb::gemm_bf16_peers(A, B, M, N, K, e, peers, static_cast<int>(split_k), static_cast<int>(bn),
                                     sms > 0 ? static_cast<int>(sms) : sm_count(), cur_stream());
  TORCH_CHECK(rc == 0, "terra_b200 gemm launch failed, code ", rc, " (M=", M, " N=", N, " K=", K, ")");
}

// x: [B,H,W,Cin] bf16 NHWC, w: [Cout, 9*Cin_pad] bf16, y: [B,Ho,Wo,Cout]
void conv3x3_fwd(const torch::Tensor& x, const torch::Tensor& w, torch::Tensor& y, int64_t stride, int64_t flags,
                 const c10::optional<torch::Tensor>& bias, const c10::optional<torch::Tensor>& residual,
                 const c10::optional<torch::Tensor>& status, const c10::optional<torch::Tensor>& halo_lo,
                 const c10::optional<torch::Tensor>& halo_hi) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 4, "x: NHWC bf16");
  TORCH_CHECK(w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && w.dim() == 2, "w: [Cout, 9*Cin_pad] bf16");
  for (const auto* h : {&halo_lo, &halo_hi})
    TORCH_CHECK(!h->has_value() || ((*h)->is_contiguous() && (*h)->scalar_type() == torch::kBFloat16 &&
                                    (*h)->numel() == x.size(0) * x.size(2) * x.size(3)),
                "halo rows must be contiguous bf16 [B, 1, W, Cin]");
  TORCH_CHECK(y.is_contiguous(), "y must be contiguous");
  const c10::cuda::CUDAGuard guard(x.device());
  tb::GemmEpilogue e{};
  e.flags = static_cast<int>(flags);
  e.C = y.data_ptr();
  e.ldc = y.size(3);
  e.bias = opt_ptr(bias);
  e.residual = opt_ptr(residual);
  e.ldr = y.size(3);
  e.alpha = 1.0f;
  e.status = status.has_value() ? status->data_ptr() : nullptr;
  tb::note_launch();
  const int rc = tb::conv3x3_fwd_bf16(x.data_ptr(), w.data_ptr(), x.size(0), x.size(1), x.size(2), x.size(3), w.size(0),
                                      static_cast<int>(stride), e, sm_count(), cur_stream(), opt_ptr(halo_lo),
                                      opt_ptr(halo_hi));
  TORCH_CHECK(rc == 0, "terra_b200 conv3x3_fwd launch failed, code ", rc);
}

// dw: [9, Cout, Cin] fp32 (zeroed by the caller)
void conv3x3_wgrad(const torch::Tensor& x, const torch::Tensor& dy, torch::Tensor& dw, int64_t stride, int64_t split_k,
                   const c10::optional<torch::Tensor>& status, const c10::optional<torch::Tensor>& halo_lo,
                   const c10::optional<torch::Tensor>& halo_hi, const c10::optional<torch::Tensor>& bias_grad) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 4, "x: NHWC bf16");
  TORCH_CHECK(dy.scalar_type() == torch::kBFloat16 && dy.is_contiguous() && dy.dim() == 4, "dy: NHWC bf16");
  TORCH_CHECK(!bias_grad.has_value() || (bias_grad->scalar_type() == torch::kFloat32 && bias_grad->is_contiguous() &&
                                         bias_grad->numel() == dy.size(3)),
              "bias_grad: contiguous fp32 [Cout]");
  TORCH_CHECK(dw.scalar_type() == torch::kFloat32 && dw.is_contiguous(), "dw: fp32 [9,Cout,Cin]");
  const c10::cuda::CUDAGuard guard(x.device());
  tb::note_launch();
  const int rc = tb::conv3x3_wgrad_bf16(x.data_ptr(), dy.data_ptr(), dw.data_ptr<float>(), x.size(0), x.size(1),
                                        x.size(2), x.size(3), dy.size(3), static_cast<int>(stride),
                                        static_cast<int>(split_k), status.has_value() ? status->data_ptr() : nullptr,
                                        sm_count(), cur_stream(), opt_ptr(halo_lo), opt_ptr(halo_hi),
                                        bias_grad.has_value() ? bias_grad->data_ptr<float>() : nullptr);
  TORCH_CHECK(rc == 0, "terra_b200 conv3x3_wgrad launch failed, code ", rc);
}

}  // namespace

void bind_elementwise(pybind11::module_& m);
void bind_attention(pybind11::module_& m);
void bind_copy_engine(pybind11::module_& m);
void bind_comm(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("launch_count", []() { return static_cast<int64_t>(tb::g_kernel_launches.load()); });
  m.def("gemm_stall_counters", [](bool reset) {
    unsigned long long v[8];
    TORCH_CHECK(tb::gemm_stall_counters(v, reset ? 1 : 0) == 0, "gemm_stall_counters failed");
    std::vector<int64_t> out(v, v + 8);
    return out;
  });
  namespace py = pybind11;
  m.def("gemm", &gemm, "tcgen05 bf16 GEMM with fused epilogues", py::arg("a"), py::arg("a_mn"), py::arg("b"),
        py::arg("b_mn"), py::arg("c"), py::arg("flags"), py::arg("bias"), py::arg("residual"), py::arg("aux"),
        py::arg("c2"), py::arg("alpha"), py::arg("split_k"), py::arg("bn"), py::arg("status"), py::arg("shuffle_cout"),
        py::arg("out_w"), py::arg("out_h"), py::arg("sms"), py::arg("a_peer_ptrs"), py::arg("rank"),
        py::arg("c_peer_ptrs"), py::arg("a_flags_ptr"), py::arg("a_epoch"), py::arg("a_budget_ns"),
        py::arg("a_interleave"), py::arg("a_chunks"), py::arg("colsum") = py::none());
  m.def("conv3x3_fwd", &conv3x3_fwd, "implicit-GEMM 3x3 convolution (NHWC bf16)");
  m.def("conv3x3_wgrad", &conv3x3_wgrad, "3x3 convolution weight gradient (fp32 atomics)", py::arg("x"), py::arg("dy"),
        py::arg("dw"), py::arg("stride"), py::arg("split_k"), py::arg("status"), py::arg("halo_lo"), py::arg("halo_hi"),
        py::arg("bias_grad") = py::none());
  bind_elementwise(m);
  bind_attention(m);
  bind_copy_engine(m);
  bind_comm(m);
}
