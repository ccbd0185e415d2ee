// Bindings for the memory-bound kernels and window attention.
#include <stdexcept>
#include <string>
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include "host_api.h"
#include "launch_count.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }
const void* opt_ptr(const c10::optional<torch::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }
void* opt_mut(const c10::optional<torch::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// Plain std::runtime_error (pybind11 turns it into RuntimeError): no backtrace collection on the error path.
void need(bool ok, const char* what) {
  if (!ok) throw std::runtime_error(std::string("terra_b200: ") + what);
}
void rc_check(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string("terra_b200: ") + what + " failed with code " + std::to_string(rc));
}

void layernorm_fwd(const torch::Tensor& x, const torch::Tensor& g, const torch::Tensor& b, torch::Tensor& y,
                   torch::Tensor& mean, torch::Tensor& rstd, double eps) {
  need(x.is_cuda() && x.is_contiguous() && x.scalar_type() == torch::kBFloat16, "layernorm_fwd: x bf16 contiguous");
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = x.size(-1);
  tb::note_launch();
  rc_check(tb::layernorm_fwd(x.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr<float>(),
                             rstd.data_ptr<float>(), x.numel() / C, C, static_cast<float>(eps), cur_stream()),
           "layernorm_fwd");
}

void layernorm_bwd(const torch::Tensor& dy, const torch::Tensor& x, const torch::Tensor& g, const torch::Tensor& mean,
                   const torch::Tensor& rstd, torch::Tensor& dx, torch::Tensor& dg, torch::Tensor& db,
                   const c10::optional<torch::Tensor>& dres) {
  need(dy.is_contiguous() && x.is_contiguous(), "layernorm_bwd: contiguous inputs");
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = x.size(-1);
  tb::note_launch();
  rc_check(tb::layernorm_bwd(dy.data_ptr(), x.data_ptr(), g.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                             dx.data_ptr(), dg.data_ptr<float>(), db.data_ptr<float>(), opt_ptr(dres), x.numel() / C, C,
                             cur_stream()),
           "layernorm_bwd");
}

void colsum(const torch::Tensor& x, torch::Tensor& out) {
  need(x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == torch::kBFloat16, "colsum: 2-D bf16");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t nparts = (x.size(0) + tb::colsum_rows_per_block() - 1) / tb::colsum_rows_per_block();
  auto partials = torch::empty({nparts, x.size(1)}, x.options().dtype(torch::kFloat32));
  tb::note_launch();
  rc_check(tb::colsum_bf16(x.data_ptr(), out.data_ptr<float>(), partials.data_ptr<float>(), x.size(0), x.size(1), x.stride(0),
                           cur_stream()),
           "colsum");
}

void groupnorm_stats(const torch::Tensor& x, torch::Tensor& sums, int64_t groups) {
  need(x.is_contiguous() && x.dim() == 3 && x.scalar_type() == torch::kBFloat16, "groupnorm_stats: [B,HW,C] bf16");
  const c10::cuda::CUDAGuard guard(x.device());
  tb::note_launch();
  rc_check(tb::groupnorm_stats(x.data_ptr(), sums.data_ptr<float>(), x.size(0), x.size(1), x.size(2), groups, cur_stream()),
           "groupnorm_stats");
}

void groupnorm_silu_apply(const torch::Tensor& x, const torch::Tensor& stats, const torch::Tensor& g,
                          const torch::Tensor& b, const c10::optional<torch::Tensor>& res, torch::Tensor& y, int64_t groups) {
  need(x.is_contiguous() && x.dim() == 3, "groupnorm_silu_apply: [B,HW,C]");
  const c10::cuda::CUDAGuard guard(x.device());
  tb::note_launch();
  rc_check(tb::groupnorm_silu_apply(x.data_ptr(), stats.data_ptr<float>(), g.data_ptr(), b.data_ptr(), opt_ptr(res), y.data_ptr(),
                                    x.size(0), x.size(1), x.size(2), groups, cur_stream()),
           "groupnorm_silu_apply");
}

// dgamma / dbeta (optional, fp32 [C]): accumulated in place (the gradient views of the affine parameters)
void groupnorm_silu_bwd_reduce(const torch::Tensor& dy, const torch::Tensor& x, const torch::Tensor& stats,
                               const torch::Tensor& g, const torch::Tensor& b, torch::Tensor& red, int64_t groups,
                               const c10::optional<torch::Tensor>& dgamma, const c10::optional<torch::Tensor>& dbeta) {
  need(x.is_contiguous() && dy.is_contiguous() && x.dim() == 3, "groupnorm_silu_bwd_reduce: [B,HW,C]");
  need(!dgamma.has_value() || (dgamma->scalar_type() == torch::kFloat32 && dgamma->is_contiguous()), "dgamma: fp32 contiguous");
  need(!dbeta.has_value() || (dbeta->scalar_type() == torch::kFloat32 && dbeta->is_contiguous()), "dbeta: fp32 contiguous");
  const c10::cuda::CUDAGuard guard(x.device());
  tb::note_launch();
  rc_check(tb::groupnorm_silu_bwd_reduce(dy.data_ptr(), x.data_ptr(), stats.data_ptr<float>(), g.data_ptr(), b.data_ptr(),
                                         red.data_ptr<float>(), dgamma.has_value() ? dgamma->data_ptr<float>() : nullptr,
                                         dbeta.has_value() ? dbeta->data_ptr<float>() : nullptr, x.size(0), x.size(1),
                                         x.size(2), groups, cur_stream()),
           "groupnorm_silu_bwd_reduce");
}

void groupnorm_finalize(torch::Tensor& sums, torch::Tensor& stats, double inv_count, double eps, bool clear) {
  need(sums.is_cuda() && sums.is_contiguous() && stats.is_contiguous() && sums.scalar_type() == torch::kFloat32 &&
           stats.scalar_type() == torch::kFloat32 && sums.numel() == stats.numel() && sums.numel() % 2 == 0,
       "groupnorm_finalize: fp32 [cells, 2] sums and stats");
  const c10::cuda::CUDAGuard guard(sums.device());
  tb::note_launch();
  rc_check(tb::groupnorm_finalize(sums.data_ptr<float>(), stats.data_ptr<float>(), static_cast<int>(sums.numel() / 2),
                                  static_cast<float>(inv_count), static_cast<float>(eps), clear ? 1 : 0, cur_stream()),
           "groupnorm_finalize");
}

void strided_add(torch::Tensor& src, torch::Tensor& dst, int64_t sa, int64_t sb, int64_t sc, bool clear) {
  need(src.is_cuda() && src.is_contiguous() && src.dim() == 3 && src.scalar_type() == torch::kFloat32 &&
           dst.scalar_type() == torch::kFloat32 && dst.is_contiguous() && dst.numel() == src.numel(),
       "strided_add: fp32 src [a, b, c] contiguous, dst contiguous with as many elements");
  const c10::cuda::CUDAGuard guard(src.device());
  tb::note_launch();
  rc_check(tb::strided_add_f32(src.data_ptr<float>(), dst.data_ptr<float>(), static_cast<int>(src.size(0)),
                               static_cast<int>(src.size(1)), static_cast<int>(src.size(2)), sa, sb, sc, clear ? 1 : 0,
                               cur_stream()),
           "strided_add");
}

void groupnorm_silu_bwd_apply(const torch::Tensor& dy, const torch::Tensor& x, const torch::Tensor& stats,
                              const torch::Tensor& red, const torch::Tensor& g, const torch::Tensor& b,
                              torch::Tensor& dx, int64_t groups, double inv_count) {
  need(x.is_contiguous() && dy.is_contiguous() && x.dim() == 3, "groupnorm_silu_bwd_apply: [B,HW,C]");
  const c10::cuda::CUDAGuard guard(x.device());
  tb::note_launch();
  rc_check(tb::groupnorm_silu_bwd_apply(dy.data_ptr(), x.data_ptr(), stats.data_ptr<float>(), red.data_ptr<float>(),
                                        g.data_ptr(), b.data_ptr(), dx.data_ptr(), x.size(0), x.size(1), x.size(2),
                                        groups, static_cast<float>(inv_count), cur_stream()),
           "groupnorm_silu_bwd_apply");
}

void masked_loss(const torch::Tensor& pred, const torch::Tensor& label, const c10::optional<torch::Tensor>& mask,
                 int64_t kind, double grad_scale, torch::Tensor& loss_sum, const c10::optional<torch::Tensor>& grad) {
  need(pred.is_contiguous() && label.is_contiguous() && pred.scalar_type() == torch::kBFloat16 &&
           label.scalar_type() == torch::kBFloat16,
       "masked_loss: bf16 contiguous pred/label");
  const c10::cuda::CUDAGuard guard(pred.device());
  tb::note_launch();
  rc_check(tb::masked_loss_fwd_bwd(pred.data_ptr(), label.data_ptr(), opt_ptr(mask), pred.numel(),
                                   mask.has_value() ? mask->numel() : 0, static_cast<int>(kind),
                                   static_cast<float>(grad_scale), loss_sum.data_ptr<float>(), opt_mut(grad), cur_stream()),
           "masked_loss");
}

void adamw_step(torch::Tensor& master, torch::Tensor& m, torch::Tensor& v, const torch::Tensor& grad,
                const c10::optional<torch::Tensor>& param_bf16, double lr, double b1, double b2, double eps, double wd,
                int64_t step, double grad_scale) {
  need(master.is_contiguous() && m.is_contiguous() && v.is_contiguous() && grad.is_contiguous(), "adamw: contiguous");
  need(master.scalar_type() == torch::kFloat32, "adamw: fp32 master");
  const c10::cuda::CUDAGuard guard(master.device());
  const double bc1 = 1.0 - std::pow(b1, static_cast<double>(step));
  const double bc2 = 1.0 - std::pow(b2, static_cast<double>(step));
  tb::note_launch();
  rc_check(tb::adamw_step(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr(),
                          grad.scalar_type() == torch::kBFloat16 ? 1 : 0, opt_mut(param_bf16), master.numel(),
                          static_cast<float>(lr), static_cast<float>(b1), static_cast<float>(b2), static_cast<float>(eps),
                          static_cast<float>(wd), static_cast<float>(bc1), static_cast<float>(std::sqrt(bc2)),
                          static_cast<float>(grad_scale), cur_stream()),
           "adamw_step");
}

void attn_rowdot(const torch::Tensor& o, const torch::Tensor& dout, torch::Tensor& drow, int64_t heads) {
  need(o.is_cuda() && o.is_contiguous() && dout.is_contiguous() && o.scalar_type() == torch::kBFloat16 &&
           dout.scalar_type() == torch::kBFloat16 && o.dim() == 2 && o.sizes() == dout.sizes(),
       "attn_rowdot: o, dout bf16 [rows, C] contiguous");
  need(drow.scalar_type() == torch::kFloat32 && drow.is_contiguous() && drow.numel() == o.size(0) * heads,
       "attn_rowdot: drow fp32 [rows, heads]");
  const c10::cuda::CUDAGuard guard(o.device());
  tb::note_launch();
  rc_check(tb::attn_rowdot(o.data_ptr(), dout.data_ptr(), drow.data_ptr<float>(), o.size(0), static_cast<int>(o.size(1)),
                           static_cast<int>(heads), cur_stream()),
           "attn_rowdot");
}

void grad_inspect(const torch::Tensor& grad, torch::Tensor& out2) {
  need(grad.is_cuda() && grad.is_contiguous() && grad.scalar_type() == torch::kFloat32, "grad_inspect: fp32 contiguous");
  need(out2.scalar_type() == torch::kFloat32 && out2.numel() >= 2, "grad_inspect: out2 fp32 [2]");
  const c10::cuda::CUDAGuard guard(grad.device());
  tb::note_launch();
  rc_check(tb::grad_inspect(grad.data_ptr<float>(), grad.numel(), out2.data_ptr<float>(), cur_stream()), "grad_inspect");
}

// Peer buffers are passed as raw device addresses (int64) so that symmetric-memory peers can be addressed;
// for a single rank the lists hold one entry each.
// Status word that the bounds-checked debug build of the attention kernels reports to (set once from Python).
void* g_debug_status = nullptr;
void set_debug_status(const c10::optional<torch::Tensor>& status) {
  g_debug_status = status.has_value() ? status->data_ptr() : nullptr;
}
bool debug_bounds_build() {
#ifdef TERRA_DEBUG_BOUNDS
  return true;
#else
  return false;
#endif
}

tb::WindowAttnArgs make_wa(const std::vector<int64_t>& win_start, int64_t my_wg, int64_t sp, int64_t my_sp,
                           int64_t shardN, int64_t B, int64_t nWh, int64_t nWw, int64_t C, int64_t heads, int64_t wh,
                           int64_t ww, int64_t sh, int64_t sw, bool use_mask, double scale, int64_t tp) {
  tb::WindowAttnArgs a{};
  a.tp = static_cast<int>(tp < 1 ? 1 : tp);
  need(win_start.size() >= 2 && win_start.size() <= 9, "window_attn: win_start must have n_wg+1 <= 9 entries");
  a.n_wg = static_cast<int>(win_start.size()) - 1;
  for (size_t i = 0; i < win_start.size(); ++i) a.win_start[i] = static_cast<int>(win_start[i]);
  a.my_wg = my_wg; a.sp = sp; a.my_sp = my_sp; a.shardN = shardN;
  a.B = B; a.nWh = nWh; a.nWw = nWw; a.C = C; a.num_heads = heads;
  a.wh = wh; a.ww = ww; a.sh = sh; a.sw = sw;
  a.use_mask = use_mask ? 1 : 0;
  a.scale = static_cast<float>(scale);
  a.debug_status = g_debug_status;
  need(a.n_wg * a.sp <= tb::WA_MAX_PEERS, "window_attn: too many peer slots");
  return a;
}

void window_attn(const std::vector<int64_t>& qkv_ptrs, const std::vector<int64_t>& out_ptrs,
                 const c10::optional<torch::Tensor>& bias_table, const std::vector<int64_t>& win_start, int64_t my_wg,
                 int64_t sp, int64_t my_sp, int64_t shardN, int64_t B, int64_t nWh, int64_t nWw, int64_t C,
                 int64_t heads, int64_t wh, int64_t ww, int64_t sh, int64_t sw, bool use_mask, double scale, int64_t tp) {
  tb::WindowAttnArgs a = make_wa(win_start, my_wg, sp, my_sp, shardN, B, nWh, nWw, C, heads, wh, ww, sh, sw, use_mask, scale, tp);
  need(qkv_ptrs.size() == static_cast<size_t>(a.n_wg * a.sp) && out_ptrs.size() == qkv_ptrs.size(),
       "window_attn: one buffer per peer slot");
  for (size_t i = 0; i < qkv_ptrs.size(); ++i) {
    a.qkv[i] = reinterpret_cast<const void*>(qkv_ptrs[i]);
    a.out[i] = reinterpret_cast<void*>(out_ptrs[i]);
  }
  a.bias_table = bias_table.has_value() ? bias_table->data_ptr<float>() : nullptr;
  tb::note_launch();
  rc_check(tb::window_attn_fwd(a, cur_stream()), "window_attn_fwd");
}

// Forward on the tensor-core (tcgen05) kernel: any window size. `lse_ptrs`: optional per-slot fp32 [rows, heads] buffers
// that receive the base-2 log-sum-exp of every row (empty list: not stored).
void window_attn_tc(const std::vector<int64_t>& qkv_ptrs, const std::vector<int64_t>& out_ptrs,
                    const c10::optional<torch::Tensor>& bias_table, const std::vector<int64_t>& win_start, int64_t my_wg,
                    int64_t sp, int64_t my_sp, int64_t shardN, int64_t B, int64_t nWh, int64_t nWw, int64_t C,
                    int64_t heads, int64_t wh, int64_t ww, int64_t sh, int64_t sw, bool use_mask, double scale, int64_t tp,
                    const c10::optional<torch::Tensor>& status, const std::vector<int64_t>& lse_ptrs) {
  tb::WindowAttnArgs a = make_wa(win_start, my_wg, sp, my_sp, shardN, B, nWh, nWw, C, heads, wh, ww, sh, sw, use_mask, scale, tp);
  need(qkv_ptrs.size() == static_cast<size_t>(a.n_wg * a.sp) && out_ptrs.size() == qkv_ptrs.size(),
       "window_attn_tc: one buffer per peer slot");
  need(lse_ptrs.empty() || lse_ptrs.size() == qkv_ptrs.size(), "window_attn_tc: one lse buffer per peer slot (or none)");
  for (size_t i = 0; i < qkv_ptrs.size(); ++i) {
    a.qkv[i] = reinterpret_cast<const void*>(qkv_ptrs[i]);
    a.out[i] = reinterpret_cast<void*>(out_ptrs[i]);
    a.lse[i] = lse_ptrs.empty() ? nullptr : reinterpret_cast<float*>(lse_ptrs[i]);
  }
  a.bias_table = bias_table.has_value() ? bias_table->data_ptr<float>() : nullptr;
  tb::note_launch();
  rc_check(tb::window_attn_tc_fwd(a, status.has_value() ? status->data_ptr() : nullptr, cur_stream()), "window_attn_tc_fwd");
}

std::vector<int64_t> window_attn_tc_stalls(bool reset) {
  unsigned long long c[16];
  rc_check(tb::window_attn_tc_stalls(c, reset ? 1 : 0), "window_attn_tc_stalls");
  return std::vector<int64_t>(c, c + 16);
}

void window_attn_bwd(const std::vector<int64_t>& qkv_ptrs, const std::vector<int64_t>& dout_ptrs,
                     const std::vector<int64_t>& dqkv_ptrs, const c10::optional<torch::Tensor>& bias_table,
                     const c10::optional<torch::Tensor>& dbias_table, const std::vector<int64_t>& win_start,
                     int64_t my_wg, int64_t sp, int64_t my_sp, int64_t shardN, int64_t B, int64_t nWh, int64_t nWw,
                     int64_t C, int64_t heads, int64_t wh, int64_t ww, int64_t sh, int64_t sw, bool use_mask,
                     double scale, int64_t tp) {
  tb::WindowAttnArgs a = make_wa(win_start, my_wg, sp, my_sp, shardN, B, nWh, nWw, C, heads, wh, ww, sh, sw, use_mask, scale, tp);
  need(qkv_ptrs.size() == static_cast<size_t>(a.n_wg * a.sp) && dout_ptrs.size() == qkv_ptrs.size() &&
           dqkv_ptrs.size() == qkv_ptrs.size(),
       "window_attn_bwd: one buffer per peer slot");
  for (size_t i = 0; i < qkv_ptrs.size(); ++i) {
    a.qkv[i] = reinterpret_cast<const void*>(qkv_ptrs[i]);
    a.dout[i] = reinterpret_cast<const void*>(dout_ptrs[i]);
    a.dqkv[i] = reinterpret_cast<void*>(dqkv_ptrs[i]);
  }
  a.bias_table = bias_table.has_value() ? bias_table->data_ptr<float>() : nullptr;
  a.dbias_table = dbias_table.has_value() ? dbias_table->data_ptr<float>() : nullptr;
  tb::note_launch();
  rc_check(tb::window_attn_bwd(a, cur_stream()), "window_attn_bwd");
}

void window_attn_tc_bwd(const std::vector<int64_t>& qkv_ptrs, const std::vector<int64_t>& dout_ptrs,
                        const std::vector<int64_t>& dqkv_ptrs, const c10::optional<torch::Tensor>& bias_table,
                        const c10::optional<torch::Tensor>& dbias_table, const std::vector<int64_t>& win_start,
                        int64_t my_wg, int64_t sp, int64_t my_sp, int64_t shardN, int64_t B, int64_t nWh, int64_t nWw,
                        int64_t C, int64_t heads, int64_t wh, int64_t ww, int64_t sh, int64_t sw, bool use_mask,
                        double scale, int64_t tp, const c10::optional<torch::Tensor>& status,
                        const std::vector<int64_t>& lse_ptrs, const std::vector<int64_t>& drow_ptrs) {
  tb::WindowAttnArgs a = make_wa(win_start, my_wg, sp, my_sp, shardN, B, nWh, nWw, C, heads, wh, ww, sh, sw, use_mask, scale, tp);
  need(qkv_ptrs.size() == static_cast<size_t>(a.n_wg * a.sp) && dout_ptrs.size() == qkv_ptrs.size() &&
           dqkv_ptrs.size() == qkv_ptrs.size(),
       "window_attn_tc_bwd: one buffer per peer slot");
  need((lse_ptrs.empty() || lse_ptrs.size() == qkv_ptrs.size()) && drow_ptrs.size() == lse_ptrs.size(),
       "window_attn_tc_bwd: lse / drow buffers per peer slot (or none)");
  for (size_t i = 0; i < qkv_ptrs.size(); ++i) {
    a.qkv[i] = reinterpret_cast<const void*>(qkv_ptrs[i]);
    a.dout[i] = reinterpret_cast<const void*>(dout_ptrs[i]);
    a.dqkv[i] = reinterpret_cast<void*>(dqkv_ptrs[i]);
    a.lse[i] = lse_ptrs.empty() ? nullptr : reinterpret_cast<float*>(lse_ptrs[i]);
    a.drow[i] = drow_ptrs.empty() ? nullptr : reinterpret_cast<const float*>(drow_ptrs[i]);
  }
  a.bias_table = bias_table.has_value() ? bias_table->data_ptr<float>() : nullptr;
  a.dbias_table = dbias_table.has_value() ? dbias_table->data_ptr<float>() : nullptr;
  tb::note_launch();
  rc_check(tb::window_attn_tc_bwd(a, status.has_value() ? status->data_ptr() : nullptr, cur_stream()), "window_attn_tc_bwd");
}

void conv_s2_col2im(const torch::Tensor& dcol, torch::Tensor& out, int64_t W, int64_t r0) {
  need(dcol.is_cuda() && dcol.is_contiguous() && dcol.scalar_type() == torch::kBFloat16 && dcol.dim() == 5 && dcol.size(3) == 9,
       "conv_s2_col2im: dcol [B, Ho, Wo, 9, C] bf16 contiguous");
  need(out.is_contiguous() && out.dim() == 4 && out.size(0) == dcol.size(0) && out.size(2) == W && out.size(3) == dcol.size(4) &&
           (out.scalar_type() == torch::kBFloat16 || out.scalar_type() == torch::kFloat32),
       "conv_s2_col2im: out [B, rows, W, C] bf16 or fp32 contiguous");
  const c10::cuda::CUDAGuard guard(dcol.device());
  tb::note_launch();
  rc_check(tb::conv_s2_col2im(dcol.data_ptr(), out.data_ptr(), static_cast<int>(dcol.size(0)), static_cast<int>(dcol.size(1)),
                              static_cast<int>(dcol.size(2)), static_cast<int>(W), static_cast<int>(dcol.size(4)),
                              static_cast<int>(r0), static_cast<int>(out.size(1)),
                              out.scalar_type() == torch::kFloat32 ? 1 : 0, cur_stream()),
           "conv_s2_col2im");
}

void sum_slots(const torch::Tensor& slots, torch::Tensor& out, const c10::optional<torch::Tensor>& bias,
               const c10::optional<torch::Tensor>& residual) {
  need(slots.is_cuda() && slots.is_contiguous() && slots.scalar_type() == torch::kBFloat16 && slots.dim() >= 2,
       "sum_slots: [slots, ...] bf16 contiguous");
  need(out.is_contiguous() && out.scalar_type() == torch::kBFloat16 && out.numel() * slots.size(0) == slots.numel(),
       "sum_slots: out must hold one slot");
  need(!bias.has_value() || (bias->scalar_type() == torch::kBFloat16 && bias->is_contiguous() && bias->numel() == out.size(-1)),
       "sum_slots: bias must be bf16 [cols]");
  need(!residual.has_value() || (residual->scalar_type() == torch::kBFloat16 && residual->is_contiguous() &&
                                 residual->numel() == out.numel()),
       "sum_slots: residual must be bf16 with the shape of out");
  const c10::cuda::CUDAGuard guard(slots.device());
  tb::note_launch();
  rc_check(tb::sum_slots_bf16(slots.data_ptr(), out.data_ptr(), static_cast<int>(slots.size(0)), out.numel(), cur_stream(),
                              opt_ptr(bias), opt_ptr(residual), static_cast<int>(out.size(-1))),
           "sum_slots");
}

}  // namespace

void bind_elementwise(pybind11::module_& m) {
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("colsum", &colsum);
  m.def("groupnorm_stats", &groupnorm_stats);
  m.def("groupnorm_silu_apply", &groupnorm_silu_apply);
  m.def("groupnorm_silu_bwd_reduce", &groupnorm_silu_bwd_reduce, pybind11::arg("dy"), pybind11::arg("x"), pybind11::arg("stats"),
        pybind11::arg("gamma"), pybind11::arg("beta"), pybind11::arg("red"), pybind11::arg("groups"),
        pybind11::arg("dgamma") = pybind11::none(), pybind11::arg("dbeta") = pybind11::none());
  m.def("groupnorm_finalize", &groupnorm_finalize);
  m.def("strided_add", &strided_add);
  m.def("groupnorm_silu_bwd_apply", &groupnorm_silu_bwd_apply);
  m.def("masked_loss", &masked_loss);
  m.def("adamw_step", &adamw_step);
  m.def("grad_inspect", &grad_inspect);
  m.def("attn_rowdot", &attn_rowdot);
  m.def("sum_slots", &sum_slots, pybind11::arg("slots"), pybind11::arg("out"), pybind11::arg("bias") = pybind11::none(),
        pybind11::arg("residual") = pybind11::none());
  m.def("conv_s2_col2im", &conv_s2_col2im);
}

void bind_attention(pybind11::module_& m) {
  m.def("window_attn_fwd", &window_attn);
  m.def("window_attn_bwd", &window_attn_bwd);
  m.def("window_attn_tc_fwd", &window_attn_tc);
  m.def("window_attn_tc_stalls", &window_attn_tc_stalls);
  m.def("window_attn_tc_bwd", &window_attn_tc_bwd);
  m.def("set_debug_status", &set_debug_status, "status word for the bounds-checked debug build of the attention kernels");
  m.def("debug_bounds_build", &debug_bounds_build, "whether this extension was compiled with -DTERRA_DEBUG_BOUNDS");
}
