// Plain C++ host API of the terra_b200 CUDA kernels (no torch types). The Python binding layer
// (bindings.cpp) and C callers use these entry points; none of them allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

struct GemmOperand {
  const void* ptr;   // bf16
  long long ld;      // leading dimension in elements (stride of the outer stored dimension)
  int mn_major;      // 0: stored [rows][K] (K contiguous); 1: stored [K][rows] (rows contiguous)
};

struct GemmEpilogue {
  int flags;          // EPI_* bit mask (gemm_sm100.cuh)
  void* C;
  void* C2;
  const void* bias;
  const void* residual;
  const void* aux;
  long long ldc, ldc2, ldr, ldaux;
  float alpha;
  int out_w, out_h, shuffle_cout;
  void* status;       // KernelStatus* (device), may be null
  // Weight-gradient form (A read MN-major, fp32 atomic output): also accumulate the sums of A's columns over the
  // contraction (sum over tokens of dy[token][n], the bias gradient) into colsum[n] (fp32), from an extra
  // 16-column MMA against a tile of ones. Null: off. Tile widths up to 192.
  float* colsum;
};

// Tensor-parallel fusions over peer memory. a_ptr[i]: GPU i's [a_rows, K] bf16 shard (K-major, leading dimension of
// operand A) - A is their concatenation, read tile by tile over NVLink. c_ptr[i]: GPU i's fp32 [c_rows, N] accumulation
// buffer - output row g is reduced into c_ptr[g / c_rows]. Either part may be unused (count 0 or 1).
struct GemmPeers {
  int a_peers;
  const void* a_ptr[8];
  long long a_rows;
  int rank;          // this GPU's index: its own shard's tiles are scheduled first; its slot in the owners' staging
  const void* a_flags;        // optional: uint32 flags, one per peer, in this GPU's memory; a_flags[i] >= a_epoch means
  unsigned int a_epoch;       // "peer i's shard is written"; the kernel waits for it (at most a_budget_ns) itself
  unsigned long long a_budget_ns;
  int a_interleave;           // 1: alternate local / remote tiles (direct peer loads); 0: own shard first
  int a_chunks;               // flags per peer (1..4); flag [i * a_chunks + c] covers chunk c of peer i's rows
  int c_peers;
  void* c_ptr[8];    // fp32 [c_rows, N] accumulation buffers (atomic epilogue) or bf16 [c_peers][c_rows, N] staging (plain)
  long long c_rows;
};

// gemm_host.cu
int gemm_bf16_peers(const GemmOperand& A, const GemmOperand& B, long long M, long long N, long long K,
                    const GemmEpilogue& epi, const GemmPeers& peers, int split_k, int bn_request, int num_sms,
                    cudaStream_t stream);
int gemm_bf16(const GemmOperand& A, const GemmOperand& B, long long M, long long N, long long K,
              const GemmEpilogue& epi, int split_k, int bn_request, int num_sms, cudaStream_t stream);
// halo_lo / halo_hi: optional one-row images [B, 1, W, Cin] holding the row above / below a row stripe
// (null: rows outside the image are zero).
// Cycle counters of the GEMM kernel's roles summed over CTAs and launches since the last reset:
// [0] MMA span, [1] MMA waiting for an accumulator, [2] MMA waiting for operands, [3] TMA span, [4] TMA waiting for
// free stages, [5] epilogue span, [6] epilogue waiting for tiles. Synchronises the device.
int gemm_stall_counters(unsigned long long* out8, int reset);

int conv3x3_fwd_bf16(const void* x, const void* w, int B, int H, int W, int Cin, int Cout, int stride,
                     const GemmEpilogue& epi, int num_sms, cudaStream_t stream, const void* halo_lo = nullptr,
                     const void* halo_hi = nullptr);
int conv3x3_wgrad_bf16(const void* x, const void* dy, float* dw, int B, int H, int W, int Cin, int Cout, int stride,
                       int split_k, void* status, int num_sms, cudaStream_t stream, const void* halo_lo = nullptr,
                       const void* halo_hi = nullptr, float* bias_grad = nullptr);   // bias_grad[Cout] += sums of dy

// elementwise.cu -------------------------------------------------------------------------------
// LayerNorm over the last dimension (C <= 8192, C % 8 == 0), bf16 in/out, fp32 statistics.
int layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                  long long rows, int C, float eps, cudaStream_t stream);
// dx (bf16, plus `dres` when given); dgamma/dbeta accumulated atomically into fp32 buffers that the caller zeroed.
int layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                  float* dgamma, float* dbeta, const void* dres, long long rows, int C, cudaStream_t stream);
// Column sums of a bf16 [rows, C] matrix into fp32 out[C] (atomic accumulate; caller zeroes out).
int colsum_rows_per_block();
// out[c] += column sums of the bf16 matrix x; partials: fp32 scratch of ceil(rows / colsum_rows_per_block()) x C
int colsum_bf16(const void* x, float* out, float* partials, long long rows, int C, long long ld, cudaStream_t stream);
// GroupNorm statistics over NHWC bf16 [B, HW, C]: accumulates per (b, group) sum and sum of squares (fp32, zeroed).
int groupnorm_stats(const void* x, float* sums, int B, long long HW, int C, int groups, cudaStream_t stream);
// y = silu((x - mean) * rstd * gamma + beta) [+ res]; `stats` holds {mean, rstd} per (b, group).
int groupnorm_silu_apply(const void* x, const float* stats, const void* gamma, const void* beta, const void* res, void* y,
                         int B, long long HW, int C, int groups, cudaStream_t stream);
// Backward of GroupNorm+SiLU. Pass 1 accumulates per (b,group) {sum(dz), sum(dz*xhat)} and per-channel dgamma/dbeta;
// pass 2 produces dx. dz = dy * silu'(z).
int groupnorm_silu_bwd_reduce(const void* dy, const void* x, const float* stats, const void* gamma, const void* beta,
                              float* red, float* dgamma, float* dbeta, int B, long long HW, int C, int groups,
                              cudaStream_t stream);
int groupnorm_silu_bwd_apply(const void* dy, const void* x, const float* stats, const float* red, const void* gamma,
                             const void* beta, void* dx, int B, long long HW, int C, int groups, float inv_count,
                             cudaStream_t stream);
// {sum, sumsq} per (sample, group) cell -> {mean, rstd}; `clear` zeroes the sums afterwards (persistent scratch).
int groupnorm_finalize(float* sums, float* stats, int cells, float inv_count, float eps, int clear, cudaStream_t stream);
// dst[a*sa + b*sb + c*sc] += src[a][b][c] (fp32, src contiguous [na][nb][nc]); `clear` zeroes src behind the read.
int strided_add_f32(float* src, float* dst, int na, int nb, int nc, long long sa, long long sb, long long sc, int clear,
                    cudaStream_t stream);
// Masked loss: loss_sum += sum(f(pred * mask - label)), f = |.| (kind 0) or square (kind 1);
// grad = mask * f'(.) * scale (bf16). `mask` may be null. Partial sums are fp32 atomics on loss_sum[0].
int masked_loss_fwd_bwd(const void* pred, const void* label, const void* mask, long long n, long long mask_period,
                        int kind, float grad_scale, float* loss_sum, void* grad, cudaStream_t stream);
// Fused AdamW on an fp32 master with a bf16 (or fp32) gradient, writing the bf16 working copy.
int adamw_step(float* master, float* exp_avg, float* exp_avg_sq, const void* grad, int grad_is_bf16, void* param_bf16,
               long long n, float lr, float beta1, float beta2, float eps, float weight_decay, float bias_corr1,
               float bias_corr2_sqrt, float grad_scale, cudaStream_t stream);
// Loss-scaling support: out2[0] += sum of squares of the fp32 buffer, out2[1] = 1 when any element is inf / nan
// (caller zeroes out2).
int grad_inspect(const float* grad, long long n, float* out2, cudaStream_t stream);
// bf16 <-> fp32 helpers
int cast_f32_to_bf16(const float* src, void* dst, long long n, cudaStream_t stream);
// out[b, i, j, c] = a + b elementwise (bf16)
int add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream);
// Input gradient of the 3x3 stride-2 convolution gathered from per-tap columns dcol[B, Ho, Wo, 9, C] (bf16): padded
// input rows [r0, r0 + rows) x columns [1, W + 1) -> out[B, rows, W, C] (fp32 when out_f32, else bf16).
int conv_s2_col2im(const void* dcol, void* out, int B, int Ho, int Wo, int W, int C, int r0, int rows, int out_f32,
                   cudaStream_t stream);
// out[n] = sum of `slots` consecutive bf16 buffers of n elements (fp32 accumulation); the owner's side of the
// slot-staged reduce-scatter. Optional: + bias[col] (bf16, `cols` columns per row) and + residual (bf16, n elements).
int sum_slots_bf16(const void* src, void* out, int slots, long long n, cudaStream_t stream, const void* bias = nullptr,
                   const void* residual = nullptr, int cols = 0);

// window_attn.cu -------------------------------------------------------------------------------
constexpr int WA_MAX_PEERS = 16;
// Window attention over window-major activations (see window_attn.cu). Peer slot = wg_rank * sp + sp_rank.
struct WindowAttnArgs {
  const void* qkv[WA_MAX_PEERS];   // bf16 [B * nW_p * shardN, 3*C] per peer slot (q | k | v, head-major inside each)
  void* out[WA_MAX_PEERS];         // forward: bf16 [B * nW_p * shardN, C] per peer slot
  const void* dout[WA_MAX_PEERS];  // backward: gradient of out
  void* dqkv[WA_MAX_PEERS];        // backward: gradient of qkv
  const float* bias_table;         // fp32 [(2wh-1)*(2ww-1), num_heads] or null
  float* dbias_table;              // backward, fp32 atomics (caller zeroes), or null
  float* lse[WA_MAX_PEERS];        // optional, tensor-core forward: base-2 log-sum-exp per (row, head), fp32 [rows, num_heads]
  const float* drow[WA_MAX_PEERS]; // tensor-core backward of large windows: rowsum(dO o O) per (row, head), fp32 [rows, num_heads]
  int win_start[9];                // flat window range of window-group rank p: [win_start[p], win_start[p+1])
  int n_wg, my_wg;                 // ranks along the window dimension, and mine
  int sp, my_sp, shardN;           // tokens of a window are split into sp shards of shardN tokens
  int tp;                          // > 1: every buffer is the concatenation of tp chunks [B, ceil(nW_p / tp) windows]
                                   // (rows all-gathered over a tensor-parallel group); else [B, nW_p windows]
  int B, nWh, nWw;                 // batch and global window grid
  int wh, ww, sh, sw;              // window and cyclic shift (0 for regular blocks)
  int use_mask;                    // shifted-window region mask (-100)
  int C, num_heads;                // channels / heads held by this rank (C/tp, nH/tp)
  int heads_per_cta;               // filled by the launcher
  float scale;
  void* debug_status;              // KernelStatus* for the bounds-checked debug build (token locations), may be null
};
int window_attn_fwd(const WindowAttnArgs& a, cudaStream_t stream);
int window_attn_bwd(const WindowAttnArgs& a, cudaStream_t stream);
// window_attn_tc.cu: forward on tcgen05 / TMEM, any window size (flash-style K/V streaming above 64 tokens).
// `status`: KernelStatus* (device) for the bounded waits, may be null.
int window_attn_tc_fwd(const WindowAttnArgs& a, void* status, cudaStream_t stream);
// Cycle counters of the tensor-core attention kernel's roles since the last reset: [0] producer span, [1] of it waiting
// for a free buffer, [2] MMA thread span, [3] waiting for operands, [4] waiting for probabilities, [5] softmax thread
// span, [6] waiting for scores, [7] waiting for outputs. Synchronises the device.
int window_attn_tc_stalls(unsigned long long* out16, int reset);   // [8..13]: softmax thread segments, see window_attn_tc.cu
// Backward on tcgen05, head dims 16 / 32 / 64: one pass for windows of at most 64 tokens, two passes (dQ; dK, dV) with
// `lse` and `drow` for larger ones.
int window_attn_tc_bwd(const WindowAttnArgs& a, void* status, cudaStream_t stream);
// drow[row, head] = sum over the head's channels of dO * O (bf16 [rows, C] inputs, fp32 [rows, heads] output).
int attn_rowdot(const void* o, const void* dout, float* drow, long long rows, int C, int heads, cudaStream_t stream);

}  // namespace tb
