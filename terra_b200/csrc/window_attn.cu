// Swin window attention (forward and backward) over a window-major activation layout, with the
// shifted-window roll / partition / reverse, the window-parallel halo and the sequence-parallel K/V
// gather all expressed as index math on the loads and stores:
//
//   * activations are stored unshifted, window-major: rank p of the window dimension holds
//     [B, nW_p, shardN, *] rows for its flat window range [win_start[p], win_start[p+1]);
//   * a CTA owns one window of the *shifted* frame and a group of heads; every token of that window is
//     located (owner rank, row) in closed form and its Q/K/V row is read from the owner's buffer
//     (a peer pointer over NVLink when the owner is another GPU); outputs are stored to the token's
//     home row, again possibly on a peer;
//   * relative-position bias comes from a shared-memory copy of the table, the shifted-window mask
//     from the token's region id in the rolled frame; nothing of size [nW, N, N] is materialised.
//
// Windows here are small (N = wh*ww <= 128 keys), far below the tile sizes at which tcgen05 pays off,
// and the op is bound by the Q/K/V/O traffic, so the products run on warp-level mma.sync with operands
// staged in shared memory by 16-byte gathers.
#include "common.cuh"
#include "host_api.h"
#include "window_geo.cuh"

namespace tb {
namespace {

constexpr int WA_THREADS = 128;
constexpr int WA_WARPS = 4;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

// 16-byte asynchronous copy global -> shared; `valid == false` writes zeros without reading the source.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// 32-bit shared-memory load by address (keeps the table lookups of the softmax on LDS with one integer add each).
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));   // the table is read-only inside the item loop
  return v;
}

constexpr float WA_LOG2E = 1.4426950408889634f;

// Kernel layout.
//   A CTA (4 warps) loops over (batch, window) items for one group of heads (G = heads_per_cta * HD channels).
//   Per item: locate the window's tokens, gather Q/K/V [dO] rows into shared memory, then per head
//     phase 1 (a warp per 16 query rows): S = Q K^T, P = softmax(scale S + bias [+ mask]) with the scores kept in the
//       mma accumulator registers; forward: O = P V; backward: dP = dO V^T, dS = P (dP - rowsum(P dP)), dQ = dS K,
//       P and dS stashed as bf16 for phase 2, bias gradient by shared-memory reductions;
//     phase 2 (backward, a warp per 16 keys): dV = P^T dO, dK = dS^T Q;
//   finally the results are scattered to the tokens' home rows.
//   Softmax runs in the base-2 domain: the table is stored pre-multiplied by log2(e) and the scale carries the same
//   factor, so an element costs one fused multiply-add, one table read, one max, one subtract and one ex2.
//   Windows whose tokens share one mask region (all windows of unshifted layers, the interior windows of shifted
//   ones) with N == NPAD take a branch-free path; the others a general one with the mask and padding tests.
template <int HD, int NPAD, bool BWD>
__global__ void __launch_bounds__(WA_THREADS, NPAD > 64 ? 1 : (BWD ? 3 : 5)) window_attn_kernel(const __grid_constant__ WindowAttnArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int hpc = a.heads_per_cta;
  const int G = hpc * HD;
  const int stride = G + 8;
  constexpr int pstride = NPAD + 8;
  Geo geo;
  geo.N = a.wh * a.ww;
  geo.nrel = (2 * a.wh - 1) * (2 * a.ww - 1);
  geo.Hg = a.nWh * a.wh;
  geo.Wg = a.nWw * a.ww;
  const int N = geo.N;

  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* Ks = Qs + NPAD * stride;
  __nv_bfloat16* Vs = Ks + NPAD * stride;
  __nv_bfloat16* dOs = Vs + NPAD * stride;                              // BWD only
  __nv_bfloat16* dQs = dOs + (BWD ? NPAD * stride : 0);                 // BWD only
  __nv_bfloat16* Ps = dQs + (BWD ? NPAD * stride : 0);                  // BWD only [NPAD][pstride]
  __nv_bfloat16* dSs = Ps + (BWD ? NPAD * pstride : 0);                 // BWD only
  float* bias_s = reinterpret_cast<float*>(dSs + (BWD ? NPAD * pstride : 0));   // [hpc][nrel], times log2(e)
  float* dbias_s = bias_s + hpc * geo.nrel;                                      // BWD only [hpc][nrel]
  // the float tables have an arbitrary length: round up so that the 8-byte row offsets are aligned
  // (offset arithmetic on the shared array itself, so the compiler keeps these accesses in the shared state space)
  const size_t tables_off =
      (static_cast<size_t>(reinterpret_cast<uint8_t*>(dbias_s + (BWD ? hpc * geo.nrel : 0)) - smem) + 15) & ~size_t(15);
  long long* rowofs = reinterpret_cast<long long*>(smem + tables_off);                       // [NPAD]
  int* rowslot = reinterpret_cast<int*>(rowofs + NPAD);                                      // [NPAD]
  int* rowreg = rowslot + NPAD;                                                              // [NPAD]
  // cofs[t] = 4 * ((t / ww) * (2 ww - 1) + (t % ww)): the byte offset into a head's table of the relative position
  // of (query r, key c) is cofs[r] - cofs[c] + 4 * rel0, so the inner loops need no division.
  int* cofs = rowreg + NPAD;                                                                 // [NPAD]
  // bias gradient (BWD): posofs[tj * ww + cj] = tj * pstride + cj (low 16 bits) | tj << 16; one ww*ww fp32 scratch per warp
  int* posofs = cofs + NPAD;                                                                 // [ww*ww]
  float* mbuf = reinterpret_cast<float*>(posofs + (BWD ? a.ww * a.ww : 0));                  // [WA_WARPS][ww*ww]
  const int rel0 = (a.wh - 1) * (2 * a.ww - 1) + (a.ww - 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int cg = blockIdx.y;            // head group
  const int head0 = cg * hpc;
  const bool use_bias = a.bias_table != nullptr;
  const bool bias_grad = BWD && use_bias && a.dbias_table != nullptr;
  const int my_nw = a.win_start[a.my_wg + 1] - a.win_start[a.my_wg];
  const int q0 = a.my_sp * a.shardN;
  const int q1 = min(N, q0 + a.shardN);
  const float scale2 = a.scale * WA_LOG2E;

  for (int i = tid; i < hpc * geo.nrel; i += WA_THREADS) {
    const int h = i / geo.nrel, r = i % geo.nrel;
    bias_s[i] = use_bias ? a.bias_table[r * a.num_heads + head0 + h] * WA_LOG2E : 0.f;
    if (BWD) dbias_s[i] = 0.f;
  }
  for (int t = tid; t < NPAD; t += WA_THREADS) cofs[t] = 4 * ((t / a.ww) * (2 * a.ww - 1) + (t % a.ww));
  if (BWD)
    for (int t = tid; t < a.ww * a.ww; t += WA_THREADS) posofs[t] = ((t / a.ww) * pstride + (t % a.ww)) | ((t / a.ww) << 16);
  // Row-wise copies between global and shared memory: a warp takes whole rows, lane l moves the 16-byte vectors
  // l and l + 32 of the row's (matrix, vector) list. The (matrix, vector) split is computed once here, so the
  // copy loops contain no division.
  const int vpr = G / 8;                       // 16-byte vectors per row and matrix
  const int gather_mats = BWD ? 4 : 3;         // q, k, v [, dO]
  int gm[2], gv[2];
  bool gok[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int idx = lane + 32 * k;
    gok[k] = idx < gather_mats * vpr;
    gm[k] = gok[k] ? idx / vpr : 0;
    gv[k] = gok[k] ? idx % vpr : 0;
  }

  const int items = a.B * my_nw;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int b = item / my_nw, lw = item % my_nw;
    const int flat = a.win_start[a.my_wg] + lw;
    const int ii = flat / a.nWw, jj = flat % a.nWw;
    __syncthreads();   // previous item fully consumed
    int differs = 0;
    if (tid < NPAD) {
      if (tid < N) {
        const Home h = locate(a, geo, b, ii, jj, tid);
        rowofs[tid] = h.row;
        rowslot[tid] = h.slot;
        rowreg[tid] = h.region;
        differs = h.region != region_of(a, geo, ii * a.wh, jj * a.ww);
      } else {
        rowofs[tid] = -1;
        rowslot[tid] = 0;
        rowreg[tid] = 15;
      }
    }
    // (also the barrier that publishes the row tables)
    const bool general = (__syncthreads_or(differs) != 0 && a.use_mask) || N != NPAD;
    // ---- gather Q (query rows), K, V (all rows) [and dO] for this head group with 16-byte asynchronous copies
    //      (global or peer memory -> shared memory, zero fill for rows outside the window / shard): all of a lane's
    //      copies are in flight at once, one memory round trip per item
    for (int r = warp; r < NPAD; r += WA_WARPS) {
      const long long ro = rowofs[r];
      const int sl = rowslot[r];
      const bool in_win = r < N;
      const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(a.qkv[sl]) + (in_win ? ro * (3LL * a.C) + cg * G : 0);
      const __nv_bfloat16* db =
          BWD ? static_cast<const __nv_bfloat16*>(a.dout[sl]) + (in_win ? ro * a.C + cg * G : 0) : nullptr;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (gok[k]) {
          const int m = gm[k];
          const bool q_like = (m == 0 || m == 3);
          const bool valid = in_win && (!q_like || BWD || (r >= q0 && r < q1));
          const __nv_bfloat16* src = (m < 3) ? qb + (valid ? m * a.C + gv[k] * 8 : 0) : db + (valid ? gv[k] * 8 : 0);
          __nv_bfloat16* dst = (m == 0 ? Qs : (m == 1 ? Ks : (m == 2 ? Vs : dOs))) + r * stride + gv[k] * 8;
          cp_async16(dst, src, valid);
        }
      }
    }
    cp_async_wait_all();
    __syncthreads();

    constexpr int rblocks = NPAD / 16;
    for (int hh = 0; hh < hpc; ++hh) {
      const uint32_t btb = smem_u32(bias_s + hh * geo.nrel);
      // =============================== phase 1: per 16-query-row block
      for (int rb = warp; rb < rblocks; rb += WA_WARPS) {
        if (rb * 16 >= N) continue;
        if (!BWD && (rb * 16 >= q1 || rb * 16 + 16 <= q0)) continue;
        float s[NPAD / 8][4];
#pragma unroll
        for (int nb = 0; nb < NPAD / 8; ++nb)
#pragma unroll
          for (int k = 0; k < 4; ++k) s[nb][k] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          uint32_t af[4];
          ldsm_x4(af, Qs + (rb * 16 + (lane & 15)) * stride + hh * HD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int nb = 0; nb < NPAD / 8; nb += 2) {
            uint32_t bf[4];
            ldsm_x4(bf, Ks + (nb * 8 + (lane & 7) + (lane >> 4) * 8) * stride + hh * HD + kk * 16 + ((lane >> 3) & 1) * 8);
            const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
            mma_bf16_16816(s[nb], af, b0);
            mma_bf16_16816(s[nb + 1], af, b1);
          }
        }
        // scale, bias, mask, softmax numerators (rows gq and gq+8 of the block), base-2 domain
        const int r0 = rb * 16 + gq, r1 = r0 + 8;
        const int ro0 = cofs[r0] + 4 * rel0, ro1 = cofs[r1] + 4 * rel0;   // r1 < NPAD always
        float mx0 = -1e30f, mx1 = -1e30f;
        if (!general) {
#pragma unroll
          for (int nb = 0; nb < NPAD / 8; ++nb) {
            const int2 co = *reinterpret_cast<const int2*>(cofs + nb * 8 + tq * 2);
            s[nb][0] = fmaf(s[nb][0], scale2, lds_f32(btb + (ro0 - co.x)));
            s[nb][1] = fmaf(s[nb][1], scale2, lds_f32(btb + (ro0 - co.y)));
            s[nb][2] = fmaf(s[nb][2], scale2, lds_f32(btb + (ro1 - co.x)));
            s[nb][3] = fmaf(s[nb][3], scale2, lds_f32(btb + (ro1 - co.y)));
            mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
          }
        } else {
          const int reg0 = rowreg[r0], reg1 = rowreg[r1];
          const bool row0 = r0 < N, row1 = r1 < N;
#pragma unroll
          for (int nb = 0; nb < NPAD / 8; ++nb) {
            const int2 co = *reinterpret_cast<const int2*>(cofs + nb * 8 + tq * 2);
            const int2 cr = *reinterpret_cast<const int2*>(rowreg + nb * 8 + tq * 2);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int col = nb * 8 + tq * 2 + (k & 1);
              const bool lo = k < 2;
              float v = s[nb][k] * scale2;
              if (col < N) {
                if (lo ? row0 : row1) v += lds_f32(btb + ((lo ? ro0 : ro1) - ((k & 1) ? co.y : co.x)));
                if (a.use_mask && ((k & 1) ? cr.y : cr.x) != (lo ? reg0 : reg1)) v += -100.f * WA_LOG2E;
              } else {
                v = -1e30f;
              }
              s[nb][k] = v;
              if (lo) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
            }
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nb = 0; nb < NPAD / 8; ++nb) {
          s[nb][0] = exp2f(s[nb][0] - mx0);
          s[nb][1] = exp2f(s[nb][1] - mx0);
          s[nb][2] = exp2f(s[nb][2] - mx1);
          s[nb][3] = exp2f(s[nb][3] - mx1);
          sum0 += s[nb][0] + s[nb][1];
          sum1 += s[nb][2] + s[nb][3];
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        const float inv0 = 1.f / sum0, inv1 = 1.f / sum1;
        if (!BWD) {
          // O = P V with the numerators as P; the row normalisation is applied to the (much smaller) output.
          // Staged over this warp's own Q rows (no other warp reads them).
          float o[HD / 8][4];
#pragma unroll
          for (int nb = 0; nb < HD / 8; ++nb)
#pragma unroll
            for (int k = 0; k < 4; ++k) o[nb][k] = 0.f;
#pragma unroll
          for (int j = 0; j < NPAD / 16; ++j) {
            const uint32_t pf[4] = {pack_bf16x2(s[2 * j][0], s[2 * j][1]), pack_bf16x2(s[2 * j][2], s[2 * j][3]),
                                    pack_bf16x2(s[2 * j + 1][0], s[2 * j + 1][1]),
                                    pack_bf16x2(s[2 * j + 1][2], s[2 * j + 1][3])};
#pragma unroll
            for (int nb = 0; nb < HD / 8; nb += 2) {
              uint32_t bf[4];
              ldsm_x4_t(bf, Vs + (j * 16 + (lane & 15)) * stride + hh * HD + nb * 8 + (lane >> 4) * 8);
              const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
              mma_bf16_16816(o[nb], pf, b0);
              mma_bf16_16816(o[nb + 1], pf, b1);
            }
          }
          __syncwarp();
#pragma unroll
          for (int nb = 0; nb < HD / 8; ++nb) {
            *reinterpret_cast<uint32_t*>(Qs + r0 * stride + hh * HD + nb * 8 + tq * 2) =
                pack_bf16x2(o[nb][0] * inv0, o[nb][1] * inv0);
            *reinterpret_cast<uint32_t*>(Qs + r1 * stride + hh * HD + nb * 8 + tq * 2) =
                pack_bf16x2(o[nb][2] * inv1, o[nb][3] * inv1);
          }
        } else {
#pragma unroll
          for (int nb = 0; nb < NPAD / 8; ++nb) {
            s[nb][0] *= inv0;
            s[nb][1] *= inv0;
            s[nb][2] *= inv1;
            s[nb][3] *= inv1;
          }
          // dP = dO V^T
          float dp[NPAD / 8][4];
#pragma unroll
          for (int nb = 0; nb < NPAD / 8; ++nb)
#pragma unroll
            for (int k = 0; k < 4; ++k) dp[nb][k] = 0.f;
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            uint32_t af[4];
            ldsm_x4(af, dOs + (rb * 16 + (lane & 15)) * stride + hh * HD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < NPAD / 8; nb += 2) {
              uint32_t bf[4];
              ldsm_x4(bf, Vs + (nb * 8 + (lane & 7) + (lane >> 4) * 8) * stride + hh * HD + kk * 16 + ((lane >> 3) & 1) * 8);
              const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
              mma_bf16_16816(dp[nb], af, b0);
              mma_bf16_16816(dp[nb + 1], af, b1);
            }
          }
          float d0 = 0.f, d1 = 0.f;
#pragma unroll
          for (int nb = 0; nb < NPAD / 8; ++nb) {
            d0 += s[nb][0] * dp[nb][0] + s[nb][1] * dp[nb][1];
            d1 += s[nb][2] * dp[nb][2] + s[nb][3] * dp[nb][3];
          }
          d0 += __shfl_xor_sync(0xffffffffu, d0, 1);
          d0 += __shfl_xor_sync(0xffffffffu, d0, 2);
          d1 += __shfl_xor_sync(0xffffffffu, d1, 1);
          d1 += __shfl_xor_sync(0xffffffffu, d1, 2);
          // dS = P * (dP - D); stash P and dS (bf16) for phase 2 and the bias gradient
#pragma unroll
          for (int nb = 0; nb < NPAD / 8; ++nb) {
            float ds[4];
            ds[0] = s[nb][0] * (dp[nb][0] - d0);
            ds[1] = s[nb][1] * (dp[nb][1] - d0);
            ds[2] = s[nb][2] * (dp[nb][2] - d1);
            ds[3] = s[nb][3] * (dp[nb][3] - d1);
            const int col = nb * 8 + tq * 2;
            *reinterpret_cast<uint32_t*>(Ps + r0 * pstride + col) = pack_bf16x2(s[nb][0], s[nb][1]);
            *reinterpret_cast<uint32_t*>(Ps + r1 * pstride + col) = pack_bf16x2(s[nb][2], s[nb][3]);
            *reinterpret_cast<uint32_t*>(dSs + r0 * pstride + col) = pack_bf16x2(ds[0], ds[1]);
            *reinterpret_cast<uint32_t*>(dSs + r1 * pstride + col) = pack_bf16x2(ds[2], ds[3]);
            dp[nb][0] = ds[0]; dp[nb][1] = ds[1]; dp[nb][2] = ds[2]; dp[nb][3] = ds[3];
          }
          // dQ = scale * dS K
          float dq[HD / 8][4];
#pragma unroll
          for (int nb = 0; nb < HD / 8; ++nb)
#pragma unroll
            for (int k = 0; k < 4; ++k) dq[nb][k] = 0.f;
#pragma unroll
          for (int j = 0; j < NPAD / 16; ++j) {
            const uint32_t pf[4] = {pack_bf16x2(dp[2 * j][0], dp[2 * j][1]), pack_bf16x2(dp[2 * j][2], dp[2 * j][3]),
                                    pack_bf16x2(dp[2 * j + 1][0], dp[2 * j + 1][1]),
                                    pack_bf16x2(dp[2 * j + 1][2], dp[2 * j + 1][3])};
#pragma unroll
            for (int nb = 0; nb < HD / 8; nb += 2) {
              uint32_t bf[4];
              ldsm_x4_t(bf, Ks + (j * 16 + (lane & 15)) * stride + hh * HD + nb * 8 + (lane >> 4) * 8);
              const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
              mma_bf16_16816(dq[nb], pf, b0);
              mma_bf16_16816(dq[nb + 1], pf, b1);
            }
          }
#pragma unroll
          for (int nb = 0; nb < HD / 8; ++nb) {
            *reinterpret_cast<uint32_t*>(dQs + r0 * stride + hh * HD + nb * 8 + tq * 2) =
                pack_bf16x2(dq[nb][0] * a.scale, dq[nb][1] * a.scale);
            *reinterpret_cast<uint32_t*>(dQs + r1 * stride + hh * HD + nb * 8 + tq * 2) =
                pack_bf16x2(dq[nb][2] * a.scale, dq[nb][3] * a.scale);
          }
        }
      }
      if (BWD) {
        __syncthreads();
        // Bias gradient: entry (di, dj) of the table collects dS[r][c] over the pairs with r - c = (di, dj), for
        // this rank's query rows. A warp takes the row displacements di, di + 4, ...: its lanes first add up, for
        // each in-row position pair (tj, cj), the ww x ww blocks (ti, ci = ti - di) of dS (conflict-free reads,
        // balanced over the warps), then lanes sum the diagonals tj - cj = dj of that small matrix. Every entry
        // has one owner, so no atomics are needed inside the CTA.
        if (bias_grad) {
          const int ww2 = a.ww * a.ww, ndi = 2 * a.wh - 1, ndj = 2 * a.ww - 1;
          const bool partial = q0 > 0 || q1 < N;
          float* Mw = mbuf + warp * ww2;
          for (int di_idx = warp; di_idx < ndi; di_idx += WA_WARPS) {
            const int di = di_idx - (a.wh - 1);
            const int ti_lo = max(0, di), ti_hi = min(a.wh, a.wh + di);
            for (int pos = lane; pos < ww2; pos += 32) {
              const int po = posofs[pos] & 0xffff, tj = posofs[pos] >> 16;
              float acc = 0.f;
              for (int ti = ti_lo; ti < ti_hi; ++ti) {
                const int r = ti * a.ww + tj;
                if (!partial || (r >= q0 && r < q1))
                  acc += __bfloat162float(dSs[ti * a.ww * pstride + (ti - di) * a.ww + po]);
              }
              Mw[pos] = acc;
            }
            __syncwarp();
            for (int dj_idx = lane; dj_idx < ndj; dj_idx += 32) {
              const int dj = dj_idx - (a.ww - 1);
              float acc = 0.f;
              for (int tj = max(0, dj); tj < min(a.ww, a.ww + dj); ++tj) acc += Mw[tj * (a.ww + 1) - dj];
              dbias_s[hh * geo.nrel + di_idx * ndj + dj_idx] += acc;
            }
            __syncwarp();
          }
        }
        // =============================== phase 2: per 16-key block: dV = P^T dO, dK = scale * dS^T Q
        for (int kb = warp; kb < rblocks; kb += WA_WARPS) {
          if (kb * 16 >= N) continue;
          float dv[HD / 8][4], dk[HD / 8][4];
#pragma unroll
          for (int nb = 0; nb < HD / 8; ++nb)
#pragma unroll
            for (int k = 0; k < 4; ++k) dv[nb][k] = dk[nb][k] = 0.f;
#pragma unroll
          for (int j = 0; j < NPAD / 16; ++j) {   // query blocks (contraction)
            uint32_t pa[4], sa[4];
            const int prow = j * 16 + (lane & 7) + (lane >> 4) * 8;
            const int pcol = kb * 16 + ((lane >> 3) & 1) * 8;
            ldsm_x4_t(pa, Ps + prow * pstride + pcol);
            ldsm_x4_t(sa, dSs + prow * pstride + pcol);
#pragma unroll
            for (int nb = 0; nb < HD / 8; nb += 2) {
              uint32_t bf[4];
              ldsm_x4_t(bf, dOs + (j * 16 + (lane & 15)) * stride + hh * HD + nb * 8 + (lane >> 4) * 8);
              const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
              mma_bf16_16816(dv[nb], pa, b0);
              mma_bf16_16816(dv[nb + 1], pa, b1);
              ldsm_x4_t(bf, Qs + (j * 16 + (lane & 15)) * stride + hh * HD + nb * 8 + (lane >> 4) * 8);
              const uint32_t c0[2] = {bf[0], bf[1]}, c1[2] = {bf[2], bf[3]};
              mma_bf16_16816(dk[nb], sa, c0);
              mma_bf16_16816(dk[nb + 1], sa, c1);
            }
          }
          // K and V columns of this head are dead after phase 1: reuse them as the staging of dK, dV
          const int r0 = kb * 16 + gq, r1 = r0 + 8;
          __syncwarp();
#pragma unroll
          for (int nb = 0; nb < HD / 8; ++nb) {
            const int c = hh * HD + nb * 8 + tq * 2;
            *reinterpret_cast<uint32_t*>(Ks + r0 * stride + c) = pack_bf16x2(dk[nb][0] * a.scale, dk[nb][1] * a.scale);
            *reinterpret_cast<uint32_t*>(Ks + r1 * stride + c) = pack_bf16x2(dk[nb][2] * a.scale, dk[nb][3] * a.scale);
            *reinterpret_cast<uint32_t*>(Vs + r0 * stride + c) = pack_bf16x2(dv[nb][0], dv[nb][1]);
            *reinterpret_cast<uint32_t*>(Vs + r1 * stride + c) = pack_bf16x2(dv[nb][2], dv[nb][3]);
          }
        }
        // the next head's phase 1 writes Ps/dSs again: wait for every reader
        __syncthreads();
      }
    }
    __syncthreads();
    // ---- scatter results to the home rows (a warp per row; lanes over the row's vectors)
    if (!BWD) {
      for (int r = q0 + warp; r < q1; r += WA_WARPS) {
        __nv_bfloat16* base = static_cast<__nv_bfloat16*>(a.out[rowslot[r]]) + rowofs[r] * a.C + cg * G;
        if (lane < vpr) *reinterpret_cast<uint4*>(base + lane * 8) = *reinterpret_cast<const uint4*>(Qs + r * stride + lane * 8);
      }
    } else {
      // With sequence parallelism every rank of the window recomputes the whole window (cheap) and keeps only the
      // gradients of its own token shard, so no cross-rank reduction of dK/dV is needed.
      for (int r = q0 + warp; r < q1; r += WA_WARPS) {
        __nv_bfloat16* base = static_cast<__nv_bfloat16*>(a.dqkv[rowslot[r]]) + rowofs[r] * (3LL * a.C) + cg * G;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int m = gm[k];
          if (gok[k] && m < 3)
            *reinterpret_cast<uint4*>(base + m * a.C + gv[k] * 8) =
                *reinterpret_cast<const uint4*>((m == 0 ? dQs : (m == 1 ? Ks : Vs)) + r * stride + gv[k] * 8);
        }
      }
    }
  }
  if (bias_grad) {
    __syncthreads();
    for (int i = tid; i < hpc * geo.nrel; i += WA_THREADS) {
      const int h = i / geo.nrel, r = i % geo.nrel;
      atomicAdd(&a.dbias_table[r * a.num_heads + head0 + h], dbias_s[i]);
    }
  }
}

template <int HD, int NPAD, bool BWD>
size_t smem_bytes(int hpc, int nrel, int ww) {
  const int G = hpc * HD, stride = G + 8, pstride = NPAD + 8;
  size_t b = static_cast<size_t>(NPAD) * stride * 2 * (BWD ? 5 : 3);
  if (BWD) b += static_cast<size_t>(NPAD) * pstride * 2 * 2;
  b += static_cast<size_t>(hpc) * nrel * 4 * (BWD ? 2 : 1);
  b += 16;   // alignment slack before the row tables
  b += NPAD * (8 + 4 + 4 + 4);
  if (BWD) b += static_cast<size_t>(ww) * ww * 4 * (1 + WA_WARPS);
  return b;
}

template <int HD, int NPAD, bool BWD>
int launch(WindowAttnArgs a, cudaStream_t stream) {
  const int nrel = (2 * a.wh - 1) * (2 * a.ww - 1);
  // heads per CTA: 64 channels (128-byte row segments) keep the CTA small enough for several per SM
  int hpc = 64 / HD;
  if (hpc < 1) hpc = 1;
  while (hpc > 1 && (a.num_heads % hpc != 0 || smem_bytes<HD, NPAD, BWD>(hpc, nrel, a.ww) > 200 * 1024)) --hpc;
  const size_t sb = smem_bytes<HD, NPAD, BWD>(hpc, nrel, a.ww);
  if (sb > 227 * 1024) return -20;
  a.heads_per_cta = hpc;
  static size_t configured = 0;
  static int occupancy = 0;
  if (sb > configured) {
    if (cudaFuncSetAttribute(window_attn_kernel<HD, NPAD, BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sb)) != cudaSuccess)
      return -21;
    configured = sb;
    occupancy = 0;
  }
  if (occupancy == 0) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occupancy, window_attn_kernel<HD, NPAD, BWD>, WA_THREADS, sb) !=
            cudaSuccess || occupancy < 1)
      occupancy = 1;
  }
  const int my_nw = a.win_start[a.my_wg + 1] - a.win_start[a.my_wg];
  const int items = a.B * my_nw;
  if (items <= 0) return 0;
  const int groups = a.num_heads / hpc;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int gx = (sms * occupancy + groups - 1) / groups;
  if (gx > items) gx = items;
  dim3 grid(gx, groups);
  window_attn_kernel<HD, NPAD, BWD><<<grid, WA_THREADS, sb, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -22;
}

template <bool BWD>
int dispatch(const WindowAttnArgs& a, cudaStream_t stream) {
  const int N = a.wh * a.ww;
  if (a.num_heads <= 0 || a.C % a.num_heads != 0) return -10;
  const int hd = a.C / a.num_heads;
  if (N > 128) return -11;
  if (a.sp < 1 || a.shardN < 1 || a.n_wg < 1 || a.n_wg > 8 || a.n_wg * a.sp > WA_MAX_PEERS) return -12;
  const int npad = N <= 64 ? 64 : (N <= 96 ? 96 : 128);
#define TB_WA_CASE(HD_, NP_) \
  if (hd == HD_ && npad == NP_) return launch<HD_, NP_, BWD>(a, stream);
  TB_WA_CASE(16, 64) TB_WA_CASE(32, 64) TB_WA_CASE(64, 64) TB_WA_CASE(128, 64)
  TB_WA_CASE(16, 96) TB_WA_CASE(32, 96) TB_WA_CASE(64, 96) TB_WA_CASE(128, 96)
  TB_WA_CASE(16, 128) TB_WA_CASE(32, 128) TB_WA_CASE(64, 128) TB_WA_CASE(128, 128)
#undef TB_WA_CASE
  return -13;
}

}  // namespace

int window_attn_fwd(const WindowAttnArgs& a, cudaStream_t stream) { return dispatch<false>(a, stream); }
int window_attn_bwd(const WindowAttnArgs& a, cudaStream_t stream) { return dispatch<true>(a, stream); }

}  // namespace tb
