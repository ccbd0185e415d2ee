// Memory-bound kernels: LayerNorm, GroupNorm(+SiLU), column sums, masked loss, fused AdamW.
// All are single-pass over HBM where the math allows it, with 16-byte vector accesses.
#include <cstdlib>
#include "common.cuh"
#include "host_api.h"

namespace tb {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 x = unpack_bf16x2(w[k]);
    f[2 * k] = x.x;
    f[2 * k + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// ------------------------------------------------------------------------------------------ LayerNorm
// One warp per row; the row lives in registers (VPL 16-byte vectors per lane).
template <int VPL>
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ gamma,
                                                            const __nv_bfloat16* __restrict__ beta,
                                                            __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                                                            float* __restrict__ rstd_out, long long rows, int C,
                                                            float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nvec = C >> 3;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
    float v[VPL][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        unpack8(xr[vi], v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
      }
    }
    const float mean = warp_sum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[i][j] - mean;
          q += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) / C + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + row * C);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float g[8], b[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(gamma)[vi], g);
        unpack8(reinterpret_cast<const uint4*>(beta)[vi], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j] + b[j];
        yr[vi] = pack8(o);
      }
    }
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
  }
}

template <int VPL>
__global__ void __launch_bounds__(256, (VPL <= 2) ? 2 : 1) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                            const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ gamma,
                                                            const float* __restrict__ mean, const float* __restrict__ rstd,
                                                            __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
                                                            float* __restrict__ dbeta, const __nv_bfloat16* __restrict__ dres,
                                                            long long rows, int C) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nvec = C >> 3;
  float ag[VPL][8], ab[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) ag[i][j] = ab[i][j] = 0.f;
  float g[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) unpack8(reinterpret_cast<const uint4*>(gamma)[vi], g[i]);
  }
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + row * C);
    const float mu = mean[row], rs = rstd[row];
    // all of the row's loads (x, dy and the residual-path gradient) are issued before the first use
    uint4 xq[VPL], dq[VPL], rq[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        xq[i] = xr[vi];
        dq[i] = dr[vi];
        if (dres != nullptr) rq[i] = reinterpret_cast<const uint4*>(dres + row * C)[vi];
      }
    }
    float xh[VPL][8], dv[VPL][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float xv[8], dyv[8];
        unpack8(xq[i], xv);
        unpack8(dq[i], dyv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mu) * rs;
          ag[i][j] += dyv[j] * xh[i][j];
          ab[i][j] += dyv[j];
          dv[i][j] = dyv[j] * g[i][j];
          s1 += dv[i][j];
          s2 += dv[i][j] * xh[i][j];
        }
      }
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
    uint4* or_ = reinterpret_cast<uint4*>(dx + row * C);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (dv[i][j] - s1 - xh[i][j] * s2);
        if (dres != nullptr) {
          float rr[8];
          unpack8(rq[i], rr);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rr[j];
        }
        or_[vi] = pack8(o);
      }
    }
  }
  // reduce the per-lane column partials across the block's warps through shared memory, then one atomic per column
  extern __shared__ float sh[];   // [2][C]
  for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) sh[c] = 0.f;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(&sh[vi * 8 + j], ag[i][j]);
        atomicAdd(&sh[C + vi * 8 + j], ab[i][j]);
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    atomicAdd(&dgamma[c], sh[c]);
    atomicAdd(&dbeta[c], sh[C + c]);
  }
}

// ------------------------------------------------------------------------------------------ column sums
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ partials,
                                                     long long rows, int C, long long ld, int rows_per_block) {
  // thread -> one 8-wide column vector; blockDim.y rows in flight. blockDim.x spans the whole row when it has at most
  // 64 vectors (a row is then one contiguous read), otherwise 32 vectors per block column.
  const int nvec = C >> 3;
  const int vi = blockIdx.y * blockDim.x + threadIdx.x;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const long long r0 = static_cast<long long>(blockIdx.x) * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  if (vi < nvec) {
    // four independent 16-byte loads in flight per thread
    const long long step = blockDim.y;
    long long r = r0 + threadIdx.y;
    for (; r + 3 * step < r1; r += 4 * step) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = *reinterpret_cast<const uint4*>(x + (r + u * step) * ld + vi * 8);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        unpack8(q[u], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
    for (; r < r1; r += step) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(x + r * ld + vi * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
  extern __shared__ float csh[];              // [blockDim.y][blockDim.x * 8 + 1]
  const int pitch = blockDim.x * 8 + 1;
#pragma unroll
  for (int j = 0; j < 8; ++j) csh[threadIdx.y * pitch + threadIdx.x * 8 + j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && vi < nvec) {
    // one partial row per row block: many blocks adding into the same few hundred addresses serialise in L2
    // (about 80 ns per atomic on one address), so the partials are written out and a second kernel adds them up
    float* prow = partials + static_cast<long long>(blockIdx.x) * C;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
      for (int y = 0; y < blockDim.y; ++y) s += csh[y * pitch + threadIdx.x * 8 + j];
      prow[vi * 8 + j] = s;
    }
  }
}

// out[c] += sum over r of partials[r][c]. Block = 32 columns x 32 row lanes.
__global__ void __launch_bounds__(1024) colsum_finish_kernel(const float* __restrict__ partials, float* __restrict__ out,
                                                             int nparts, int C) {
  __shared__ float sh[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < C)
    for (int r = threadIdx.y; r < nparts; r += 32) s += partials[static_cast<long long>(r) * C + c];
  sh[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += sh[y][threadIdx.x];
    out[c] += t;
  }
}

// ------------------------------------------------------------------------------------------ GroupNorm
// x: [B, HW, C] bf16. Block = (C/8 column vectors) x (rows in flight); per-channel partials in shared memory,
// folded to groups, two atomics per (block, group).
__global__ void __launch_bounds__(512) groupnorm_stats_kernel(const __nv_bfloat16* __restrict__ x,
                                                              float* __restrict__ sums, long long HW, int C, int groups,
                                                              int pix_per_block) {
  extern __shared__ float sh[];  // [2][C]
  const int nvec = C >> 3;
  const int b = blockIdx.y;
  for (int c = threadIdx.y * blockDim.x + threadIdx.x; c < 2 * C; c += blockDim.x * blockDim.y) sh[c] = 0.f;
  __syncthreads();
  const long long p0 = static_cast<long long>(blockIdx.x) * pix_per_block;
  const long long p1 = min(HW, p0 + pix_per_block);
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0}, q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long p = p0 + threadIdx.y; p < p1; p += blockDim.y) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(x + (static_cast<long long>(b) * HW + p) * C + vi * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j] += f[j];
        q[j] += f[j] * f[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(&sh[vi * 8 + j], s[j]);
      atomicAdd(&sh[C + vi * 8 + j], q[j]);
    }
  }
  __syncthreads();
  const int cpg = C / groups;
  for (int g = threadIdx.y * blockDim.x + threadIdx.x; g < groups; g += blockDim.x * blockDim.y) {
    float s = 0.f, q = 0.f;
    for (int c = g * cpg; c < (g + 1) * cpg; ++c) {
      s += sh[c];
      q += sh[C + c];
    }
    atomicAdd(&sums[(b * groups + g) * 2 + 0], s);
    atomicAdd(&sums[(b * groups + g) * 2 + 1], q);
  }
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + __expf(-z)); }

__global__ void __launch_bounds__(256) groupnorm_silu_apply_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   const float* __restrict__ stats,
                                                                   const __nv_bfloat16* __restrict__ gamma,
                                                                   const __nv_bfloat16* __restrict__ beta,
                                                                   const __nv_bfloat16* __restrict__ res,
                                                                   __nv_bfloat16* __restrict__ y, long long HW, int C,
                                                                   int groups, long long total_vec) {
  const int nvec = C >> 3;
  const int cpg = C / groups;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vi = static_cast<int>(i % nvec);
    const long long pix = i / nvec;
    const int b = static_cast<int>(pix / HW);
    float f[8], g[8], bt[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], f);
    unpack8(reinterpret_cast<const uint4*>(gamma)[vi], g);
    unpack8(reinterpret_cast<const uint4*>(beta)[vi], bt);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int grp = (vi * 8 + j) / cpg;
      const float mu = stats[(b * groups + grp) * 2], rs = stats[(b * groups + grp) * 2 + 1];
      const float z = (f[j] - mu) * rs * g[j] + bt[j];
      o[j] = z * sigmoidf_(z);
    }
    if (res != nullptr) {
      float rr[8];
      unpack8(reinterpret_cast<const uint4*>(res)[i], rr);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += rr[j];
    }
    reinterpret_cast<uint4*>(y)[i] = pack8(o);
  }
}

// pass 1 of the backward: red[b][c] = {sum dz, sum dz * xhat}
__global__ void __launch_bounds__(512) groupnorm_silu_bwd_reduce_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ stats,
    const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta, float* __restrict__ red,
    long long HW, int C, int groups, int pix_per_block, float* __restrict__ dgamma, float* __restrict__ dbeta) {
  extern __shared__ float sh[];  // [2][C]
  const int nvec = C >> 3;
  const int cpg = C / groups;
  const int b = blockIdx.y;
  for (int c = threadIdx.y * blockDim.x + threadIdx.x; c < 2 * C; c += blockDim.x * blockDim.y) sh[c] = 0.f;
  __syncthreads();
  const long long p0 = static_cast<long long>(blockIdx.x) * pix_per_block;
  const long long p1 = min(HW, p0 + pix_per_block);
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    float g[8], bt[8], mu[8], rs[8];
    unpack8(reinterpret_cast<const uint4*>(gamma)[vi], g);
    unpack8(reinterpret_cast<const uint4*>(beta)[vi], bt);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int grp = (vi * 8 + j) / cpg;
      mu[j] = stats[(b * groups + grp) * 2];
      rs[j] = stats[(b * groups + grp) * 2 + 1];
    }
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0}, q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long p = p0 + threadIdx.y; p < p1; p += blockDim.y) {
      const long long off = (static_cast<long long>(b) * HW + p) * C + vi * 8;
      float f[8], d[8];
      unpack8(*reinterpret_cast<const uint4*>(x + off), f);
      unpack8(*reinterpret_cast<const uint4*>(dy + off), d);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (f[j] - mu[j]) * rs[j];
        const float z = xh * g[j] + bt[j];
        const float sg = sigmoidf_(z);
        const float dz = d[j] * sg * (1.f + z * (1.f - sg));
        s[j] += dz;
        q[j] += dz * xh;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(&sh[vi * 8 + j], s[j]);
      atomicAdd(&sh[C + vi * 8 + j], q[j]);
    }
  }
  __syncthreads();
  for (int c = threadIdx.y * blockDim.x + threadIdx.x; c < C; c += blockDim.x * blockDim.y) {
    atomicAdd(&red[(static_cast<long long>(b) * C + c) * 2 + 0], sh[c]);
    atomicAdd(&red[(static_cast<long long>(b) * C + c) * 2 + 1], sh[C + c]);
    // the affine parameters' gradients are the same sums taken over the batch as well
    if (dbeta != nullptr) atomicAdd(&dbeta[c], sh[c]);
    if (dgamma != nullptr) atomicAdd(&dgamma[c], sh[C + c]);
  }
}

// {sum, sum of squares} per (sample, group) -> {mean, rstd}; the sums are cleared for their next use
__global__ void groupnorm_finalize_kernel(float* __restrict__ sums, float* __restrict__ stats, int cells, float inv_count,
                                          float eps, int clear) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cells) {
    const float mean = sums[2 * i] * inv_count;
    const float var = fmaxf(sums[2 * i + 1] * inv_count - mean * mean, 0.f);
    stats[2 * i] = mean;
    stats[2 * i + 1] = rsqrtf(var + eps);
    if (clear) {
      sums[2 * i] = 0.f;
      sums[2 * i + 1] = 0.f;
    }
  }
}

// dst[a * sa + b * sb + c * sc] += src[(a * nb + b) * nc + c] (fp32); with `clear` the source is zeroed behind the read,
// so that a persistent staging buffer is clean for its next accumulation. Used to fold tap-major convolution weight
// gradients into the (Cout, Cin, kh, kw) layout of the gradient arena.
__global__ void __launch_bounds__(256) strided_add_kernel(float* __restrict__ src, float* __restrict__ dst, int na, int nb,
                                                          int nc, long long sa, long long sb, long long sc, int clear) {
  const long long total = static_cast<long long>(na) * nb * nc;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % nc);
    const long long t = i / nc;
    const int b = static_cast<int>(t % nb), a2 = static_cast<int>(t / nb);
    const float v = src[i];
    dst[a2 * sa + b * sb + c * sc] += v;
    if (clear) src[i] = 0.f;
  }
}

// pass 2: dx = rstd * (dz*gamma - s1/n - xhat * s2/n), s1 = sum_c gamma_c red[b][c][0], s2 likewise with [1]
__global__ void __launch_bounds__(256) groupnorm_silu_bwd_apply_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ stats,
    const float* __restrict__ red, const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
    __nv_bfloat16* __restrict__ dx, int B, long long HW, int C, int groups, float inv_count, long long total_vec) {
  extern __shared__ float gs[];  // [B][groups][2]
  const int cpg = C / groups;
  for (int i = threadIdx.x; i < B * groups; i += blockDim.x) {
    const int b = i / groups, g = i % groups;
    float s1 = 0.f, s2 = 0.f;
    for (int c = g * cpg; c < (g + 1) * cpg; ++c) {
      const float gm = __bfloat162float(gamma[c]);
      s1 += gm * red[(static_cast<long long>(b) * C + c) * 2];
      s2 += gm * red[(static_cast<long long>(b) * C + c) * 2 + 1];
    }
    gs[i * 2] = s1 * inv_count;
    gs[i * 2 + 1] = s2 * inv_count;
  }
  __syncthreads();
  const int nvec = C >> 3;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vi = static_cast<int>(i % nvec);
    const long long pix = i / nvec;
    const int b = static_cast<int>(pix / HW);
    float f[8], d[8], g[8], bt[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], f);
    unpack8(reinterpret_cast<const uint4*>(dy)[i], d);
    unpack8(reinterpret_cast<const uint4*>(gamma)[vi], g);
    unpack8(reinterpret_cast<const uint4*>(beta)[vi], bt);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int grp = (vi * 8 + j) / cpg;
      const float mu = stats[(b * groups + grp) * 2], rs = stats[(b * groups + grp) * 2 + 1];
      const float xh = (f[j] - mu) * rs;
      const float z = xh * g[j] + bt[j];
      const float sg = sigmoidf_(z);
      const float dz = d[j] * sg * (1.f + z * (1.f - sg));
      o[j] = rs * (dz * g[j] - gs[(b * groups + grp) * 2] - xh * gs[(b * groups + grp) * 2 + 1]);
    }
    reinterpret_cast<uint4*>(dx)[i] = pack8(o);
  }
}

// ------------------------------------------------------------------------------------------ masked loss
__global__ void __launch_bounds__(256) masked_loss_kernel(const __nv_bfloat16* __restrict__ pred,
                                                          const __nv_bfloat16* __restrict__ label,
                                                          const __nv_bfloat16* __restrict__ mask, long long nvec,
                                                          long long mask_period_vec, int kind, float grad_scale,
                                                          float* __restrict__ loss_sum, __nv_bfloat16* __restrict__ grad) {
  float acc = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p[8], l[8], m[8], g[8];
    unpack8(reinterpret_cast<const uint4*>(pred)[i], p);
    unpack8(reinterpret_cast<const uint4*>(label)[i], l);
    if (mask != nullptr) {
      unpack8(reinterpret_cast<const uint4*>(mask)[i % mask_period_vec], m);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) m[j] = 1.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float d = p[j] * m[j] - l[j];
      if (kind == 0) {
        acc += fabsf(d);
        g[j] = (d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f)) * m[j] * grad_scale;
      } else {
        acc += d * d;
        g[j] = 2.f * d * m[j] * grad_scale;
      }
    }
    if (grad != nullptr) reinterpret_cast<uint4*>(grad)[i] = pack8(g);
  }
  acc = warp_sum(acc);
  __shared__ float sh[8];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) s += sh[w];
    atomicAdd(loss_sum, s);
  }
}

// ------------------------------------------------------------------------------------------ attention row dots
// drow[row, head] = sum over the head's channels of dO * O: the "D" term of the attention backward pass. A warp per row;
// lanes stride over the row's 16-byte vectors, then the lanes of one head are summed.
__global__ void __launch_bounds__(256) attn_rowdot_kernel(const uint4* __restrict__ o, const uint4* __restrict__ dout,
                                                          float* __restrict__ drow, long long rows, int vec_per_row,
                                                          int vec_per_head, int heads) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    for (int v0 = 0; v0 < vec_per_row; v0 += 32) {
      const int v = v0 + lane;
      float acc = 0.f;
      if (v < vec_per_row) {
        float x[8], y[8];
        unpack8(o[r * vec_per_row + v], x);
        unpack8(dout[r * vec_per_row + v], y);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(x[j], y[j], acc);
      }
      // vec_per_head is 2, 4, 8 or 16 (head dims 16 .. 128): sum groups of that many neighbouring lanes
      for (int d = 1; d < vec_per_head && d < 32; d <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
      if (v < vec_per_row && (v % vec_per_head) == 0) drow[r * heads + v / vec_per_head] = acc;
    }
  }
}

// ------------------------------------------------------------------------------------------ gradient inspection
// One pass over a flat fp32 gradient buffer for the loss-scaling path: out[0] += sum of squares (for the clipping
// norm), out[1] becomes non-zero when any element is inf or nan (the step is then skipped and the scale backed off).
__global__ void __launch_bounds__(256) grad_inspect_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  float acc = 0.f;
  bool bad = false;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = g[i];
    bad |= !(fabsf(v) <= 3.0e38f);     // false for inf and for nan
    acc = fmaf(v, v, acc);
  }
  acc = warp_sum(acc);
  const unsigned int any_bad = __ballot_sync(0xffffffffu, bad);
  __shared__ float sh[8];
  __shared__ unsigned int shb[8];
  if ((threadIdx.x & 31) == 0) {
    sh[threadIdx.x >> 5] = acc;
    shb[threadIdx.x >> 5] = any_bad;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    unsigned int b = 0u;
    for (int w = 0; w < (blockDim.x >> 5); ++w) {
      s += sh[w];
      b |= shb[w];
    }
    if (b == 0u) atomicAdd(out, s);           // a poisoned sum would only hide the flag's meaning
    else out[1] = 1.f;
  }
}

// ------------------------------------------------------------------------------------------ AdamW
template <bool GRAD_BF16>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ master, float* __restrict__ m,
                                                    float* __restrict__ v, const void* __restrict__ grad,
                                                    __nv_bfloat16* __restrict__ param, long long n, float lr, float b1,
                                                    float b2, float eps, float wd, float bc1, float bc2s,
                                                    float gscale) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g = GRAD_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(grad)[i])
                        : static_cast<const float*>(grad)[i];
    g *= gscale;
    float p = master[i];
    p *= 1.f - lr * wd;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    const float denom = sqrtf(vi) / bc2s + eps;
    p -= (lr / bc1) * (mi / denom);
    m[i] = mi;
    v[i] = vi;
    master[i] = p;
    if (param != nullptr) param[i] = __float2bfloat16(p);
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    d[i] = __float2bfloat16(s[i]);
}

__global__ void add_bf16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ o,
                                long long nvec) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    unpack8(a[i], x);
    unpack8(b[i], y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    o[i] = pack8(x);
  }
}

// Input gradient of the 3x3 stride-2 convolution from its per-tap columns: dcol[b, ho, wo, tap, c] (tap = ky * 3 + kx)
// is the contribution of output pixel (ho, wo) to padded input pixel (2 ho + ky, 2 wo + kx). Every padded input pixel
// gathers its (at most four) contributions; the result is written for padded rows [r0, r0 + rows) and padded columns
// [1, W + 1) as fp32 (F32: with the halo rows, for the multi-rank fold) or bf16.
template <bool F32>
__global__ void conv_s2_col2im_kernel(const uint4* __restrict__ dcol, void* __restrict__ out, int B, int Ho, int Wo, int W,
                                      int cvec, int r0, int rows) {
  const long long total = static_cast<long long>(B) * rows * W * cvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cv = static_cast<int>(i % cvec);
    long long t = i / cvec;
    const int w = static_cast<int>(t % W);
    t /= W;
    const int r = static_cast<int>(t % rows);
    const int b = static_cast<int>(t / rows);
    const int ph = r0 + r, pw = w + 1;                     // padded coordinates
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // ky in {ph & 1, (ph & 1) + 2 if even}: ph = 2 ho + ky
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int ky = (ph & 1) + 2 * a;
      if (ky > 2) continue;
      const int ho = (ph - ky) >> 1;
      if (ph - ky < 0 || ho >= Ho) continue;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int kx = (pw & 1) + 2 * c;
        if (kx > 2) continue;
        const int wo = (pw - kx) >> 1;
        if (pw - kx < 0 || wo >= Wo) continue;
        float f[8];
        unpack8(dcol[((static_cast<long long>(b) * Ho + ho) * Wo + wo) * 9 * cvec + (ky * 3 + kx) * cvec + cv], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
    if (F32) {
      float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + i * 8);
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      reinterpret_cast<uint4*>(out)[i] = pack8(acc);
    }
  }
}

// out = sum over `slots` consecutive bf16 buffers of `nvec` 16-byte vectors each (fp32 accumulation), optionally
// + bias[col] (bf16, `cvec` vectors per row) + residual (bf16, same shape as out): the owner's side of the slot-staged
// reduce-scatter with the row-parallel layer's bias and the block's shortcut folded in.
__global__ void sum_slots_bf16_kernel(const uint4* __restrict__ src, uint4* __restrict__ o, int slots, long long nvec,
                                      const uint4* __restrict__ bias, const uint4* __restrict__ res, int cvec) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
    unpack8(src[i], acc);
    for (int s = 1; s < slots; ++s) {
      float y[8];
      unpack8(src[i + s * nvec], y);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += y[j];
    }
    if (bias != nullptr) {
      float y[8];
      unpack8(bias[i % cvec], y);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += y[j];
    }
    if (res != nullptr) {
      float y[8];
      unpack8(res[i], y);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += y[j];
    }
    o[i] = pack8(acc);
  }
}

int grid_for(long long work_items, int block, int max_blocks = 148 * 16) {
  long long g = (work_items + block - 1) / block;
  if (g > max_blocks) g = max_blocks;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace

#define TB_LN_DISPATCH(VPL_EXPR, CALL)                      \
  switch (VPL_EXPR) {                                       \
    case 1: { constexpr int VPL = 1; CALL; break; }         \
    case 2: { constexpr int VPL = 2; CALL; break; }         \
    case 3: { constexpr int VPL = 3; CALL; break; }         \
    case 4: { constexpr int VPL = 4; CALL; break; }         \
    case 5: case 6: { constexpr int VPL = 6; CALL; break; } \
    case 7: case 8: { constexpr int VPL = 8; CALL; break; } \
    default: return -1;                                     \
  }

int layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                  long long rows, int C, float eps, cudaStream_t stream) {
  if (C % 8 != 0 || C > 2048) return -1;
  const int vpl = (C / 8 + 31) / 32;
  const int grid = grid_for(rows, 8);
  TB_LN_DISPATCH(vpl, (layernorm_fwd_kernel<VPL><<<grid, 256, 0, stream>>>(
                          static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),
                          static_cast<const __nv_bfloat16*>(beta), static_cast<__nv_bfloat16*>(y), mean, rstd, rows, C,
                          eps)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                  float* dgamma, float* dbeta, const void* dres, long long rows, int C, cudaStream_t stream) {
  if (C % 8 != 0 || C > 2048) return -1;
  const int vpl = (C / 8 + 31) / 32;
  const int grid = grid_for(rows, 8, 148 * 4);
  const size_t sh = 2 * C * sizeof(float);
  TB_LN_DISPATCH(vpl, (layernorm_bwd_kernel<VPL><<<grid, 256, sh, stream>>>(
                          static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                          static_cast<const __nv_bfloat16*>(gamma), mean, rstd, static_cast<__nv_bfloat16*>(dx), dgamma,
                          dbeta, static_cast<const __nv_bfloat16*>(dres), rows, C)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int colsum_rows_per_block() { return 256; }

// out[c] += sum over rows of x[r][c]. `partials`: fp32 scratch of ceil(rows / colsum_rows_per_block()) x C elements.
int colsum_bf16(const void* x, float* out, float* partials, long long rows, int C, long long ld, cudaStream_t stream) {
  if (C % 8 != 0 || partials == nullptr) return -1;
  const int nvec = C / 8;
  const int bx = nvec <= 64 ? nvec : 32;
  const int by = 256 / bx > 0 ? 256 / bx : 1;
  dim3 block(bx, by);
  const int rows_per_block = colsum_rows_per_block();
  const int nparts = static_cast<int>((rows + rows_per_block - 1) / rows_per_block);
  dim3 grid(static_cast<unsigned>(nparts), (nvec + bx - 1) / bx);
  const size_t sh = static_cast<size_t>(by) * (bx * 8 + 1) * sizeof(float);
  colsum_kernel<<<grid, block, sh, stream>>>(static_cast<const __nv_bfloat16*>(x), partials, rows, C, ld, rows_per_block);
  colsum_finish_kernel<<<(C + 31) / 32, dim3(32, 32), 0, stream>>>(partials, out, nparts, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int groupnorm_stats(const void* x, float* sums, int B, long long HW, int C, int groups, cudaStream_t stream) {
  if (C % 8 != 0 || C % groups != 0) return -1;
  const int nvec = C / 8;
  const int bx = nvec < 64 ? nvec : 64;
  dim3 block(bx, 512 / bx > 0 ? 512 / bx : 1);
  const int pix_per_block = 1024;
  dim3 grid(static_cast<unsigned>((HW + pix_per_block - 1) / pix_per_block), B);
  groupnorm_stats_kernel<<<grid, block, 2 * C * sizeof(float), stream>>>(static_cast<const __nv_bfloat16*>(x), sums, HW,
                                                                         C, groups, pix_per_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int groupnorm_silu_apply(const void* x, const float* stats, const void* gamma, const void* beta, const void* res, void* y,
                         int B, long long HW, int C, int groups, cudaStream_t stream) {
  if (C % 8 != 0 || C % groups != 0) return -1;
  const long long total_vec = static_cast<long long>(B) * HW * (C / 8);
  groupnorm_silu_apply_kernel<<<grid_for(total_vec, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), stats, static_cast<const __nv_bfloat16*>(gamma),
      static_cast<const __nv_bfloat16*>(beta), static_cast<const __nv_bfloat16*>(res), static_cast<__nv_bfloat16*>(y), HW,
      C, groups, total_vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int groupnorm_silu_bwd_reduce(const void* dy, const void* x, const float* stats, const void* gamma, const void* beta,
                              float* red, float* dgamma, float* dbeta, int B, long long HW, int C, int groups,
                              cudaStream_t stream) {
  if (C % 8 != 0 || C % groups != 0) return -1;
  const int nvec = C / 8;
  const int bx = nvec < 64 ? nvec : 64;
  dim3 block(bx, 512 / bx > 0 ? 512 / bx : 1);
  const int pix_per_block = 1024;
  dim3 grid(static_cast<unsigned>((HW + pix_per_block - 1) / pix_per_block), B);
  groupnorm_silu_bwd_reduce_kernel<<<grid, block, 2 * C * sizeof(float), stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), stats,
      static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta), red, HW, C, groups,
      pix_per_block, dgamma, dbeta);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int groupnorm_finalize(float* sums, float* stats, int cells, float inv_count, float eps, int clear, cudaStream_t stream) {
  if (cells <= 0) return 0;
  groupnorm_finalize_kernel<<<(cells + 255) / 256, 256, 0, stream>>>(sums, stats, cells, inv_count, eps, clear);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int strided_add_f32(float* src, float* dst, int na, int nb, int nc, long long sa, long long sb, long long sc, int clear,
                    cudaStream_t stream) {
  const long long total = static_cast<long long>(na) * nb * nc;
  if (total <= 0) return 0;
  strided_add_kernel<<<grid_for(total, 256), 256, 0, stream>>>(src, dst, na, nb, nc, sa, sb, sc, clear);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int groupnorm_silu_bwd_apply(const void* dy, const void* x, const float* stats, const float* red, const void* gamma,
                             const void* beta, void* dx, int B, long long HW, int C, int groups, float inv_count,
                             cudaStream_t stream) {
  if (C % 8 != 0 || C % groups != 0) return -1;
  const long long total_vec = static_cast<long long>(B) * HW * (C / 8);
  groupnorm_silu_bwd_apply_kernel<<<grid_for(total_vec, 256), 256, B * groups * 2 * sizeof(float), stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), stats, red,
      static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta),
      static_cast<__nv_bfloat16*>(dx), B, HW, C, groups, inv_count, total_vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int masked_loss_fwd_bwd(const void* pred, const void* label, const void* mask, long long n, long long mask_period,
                        int kind, float grad_scale, float* loss_sum, void* grad, cudaStream_t stream) {
  if (n % 8 != 0 || (mask != nullptr && mask_period % 8 != 0)) return -1;
  const long long nvec = n / 8;
  masked_loss_kernel<<<grid_for(nvec, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(pred), static_cast<const __nv_bfloat16*>(label),
      static_cast<const __nv_bfloat16*>(mask), nvec, mask != nullptr ? mask_period / 8 : 1, kind, grad_scale, loss_sum,
      static_cast<__nv_bfloat16*>(grad));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int adamw_step(float* master, float* exp_avg, float* exp_avg_sq, const void* grad, int grad_is_bf16, void* param_bf16,
               long long n, float lr, float beta1, float beta2, float eps, float weight_decay, float bias_corr1,
               float bias_corr2_sqrt, float grad_scale, cudaStream_t stream) {
  const int grid = grid_for(n, 256);
  if (grad_is_bf16)
    adamw_kernel<true><<<grid, 256, 0, stream>>>(master, exp_avg, exp_avg_sq, grad,
                                                 static_cast<__nv_bfloat16*>(param_bf16), n, lr, beta1, beta2, eps,
                                                 weight_decay, bias_corr1, bias_corr2_sqrt, grad_scale);
  else
    adamw_kernel<false><<<grid, 256, 0, stream>>>(master, exp_avg, exp_avg_sq, grad,
                                                  static_cast<__nv_bfloat16*>(param_bf16), n, lr, beta1, beta2, eps,
                                                  weight_decay, bias_corr1, bias_corr2_sqrt, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int cast_f32_to_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  cast_f32_bf16_kernel<<<grid_for(n, 256), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  if (n % 8 != 0) return -1;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(static_cast<const uint4*>(a), static_cast<const uint4*>(b),
                                                            static_cast<uint4*>(out), n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int conv_s2_col2im(const void* dcol, void* out, int B, int Ho, int Wo, int W, int C, int r0, int rows, int out_f32,
                   cudaStream_t stream) {
  if (C % 8 != 0 || rows <= 0) return -1;
  const long long total = static_cast<long long>(B) * rows * W * (C / 8);
  if (out_f32)
    conv_s2_col2im_kernel<true><<<grid_for(total, 256), 256, 0, stream>>>(static_cast<const uint4*>(dcol), out, B, Ho, Wo, W,
                                                                          C / 8, r0, rows);
  else
    conv_s2_col2im_kernel<false><<<grid_for(total, 256), 256, 0, stream>>>(static_cast<const uint4*>(dcol), out, B, Ho, Wo, W,
                                                                           C / 8, r0, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int attn_rowdot(const void* o, const void* dout, float* drow, long long rows, int C, int heads, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || C % heads != 0) return -1;
  const int hd = C / heads;
  if (hd != 16 && hd != 32 && hd != 64 && hd != 128) return -1;
  attn_rowdot_kernel<<<grid_for(rows * 32, 256), 256, 0, stream>>>(static_cast<const uint4*>(o), static_cast<const uint4*>(dout),
                                                                  drow, rows, C / 8, hd / 8, heads);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int grad_inspect(const float* grad, long long n, float* out2, cudaStream_t stream) {
  if (n <= 0) return 0;
  grad_inspect_kernel<<<grid_for(n, 256 * 8, 148 * 8), 256, 0, stream>>>(grad, n, out2);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sum_slots_bf16(const void* src, void* out, int slots, long long n, cudaStream_t stream, const void* bias,
                   const void* residual, int cols) {
  if (n % 8 != 0 || slots < 1) return -1;
  if (bias != nullptr && (cols <= 0 || cols % 8 != 0 || n % cols != 0)) return -1;
  sum_slots_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(out),
                                                                  slots, n / 8, static_cast<const uint4*>(bias),
                                                                  static_cast<const uint4*>(residual), cols > 0 ? cols / 8 : 1);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace tb
