// Shared device-side helpers for the sm_100a kernels of terra_b200:
// mbarrier / TMA / tcgen05 PTX wrappers, bounded waits and the status word that
// kernels use to report a wait that ran out instead of hanging the GPU.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>

namespace tb {

// Error codes written to KernelStatus::error (0 = ok).
enum : unsigned int {
  TB_OK = 0,
  TB_ERR_MBAR_TIMEOUT = 1,   // an mbarrier wait inside a CTA ran out
  TB_ERR_PEER_TIMEOUT = 2,   // a wait on a flag written by another GPU ran out
  TB_ERR_BAD_ARG = 3,
  TB_ERR_BOUNDS = 4,         // TERRA_DEBUG_BOUNDS build: an index computed from a table or across ranks left its buffer
};

// One status record per launch family, in global memory. Kernels only ever write
// to it on failure (first writer wins), the host reads it after synchronising.
struct KernelStatus {
  unsigned int error;
  unsigned int where;   // role / site id
  unsigned int info0;   // e.g. stage or peer
  unsigned int info1;   // e.g. expected parity / epoch
};

__device__ __forceinline__ void report_error(KernelStatus* st, unsigned int code, unsigned int where,
                                             unsigned int i0, unsigned int i1) {
  if (st != nullptr && atomicCAS(&st->error, 0u, code) == 0u) {
    st->where = where;
    st->info0 = i0;
    st->info1 = i1;
  }
}

// Bounds-checked debug build (-DTERRA_DEBUG_BOUNDS, `TERRA_DEBUG_BOUNDS=1` for terra_b200/_ext.py): accesses whose
// index comes from a table or from cross-rank arithmetic (a token's home buffer and row, a relayout route) go through
// tb_index_ok first. A violation is recorded once in the status word {TB_ERR_BOUNDS, site, two words of the index}
// and the caller skips or redirects the access: nothing traps, the host raises from the status word after the step.
// In the normal build the check is a compile-time constant and disappears.
#ifdef TERRA_DEBUG_BOUNDS
constexpr bool TB_DEBUG_BOUNDS = true;
#else
constexpr bool TB_DEBUG_BOUNDS = false;
#endif
__device__ __forceinline__ bool tb_index_ok(bool ok, KernelStatus* st, unsigned int site, unsigned int i0, unsigned int i1) {
  if (!TB_DEBUG_BOUNDS || ok) return true;
  report_error(st, TB_ERR_BOUNDS, site, i0, i1);
  return false;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .b32 rx;\n"
      ".reg .pred px;\n"
      "elect.sync rx|px, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, px;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// ----------------------------------------------------------------------------- CTA pairs (cluster of two)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a shared-memory pointer of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t ld_shared_cluster_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
// Bounded wait. `abort_flag` lives in shared memory; once any role of the CTA gives up,
// every later wait of the CTA returns false at once so that all roles drain and the CTA
// reaches its teardown (TMEM release) instead of spinning for ever. The bound is a poll count (about a second of
// polling at TB_MBAR_SPIN_LIMIT: 64 ns of sleep per 256 polls plus the polls themselves) times `scale`. A kernel
// whose producer may itself wait for another GPU (bounded there by the global timer) passes a scale that makes the
// consumer roles outlast that wait, so that rank skew cannot abort a tile whose data would have arrived in time.
#ifndef TB_MBAR_SPIN_LIMIT
#define TB_MBAR_SPIN_LIMIT (1u << 24)
#endif
// CLUSTER marks waits on barriers that the other CTA of a pair (or its tensor core) signals. They use the same
// CTA-scope wait: a cluster-scope acquire on every poll costs about a microsecond per hand-over (measured).
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          KernelStatus* st, unsigned int where, uint32_t scale = 1u) {
  for (uint32_t round = 0; round < scale; ++round) {
    for (uint32_t i = 0; i < TB_MBAR_SPIN_LIMIT; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 255u) == 255u) {
        if (*abort_flag) return false;
        __nanosleep(64);
      }
    }
  }
  *abort_flag = 1;
  report_error(st, TB_ERR_MBAR_TIMEOUT, where, smem_u32(bar), parity);
  return false;
}

// ----------------------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------- TMA (no cluster fan-out: every CTA loads for itself)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, "
      "%7}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// Shared memory -> global memory through a tensor map (clipped at the tensor's bounds). The issuing thread owns the
// bulk group: it commits, and waits for the source to have been read before the buffer is written again.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src_smem, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(src_smem), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------- tcgen05 / TMEM
// CTAS = 1: the CTA works alone. CTAS = 2: the two CTAs of a cluster drive one MMA over both SMs (cta_group::2); the
// allocation calls are then made by one warp of each CTA.
template <int NCOLS, int CTAS = 1>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result) {
  if (CTAS == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(NCOLS)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(NCOLS)
                 : "memory");
}
template <int CTAS = 1>
__device__ __forceinline__ void tmem_relinquish() {
  if (CTAS == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int NCOLS, int CTAS = 1>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr) {
  if (CTAS == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS) : "memory");
  else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate. One thread issues (of the leader CTA when
// CTAS = 2: the descriptors then name the same shared-memory offsets in both CTAs, each holding its 128 rows of A and
// its half of B, and each CTA's tensor memory receives its 128 rows of D).
template <int CTAS = 1>
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  if (CTAS == 1)
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Makes `bar` complete once all previously issued tcgen05.mma of this thread are done. With CTAS = 2 the arrival is
// delivered to the barrier at the same shared-memory offset in both CTAs of the pair.
template <int CTAS = 1>
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  if (CTAS == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
  } else {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"(mask)
                 : "memory");
  }
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
//  K-major operand: rows of 64 bf16 (128 B), 8-row groups 1024 B apart (SBO); LBO unused.
//  MN-major operand: 8 K-rows of 64 MN elements (128 B each) form a 1024 B atom; atoms along
//  K are SBO apart, atoms along MN are LBO apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;   // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;   // 128-byte swizzle
  return d;
}

// K-major operand without swizzle: core matrices of 8 rows x 16 bytes (128 B, contiguous), LBO apart along K and SBO
// apart along the rows.
__device__ __forceinline__ uint64_t make_smem_desc_plain(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;   // descriptor version for sm_100
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 D.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// ----------------------------------------------------------------------------- small math
// GELU in its exact (erf) definition, evaluated as 0.5 x (1 + tanh(u(x))) with u(x) = x (c0 + c1 x^2 + c2 x^4):
// for this u, tanh(u(x)) reproduces erf(x / sqrt 2) closely enough that the GELU value differs from the erf form by at
// most 2.6e-5 and its derivative by at most 1.2e-4 (coefficients from a minimax fit on [-8, 8]; the argument of u is
// clamped there, where tanh has long saturated). One special-function instruction (tanh.approx) per element instead of
// the exponential + reciprocal of a rational erf, which matters where the GELU runs in a GEMM epilogue. The gradient
// is the derivative of the same expression, so forward and backward stay consistent.
constexpr float GELU_C0 = 0.7975052753853628f;
constexpr float GELU_C1 = 0.03700801999616438f;
constexpr float GELU_C2 = -0.000351902394432035f;
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
#ifdef TERRA_GELU_EXACT_ERF
// Build switch (TERRA_GELU_EXACT=1 for terra_b200/_ext.py): the erf form itself, 0.5 x (1 + erf(x / sqrt 2)), and its
// derivative Phi(x) + x phi(x), for runs that must not depend on the fit below (a few more instructions per element
// in the fc1 / d(fc2) epilogues).
__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
  const float pdf = 0.39894228040143268f * __expf(-0.5f * x * x);
  return fmaf(x, pdf, cdf);
}
#else
__device__ __forceinline__ float gelu_erf(float x) {
  const float xc = fminf(fmaxf(x, -8.0f), 8.0f);
  const float x2 = xc * xc;
  const float u = xc * fmaf(x2, fmaf(x2, GELU_C2, GELU_C1), GELU_C0);
  const float h = 0.5f * x;
  return fmaf(h, tanh_fast(u), h);
}
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float xc = fminf(fmaxf(x, -8.0f), 8.0f);
  const float x2 = xc * xc;
  const float t = tanh_fast(xc * fmaf(x2, fmaf(x2, GELU_C2, GELU_C1), GELU_C0));
  const float du = fmaf(x2, fmaf(x2, 5.0f * GELU_C2, 3.0f * GELU_C1), GELU_C0);
  const float sech2 = fmaf(-t, t, 1.0f);
  return fmaf(0.5f * xc * sech2, du, fmaf(0.5f, t, 0.5f));
}
#endif
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

}  // namespace tb
