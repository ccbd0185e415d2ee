// Window attention, forward, on the 5th-generation tensor cores (tcgen05 / TMEM), for any window size.
//
// Same contract as window_attn.cu (window-major activations, shifted windows / halos / token shards located by index
// arithmetic, rows of other GPUs read and written through peer pointers), different engine:
//
//   * a tile is 128 query rows x one group of heads (64 channels, or one head of 128). Small windows (N <= 64 tokens)
//     are packed two to a tile (rows 0-63 / 64-127), each half attending to its own 64-key slot; larger windows are cut
//     into blocks of 128 queries that stream the window's keys and values in slots of 64 (flash-style, online softmax);
//   * two producer warps gather Q / K / V rows (local or peer memory, plain 16-byte asynchronous copies) into
//     128-byte-swizzled shared-memory tiles, two Q tiles and a ring of K/V slots ahead of the math;
//   * one warp (one elected lane) issues tcgen05.mma: S = Q K^T (M = 128, N = 64 per slot, K = head dim) into one of two
//     score buffers in tensor memory, and O_step = P V (M = 128, N = head dim, K = keys of the slots) into one of two
//     output buffers;
//   * four warps own one query row each (row = TMEM lane): tcgen05.ld the scores, add the relative-position bias (table
//     in shared memory) and the shifted-window mask (region ids), exponentiate in base 2, write the probabilities
//     (bf16, unnormalised) back to shared memory as the A operand of P V, fold each step's O into fp32 accumulators with
//     the online-softmax rescaling, normalise at the end and store the row to its home (possibly on a peer).
//
// The MMA thread runs one S product ahead of the softmax warps; score, probability and output buffers alternate by
// step parity, and "probabilities written" doubles as "scores and previous output consumed", so three barrier pairs
// carry the whole hand-over. Every wait is bounded; on expiry the CTA sets its abort flag, reports through the status
// word, drains and releases its tensor memory.
#include "common.cuh"
#include "host_api.h"
#include "window_geo.cuh"

namespace tb {
namespace {

constexpr int TC_PROD = 2;                              // producer warps
constexpr int TC_MMA_WARP = TC_PROD;                    // the warp that owns tensor memory and issues the products
constexpr int TC_THREADS = 32 * (TC_PROD + 1 + 4);      // + four softmax warps
constexpr int TC_ROWS = 128;
constexpr int TC_KV = 64;
constexpr float TC_LOG2E = 1.4426950408889634f;
constexpr float TC_NEG = -1.0e30f;

template <int HD>
struct TcCfg {
  static constexpr int G = HD < 64 ? 64 : HD;            // channels of a head group
  static constexpr int NSUB = G / 64;                    // 64-channel sub-tiles per row
  static constexpr int HPG = G / HD;                     // heads per group
  static constexpr int Q_BYTES = TC_ROWS * 128 * NSUB;
  static constexpr int KV_BYTES = TC_KV * 128 * NSUB;    // K (or V) of one slot
  static constexpr int SLOT_BYTES = 2 * KV_BYTES;
  static constexpr int NSLOT = NSUB == 1 ? 4 : 2;
  static constexpr int P_TILE = TC_ROWS * 128;           // [128 rows][64 keys] bf16
  static constexpr int P_BYTES = 2 * P_TILE;             // two key blocks (pair mode) per buffer
  static constexpr int TILE_BYTES = 2 * Q_BYTES + NSLOT * SLOT_BYTES + 2 * P_BYTES;
  static constexpr int TMEM_COLS = 512;                  // 2 x 128 score columns + 2 x HD output columns
  static constexpr int O_COL = 256;
};

struct TcBars {
  uint64_t q_full[2], q_empty[2];
  uint64_t kv_full[4], kv_empty[4];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint64_t rows_sync;   // barrier among the 128 softmax threads (bounded, unlike bar.sync)
};

// Work item -> what every role needs to know about it.
struct TcItem {
  int b, hg, w0, nwin, qb, nkv, T;
};

struct TcPlan {
  int pair;        // 1: two windows of <= 64 tokens per tile; 0: 128-query blocks of one window
  int my_nw, q0, q1, nqb, tiles_per_b, hgroups, items, N;
};

template <int HPG>
__device__ __forceinline__ TcItem tc_decode(const TcPlan& pl, int item) {
  TcItem it;
  // head group slowest: a CTA's consecutive items mostly share it, so the bias table in shared memory is rarely reloaded
  const int per_hg = pl.items / pl.hgroups;
  it.hg = item / per_hg;
  const int t = item % per_hg;
  it.b = t / pl.tiles_per_b;
  const int tile = t % pl.tiles_per_b;
  if (pl.pair) {
    it.w0 = 2 * tile;
    it.nwin = min(2, pl.my_nw - it.w0);
    it.qb = 0;
    it.nkv = 1;
  } else {
    it.w0 = tile / pl.nqb;
    it.qb = tile % pl.nqb;
    it.nwin = 1;
    it.nkv = (pl.N + TC_KV - 1) / TC_KV;
  }
  it.T = it.nkv * HPG;
  return it;
}

__device__ __forceinline__ void tc_cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tc_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Explicit shared-memory loads by 32-bit address: through a generic pointer the compiler emits generic loads, which wait
// on the long scoreboard like global memory.
__device__ __forceinline__ float tc_lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ int4 tc_lds_i4(uint32_t addr) {
  int4 v;
  asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

__device__ __forceinline__ void tc_sts_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void tc_red_f32(uint32_t addr, float v) {
  asm volatile("red.shared.add.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// Cycle counters of the roles, summed over CTAs and launches since the last reset (window_attn_tc_stalls):
// [0] producer span, [1] of it waiting for a free buffer, [2] MMA thread span, [3] of it waiting for operands,
// [4] of it waiting for probabilities, [5] softmax thread span, [6] of it waiting for scores, [7] for outputs.
__device__ unsigned long long g_tc_stalls[16];   // [8..13] softmax thread: item prologue, score load, math, store + signal, output fold, row store

template <int HD, bool PAIR>
__global__ void __launch_bounds__(TC_THREADS, 1) wattn_tc_fwd_kernel(const __grid_constant__ WindowAttnArgs a,
                                                                     const __grid_constant__ TcPlan pl,
                                                                     KernelStatus* status, int bias_in_smem) {
  using Cfg = TcCfg<HD>;
  constexpr int G = Cfg::G, NSUB = Cfg::NSUB, HPG = Cfg::HPG;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_tiles = smem;                                     // [2][Q_BYTES]
  uint8_t* kv_slots = q_tiles + 2 * Cfg::Q_BYTES;              // [NSLOT][K | V]
  uint8_t* p_bufs = kv_slots + Cfg::NSLOT * Cfg::SLOT_BYTES;   // [2][2][P_TILE]
  uint8_t* tail = p_bufs + 2 * Cfg::P_BYTES;
  TcBars* bars = reinterpret_cast<TcBars*>(tail);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + sizeof(TcBars));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  long long* prow_ofs = reinterpret_cast<long long*>(tail + 256);        // producer: [128] home row of the rows being gathered
  int* prow_slot = reinterpret_cast<int*>(prow_ofs + TC_ROWS);           // producer: [128] peer slot (-1: zero fill)
  int* key_term = prow_slot + TC_ROWS;                                   // [2][64] bias-table term of the keys of a slot
  int* key_reg = key_term + 2 * TC_KV;                                   // [2][64] mask region of the keys (15: padding)
  int* tok_ij = key_reg + 2 * TC_KV;                                     // [64] (ti << 16 | tj) of the tokens of a small window
  float* bias_s = reinterpret_cast<float*>(tok_ij + TC_KV);              // [HPG][nrel] x log2(e), when it fits

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Geo geo;
  geo.N = pl.N;
  geo.nrel = (2 * a.wh - 1) * (2 * a.ww - 1);
  geo.Hg = a.nWh * a.wh;
  geo.Wg = a.nWw * a.ww;
  const int N = pl.N;
  const int rel0 = (a.wh - 1) * (2 * a.ww - 1) + (a.ww - 1);
  const int row_ld = 3 * a.C;   // elements between rows of a q|k|v buffer

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 32 * TC_PROD);
      mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 4);
      mbar_init(&bars->o_full[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars->kv_full[i], 32 * TC_PROD);
      mbar_init(&bars->kv_empty[i], 1);
    }
    mbar_init(&bars->rows_sync, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == TC_MMA_WARP) {
    tmem_alloc<Cfg::TMEM_COLS>(tmem_slot);
    tmem_relinquish();
  }
  if (threadIdx.x < TC_KV) {
    const int t = min(static_cast<int>(threadIdx.x), N - 1);
    tok_ij[threadIdx.x] = ((t / a.ww) << 16) | (t % a.ww);
    if (pl.pair) {
      // keys of a small window are its own tokens: their bias terms never change, padding keys are marked once
      for (int sl2 = 0; sl2 < 2; ++sl2) {
        key_term[sl2 * TC_KV + threadIdx.x] = (t / a.ww) * (2 * a.ww - 1) + (t % a.ww);
        key_reg[sl2 * TC_KV + threadIdx.x] = static_cast<int>(threadIdx.x) < N ? 0 : 15;
      }
    }
  }
  // probability tiles start as zeros: in pair mode each half of the rows writes only its own key block, the other
  // block must contribute nothing to P V
  for (int i = threadIdx.x; i < 2 * Cfg::P_BYTES / 16; i += TC_THREADS)
    reinterpret_cast<uint4*>(p_bufs)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < TC_PROD) {
    // ================================================================== producers: gather into swizzled tiles
    // Rows are dealt to the producer warps in groups of 32 (group g belongs to warp g % TC_PROD); a warp fills the
    // table entries of its own rows and copies only those, so the warps never wait for each other. Each lane counts
    // itself in on the tile's barrier once its own copies have landed.
    uint64_t* fifo[3] = {nullptr, nullptr, nullptr};   // barriers of this lane's copy groups in flight (oldest first)
    int pending = 0;
    const long long t_begin = clock64();
    long long t_wait = 0;
    auto retire_oldest = [&]() {
      fence_proxy_async_smem();      // generic-proxy writes of the copies -> visible to the tensor core's reads
      mbar_arrive(fifo[0]);
      fifo[0] = fifo[1];
      fifo[1] = fifo[2];
      fifo[2] = nullptr;
      --pending;
    };
    auto submit = [&](uint64_t* bar) {
      tc_cp_commit();
      fifo[pending++] = bar;
      if (pending == 3) {
        tc_cp_wait<2>();
        retire_oldest();
      }
    };
    auto wait_empty = [&](uint64_t* bar, uint32_t parity, unsigned where) -> bool {
      int ok = 1;
      const long long w0 = clock64();
      if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, where) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      t_wait += clock64() - w0;
      return ok != 0;
    };
    // Rows [0, nrows) of a tile hold tokens tok0 + (r - row0) of window `flat` for r in [row0, row0 + nspan) (-1: no
    // window; tokens at or beyond tok_end do not exist): copy matrix m0 (0 q, 1 k) into dst0 and, with dst1, matrix
    // m0 + 1 (v) into dst1; rows without a home are zero filled. Tile layout: 64-channel sub-tiles of nrows x 128 bytes,
    // 16-byte chunks XOR-swizzled by row.
    auto gather = [&](uint8_t* dst0, uint8_t* dst1, int nrows, int row0, int nspan, int b, int flat, int tok0, int tok_end,
                      int hg, int m0) {
      const int ii = flat >= 0 ? flat / a.nWw : 0, jj = flat >= 0 ? flat % a.nWw : 0;
      const uint32_t d0 = smem_u32(dst0), d1 = dst1 != nullptr ? smem_u32(dst1) : 0u;
      constexpr int per_row = 8 * NSUB;
      for (int g0 = warp * 32; g0 < nspan; g0 += 32 * TC_PROD) {
        const int r = row0 + g0 + lane;
        const int tok = tok0 + g0 + lane;
        long long ofs = 0;
        int slot = -1;
        if (flat >= 0 && g0 + lane < nspan && tok < tok_end) {
          int ti, tj;
          if (pl.pair) {
            ti = tok_ij[tok] >> 16;
            tj = tok_ij[tok] & 0xffff;
          } else {
            ti = tok / a.ww;
            tj = tok - ti * a.ww;
          }
          const Home h = locate_ij(a, geo, b, ii, jj, ti, tj);
          ofs = h.row * row_ld + m0 * a.C + hg * G;
          slot = h.slot;
        }
        // 32 rows x per_row chunks: lane l copies chunk (l % per_row) of rows (l / per_row) + k * (32 / per_row)
#pragma unroll
        for (int k = 0; k < per_row; ++k) {
          const int idx = k * 32 + lane;
          const int rr = idx / per_row, ch = idx % per_row;
          const long long o = __shfl_sync(0xffffffffu, ofs, rr);
          const int sl = __shfl_sync(0xffffffffu, slot, rr);
          const int row = row0 + g0 + rr;
          if (g0 + rr < nspan) {
            const bool valid = sl >= 0;
            const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(a.qkv[valid ? sl : 0]) + (valid ? o + ch * 8 : 0);
            const uint32_t off = (ch >> 3) * (nrows * 128) + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
            tc_cp_async16(d0 + off, src, valid);
            if (dst1 != nullptr) tc_cp_async16(d1 + off, src + (valid ? a.C : 0), valid);
          }
        }
        (void)r;
      }
    };
    uint32_t q_it = 0, kv_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < pl.items && ok && !*abort_flag; item += gridDim.x) {
      const TcItem it = tc_decode<HPG>(pl, item);
      const int flat0 = a.win_start[a.my_wg] + it.w0;
      // ---- Q tile
      {
        const int qb = q_it & 1;
        if (!(ok = wait_empty(&bars->q_empty[qb], ((q_it >> 1) & 1u) ^ 1u, 0x1100u + qb))) break;
        uint8_t* qt = q_tiles + qb * Cfg::Q_BYTES;
        if (pl.pair) {
          // two windows of up to 64 tokens: rows 0-63 and 64-127
          gather(qt, nullptr, TC_ROWS, 0, 64, it.b, flat0, 0, N, it.hg, 0);
          gather(qt, nullptr, TC_ROWS, 64, 64, it.b, it.nwin > 1 ? flat0 + 1 : -1, 0, N, it.hg, 0);
        } else {
          gather(qt, nullptr, TC_ROWS, 0, TC_ROWS, it.b, flat0, pl.q0 + it.qb * TC_ROWS, pl.q1, it.hg, 0);
        }
        submit(&bars->q_full[qb]);
        ++q_it;
      }
      // ---- K / V slots in the order the math consumes them
      const int nslots = pl.pair ? it.nwin : it.nkv;
      for (int s = 0; s < nslots && ok; ++s) {
        const int ks = kv_it % Cfg::NSLOT;
        if (!(ok = wait_empty(&bars->kv_empty[ks], ((kv_it / Cfg::NSLOT) & 1u) ^ 1u, 0x1200u + ks))) break;
        uint8_t* kt = kv_slots + ks * Cfg::SLOT_BYTES;
        if (pl.pair) gather(kt, kt + Cfg::KV_BYTES, TC_KV, 0, TC_KV, it.b, flat0 + s, 0, N, it.hg, 1);
        else gather(kt, kt + Cfg::KV_BYTES, TC_KV, 0, TC_KV, it.b, flat0, s * TC_KV, N, it.hg, 1);
        submit(&bars->kv_full[ks]);
        ++kv_it;
      }
    }
    tc_cp_wait<0>();
    while (pending > 0) retire_oldest();
    if (warp == 0 && lane == 0) {
      atomicAdd(&g_tc_stalls[0], static_cast<unsigned long long>(clock64() - t_begin));
      atomicAdd(&g_tc_stalls[1], static_cast<unsigned long long>(t_wait));
    }
  } else if (warp == TC_MMA_WARP) {
    // ================================================================== MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(TC_ROWS, TC_KV, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TC_ROWS, HD, 0, 1);
      uint32_t q_it = 0, kv_it = 0, gs = 0;   // Q tiles, K/V slots and steps consumed so far
      bool ok = true;
      const long long t_begin = clock64();
      long long t_ops = 0, t_prob = 0;
      for (int item = blockIdx.x; item < pl.items && ok && !*abort_flag; item += gridDim.x) {
        const TcItem it = tc_decode<HPG>(pl, item);
        const int qb = q_it & 1;
        {
          const long long w0 = clock64();
          ok = mbar_wait(&bars->q_full[qb], (q_it >> 1) & 1u, abort_flag, status, 0x2100u + qb);
          t_ops += clock64() - w0;
          if (!ok) break;
        }
        const uint32_t q_addr = smem_u32(q_tiles + qb * Cfg::Q_BYTES);
        const int spi = pl.pair ? it.nwin : 1;   // slots per iteration
        auto issue_qk = [&](int n, uint32_t step) -> bool {
          const int j = n / HPG, h = n % HPG;
          const uint32_t buf = step & 1u;
          for (int s = 0; s < spi; ++s) {
            const uint32_t kslot = kv_it + (pl.pair ? s : j);
            const int ks = kslot % Cfg::NSLOT;
            if (h == 0) {
              const long long w0 = clock64();
              const bool got = mbar_wait(&bars->kv_full[ks], (kslot / Cfg::NSLOT) & 1u, abort_flag, status, 0x2200u + ks);
              t_ops += clock64() - w0;
              if (!got) return false;
            }
            tc_fence_after();
            const uint32_t k_addr = smem_u32(kv_slots + ks * Cfg::SLOT_BYTES);
            const uint32_t d = tmem_base + buf * 128 + s * TC_KV;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
              const int cb = h * HD + kk * 16;
              const uint32_t sub = cb >> 6, off = (cb & 63) * 2;
              umma_bf16(d, make_smem_desc(q_addr + sub * (TC_ROWS * 128) + off, 16, 1024),
                        make_smem_desc(k_addr + sub * (TC_KV * 128) + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
            }
          }
          umma_commit(&bars->s_full[buf]);
          if (n == it.T - 1) umma_commit(&bars->q_empty[qb]);   // last use of this Q tile
          return true;
        };
        if (!(ok = issue_qk(0, gs))) break;
        for (int n = 0; n < it.T && ok; ++n, ++gs) {
          if (n + 1 < it.T && !(ok = issue_qk(n + 1, gs + 1))) break;
          const int j = n / HPG, h = n % HPG;
          const uint32_t buf = gs & 1u;
          {
            const long long w0 = clock64();
            ok = mbar_wait(&bars->p_full[buf], (gs >> 1) & 1u, abort_flag, status, 0x2300u + buf);
            t_prob += clock64() - w0;
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t d = tmem_base + Cfg::O_COL + buf * HD;
          const uint32_t p_addr = smem_u32(p_bufs + buf * Cfg::P_BYTES);
          uint32_t first = 1u;
          for (int s = 0; s < spi; ++s) {
            const uint32_t kslot = kv_it + (pl.pair ? s : j);
            const int ks = kslot % Cfg::NSLOT;
            const int cb = h * HD;
            const uint32_t v_addr = smem_u32(kv_slots + ks * Cfg::SLOT_BYTES + Cfg::KV_BYTES) + (cb >> 6) * (TC_KV * 128) +
                                    (cb & 63) * 2;
#pragma unroll
            for (int k4 = 0; k4 < TC_KV / 16; ++k4) {
              umma_bf16(d, make_smem_desc(p_addr + s * Cfg::P_TILE + k4 * 32, 16, 1024),
                        make_smem_desc(v_addr + k4 * (16 * 128), TC_KV * 128, 1024), idesc_pv, first ? 0u : 1u);
              first = 0u;
            }
            if (h == HPG - 1) umma_commit(&bars->kv_empty[ks]);   // last head: the slot may be refilled
          }
          umma_commit(&bars->o_full[buf]);
        }
        kv_it += pl.pair ? it.nwin : it.nkv;
        ++q_it;
      }
      atomicAdd(&g_tc_stalls[2], static_cast<unsigned long long>(clock64() - t_begin));
      atomicAdd(&g_tc_stalls[3], static_cast<unsigned long long>(t_ops));
      atomicAdd(&g_tc_stalls[4], static_cast<unsigned long long>(t_prob));
    }
  } else {
    // ================================================================== softmax / epilogue: one query row per thread
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const bool use_bias = a.bias_table != nullptr;
    const float scale2 = a.scale * TC_LOG2E;
    uint32_t gs = 0, syncs = 0;
    bool ok = true;
    int cur_hg = -1;
    const long long t_begin = clock64();
    long long t_score = 0, t_out = 0, t_seg[6] = {0, 0, 0, 0, 0, 0};
    // barrier among the softmax threads; bounded like every other wait, so a failed CTA cannot hang in it
    auto rows_barrier = [&]() {
      mbar_arrive(&bars->rows_sync);
      if (ok) ok = mbar_wait(&bars->rows_sync, syncs & 1u, abort_flag, status, 0x3500u);
      ++syncs;
      ok = __all_sync(0xffffffffu, ok);
    };
    for (int item = blockIdx.x; item < pl.items && ok; item += gridDim.x) {
      long long tq = clock64();
      const TcItem it = tc_decode<HPG>(pl, item);
      if (bias_in_smem && it.hg != cur_hg) {
        // relative-position bias of this head group, pre-multiplied by log2(e)
        rows_barrier();      // nobody reads the previous group's table any more
        for (int i = threadIdx.x - 32 * (TC_PROD + 1); i < HPG * geo.nrel; i += 128) {
          const int h = i / geo.nrel, e = i % geo.nrel;
          bias_s[i] = a.bias_table[static_cast<long long>(e) * a.num_heads + it.hg * HPG + h] * TC_LOG2E;
        }
        rows_barrier();
        cur_hg = it.hg;
        if (!ok) break;
      }
      const int sl = PAIR ? (r >> 6) : 0;
      const int flat = a.win_start[a.my_wg] + it.w0 + sl;
      const int tok = PAIR ? (r & 63) : pl.q0 + it.qb * TC_ROWS + r;
      const bool active = PAIR ? (sl < it.nwin && tok < N) : (tok < pl.q1);
      const int fl = (PAIR && sl >= it.nwin) ? flat - sl : flat;   // clamp to an existing window
      const int ii = fl / a.nWw, jj = fl % a.nWw;
      const int tk = min(tok, N - 1);
      int ti, tj;
      if (PAIR) {
        ti = tok_ij[tk] >> 16;
        tj = tok_ij[tk] & 0xffff;
      } else {
        ti = tk / a.ww;
        tj = tk - ti * a.ww;
      }
      const Home home = locate_ij(a, geo, it.b, ii, jj, ti, tj);
      const int row_term = ti * (2 * a.ww - 1) + tj + rel0;
      const bool general = a.use_mask && ((a.sh > 0 && ii == a.nWh - 1) || (a.sw > 0 && jj == a.nWw - 1));
      const bool store_row = active && (!PAIR || (tok >= pl.q0 && tok < pl.q1));
      // Small windows: the keys of a slot are the window's own tokens. Their bias terms are static; their mask regions
      // matter only in the windows of the last row / column of a shifted frame, where every row publishes its region.
      bool tile_general = false;
      if (PAIR && a.use_mask) {
        const int fa = a.win_start[a.my_wg] + it.w0, fb = fa + (it.nwin > 1 ? 1 : 0);
        tile_general = (a.sh > 0 && (fa / a.nWw == a.nWh - 1 || fb / a.nWw == a.nWh - 1)) ||
                       (a.sw > 0 && (fa % a.nWw == a.nWw - 1 || fb % a.nWw == a.nWw - 1));
      }
      if (tile_general) {
        key_reg[sl * TC_KV + (r & 63)] = (tok < N) ? home.region : 15;
        rows_barrier();
        if (!ok) break;
      }
      // Small windows see all their keys in one step, so a head's output is final after its single product and goes
      // straight to memory; large windows accumulate over the key slots with the online-softmax rescaling.
      float m_run[HPG], l_run[HPG], oacc[PAIR ? 1 : G];
#pragma unroll
      for (int h = 0; h < HPG; ++h) {
        m_run[h] = TC_NEG;
        l_run[h] = 0.f;
      }
#pragma unroll
      for (int c = 0; c < (PAIR ? 1 : G); ++c) oacc[c] = 0.f;
      __nv_bfloat16* const out_row =
          static_cast<__nv_bfloat16*>(a.out[home.slot]) + home.row * a.C + it.hg * G;
      float alpha_prev = 0.f;
      int h_prev = 0;
      t_seg[0] += clock64() - tq;

      auto fold_output = [&](uint32_t step, int h, float alpha) {
        // O of `step` (head h) is complete in tensor memory. Large windows: acc = acc * alpha + O (alpha: the rescaling
        // of that step). Small windows: alpha is 1 / (sum of the row's numerators) and the normalised row is stored.
        const uint32_t buf = step & 1u;
        const long long w0 = clock64();
        if (ok) ok = mbar_wait(&bars->o_full[buf], (step >> 1) & 1u, abort_flag, status, 0x3300u + buf);
        ok = __all_sync(0xffffffffu, ok);
        t_out += clock64() - w0;
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + Cfg::O_COL + buf * HD + c0 + lane_base, v);
          tmem_ld_wait();
          if (PAIR) {
            if (store_row) {
#pragma unroll
              for (int c = 0; c < 32 && c0 + c < HD; c += 8)
                *reinterpret_cast<uint4*>(out_row + h * HD + c0 + c) = make_uint4(
                    pack_bf16x2(__uint_as_float(v[c]) * alpha, __uint_as_float(v[c + 1]) * alpha),
                    pack_bf16x2(__uint_as_float(v[c + 2]) * alpha, __uint_as_float(v[c + 3]) * alpha),
                    pack_bf16x2(__uint_as_float(v[c + 4]) * alpha, __uint_as_float(v[c + 5]) * alpha),
                    pack_bf16x2(__uint_as_float(v[c + 6]) * alpha, __uint_as_float(v[c + 7]) * alpha));
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              if (c0 + c < HD) {
#pragma unroll
                for (int hh = 0; hh < HPG; ++hh)
                  if (hh == h) oacc[(PAIR ? 0 : hh * HD + c0 + c)] = fmaf(oacc[(PAIR ? 0 : hh * HD + c0 + c)], alpha, __uint_as_float(v[c]));
              }
            }
          }
        }
        tc_fence_before();
      };

      for (int n = 0; n < it.T; ++n, ++gs) {
        const int j = n / HPG, h = n % HPG;
        const uint32_t buf = gs & 1u;
        const int kt = PAIR ? sl : (j & 1);   // which key table
        if (!PAIR && h == 0) {
          // keys j*64 .. j*64+63 of this window: bias term, mask region, validity
          if (r < TC_KV) {
            const int key = j * TC_KV + r;
            const int kk = min(key, N - 1);
            key_term[kt * TC_KV + r] = (kk / a.ww) * (2 * a.ww - 1) + (kk % a.ww);
            key_reg[kt * TC_KV + r] = key < N ? region_of(a, geo, ii * a.wh + kk / a.ww, jj * a.ww + kk % a.ww) : 15;
          }
          rows_barrier();
          if (!ok) break;
        }
        {
          const long long w0 = clock64();
          if (ok) ok = mbar_wait(&bars->s_full[buf], (gs >> 1) & 1u, abort_flag, status, 0x3100u + buf);
          ok = __all_sync(0xffffffffu, ok);
          t_score += clock64() - w0;
        }
        if (!ok) break;
        tc_fence_after();
        tq = clock64();
        float s[TC_KV];
        {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + buf * 128 + sl * TC_KV + lane_base, v);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) s[c] = __uint_as_float(v[c]);
          tmem_ld_32x32(tmem_base + buf * 128 + sl * TC_KV + 32 + lane_base, v);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) s[32 + c] = __uint_as_float(v[c]);
        }
        tc_fence_before();
        t_seg[1] += clock64() - tq;
        tq = clock64();
        // ---- scale, bias, mask (base-2 domain)
        const uint32_t kterm = smem_u32(key_term + kt * TC_KV);
        const uint32_t kreg = smem_u32(key_reg + kt * TC_KV);
        const bool padded = PAIR ? (N < TC_KV) : ((j + 1) * TC_KV > N);
        float mx = TC_NEG;
        if (use_bias && bias_in_smem) {
          const uint32_t table = smem_u32(bias_s + h * geo.nrel) + 4u * row_term;     // entry of (this row, key term 0)
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 t4 = tc_lds_i4(kterm + 4 * c4);
            s[c4] = fmaf(s[c4], scale2, tc_lds_f32(table - 4u * t4.x));
            s[c4 + 1] = fmaf(s[c4 + 1], scale2, tc_lds_f32(table - 4u * t4.y));
            s[c4 + 2] = fmaf(s[c4 + 2], scale2, tc_lds_f32(table - 4u * t4.z));
            s[c4 + 3] = fmaf(s[c4 + 3], scale2, tc_lds_f32(table - 4u * t4.w));
          }
        } else if (use_bias) {
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 t4 = tc_lds_i4(kterm + 4 * c4);
            const int tt[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              s[c4 + e] = fmaf(s[c4 + e], scale2,
                               __ldg(a.bias_table + static_cast<long long>(row_term - tt[e]) * a.num_heads + it.hg * HPG + h) * TC_LOG2E);
          }
        } else {
#pragma unroll
          for (int c = 0; c < TC_KV; ++c) s[c] *= scale2;
        }
        if (general || padded) {
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 g4 = tc_lds_i4(kreg + 4 * c4);
            const int gg[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (gg[e] == 15) s[c4 + e] = TC_NEG;
              else if (general && gg[e] != home.region) s[c4 + e] += -100.f * TC_LOG2E;
            }
          }
        }
#pragma unroll
        for (int c = 0; c < TC_KV; ++c) mx = fmaxf(mx, s[c]);
        // ---- online softmax state of head h
        float m_old = TC_NEG, l_old = 0.f;
#pragma unroll
        for (int hh = 0; hh < HPG; ++hh)
          if (hh == h) {
            m_old = m_run[hh];
            l_old = l_run[hh];
          }
        const float m_new = fmaxf(m_old, mx);
        const float alpha = exp2f(m_old - m_new);
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < TC_KV; ++c) {
          s[c] = exp2f(s[c] - m_new);
          sum += s[c];
        }
#pragma unroll
        for (int hh = 0; hh < HPG; ++hh)
          if (hh == h) {
            m_run[hh] = m_new;
            l_run[hh] = fmaf(l_old, alpha, sum);
          }
        t_seg[2] += clock64() - tq;
        tq = clock64();
        // ---- probabilities (bf16) into the A-operand tile: row r, 16-byte chunk c8 at (c8 ^ (r & 7))
        {
          const uint32_t prow = smem_u32(p_bufs + buf * Cfg::P_BYTES + sl * Cfg::P_TILE + r * 128);
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const uint4 pk = make_uint4(pack_bf16x2(s[8 * c8], s[8 * c8 + 1]), pack_bf16x2(s[8 * c8 + 2], s[8 * c8 + 3]),
                                        pack_bf16x2(s[8 * c8 + 4], s[8 * c8 + 5]), pack_bf16x2(s[8 * c8 + 6], s[8 * c8 + 7]));
            tc_sts_v4(prow + ((c8 ^ (r & 7)) << 4), pk);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[buf]);     // one arrival per warp: 128 threads on one word serialise
        t_seg[3] += clock64() - tq;
        // ---- the previous step's output is ready by now: fold it in while the tensor core works on this step
        tq = clock64();
        if (n > 0) fold_output(gs - 1, h_prev, alpha_prev);
        t_seg[4] += clock64() - tq;
        if (!ok) break;
        alpha_prev = PAIR ? 1.f / fmaf(l_old, alpha, sum) : alpha;
        h_prev = h;
      }
      tq = clock64();
      if (ok && it.T > 0) fold_output(gs - 1, h_prev, alpha_prev);
      t_seg[4] += clock64() - tq;
      if (!ok) break;
      tq = clock64();
      // ---- normalise and store the row to its home (this GPU's buffer or a peer's)
      if (store_row) {
        if (!PAIR) {
#pragma unroll
          for (int h = 0; h < HPG; ++h) {
            const float inv = 1.f / l_run[h];
#pragma unroll
            for (int c = 0; c < HD; c += 8) {
              const float* o = oacc + (PAIR ? 0 : h * HD + c);
              *reinterpret_cast<uint4*>(out_row + h * HD + c) =
                  make_uint4(pack_bf16x2(o[0] * inv, o[1] * inv), pack_bf16x2(o[2] * inv, o[3] * inv),
                             pack_bf16x2(o[4] * inv, o[5] * inv), pack_bf16x2(o[6] * inv, o[7] * inv));
            }
          }
        }
        if (a.lse[home.slot] != nullptr) {
          float* lse = a.lse[home.slot] + home.row * a.num_heads + it.hg * HPG;
#pragma unroll
          for (int h = 0; h < HPG; ++h) lse[h] = m_run[h] + log2f(l_run[h]);
        }
      }
      t_seg[5] += clock64() - tq;
      if (tile_general) {
        rows_barrier();               // everybody is done with the regions of this tile ...
        key_reg[sl * TC_KV + (r & 63)] = (r & 63) < N ? 0 : 15;   // ... which go back to "one region"
        rows_barrier();               // ... before anybody reads them for the next tile
      }
    }
    if (warp == TC_MMA_WARP + 1 && lane == 0) {
      atomicAdd(&g_tc_stalls[5], static_cast<unsigned long long>(clock64() - t_begin));
      atomicAdd(&g_tc_stalls[6], static_cast<unsigned long long>(t_score));
      atomicAdd(&g_tc_stalls[7], static_cast<unsigned long long>(t_out));
      for (int i = 0; i < 6; ++i) atomicAdd(&g_tc_stalls[8 + i], static_cast<unsigned long long>(t_seg[i]));
    }
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let copies and products in flight land before smem / TMEM go away
  }
  tc_fence_before();
  __syncthreads();
  if (warp == TC_MMA_WARP) {
    __syncwarp();
    tmem_dealloc<Cfg::TMEM_COLS>(tmem_base);
  }
}

// ================================================================================================ backward, N <= 64
// Two windows of at most 64 tokens per tile, one head group (64 channels), heads one after the other. Per head:
//   S = Q K^T and dP = dO V^T (M = 128, N = 128: both windows' rows against both windows' keys; each row uses its own
//   window's 64 columns), the row's thread recomputes P = softmax(S), D = sum(P dP), dS = P (dP - D) and writes P and
//   dS (bf16) as block-diagonal [row][key] tiles; then dV = P^T dO, dK = dS^T Q (A read MN-major from those tiles) and
//   dQ = dS K, all M = 128, N = head dim, K = 128, into tensor memory, from where the row's thread stores them to the
//   token's home row (q | k | v gradients side by side). The bias gradient is accumulated in shared memory and flushed
//   with one atomic per table entry when the head group changes.
template <int HD>
struct TcBwdCfg {
  static constexpr int G = 64;
  static constexpr int HPG = G / HD;
  static constexpr int MAT = TC_ROWS * 128;              // one [128 rows][64 channels] tile
  static constexpr int STAGE = 4 * MAT;                  // q, k, v, dO
  static constexpr int PS = 4 * MAT;                     // P (2 key blocks) + dS (2 key blocks)
  static constexpr int TILE_BYTES = 2 * STAGE + PS;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_DP = 128, COL_DV = 256, COL_DK = 256 + HD, COL_DQ = 256 + 2 * HD;
};

struct TcBwdBars {
  uint64_t in_full[2], in_empty[2];
  uint64_t sdp_full, pds_full, out_full, rows_sync;
};

template <int HD>
__global__ void __launch_bounds__(TC_THREADS, 1) wattn_tc_bwd_kernel(const __grid_constant__ WindowAttnArgs a,
                                                                     const __grid_constant__ TcPlan pl,
                                                                     KernelStatus* status) {
  using Cfg = TcBwdCfg<HD>;
  constexpr int G = Cfg::G, HPG = Cfg::HPG;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;                                  // [2][q | k | v | dO]
  uint8_t* p_tiles = stages + 2 * Cfg::STAGE;              // [2][MAT]: probabilities, key block 0 / 1
  uint8_t* ds_tiles = p_tiles + 2 * Cfg::MAT;              // [2][MAT]: dS
  uint8_t* tail = ds_tiles + 2 * Cfg::MAT;
  TcBwdBars* bars = reinterpret_cast<TcBwdBars*>(tail);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + sizeof(TcBwdBars));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* key_term = reinterpret_cast<int*>(tail + 128);      // [64] bias-table term of token t
  int* key_reg = key_term + TC_KV;                         // [2][64] mask region of the keys (15: padding)
  int* tok_ij = key_reg + 2 * TC_KV;                       // [64]
  float* bias_s = reinterpret_cast<float*>(tok_ij + TC_KV);   // [HPG][nrel] x log2(e)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Geo geo;
  geo.N = pl.N;
  geo.nrel = (2 * a.wh - 1) * (2 * a.ww - 1);
  geo.Hg = a.nWh * a.wh;
  geo.Wg = a.nWw * a.ww;
  const int N = pl.N;
  float* dbias_s = bias_s + HPG * geo.nrel;                // [HPG][nrel] gradient accumulator
  const int rel0 = (a.wh - 1) * (2 * a.ww - 1) + (a.ww - 1);
  const bool use_bias = a.bias_table != nullptr;
  const bool bias_grad = use_bias && a.dbias_table != nullptr;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->in_full[i], 32 * TC_PROD);
      mbar_init(&bars->in_empty[i], 1);
    }
    mbar_init(&bars->sdp_full, 1);
    mbar_init(&bars->pds_full, 4);
    mbar_init(&bars->out_full, 1);
    mbar_init(&bars->rows_sync, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == TC_MMA_WARP) {
    tmem_alloc<Cfg::TMEM_COLS>(tmem_slot);
    tmem_relinquish();
  }
  if (threadIdx.x < TC_KV) {
    const int t = min(static_cast<int>(threadIdx.x), N - 1);
    tok_ij[threadIdx.x] = ((t / a.ww) << 16) | (t % a.ww);
    key_term[threadIdx.x] = (t / a.ww) * (2 * a.ww - 1) + (t % a.ww);
    key_reg[threadIdx.x] = key_reg[TC_KV + threadIdx.x] = static_cast<int>(threadIdx.x) < N ? 0 : 15;
  }
  for (int i = threadIdx.x; i < Cfg::PS / 16; i += TC_THREADS) reinterpret_cast<uint4*>(p_tiles)[i] = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < HPG * geo.nrel; i += TC_THREADS) dbias_s[i] = 0.f;
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < TC_PROD) {
    // ================================================================== producers
    uint64_t* fifo[2] = {nullptr, nullptr};
    int pending = 0;
    auto retire_oldest = [&]() {
      fence_proxy_async_smem();
      mbar_arrive(fifo[0]);
      fifo[0] = fifo[1];
      fifo[1] = nullptr;
      --pending;
    };
    uint32_t fills = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < pl.items && ok && !*abort_flag; item += gridDim.x) {
      const TcItem it = tc_decode<HPG>(pl, item);
      const int st = fills & 1;
      {
        int got = 1;
        if (lane == 0) got = mbar_wait(&bars->in_empty[st], ((fills >> 1) & 1u) ^ 1u, abort_flag, status, 0x4100u + st) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!(ok = got != 0)) break;
      }
      const uint32_t base = smem_u32(stages + st * Cfg::STAGE);
      const int flat0 = a.win_start[a.my_wg] + it.w0;
      for (int g0 = warp * 32; g0 < TC_ROWS; g0 += 32 * TC_PROD) {
        const int r = g0 + lane;
        const int sl = r >> 6, tok = r & 63;
        long long ofs_qkv = 0, ofs_do = 0;
        int slot = -1;
        if (sl < it.nwin && tok < N) {
          const int flat = flat0 + sl;
          const Home h = locate_ij(a, geo, it.b, flat / a.nWw, flat % a.nWw, tok_ij[tok] >> 16, tok_ij[tok] & 0xffff);
          ofs_qkv = h.row * (3LL * a.C) + it.hg * G;
          ofs_do = h.row * static_cast<long long>(a.C) + it.hg * G;
          slot = h.slot;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int idx = k * 32 + lane;
          const int rr = idx >> 3, ch = idx & 7;
          const long long oq = __shfl_sync(0xffffffffu, ofs_qkv, rr);
          const long long od = __shfl_sync(0xffffffffu, ofs_do, rr);
          const int sp = __shfl_sync(0xffffffffu, slot, rr);
          const int row = g0 + rr;
          const bool valid = sp >= 0;
          const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(a.qkv[valid ? sp : 0]) + (valid ? oq + ch * 8 : 0);
          const __nv_bfloat16* sdo = static_cast<const __nv_bfloat16*>(a.dout[valid ? sp : 0]) + (valid ? od + ch * 8 : 0);
          const uint32_t off = row * 128 + ((ch ^ (row & 7)) << 4);
          tc_cp_async16(base + off, src, valid);
          tc_cp_async16(base + Cfg::MAT + off, src + (valid ? a.C : 0), valid);
          tc_cp_async16(base + 2 * Cfg::MAT + off, src + (valid ? 2 * a.C : 0), valid);
          tc_cp_async16(base + 3 * Cfg::MAT + off, sdo, valid);
        }
      }
      tc_cp_commit();
      fifo[pending++] = &bars->in_full[st];
      if (pending == 2) {
        tc_cp_wait<1>();
        retire_oldest();
      }
      ++fills;
    }
    tc_cp_wait<0>();
    while (pending > 0) retire_oldest();
  } else if (warp == TC_MMA_WARP) {
    // ================================================================== MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(TC_ROWS, 128, 0, 0);      // S, dP: K-major x K-major
      constexpr uint32_t idesc_t = make_idesc_bf16(TC_ROWS, HD, 1, 1);       // dV, dK: A = P^T / dS^T (MN-major), B MN-major
      constexpr uint32_t idesc_q = make_idesc_bf16(TC_ROWS, HD, 0, 1);       // dQ: A = dS (K-major), B = K (MN-major)
      uint32_t fills = 0, gs = 0;
      bool ok = true;
      const uint32_t p_addr = smem_u32(p_tiles), ds_addr = smem_u32(ds_tiles);
      auto issue_sdp = [&](uint32_t base, int h) {
        // S = Q K^T -> columns [0, 128); dP = dO V^T -> columns [128, 256)
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (h * HD + kk * 16) * 2;
          umma_bf16(tmem_base, make_smem_desc(base + off, 16, 1024), make_smem_desc(base + Cfg::MAT + off, 16, 1024), idesc_s,
                    kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (h * HD + kk * 16) * 2;
          umma_bf16(tmem_base + Cfg::COL_DP, make_smem_desc(base + 3 * Cfg::MAT + off, 16, 1024),
                    make_smem_desc(base + 2 * Cfg::MAT + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->sdp_full);
      };
      for (int item = blockIdx.x; item < pl.items && ok && !*abort_flag; item += gridDim.x) {
        const int st = fills & 1;
        if (!(ok = mbar_wait(&bars->in_full[st], (fills >> 1) & 1u, abort_flag, status, 0x4200u + st))) break;
        tc_fence_after();
        const uint32_t base = smem_u32(stages + st * Cfg::STAGE);
        issue_sdp(base, 0);
        for (int h = 0; h < HPG && ok; ++h, ++gs) {
          if (!(ok = mbar_wait(&bars->pds_full, gs & 1u, abort_flag, status, 0x4300u))) break;
          tc_fence_after();
          const uint32_t hb = h * HD * 2;   // byte offset of the head's channels inside a 128-byte row
          // dV = P^T dO, dK = dS^T Q: contraction over the 128 rows (8 steps of 16), A tiles read MN-major
#pragma unroll
          for (int k8 = 0; k8 < 8; ++k8) {
            umma_bf16(tmem_base + Cfg::COL_DV, make_smem_desc(p_addr + k8 * 2048, Cfg::MAT, 1024),
                      make_smem_desc(base + 3 * Cfg::MAT + hb + k8 * 2048, TC_ROWS * 128, 1024), idesc_t, k8 > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int k8 = 0; k8 < 8; ++k8) {
            umma_bf16(tmem_base + Cfg::COL_DK, make_smem_desc(ds_addr + k8 * 2048, Cfg::MAT, 1024),
                      make_smem_desc(base + hb + k8 * 2048, TC_ROWS * 128, 1024), idesc_t, k8 > 0 ? 1u : 0u);
          }
          // dQ = dS K: contraction over the 128 keys: key block t (tile t of dS), 4 steps of 16 each
#pragma unroll
          for (int k8 = 0; k8 < 8; ++k8) {
            umma_bf16(tmem_base + Cfg::COL_DQ, make_smem_desc(ds_addr + (k8 >> 2) * Cfg::MAT + (k8 & 3) * 32, 16, 1024),
                      make_smem_desc(base + Cfg::MAT + hb + k8 * 2048, TC_ROWS * 128, 1024), idesc_q, k8 > 0 ? 1u : 0u);
          }
          umma_commit(&bars->out_full);
          if (h == HPG - 1) umma_commit(&bars->in_empty[st]);
          else issue_sdp(base, h + 1);
        }
        ++fills;
      }
    }
  } else {
    // ================================================================== softmax / gradient rows
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float scale2 = a.scale * TC_LOG2E;
    const int sl = r >> 6, tok = r & 63;
    uint32_t gs = 0, syncs = 0;
    bool ok = true;
    int cur_hg = -1;
    auto rows_barrier = [&]() {
      mbar_arrive(&bars->rows_sync);
      if (ok) ok = mbar_wait(&bars->rows_sync, syncs & 1u, abort_flag, status, 0x5500u);
      ++syncs;
      ok = __all_sync(0xffffffffu, ok);
    };
    auto flush_dbias = [&](int hg) {
      // one atomic per table entry and head of the group that was just finished
      rows_barrier();
      if (bias_grad && hg >= 0) {
        for (int i = threadIdx.x - 32 * (TC_PROD + 1); i < HPG * geo.nrel; i += 128) {
          const int h = i / geo.nrel, e = i % geo.nrel;
          const float v = dbias_s[i];
          if (v != 0.f) atomicAdd(&a.dbias_table[static_cast<long long>(e) * a.num_heads + hg * HPG + h], v);
          dbias_s[i] = 0.f;
        }
      }
    };
    const int tk = min(tok, N - 1);
    const int ti = tok_ij[tk] >> 16, tj = tok_ij[tk] & 0xffff;
    const int row_term = ti * (2 * a.ww - 1) + tj + rel0;
    for (int item = blockIdx.x; item < pl.items && ok; item += gridDim.x) {
      const TcItem it = tc_decode<HPG>(pl, item);
      if (it.hg != cur_hg) {
        flush_dbias(cur_hg);
        if (use_bias) {
          for (int i = threadIdx.x - 32 * (TC_PROD + 1); i < HPG * geo.nrel; i += 128) {
            const int h = i / geo.nrel, e = i % geo.nrel;
            bias_s[i] = a.bias_table[static_cast<long long>(e) * a.num_heads + it.hg * HPG + h] * TC_LOG2E;
          }
        }
        rows_barrier();
        cur_hg = it.hg;
        if (!ok) break;
      }
      const bool active = sl < it.nwin && tok < N;
      const int flat = a.win_start[a.my_wg] + it.w0 + (sl < it.nwin ? sl : 0);
      const int ii = flat / a.nWw, jj = flat % a.nWw;
      const Home home = locate_ij(a, geo, it.b, ii, jj, ti, tj);
      const bool general = a.use_mask && ((a.sh > 0 && ii == a.nWh - 1) || (a.sw > 0 && jj == a.nWw - 1));
      const bool mine = active && tok >= pl.q0 && tok < pl.q1;     // this rank keeps the gradients of its own token shard
      bool tile_general = false;
      if (a.use_mask) {
        const int fa = a.win_start[a.my_wg] + it.w0, fb = fa + (it.nwin > 1 ? 1 : 0);
        tile_general = (a.sh > 0 && (fa / a.nWw == a.nWh - 1 || fb / a.nWw == a.nWh - 1)) ||
                       (a.sw > 0 && (fa % a.nWw == a.nWw - 1 || fb % a.nWw == a.nWw - 1));
      }
      if (tile_general) {
        key_reg[sl * TC_KV + tok] = (tok < N) ? home.region : 15;
        rows_barrier();
        if (!ok) break;
      }
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.dqkv[home.slot]) + home.row * (3LL * a.C) + it.hg * G;

      auto store_outputs = [&](int h) {
        // dV, dK, dQ of head h are complete in tensor memory: row r of each is this token's gradient
        if (ok) ok = mbar_wait(&bars->out_full, (gs - 1) & 1u, abort_flag, status, 0x5300u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int m = 0; m < 3; ++m) {
          const uint32_t col = m == 0 ? Cfg::COL_DQ : (m == 1 ? Cfg::COL_DK : Cfg::COL_DV);
          const float mul = m == 2 ? 1.f : a.scale;
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + col + c0 + lane_base, v);
            tmem_ld_wait();
            if (mine) {
#pragma unroll
              for (int c = 0; c < 32 && c0 + c < HD; c += 8) {
                *reinterpret_cast<uint4*>(dst + m * a.C + h * HD + c0 + c) = make_uint4(
                    pack_bf16x2(__uint_as_float(v[c]) * mul, __uint_as_float(v[c + 1]) * mul),
                    pack_bf16x2(__uint_as_float(v[c + 2]) * mul, __uint_as_float(v[c + 3]) * mul),
                    pack_bf16x2(__uint_as_float(v[c + 4]) * mul, __uint_as_float(v[c + 5]) * mul),
                    pack_bf16x2(__uint_as_float(v[c + 6]) * mul, __uint_as_float(v[c + 7]) * mul));
              }
            }
          }
        }
        tc_fence_before();
      };

      for (int h = 0; h < HPG; ++h, ++gs) {
        if (ok) ok = mbar_wait(&bars->sdp_full, gs & 1u, abort_flag, status, 0x5100u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float s[TC_KV], dp[TC_KV];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + sl * TC_KV + half * 32 + lane_base, v);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) s[half * 32 + c] = __uint_as_float(v[c]);
          tmem_ld_32x32(tmem_base + Cfg::COL_DP + sl * TC_KV + half * 32 + lane_base, v);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) dp[half * 32 + c] = __uint_as_float(v[c]);
        }
        tc_fence_before();
        const uint32_t kreg = smem_u32(key_reg + sl * TC_KV);
        const uint32_t kterm = smem_u32(key_term);
        if (use_bias) {
          const uint32_t table = smem_u32(bias_s + h * geo.nrel) + 4u * row_term;
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 t4 = tc_lds_i4(kterm + 4 * c4);
            s[c4] = fmaf(s[c4], scale2, tc_lds_f32(table - 4u * t4.x));
            s[c4 + 1] = fmaf(s[c4 + 1], scale2, tc_lds_f32(table - 4u * t4.y));
            s[c4 + 2] = fmaf(s[c4 + 2], scale2, tc_lds_f32(table - 4u * t4.z));
            s[c4 + 3] = fmaf(s[c4 + 3], scale2, tc_lds_f32(table - 4u * t4.w));
          }
        } else {
#pragma unroll
          for (int c = 0; c < TC_KV; ++c) s[c] *= scale2;
        }
        if (general || N < TC_KV) {
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 g4 = tc_lds_i4(kreg + 4 * c4);
            const int gg[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (gg[e] == 15) s[c4 + e] = TC_NEG;
              else if (general && gg[e] != home.region) s[c4 + e] += -100.f * TC_LOG2E;
            }
          }
        }
        float mx = TC_NEG;
#pragma unroll
        for (int c = 0; c < TC_KV; ++c) mx = fmaxf(mx, s[c]);
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < TC_KV; ++c) {
          s[c] = exp2f(s[c] - mx);
          sum += s[c];
        }
        const float inv = 1.f / sum;
        float dsum = 0.f;
#pragma unroll
        for (int c = 0; c < TC_KV; ++c) {
          s[c] *= inv;
          dsum = fmaf(s[c], dp[c], dsum);
        }
#pragma unroll
        for (int c = 0; c < TC_KV; ++c) dp[c] = s[c] * (dp[c] - dsum);      // dS (before the 1/sqrt(d) factor)
        if (bias_grad && mine) {
          const uint32_t gtab = smem_u32(dbias_s + h * geo.nrel) + 4u * row_term;
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 t4 = tc_lds_i4(kterm + 4 * c4);
            const int tt[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (c4 + e < N) tc_red_f32(gtab - 4u * tt[e], dp[c4 + e]);
          }
        }
        // the tiles are read by the previous head's products until out_full: wait for it (and take its results)
        if (h > 0) store_outputs(h - 1);
        if (!ok) break;
        {
          const uint32_t prow = smem_u32(p_tiles + sl * Cfg::MAT + r * 128);
          const uint32_t drow = smem_u32(ds_tiles + sl * Cfg::MAT + r * 128);
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const int o = (c8 ^ (r & 7)) << 4;
            tc_sts_v4(prow + o, make_uint4(pack_bf16x2(s[8 * c8], s[8 * c8 + 1]), pack_bf16x2(s[8 * c8 + 2], s[8 * c8 + 3]),
                                           pack_bf16x2(s[8 * c8 + 4], s[8 * c8 + 5]), pack_bf16x2(s[8 * c8 + 6], s[8 * c8 + 7])));
            tc_sts_v4(drow + o, make_uint4(pack_bf16x2(dp[8 * c8], dp[8 * c8 + 1]), pack_bf16x2(dp[8 * c8 + 2], dp[8 * c8 + 3]),
                                           pack_bf16x2(dp[8 * c8 + 4], dp[8 * c8 + 5]), pack_bf16x2(dp[8 * c8 + 6], dp[8 * c8 + 7])));
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->pds_full);
      }
      if (!ok) break;
      store_outputs(HPG - 1);      // gs already counts the last head
      if (!ok) break;
      if (tile_general) {
        rows_barrier();
        key_reg[sl * TC_KV + tok] = tok < N ? 0 : 15;
        rows_barrier();
      }
    }
    if (ok) flush_dbias(cur_hg);
  }

  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == TC_MMA_WARP) {
    __syncwarp();
    tmem_dealloc<Cfg::TMEM_COLS>(tmem_base);
  }
}

template <int HD>
int launch_tc_bwd(const WindowAttnArgs& a, void* status, cudaStream_t stream) {
  using Cfg = TcBwdCfg<HD>;
  TcPlan pl;
  pl.N = a.wh * a.ww;
  if (pl.N > TC_KV) return -34;
  pl.pair = 1;
  pl.my_nw = a.win_start[a.my_wg + 1] - a.win_start[a.my_wg];
  pl.q0 = a.my_sp * a.shardN;
  pl.q1 = pl.q0 + a.shardN < pl.N ? pl.q0 + a.shardN : pl.N;
  pl.nqb = 1;
  pl.tiles_per_b = (pl.my_nw + 1) / 2;
  pl.hgroups = a.C / Cfg::G;
  pl.items = a.B * pl.tiles_per_b * pl.hgroups;
  if (pl.items <= 0) return 0;
  if (a.C % Cfg::G != 0) return -31;
  const int nrel = (2 * a.wh - 1) * (2 * a.ww - 1);
  const size_t sb = 1024 + Cfg::TILE_BYTES + 128 + 4 * TC_KV * 4 + static_cast<size_t>(2) * Cfg::HPG * nrel * 4 + 64;
  if (sb > 232448) return -35;
  static size_t configured = 0;
  if (sb > configured) {
    if (cudaFuncSetAttribute(wattn_tc_bwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb)) !=
        cudaSuccess)
      return -32;
    configured = sb;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = pl.items < sms ? pl.items : sms;
  wattn_tc_bwd_kernel<HD><<<grid, TC_THREADS, sb, stream>>>(a, pl, static_cast<KernelStatus*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -33;
}

// ================================================================================================ backward, N > 64
// Large windows: two passes over 128 x 128 blocks of the score matrix, both without atomics or cross-rank reductions.
//   PASS 0 (dQ):      an item is a block of 128 of this rank's queries; the window's keys stream by in blocks of 128:
//                     dQ += dS K, accumulated in tensor memory over the key blocks.
//   PASS 1 (dK, dV):  an item is a block of 128 of this rank's keys; all of the window's queries (with their dO, LSE and
//                     D = rowsum(dO o O), read from their home rows, possibly on peers) stream by in blocks of 128:
//                     dV += P^T dO, dK += dS^T Q.
// Per step and head: S = Q K^T and dP = dO V^T (M = N = 128); the row's thread turns them into P = exp2(S' - LSE) and
// dS = P (dP - D) 32 columns at a time - the softmax statistics come from the forward pass, so no row-wide reduction
// is needed - and writes them as [row][key] tiles, the operands of the output products.
template <int HD, int PASS>
__global__ void __launch_bounds__(TC_THREADS, 1) wattn_tc_bwd_block_kernel(const __grid_constant__ WindowAttnArgs a,
                                                                           const __grid_constant__ TcPlan pl,
                                                                           KernelStatus* status) {
  constexpr int G = 64, HPG = G / HD;
  constexpr int MAT = TC_ROWS * 128;
  constexpr int COL_DP = 128, COL_OUT = 256;      // PASS 0: dQ [G]; PASS 1: dV [G] then dK [G]
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* fixed_set = smem;                         // [2][MAT]: PASS 0: q, dO of the item's queries; PASS 1: k, v of its keys
  uint8_t* stream_set = fixed_set + 2 * MAT;         // [2 stages][2][MAT]: the other side, block by block
  uint8_t* p_tiles = stream_set + 4 * MAT;           // [2][MAT] key block 0 / 1
  uint8_t* ds_tiles = p_tiles + 2 * MAT;
  uint8_t* tail = ds_tiles + 2 * MAT;
  struct Bars {
    uint64_t fixed_full, fixed_empty, st_full[2], st_empty[2], sdp_full, pds_full, out_done, item_done, rows_sync;
  };
  Bars* bars = reinterpret_cast<Bars*>(tail);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + sizeof(Bars));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* key_term = reinterpret_cast<int*>(tail + 128);   // [2][128] bias term of the keys of the current key block
  int* key_reg = key_term + 2 * TC_ROWS;                // [2][128] their mask region (15: beyond the window)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Geo geo;
  geo.N = pl.N;
  geo.nrel = (2 * a.wh - 1) * (2 * a.ww - 1);
  geo.Hg = a.nWh * a.wh;
  geo.Wg = a.nWw * a.ww;
  const int N = pl.N;
  const int rel0 = (a.wh - 1) * (2 * a.ww - 1) + (a.ww - 1);
  const int nblk = (N + TC_ROWS - 1) / TC_ROWS;          // blocks of the streamed side (all keys / all queries)
  const bool use_bias = a.bias_table != nullptr;
  const bool bias_grad = PASS == 0 && use_bias && a.dbias_table != nullptr;

  if (threadIdx.x == 0) {
    mbar_init(&bars->fixed_full, 32 * TC_PROD);
    mbar_init(&bars->fixed_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->st_full[i], 32 * TC_PROD);
      mbar_init(&bars->st_empty[i], 1);
    }
    mbar_init(&bars->sdp_full, 1);
    mbar_init(&bars->pds_full, 4);
    mbar_init(&bars->out_done, 1);
    mbar_init(&bars->item_done, 1);
    mbar_init(&bars->rows_sync, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == TC_MMA_WARP) {
    tmem_alloc<512>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // item -> (head group, batch, window, block of the fixed side); the fixed side covers this rank's token shard
  auto decode = [&](int item, int& hg, int& b, int& lw, int& fb) {
    const int per_hg = pl.items / pl.hgroups;
    hg = item / per_hg;
    const int t = item % per_hg;
    b = t / pl.tiles_per_b;
    const int tile = t % pl.tiles_per_b;
    lw = tile / pl.nqb;
    fb = tile % pl.nqb;
  };

  if (warp < TC_PROD) {
    // ================================================================== producers
    uint64_t* fifo[3] = {nullptr, nullptr, nullptr};
    int pending = 0;
    auto retire_oldest = [&]() {
      fence_proxy_async_smem();
      mbar_arrive(fifo[0]);
      fifo[0] = fifo[1];
      fifo[1] = fifo[2];
      fifo[2] = nullptr;
      --pending;
    };
    auto submit = [&](uint64_t* bar) {
      tc_cp_commit();
      fifo[pending++] = bar;
      if (pending == 3) {
        tc_cp_wait<2>();
        retire_oldest();
      }
    };
    auto wait_empty = [&](uint64_t* bar, uint32_t parity, unsigned where) -> bool {
      // The consumer may need tiles whose arrival this lane still defers (copies in flight): if the buffer is not
      // free yet, let everything land and be counted in first - otherwise producer and consumer wait for each other.
      int ready = 0;
      if (lane == 0) ready = mbar_try_wait(bar, parity) ? 1 : 0;
      if (__shfl_sync(0xffffffffu, ready, 0) != 0) return true;
      tc_cp_wait<0>();
      while (pending > 0) retire_oldest();
      int got = 1;
      if (lane == 0) got = mbar_wait(bar, parity, abort_flag, status, where) ? 1 : 0;
      return __shfl_sync(0xffffffffu, got, 0) != 0;
    };
    // 128 rows = tokens tok0 .. tok0 + 127 of window `flat` (below tok_end): `queries`: q and dO, else k and v
    auto gather = [&](uint8_t* dst, int b, int flat, int tok0, int tok_end, int hg, bool queries) {
      const int ii = flat / a.nWw, jj = flat % a.nWw;
      const uint32_t d0 = smem_u32(dst);
      for (int g0 = warp * 32; g0 < TC_ROWS; g0 += 32 * TC_PROD) {
        const int tok = tok0 + g0 + lane;
        long long o0 = 0, o1 = 0;
        int slot = -1;
        if (tok < tok_end) {
          const int ti = tok / a.ww, tj = tok - ti * a.ww;
          const Home h = locate_ij(a, geo, b, ii, jj, ti, tj);
          slot = h.slot;
          if (queries) {
            o0 = h.row * (3LL * a.C) + hg * G;                               // q
            o1 = h.row * static_cast<long long>(a.C) + hg * G;               // dO (its own buffer)
          } else {
            o0 = h.row * (3LL * a.C) + a.C + hg * G;                         // k
            o1 = o0 + a.C;                                                   // v
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int idx = k * 32 + lane;
          const int rr = idx >> 3, ch = idx & 7;
          const long long s0 = __shfl_sync(0xffffffffu, o0, rr);
          const long long s1 = __shfl_sync(0xffffffffu, o1, rr);
          const int sp = __shfl_sync(0xffffffffu, slot, rr);
          const int row = g0 + rr;
          const bool valid = sp >= 0;
          const __nv_bfloat16* base0 = static_cast<const __nv_bfloat16*>(a.qkv[valid ? sp : 0]);
          const __nv_bfloat16* base1 = queries ? static_cast<const __nv_bfloat16*>(a.dout[valid ? sp : 0]) : base0;
          const uint32_t off = row * 128 + ((ch ^ (row & 7)) << 4);
          tc_cp_async16(d0 + off, base0 + (valid ? s0 + ch * 8 : 0), valid);
          tc_cp_async16(d0 + MAT + off, base1 + (valid ? s1 + ch * 8 : 0), valid);
        }
      }
    };
    uint32_t items_done = 0, st_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < pl.items && ok && !*abort_flag; item += gridDim.x, ++items_done) {
      int hg, b, lw, fb;
      decode(item, hg, b, lw, fb);
      const int flat = a.win_start[a.my_wg] + lw;
      if (!(ok = wait_empty(&bars->fixed_empty, (items_done & 1u) ^ 1u, 0x6100u))) break;
      gather(fixed_set, b, flat, pl.q0 + fb * TC_ROWS, pl.q1, hg, PASS == 0);
      submit(&bars->fixed_full);
      for (int blk = 0; blk < nblk && ok; ++blk, ++st_it) {
        const int st = st_it & 1;
        if (!(ok = wait_empty(&bars->st_empty[st], ((st_it >> 1) & 1u) ^ 1u, 0x6200u + st))) break;
        gather(stream_set + st * 2 * MAT, b, flat, blk * TC_ROWS, N, hg, PASS == 1);
        submit(&bars->st_full[st]);
      }
    }
    tc_cp_wait<0>();
    while (pending > 0) retire_oldest();
  } else if (warp == TC_MMA_WARP) {
    // ================================================================== MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(TC_ROWS, 128, 0, 0);
      constexpr uint32_t idesc_t = make_idesc_bf16(TC_ROWS, HD, 1, 1);
      constexpr uint32_t idesc_q = make_idesc_bf16(TC_ROWS, HD, 0, 1);
      const uint32_t p_addr = smem_u32(p_tiles), ds_addr = smem_u32(ds_tiles), fx = smem_u32(fixed_set);
      uint32_t items_done = 0, st_it = 0, gs = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < pl.items && ok && !*abort_flag; item += gridDim.x, ++items_done) {
        if (!(ok = mbar_wait(&bars->fixed_full, items_done & 1u, abort_flag, status, 0x6300u))) break;
        // operands: Q / dO are the fixed set in PASS 0 and the streamed set in PASS 1; K / V the other way round
        auto issue_sdp = [&](uint32_t sx, int h) {
          const uint32_t q = PASS == 0 ? fx : sx, dO = q + MAT, k = PASS == 0 ? sx : fx, v = k + MAT;
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = (h * HD + kk * 16) * 2;
            umma_bf16(tmem_base, make_smem_desc(q + off, 16, 1024), make_smem_desc(k + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = (h * HD + kk * 16) * 2;
            umma_bf16(tmem_base + COL_DP, make_smem_desc(dO + off, 16, 1024), make_smem_desc(v + off, 16, 1024), idesc_s,
                      kk > 0 ? 1u : 0u);
          }
          umma_commit(&bars->sdp_full);
        };
        for (int blk = 0; blk < nblk && ok; ++blk, ++st_it) {
          const int st = st_it & 1;
          if (!(ok = mbar_wait(&bars->st_full[st], (st_it >> 1) & 1u, abort_flag, status, 0x6400u + st))) break;
          tc_fence_after();
          const uint32_t sx = smem_u32(stream_set + st * 2 * MAT);
          if (blk == 0) issue_sdp(sx, 0);
          for (int h = 0; h < HPG && ok; ++h, ++gs) {
            if (!(ok = mbar_wait(&bars->pds_full, gs & 1u, abort_flag, status, 0x6500u))) break;
            tc_fence_after();
            const uint32_t hb = h * HD * 2;
            const uint32_t acc = blk > 0 ? 1u : 0u;
            if (PASS == 0) {
              // dQ[h] += dS K: contraction over the 128 keys of this block
#pragma unroll
              for (int k8 = 0; k8 < 8; ++k8)
                umma_bf16(tmem_base + COL_OUT + h * HD, make_smem_desc(ds_addr + (k8 >> 2) * MAT + (k8 & 3) * 32, 16, 1024),
                          make_smem_desc(sx + hb + k8 * 2048, MAT, 1024), idesc_q, (acc | (k8 > 0)) ? 1u : 0u);
            } else {
              // dV[h] += P^T dO, dK[h] += dS^T Q: contraction over the 128 queries of this block
#pragma unroll
              for (int k8 = 0; k8 < 8; ++k8)
                umma_bf16(tmem_base + COL_OUT + h * HD, make_smem_desc(p_addr + k8 * 2048, MAT, 1024),
                          make_smem_desc(sx + MAT + hb + k8 * 2048, MAT, 1024), idesc_t, (acc | (k8 > 0)) ? 1u : 0u);
#pragma unroll
              for (int k8 = 0; k8 < 8; ++k8)
                umma_bf16(tmem_base + COL_OUT + G + h * HD, make_smem_desc(ds_addr + k8 * 2048, MAT, 1024),
                          make_smem_desc(sx + hb + k8 * 2048, MAT, 1024), idesc_t, (acc | (k8 > 0)) ? 1u : 0u);
            }
            umma_commit(&bars->out_done);
            if (h == HPG - 1) umma_commit(&bars->st_empty[st]);
            // next step's scores: the next head of this block, or head 0 of the next block (once it has landed)
            if (h + 1 < HPG) {
              issue_sdp(sx, h + 1);
            } else if (blk + 1 < nblk) {
              const int st2 = (st_it + 1) & 1;
              if (!(ok = mbar_wait(&bars->st_full[st2], ((st_it + 1) >> 1) & 1u, abort_flag, status, 0x6600u + st2))) break;
              tc_fence_after();
              issue_sdp(smem_u32(stream_set + st2 * 2 * MAT), 0);
            }
          }
        }
        if (!ok) break;
        umma_commit(&bars->item_done);
        umma_commit(&bars->fixed_empty);
      }
    }
  } else {
    // ================================================================== rows
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float scale2 = a.scale * TC_LOG2E;
    uint32_t gs = 0, syncs = 0, items_done = 0;
    bool ok = true;
    auto rows_barrier = [&]() {
      mbar_arrive(&bars->rows_sync);
      if (ok) ok = mbar_wait(&bars->rows_sync, syncs & 1u, abort_flag, status, 0x7500u);
      ++syncs;
      ok = __all_sync(0xffffffffu, ok);
    };
    for (int item = blockIdx.x; item < pl.items && ok; item += gridDim.x, ++items_done) {
      int hg, b, lw, fb;
      decode(item, hg, b, lw, fb);
      const int flat = a.win_start[a.my_wg] + lw;
      const int ii = flat / a.nWw, jj = flat % a.nWw;
      const bool general = a.use_mask && ((a.sh > 0 && ii == a.nWh - 1) || (a.sw > 0 && jj == a.nWw - 1));
      // the fixed-side token of this thread: a query in PASS 0 (softmax row and output row), a key in PASS 1 (output row)
      const int ftok = pl.q0 + fb * TC_ROWS + r;
      const bool factive = ftok < pl.q1;
      const int ftk = min(ftok, N - 1);
      const int fti = ftk / a.ww, ftj = ftk - fti * a.ww;
      const Home fhome = locate_ij(a, geo, b, ii, jj, fti, ftj);
      float lse_row[HPG], d_row[HPG];
      int row_term = 0, row_reg = 0;
      bool row_active = false;
      auto load_row = [&](int tok) {
        // softmax statistics of query `tok` from its home row
        row_active = tok < N;
        const int tk = min(tok, N - 1);
        const int ti = tk / a.ww, tj = tk - ti * a.ww;
        const Home h = (PASS == 0) ? fhome : locate_ij(a, geo, b, ii, jj, ti, tj);
        row_term = ti * (2 * a.ww - 1) + tj + rel0;
        row_reg = h.region;
#pragma unroll
        for (int hh = 0; hh < HPG; ++hh) {
          const long long o = h.row * a.num_heads + hg * HPG + hh;
          lse_row[hh] = row_active ? a.lse[h.slot][o] : 0.f;
          d_row[hh] = row_active ? a.drow[h.slot][o] : 0.f;
        }
      };
      if (PASS == 0) load_row(ftok);
      if (PASS == 1) {
        // the keys of the item are fixed: their bias terms and regions once per item
        key_term[r] = fti * (2 * a.ww - 1) + ftj;
        key_reg[r] = factive ? fhome.region : 15;
        rows_barrier();
        if (!ok) break;
      }
      for (int blk = 0; blk < nblk && ok; ++blk) {
        const int kt = PASS == 0 ? (blk & 1) : 0;
        if (PASS == 0) {
          const int key = blk * TC_ROWS + r;
          const int kk = min(key, N - 1);
          const int ki = kk / a.ww, kj = kk - ki * a.ww;
          key_term[kt * TC_ROWS + r] = ki * (2 * a.ww - 1) + kj;
          key_reg[kt * TC_ROWS + r] = key < N ? region_of(a, geo, ii * a.wh + ki, jj * a.ww + kj) : 15;
          rows_barrier();
          if (!ok) break;
        } else {
          load_row(blk * TC_ROWS + r);
        }
        const int* kterm = key_term + kt * TC_ROWS;
        const int* kreg = key_reg + kt * TC_ROWS;
        for (int h = 0; h < HPG; ++h, ++gs) {
          if (ok) ok = mbar_wait(&bars->sdp_full, gs & 1u, abort_flag, status, 0x7100u);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          float lse_h = 0.f, d_h = 0.f;
#pragma unroll
          for (int hh = 0; hh < HPG; ++hh)
            if (hh == h) {
              lse_h = lse_row[hh];
              d_h = d_row[hh];
            }
          // the tiles are still being read by the previous step's products until out_done
          if (gs > 0) {
            if (ok) ok = mbar_wait(&bars->out_done, (gs - 1) & 1u, abort_flag, status, 0x7200u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          }
          const int head = hg * HPG + h;
#pragma unroll
          for (int c0 = 0; c0 < TC_ROWS; c0 += 32) {
            uint32_t sv[32], dv[32];
            tmem_ld_32x32(tmem_base + c0 + lane_base, sv);
            tmem_ld_32x32(tmem_base + COL_DP + c0 + lane_base, dv);
            tmem_ld_wait();
            float p[32], ds[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int kc = c0 + c;
              float sc = __uint_as_float(sv[c]) * scale2;
              const int kr = kreg[kc];
              if (use_bias)
                sc += __ldg(a.bias_table + static_cast<long long>(row_term - kterm[kc]) * a.num_heads + head) * TC_LOG2E;
              if (general && kr != row_reg) sc += -100.f * TC_LOG2E;
              const float pv = (kr == 15 || !row_active) ? 0.f : exp2f(sc - lse_h);
              p[c] = pv;
              ds[c] = pv * (__uint_as_float(dv[c]) - d_h);
              if (bias_grad && factive && pv != 0.f)
                atomicAdd(a.dbias_table + static_cast<long long>(row_term - kterm[kc]) * a.num_heads + head, ds[c]);
            }
            // 32 columns = 4 chunks of key block (c0 / 64)
            uint8_t* prow = p_tiles + (c0 >> 6) * MAT + r * 128;
            uint8_t* drow = ds_tiles + (c0 >> 6) * MAT + r * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const int c8 = ((c0 & 63) >> 3) + q4;
              const int o = (c8 ^ (r & 7)) << 4;
              if (PASS == 1)
                *reinterpret_cast<uint4*>(prow + o) =
                    make_uint4(pack_bf16x2(p[8 * q4], p[8 * q4 + 1]), pack_bf16x2(p[8 * q4 + 2], p[8 * q4 + 3]),
                               pack_bf16x2(p[8 * q4 + 4], p[8 * q4 + 5]), pack_bf16x2(p[8 * q4 + 6], p[8 * q4 + 7]));
              *reinterpret_cast<uint4*>(drow + o) =
                  make_uint4(pack_bf16x2(ds[8 * q4], ds[8 * q4 + 1]), pack_bf16x2(ds[8 * q4 + 2], ds[8 * q4 + 3]),
                             pack_bf16x2(ds[8 * q4 + 4], ds[8 * q4 + 5]), pack_bf16x2(ds[8 * q4 + 6], ds[8 * q4 + 7]));
            }
          }
          tc_fence_before();
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->pds_full);
        }
      }
      if (!ok) break;
      // ---- all blocks accumulated: store this thread's row of the outputs to the token's home
      if (ok) ok = mbar_wait(&bars->item_done, items_done & 1u, abort_flag, status, 0x7300u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.dqkv[fhome.slot]) + fhome.row * (3LL * a.C) + hg * G;
      constexpr int NOUT = PASS == 0 ? 1 : 2;
#pragma unroll
      for (int m = 0; m < NOUT; ++m) {
        // PASS 0: dQ (x scale) -> q columns; PASS 1: m = 0 dV -> v columns, m = 1 dK (x scale) -> k columns
        const int col_off = PASS == 0 ? 0 : (m == 0 ? 2 * a.C : a.C);
        const float mul = (PASS == 1 && m == 0) ? 1.f : a.scale;
#pragma unroll
        for (int c0 = 0; c0 < G; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + COL_OUT + m * G + c0 + lane_base, v);
          tmem_ld_wait();
          if (factive) {
#pragma unroll
            for (int c = 0; c < 32; c += 8)
              *reinterpret_cast<uint4*>(dst + col_off + c0 + c) = make_uint4(
                  pack_bf16x2(__uint_as_float(v[c]) * mul, __uint_as_float(v[c + 1]) * mul),
                  pack_bf16x2(__uint_as_float(v[c + 2]) * mul, __uint_as_float(v[c + 3]) * mul),
                  pack_bf16x2(__uint_as_float(v[c + 4]) * mul, __uint_as_float(v[c + 5]) * mul),
                  pack_bf16x2(__uint_as_float(v[c + 6]) * mul, __uint_as_float(v[c + 7]) * mul));
          }
        }
      }
      tc_fence_before();
      rows_barrier();      // everybody has read the outputs (and the key tables) before the next item overwrites them
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == TC_MMA_WARP) {
    __syncwarp();
    tmem_dealloc<512>(tmem_base);
  }
}

template <int HD>
int launch_tc_bwd_block(const WindowAttnArgs& a, void* status, cudaStream_t stream) {
  TcPlan pl;
  pl.N = a.wh * a.ww;
  pl.pair = 0;
  pl.my_nw = a.win_start[a.my_wg + 1] - a.win_start[a.my_wg];
  pl.q0 = a.my_sp * a.shardN;
  pl.q1 = pl.q0 + a.shardN < pl.N ? pl.q0 + a.shardN : pl.N;
  pl.nqb = (pl.q1 - pl.q0 + TC_ROWS - 1) / TC_ROWS;
  pl.tiles_per_b = pl.my_nw * pl.nqb;
  pl.hgroups = a.C / 64;
  pl.items = a.B * pl.tiles_per_b * pl.hgroups;
  if (pl.items <= 0) return 0;
  if (a.C % 64 != 0) return -31;
  const size_t sb = 1024 + 10 * TC_ROWS * 128 + 128 + 4 * TC_ROWS * 4 + 64;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(wattn_tc_bwd_block_kernel<HD, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb)) !=
            cudaSuccess ||
        cudaFuncSetAttribute(wattn_tc_bwd_block_kernel<HD, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb)) !=
            cudaSuccess)
      return -32;
    configured = true;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = pl.items < sms ? pl.items : sms;
  wattn_tc_bwd_block_kernel<HD, 0><<<grid, TC_THREADS, sb, stream>>>(a, pl, static_cast<KernelStatus*>(status));
  if (cudaGetLastError() != cudaSuccess) return -33;
  wattn_tc_bwd_block_kernel<HD, 1><<<grid, TC_THREADS, sb, stream>>>(a, pl, static_cast<KernelStatus*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -33;
}

template <int HD>
int launch_tc(const WindowAttnArgs& a, void* status, cudaStream_t stream) {
  using Cfg = TcCfg<HD>;
  TcPlan pl;
  pl.N = a.wh * a.ww;
  pl.pair = pl.N <= TC_KV ? 1 : 0;
  pl.my_nw = a.win_start[a.my_wg + 1] - a.win_start[a.my_wg];
  pl.q0 = a.my_sp * a.shardN;
  pl.q1 = pl.q0 + a.shardN < pl.N ? pl.q0 + a.shardN : pl.N;
  pl.nqb = (pl.q1 - pl.q0 + TC_ROWS - 1) / TC_ROWS;
  pl.tiles_per_b = pl.pair ? (pl.my_nw + 1) / 2 : pl.my_nw * pl.nqb;
  pl.hgroups = a.C / Cfg::G;
  pl.items = a.B * pl.tiles_per_b * pl.hgroups;
  if (pl.items <= 0) return 0;
  if (a.C % Cfg::G != 0) return -31;
  const int nrel = (2 * a.wh - 1) * (2 * a.ww - 1);
  const size_t fixed = 1024 + Cfg::TILE_BYTES + 256 + TC_ROWS * 12 + 5 * TC_KV * 4;
  const size_t table = static_cast<size_t>(Cfg::HPG) * nrel * 4;
  const int bias_in_smem = (a.bias_table != nullptr && fixed + table + 64 <= 232448) ? 1 : 0;
  const size_t sb = fixed + (bias_in_smem ? table : 0) + 64;
  static size_t configured = 0;
  if (sb > configured) {
    if (cudaFuncSetAttribute(wattn_tc_fwd_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb)) !=
            cudaSuccess ||
        cudaFuncSetAttribute(wattn_tc_fwd_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb)) !=
            cudaSuccess)
      return -32;
    configured = sb;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = pl.items < sms ? pl.items : sms;
  if (pl.pair)
    wattn_tc_fwd_kernel<HD, true><<<grid, TC_THREADS, sb, stream>>>(a, pl, static_cast<KernelStatus*>(status), bias_in_smem);
  else
    wattn_tc_fwd_kernel<HD, false><<<grid, TC_THREADS, sb, stream>>>(a, pl, static_cast<KernelStatus*>(status), bias_in_smem);
  return cudaGetLastError() == cudaSuccess ? 0 : -33;
}

}  // namespace

int window_attn_tc_stalls(unsigned long long* out16, int reset) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(out16, g_tc_stalls, 16 * sizeof(unsigned long long)) != cudaSuccess) return -2;
  if (reset) {
    unsigned long long zero[16] = {0};
    if (cudaMemcpyToSymbol(g_tc_stalls, zero, sizeof(zero)) != cudaSuccess) return -3;
  }
  return 0;
}

int window_attn_tc_fwd(const WindowAttnArgs& a, void* status, cudaStream_t stream) {
  if (a.num_heads <= 0 || a.C % a.num_heads != 0) return -10;
  if (a.sp < 1 || a.shardN < 1 || a.n_wg < 1 || a.n_wg > 8 || a.n_wg * a.sp > WA_MAX_PEERS) return -12;
  switch (a.C / a.num_heads) {
    case 16: return launch_tc<16>(a, status, stream);
    case 32: return launch_tc<32>(a, status, stream);
    case 64: return launch_tc<64>(a, status, stream);
    case 128: return launch_tc<128>(a, status, stream);
    default: return -13;
  }
}

// Backward on tcgen05, head dims 16 / 32 / 64. Windows of at most 64 tokens: one pass, two windows per tile, softmax
// statistics recomputed. Larger windows: two passes (dQ; dK and dV) over 128 x 128 blocks, which need the forward
// pass's log-sum-exp (`lse`, as written by window_attn_tc_fwd) and `drow` = rowsum(dO o O) per (row, head).
int window_attn_tc_bwd(const WindowAttnArgs& a, void* status, cudaStream_t stream) {
  if (a.num_heads <= 0 || a.C % a.num_heads != 0) return -10;
  if (a.sp < 1 || a.shardN < 1 || a.n_wg < 1 || a.n_wg > 8 || a.n_wg * a.sp > WA_MAX_PEERS) return -12;
  const bool large = a.wh * a.ww > TC_KV;
  if (large) {
    for (int i = 0; i < a.n_wg * a.sp; ++i)
      if (a.lse[i] == nullptr || a.drow[i] == nullptr) return -14;
  }
  switch (a.C / a.num_heads) {
    case 16: return large ? launch_tc_bwd_block<16>(a, status, stream) : launch_tc_bwd<16>(a, status, stream);
    case 32: return large ? launch_tc_bwd_block<32>(a, status, stream) : launch_tc_bwd<32>(a, status, stream);
    case 64: return large ? launch_tc_bwd_block<64>(a, status, stream) : launch_tc_bwd<64>(a, status, stream);
    default: return -13;
  }
}

}  // namespace tb
