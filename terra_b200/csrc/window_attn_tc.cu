// Window attention, forward, on the 5th-generation tensor cores (tcgen05 / TMEM), for any window size.
//
// Same contract as window_attn.cu (window-major activations, shifted windows / halos / token shards located by index
// arithmetic, rows of other GPUs read and written through peer pointers), different engine:
//
//   * a tile is 128 query rows x one group of heads (64 channels, or one head of 128). Small windows (N <= 64 tokens)
//     are packed two to a tile (rows 0-63 / 64-127), each half attending to its own 64-key slot; larger windows are cut
//     into blocks of 128 queries that stream the window's keys and values in slots of 64 (flash-style, online softmax);
//   * warp 0 gathers Q / K / V rows (local or peer memory, plain 16-byte asynchronous copies) into 128-byte-swizzled
//     shared-memory tiles, two Q tiles and a ring of K/V slots ahead of the math;
//   * warp 1 (one elected lane) issues tcgen05.mma: S = Q K^T (M = 128, N = 64 per slot, K = head dim) into one of two
//     score buffers in tensor memory, and O_step = P V (M = 128, N = head dim, K = keys of the slots) into one of two
//     output buffers;
//   * warps 2-5 own one query row each (row = TMEM lane): tcgen05.ld the scores, add the relative-position bias (table
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

constexpr int TC_THREADS = 192;
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

template <int HD>
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
  float* bias_s = reinterpret_cast<float*>(key_reg + 2 * TC_KV);         // [HPG][nrel] x log2(e), when it fits

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
      mbar_init(&bars->q_full[i], 32);
      mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 128);
      mbar_init(&bars->o_full[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars->kv_full[i], 32);
      mbar_init(&bars->kv_empty[i], 1);
    }
    mbar_init(&bars->rows_sync, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<Cfg::TMEM_COLS>(tmem_slot);
    tmem_relinquish();
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

  if (warp == 0) {
    // ================================================================== producer: gathers into swizzled tiles
    uint64_t* fifo[3] = {nullptr, nullptr, nullptr};   // barriers of the copy groups still in flight (oldest first)
    int pending = 0;
    auto retire_oldest = [&]() {
      // the oldest group of this lane has landed: make it visible to the tensor core's proxy, then count the lane in
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
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, where) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      return ok != 0;
    };
    // table rows [row0, row0 + nrows): tokens tok0 .. of shifted-frame window `flat` (-1: no window), valid below tok_end
    auto fill_table = [&](int row0, int nrows, int b, int flat, int tok0, int tok_end) {
      const int ii = flat >= 0 ? flat / a.nWw : 0, jj = flat >= 0 ? flat % a.nWw : 0;
      for (int r = lane; r < nrows; r += 32) {
        const int tok = tok0 + r;
        if (flat >= 0 && tok < tok_end) {
          const Home h = locate(a, geo, b, ii, jj, tok);
          prow_ofs[row0 + r] = h.row;
          prow_slot[row0 + r] = h.slot;
        } else {
          prow_ofs[row0 + r] = 0;
          prow_slot[row0 + r] = -1;
        }
      }
    };
    // rows [0, nrows) of matrix m0 (0 q, 1 k) into dst0 and, with dst1, matrix m0 + 1 (v) into dst1; rows without a
    // home are zero filled. Tile layout: 64-channel sub-tiles of nrows x 128 bytes, 16-byte chunks XOR-swizzled by row.
    auto copy_rows = [&](uint8_t* dst0, uint8_t* dst1, int nrows, int hg, int m0) {
      __syncwarp();
      const int per_row = 8 * NSUB;
      const uint32_t d0 = smem_u32(dst0), d1 = dst1 != nullptr ? smem_u32(dst1) : 0u;
      for (int idx = lane; idx < nrows * per_row; idx += 32) {
        const int r = idx / per_row, ch = idx % per_row;
        const int sub = ch >> 3, c = ch & 7;
        const int sl = prow_slot[r];
        const bool valid = sl >= 0;
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(a.qkv[valid ? sl : 0]) +
                                   (valid ? prow_ofs[r] * row_ld + m0 * a.C + hg * G + ch * 8 : 0);
        const uint32_t off = sub * (nrows * 128) + r * 128 + ((c ^ (r & 7)) << 4);
        tc_cp_async16(d0 + off, src, valid);
        if (dst1 != nullptr) tc_cp_async16(d1 + off, src + (valid ? a.C : 0), valid);
      }
      __syncwarp();   // the table may be rewritten
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
          fill_table(0, 64, it.b, flat0, 0, N);
          fill_table(64, 64, it.b, it.nwin > 1 ? flat0 + 1 : -1, 0, N);
        } else {
          fill_table(0, TC_ROWS, it.b, flat0, pl.q0 + it.qb * TC_ROWS, pl.q1);
        }
        copy_rows(qt, nullptr, TC_ROWS, it.hg, 0);
        submit(&bars->q_full[qb]);
        ++q_it;
      }
      // ---- K / V slots in the order the math consumes them
      const int nslots = pl.pair ? it.nwin : it.nkv;
      for (int s = 0; s < nslots && ok; ++s) {
        const int ks = kv_it % Cfg::NSLOT;
        if (!(ok = wait_empty(&bars->kv_empty[ks], ((kv_it / Cfg::NSLOT) & 1u) ^ 1u, 0x1200u + ks))) break;
        uint8_t* kt = kv_slots + ks * Cfg::SLOT_BYTES;
        if (pl.pair) fill_table(0, TC_KV, it.b, flat0 + s, 0, N);
        else fill_table(0, TC_KV, it.b, flat0, s * TC_KV, N);
        copy_rows(kt, kt + Cfg::KV_BYTES, TC_KV, it.hg, 1);
        submit(&bars->kv_full[ks]);
        ++kv_it;
      }
    }
    tc_cp_wait<0>();
    while (pending > 0) retire_oldest();
  } else if (warp == 1) {
    // ================================================================== MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(TC_ROWS, TC_KV, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TC_ROWS, HD, 0, 1);
      uint32_t q_it = 0, kv_it = 0, gs = 0;   // Q tiles, K/V slots and steps consumed so far
      bool ok = true;
      for (int item = blockIdx.x; item < pl.items && ok && !*abort_flag; item += gridDim.x) {
        const TcItem it = tc_decode<HPG>(pl, item);
        const int qb = q_it & 1;
        if (!(ok = mbar_wait(&bars->q_full[qb], (q_it >> 1) & 1u, abort_flag, status, 0x2100u + qb))) break;
        const uint32_t q_addr = smem_u32(q_tiles + qb * Cfg::Q_BYTES);
        const int spi = pl.pair ? it.nwin : 1;   // slots per iteration
        auto issue_qk = [&](int n, uint32_t step) -> bool {
          const int j = n / HPG, h = n % HPG;
          const uint32_t buf = step & 1u;
          for (int s = 0; s < spi; ++s) {
            const uint32_t kslot = kv_it + (pl.pair ? s : j);
            const int ks = kslot % Cfg::NSLOT;
            if (h == 0 && !mbar_wait(&bars->kv_full[ks], (kslot / Cfg::NSLOT) & 1u, abort_flag, status, 0x2200u + ks))
              return false;
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
          if (!(ok = mbar_wait(&bars->p_full[buf], (gs >> 1) & 1u, abort_flag, status, 0x2300u + buf))) break;
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
    // barrier among the softmax threads; bounded like every other wait, so a failed CTA cannot hang in it
    auto rows_barrier = [&]() {
      mbar_arrive(&bars->rows_sync);
      if (ok) ok = mbar_wait(&bars->rows_sync, syncs & 1u, abort_flag, status, 0x3500u);
      ++syncs;
      ok = __all_sync(0xffffffffu, ok);
    };
    for (int item = blockIdx.x; item < pl.items && ok; item += gridDim.x) {
      const TcItem it = tc_decode<HPG>(pl, item);
      if (bias_in_smem && it.hg != cur_hg) {
        // relative-position bias of this head group, pre-multiplied by log2(e)
        rows_barrier();      // nobody reads the previous group's table any more
        for (int i = threadIdx.x - 64; i < HPG * geo.nrel; i += 128) {
          const int h = i / geo.nrel, e = i % geo.nrel;
          bias_s[i] = a.bias_table[static_cast<long long>(e) * a.num_heads + it.hg * HPG + h] * TC_LOG2E;
        }
        rows_barrier();
        cur_hg = it.hg;
        if (!ok) break;
      }
      const int sl = pl.pair ? (r >> 6) : 0;
      const int flat = a.win_start[a.my_wg] + it.w0 + sl;
      const int tok = pl.pair ? (r & 63) : pl.q0 + it.qb * TC_ROWS + r;
      const bool active = pl.pair ? (sl < it.nwin && tok < N) : (tok < pl.q1);
      const int fl = (pl.pair && sl >= it.nwin) ? flat - sl : flat;   // clamp to an existing window
      const int ii = fl / a.nWw, jj = fl % a.nWw;
      const int tk = min(tok, N - 1);
      const Home home = locate(a, geo, it.b, ii, jj, tk);
      const int row_term = (tk / a.ww) * (2 * a.ww - 1) + (tk % a.ww) + rel0;
      const bool general = a.use_mask && ((a.sh > 0 && ii == a.nWh - 1) || (a.sw > 0 && jj == a.nWw - 1));
      const bool store_row = active && (!pl.pair || (tok >= pl.q0 && tok < pl.q1));
      if (pl.pair) {
        // the keys of a slot are the tokens of the window itself: every row publishes its own terms
        if ((r & 63) < TC_KV) {
          key_term[sl * TC_KV + (r & 63)] = (tk / a.ww) * (2 * a.ww - 1) + (tk % a.ww);
          key_reg[sl * TC_KV + (r & 63)] = (tok < N) ? home.region : 15;
        }
        rows_barrier();
        if (!ok) break;
      }
      float m_run[HPG], l_run[HPG], oacc[G];
#pragma unroll
      for (int h = 0; h < HPG; ++h) {
        m_run[h] = TC_NEG;
        l_run[h] = 0.f;
      }
#pragma unroll
      for (int c = 0; c < G; ++c) oacc[c] = 0.f;
      float alpha_prev = 0.f;
      int h_prev = 0;

      auto fold_output = [&](uint32_t step, int h, float alpha) {
        // O of `step` (head h) is complete in tensor memory: acc = acc * alpha + O
        const uint32_t buf = step & 1u;
        if (ok) ok = mbar_wait(&bars->o_full[buf], (step >> 1) & 1u, abort_flag, status, 0x3300u + buf);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + Cfg::O_COL + buf * HD + c0 + lane_base, v);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c0 + c < HD) {
#pragma unroll
              for (int hh = 0; hh < HPG; ++hh)
                if (hh == h) oacc[hh * HD + c0 + c] = fmaf(oacc[hh * HD + c0 + c], alpha, __uint_as_float(v[c]));
            }
          }
        }
        tc_fence_before();
      };

      for (int n = 0; n < it.T; ++n, ++gs) {
        const int j = n / HPG, h = n % HPG;
        const uint32_t buf = gs & 1u;
        const int kt = pl.pair ? sl : (j & 1);   // which key table
        if (!pl.pair && h == 0) {
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
        if (ok) ok = mbar_wait(&bars->s_full[buf], (gs >> 1) & 1u, abort_flag, status, 0x3100u + buf);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
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
        // ---- scale, bias, mask (base-2 domain)
        const int* kterm = key_term + kt * TC_KV;
        const int* kreg = key_reg + kt * TC_KV;
        const bool padded = pl.pair ? (N < TC_KV) : ((j + 1) * TC_KV > N);
        float mx = TC_NEG;
        if (use_bias) {
          const float* table = bias_in_smem ? bias_s + h * geo.nrel : nullptr;
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 t4 = *reinterpret_cast<const int4*>(kterm + c4);
            const int tt[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int idx = row_term - tt[e];
              const float bv = bias_in_smem ? table[idx]
                                            : __ldg(a.bias_table + static_cast<long long>(idx) * a.num_heads + it.hg * HPG + h) * TC_LOG2E;
              s[c4 + e] = fmaf(s[c4 + e], scale2, bv);
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < TC_KV; ++c) s[c] *= scale2;
        }
        if (general || padded) {
#pragma unroll
          for (int c4 = 0; c4 < TC_KV; c4 += 4) {
            const int4 g4 = *reinterpret_cast<const int4*>(kreg + c4);
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
        // ---- probabilities (bf16) into the A-operand tile: row r, 16-byte chunk c8 at (c8 ^ (r & 7))
        {
          uint8_t* prow = p_bufs + buf * Cfg::P_BYTES + sl * Cfg::P_TILE + r * 128;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const uint4 pk = make_uint4(pack_bf16x2(s[8 * c8], s[8 * c8 + 1]), pack_bf16x2(s[8 * c8 + 2], s[8 * c8 + 3]),
                                        pack_bf16x2(s[8 * c8 + 4], s[8 * c8 + 5]), pack_bf16x2(s[8 * c8 + 6], s[8 * c8 + 7]));
            *reinterpret_cast<uint4*>(prow + ((c8 ^ (r & 7)) << 4)) = pk;
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars->p_full[buf]);
        // ---- the previous step's output is ready by now: fold it in while the tensor core works on this step
        if (n > 0) fold_output(gs - 1, h_prev, alpha_prev);
        if (!ok) break;
        alpha_prev = alpha;
        h_prev = h;
      }
      if (ok && it.T > 0) fold_output(gs - 1, h_prev, alpha_prev);
      if (!ok) break;
      // ---- normalise and store the row to its home (this GPU's buffer or a peer's)
      if (store_row) {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.out[home.slot]) + home.row * a.C + it.hg * G;
#pragma unroll
        for (int h = 0; h < HPG; ++h) {
          const float inv = 1.f / l_run[h];
#pragma unroll
          for (int c = 0; c < HD; c += 8) {
            const float* o = oacc + h * HD + c;
            *reinterpret_cast<uint4*>(dst + h * HD + c) =
                make_uint4(pack_bf16x2(o[0] * inv, o[1] * inv), pack_bf16x2(o[2] * inv, o[3] * inv),
                           pack_bf16x2(o[4] * inv, o[5] * inv), pack_bf16x2(o[6] * inv, o[7] * inv));
          }
        }
        if (a.lse[home.slot] != nullptr) {
          float* lse = a.lse[home.slot] + home.row * a.num_heads + it.hg * HPG;
#pragma unroll
          for (int h = 0; h < HPG; ++h) lse[h] = m_run[h] + log2f(l_run[h]);
        }
      }
      if (pl.pair) rows_barrier();   // the key tables are rewritten by the next item
    }
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let copies and products in flight land before smem / TMEM go away
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<Cfg::TMEM_COLS>(tmem_base);
  }
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
  const size_t fixed = 1024 + Cfg::TILE_BYTES + 256 + TC_ROWS * 12 + 4 * TC_KV * 4;
  const size_t table = static_cast<size_t>(Cfg::HPG) * nrel * 4;
  const int bias_in_smem = (a.bias_table != nullptr && fixed + table + 64 <= 232448) ? 1 : 0;
  const size_t sb = fixed + (bias_in_smem ? table : 0) + 64;
  static size_t configured = 0;
  if (sb > configured) {
    if (cudaFuncSetAttribute(wattn_tc_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb)) !=
        cudaSuccess)
      return -32;
    configured = sb;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = pl.items < sms ? pl.items : sms;
  wattn_tc_fwd_kernel<HD><<<grid, TC_THREADS, sb, stream>>>(a, pl, static_cast<KernelStatus*>(status), bias_in_smem);
  return cudaGetLastError() == cudaSuccess ? 0 : -33;
}

}  // namespace

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

}  // namespace tb
