// Persistent, warp-specialised bf16 GEMM / implicit-GEMM for sm_100a.
//
//   D[M,N] (+)= A[M,K] * B[N,K]^T, fp32 accumulation in tensor memory.
//
// Roles inside a 448-thread CTA (one CTA per SM, tiles assigned round-robin):
//   warp 0   one elected lane issues TMA loads (per-CTA, no cluster fan-out) into a ring of
//            128-byte-swizzled shared-memory stages, signalling `full[s]` by transaction bytes;
//   warp 1   owns the TMEM allocation; one elected lane issues tcgen05.mma (M=128, N=BN, K=16)
//            and commits to `empty[s]` (stage reusable) and `tfull[a]` (accumulator a complete);
//   warps 2-13 epilogue (three per 32-lane TMEM quadrant, interleaved over the column chunks): tcgen05.ld, fused
//            bias / GELU / residual / GELU-gradient / pixel-shuffle / split-K atomics; global transfers coalesced
//            through shared memory.
// Two accumulators (2*BN TMEM columns) let the epilogue of tile i overlap the main loop of tile i+1.
//
// Operand addressing is data driven (see gemm_sm100.cuh) so that the same kernel serves
//   * linear layers forward (K-major x K-major),
//   * their input gradients (B read MN-major: the weight is used untransposed),
//   * their weight gradients (both operands MN-major, contraction over tokens, split-K atomics),
//   * 3x3 convolutions (stride 1 and 2) as implicit GEMM: A rows gathered by 5-D TMA boxes with
//     zero fill outside the image, k-blocks enumerate (tap, channel chunk),
//   * convolution weight gradients (contraction over pixels, one tile group per tap).
// Two further instantiations: CTA pairs (a cluster of two drives one cta_group::2 MMA over a 256-row tile, see GemmCfg)
// and the tensor-parallel forms (A gathered from the peers' buffers, output scattered to the owners' buffers, see
// gemm_sm100.cuh).
//
// Every wait is bounded; on expiry the CTA sets its abort flag, records the site in the
// KernelStatus word, drains, releases TMEM and returns.
#include "gemm_sm100.cuh"

namespace tb {

// warp 0: TMA, warp 1: MMA, warps 2..13: epilogue (three per TMEM lane quadrant, interleaved over the 32-column
// chunks). 14 warps keep every scheduler at four warps or fewer, which allows 128 registers per thread: with 18 warps
// the cap is 96 and the epilogue spills, and its reloads miss the small L1 left beside 227 KB of shared memory.
constexpr int GEMM_EPI_WARPS = 12;
constexpr int GEMM_THREADS = 64 + 32 * GEMM_EPI_WARPS;

// CTAS = 2: a cluster of two CTAs (two SMs of one TPC) computes a 256 x BN tile with one pair-wide MMA. Each CTA stages
// its own 128 rows of A and its own half of B, so a k-block costs each SM (16 + BN / 8) KB of shared-memory fill instead
// of (16 + BN / 4) KB: the operand traffic per flop through shared memory, which bounds the single-CTA main loop, drops
// by a third at BN = 256.
template <int BN, int CTAS>
struct GemmCfg {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_ROWS = BN / CTAS;                 // rows of B staged by one CTA
  static constexpr int B_BYTES = B_ROWS * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // After the operand ring: 512 bytes of barriers, the per-warp bias slots (together 2 KB), then `bufs` buffers of
  // 2 KB per epilogue warp (1: the exchange / output staging buffer; 3: two more for the operand the epilogue reads,
  // loaded ahead by TMA). The ring takes what is left: the launcher passes the stage count to the kernel.
  static constexpr int BAR_BYTES = 512;
  static constexpr int FIXED_BASE = 2048;
  static constexpr int EPI_BUF = 2048;
  static constexpr int MAX_SMEM = 232448;   // 227 KB, the per-block limit of sm_100
  static constexpr int MAX_STAGES = 8;
  static constexpr int fixed_bytes(int bufs) { return FIXED_BASE + GEMM_EPI_WARPS * bufs * EPI_BUF; }
  static constexpr int stages_for(int bufs) {
    return (MAX_SMEM - 1024 - fixed_bytes(bufs)) / STAGE_BYTES > MAX_STAGES ? MAX_STAGES
                                                                            : (MAX_SMEM - 1024 - fixed_bytes(bufs)) / STAGE_BYTES;
  }
  static constexpr int smem_bytes(int bufs) { return stages_for(bufs) * STAGE_BYTES + fixed_bytes(bufs) + 1024; }   // + alignment slack
  // two accumulators; the allocation must be a power of two
  // behind them two 32-column accumulators of the column sums (weight-gradient form with a bias gradient, BN <= 192)
  static constexpr int SUM_COL0 = 2 * BN;
  static constexpr int TMEM_COLS = (2 * BN + 64 <= 256) ? 256 : 512;
  static constexpr bool CAN_COLSUM = CTAS == 1 && 2 * BN + 64 <= 512;
  static_assert(stages_for(3) >= 3 && smem_bytes(1) <= MAX_SMEM && smem_bytes(3) <= MAX_SMEM, "shared memory budget");
  static_assert(GEMM_EPI_WARPS * 32 * 4 + BAR_BYTES <= FIXED_BASE, "bias slots");
  static_assert(CTAS == 1 || (B_ROWS % 64 == 0), "a CTA's half of B must be whole 64-row boxes");
};

// Cycle counters of the three roles, summed over CTAs and launches since the last reset (read by gemm_read_stalls):
// [0] MMA thread busy span, [1] of it waiting for a free accumulator, [2] waiting for operand stages,
// [3] TMA thread span, [4] of it waiting for free stages, [5] first epilogue warp span, [6] of it waiting for tiles.
__device__ unsigned long long g_gemm_stalls[8];

struct TileCoord {
  int grp, m_blk, n_blk, split;
  int kb_begin, kb_end;
};

// p.num_m_tiles counts tiles of ctas * 128 rows; m_blk is returned in units of 128 rows for CTA `rank` of the pair.
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int tile, int ctas = 1, int rank = 0) {
  TileCoord t;
  t.split = tile % p.split_k;
  int r = tile / p.split_k;
  t.n_blk = r % p.num_n_tiles;
  r /= p.num_n_tiles;
  t.m_blk = (r % p.num_m_tiles) * ctas + rank;
  t.grp = r / p.num_m_tiles;
  const int per = (p.k_blocks + p.split_k - 1) / p.split_k;
  t.kb_begin = t.split * per;
  t.kb_end = min(p.k_blocks, t.kb_begin + per);
  return t;
}

// PEERS: the tensor-parallel variants (A gathered from peer buffers, output scattered to peer buffers). A separate
// instantiation, so that the plain kernel carries none of their registers and branches.
template <int BN, int CTAS, bool PEERS>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<BN, CTAS>;
  constexpr bool PAIR = CTAS == 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint8_t* fixed = smem + stages * Cfg::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(fixed);
  uint64_t* empty = full + Cfg::MAX_STAGES;
  uint64_t* tfull = empty + Cfg::MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* pfull = tempty + 2;   // pair mode, leader CTA: "the peer's half of stage s has landed"
  uint64_t* in_bar = pfull + Cfg::MAX_STAGES;   // two per epilogue warp: "the epilogue operand chunk has landed"
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(in_bar + 2 * GEMM_EPI_WARPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((3 * Cfg::MAX_STAGES + 4 + 2 * GEMM_EPI_WARPS) * 8 + 8 <= Cfg::BAR_BYTES, "barrier block");
  float* bias_slots = reinterpret_cast<float*>(fixed + Cfg::BAR_BYTES);
  uint8_t* xchg = fixed + Cfg::FIXED_BASE;
  // The ring needs a 1024-byte aligned base (128-byte swizzle atoms). The dynamic window normally starts aligned; if
  // the alignment shift does not fit into the slack the launch is refused as a whole, before any barrier exists.
  if (stages < 1 || stages > Cfg::MAX_STAGES ||
      xchg + GEMM_EPI_WARPS * p.epi_bufs * Cfg::EPI_BUF > smem_raw + p.smem_bytes) {
    if (threadIdx.x == 0) report_error(p.status, TB_ERR_BAD_ARG, 0x700u, blockIdx.x, 0u);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = PAIR ? static_cast<int>(cluster_ctarank()) : 0;     // 0 = leader (issues the MMAs)
  const int unit = PAIR ? blockIdx.x >> 1 : blockIdx.x;                 // CTA or CTA pair
  const int units = PAIR ? gridDim.x >> 1 : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::MAX_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&pfull[s], 1);
    }
    for (int i = 0; i < 2 * GEMM_EPI_WARPS; ++i) mbar_init(&in_bar[i], 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], GEMM_EPI_WARPS * CTAS);   // pair mode: both CTAs' epilogue warps release the leader's
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.map_a);
    tma_prefetch_desc(&p.map_b);
    if (p.epi_tma) {
      tma_prefetch_desc(&p.map_c);
      if (p.epi & EPI_SAVE_PRE) tma_prefetch_desc(&p.map_c2);
      if (p.epi & (EPI_RESIDUAL | EPI_MUL_DGELU)) tma_prefetch_desc(&p.map_in);
    }
    if (PEERS)
      for (int i = 0; i < p.a_peers && p.a_peers > 1; ++i) tma_prefetch_desc(&p.map_a_peer[i]);
  }
  if (warp == 1) {
    tmem_alloc<Cfg::TMEM_COLS, CTAS>(tmem_slot);
    tmem_relinquish<CTAS>();
  }
  if (Cfg::CAN_COLSUM && p.colsum != nullptr && threadIdx.x >= 64 && threadIdx.x < 64 + 128) {
    // 16 x 16 tile of ones (four 128-byte core matrices) in the bias slots, which this form does not use
    reinterpret_cast<uint32_t*>(bias_slots)[threadIdx.x - 64] = 0x3F803F80u;
    fence_proxy_async_smem();
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all(); else __syncthreads();   // barriers and allocations of both CTAs exist from here on
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (PAIR) {
    // the pair-wide MMA names one tensor-memory address for both CTAs: the two allocations must coincide
    if (threadIdx.x == 0 && ld_shared_cluster_u32(map_to_cta(tmem_slot, rank ^ 1)) != tmem_base) {
      *abort_flag = 1;
      report_error(p.status, TB_ERR_BAD_ARG, 0x701u, tmem_base, 0u);
    }
    cluster_sync_all();
    if (*abort_flag == 0 && ld_shared_cluster_u32(map_to_cta(const_cast<int*>(abort_flag), rank ^ 1)) != 0) *abort_flag = 1;
    cluster_sync_all();
  }

  const int total_tiles = p.groups * p.num_m_tiles * p.num_n_tiles * p.split_k;
  // Bound of the CTA-internal waits, in units of about a second of polling. The producer of the tensor-parallel form
  // may wait a_budget_ns (global timer) for a peer's shard; the roles that consume its stages must outlast that wait,
  // or ordinary rank skew would abort a tile whose data arrives in time. Measured polling rates put one unit between
  // 0.3 and 2 s, so 4 units per second of peer budget (+ 1) stay above it.
  const uint32_t mbar_budget = PEERS ? 1u + 4u * static_cast<uint32_t>((p.a_budget_ns + 999999999ull) / 1000000000ull) : 1u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      const long long t_begin = clock64();
      long long t_wait = 0;
      unsigned int peers_ready = 0u;   // bit per (peer, chunk) whose flag has been seen
      for (int tile = unit; tile < total_tiles && !*abort_flag; tile += units) {
        const TileCoord tc = decode_tile(p, tile, CTAS, rank);
        const int m0 = tc.m_blk * GEMM_BM;
        const int n0 = tc.n_blk * BN + rank * Cfg::B_ROWS;   // this CTA's rows of B
        int abase[5] = {0, 0, 0, 0, 0};
        if (p.a_mode == OP_TABLE_5D) {
          const int t0 = tc.m_blk % p.tile_n0;
          const int t1 = (tc.m_blk / p.tile_n0) % p.tile_n1;
          const int t2 = tc.m_blk / (p.tile_n0 * p.tile_n1);
#pragma unroll
          for (int d = 0; d < 5; ++d) abase[d] = t0 * p.a_mul0[d] + t1 * p.a_mul1[d] + t2 * p.a_mul2[d];
        }
        for (int kb = tc.kb_begin; kb < tc.kb_end; ++kb, ph ^= (s + 1 == stages), s = (s + 1 == stages) ? 0 : s + 1) {
          const long long w0 = clock64();
          if (!mbar_wait<PAIR>(&empty[s], ph ^ 1u, abort_flag, p.status, 0x100u + s, mbar_budget)) break;
          t_wait += clock64() - w0;
          uint8_t* sA = smem + s * Cfg::STAGE_BYTES;
          uint8_t* sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          int pw = 0, ph_ = 0, pb = 0;
          if (p.a_mode == OP_PIXELS_5D || p.b_mode == OP_PIXELS_5D) {
            pw = kb % p.pix_n0;
            ph_ = (kb / p.pix_n0) % p.pix_n1;
            pb = kb / (p.pix_n0 * p.pix_n1);
          }
          // ---- operand A
          if (p.a_mode == OP_KMAJOR_2D) {
            if (PEERS && p.a_peers > 1) {
              const int slot = p.a_interleave ? tc.m_blk % p.a_peers : tc.m_blk / p.a_tiles;
              const int lm = p.a_interleave ? tc.m_blk / p.a_peers : tc.m_blk % p.a_tiles;
              const int peer = (slot + p.a_first) % p.a_peers;
              const int fidx = peer * p.a_chunks + min(lm / p.a_chunk_tiles, p.a_chunks - 1);
              if (p.a_flags != nullptr && peer != p.a_first && !((peers_ready >> fidx) & 1u)) {
                // first tile from this peer: its shard must have been published (bounded wait on its flag)
                const unsigned long long w_begin = global_timer_ns();
                unsigned int seen, polls = 0;
                while (true) {
                  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.a_flags + fidx) : "memory");
                  if (static_cast<int>(seen - p.a_epoch) >= 0) break;
                  if ((++polls & 31u) == 0u && global_timer_ns() - w_begin > p.a_budget_ns) {
                    *abort_flag = 1;
                    report_error(p.status, TB_ERR_PEER_TIMEOUT, 0x500u + peer, seen, p.a_epoch);
                    break;
                  }
                  __nanosleep(50);
                }
                if (*abort_flag) break;
                fence_proxy_async_all();   // order the acquire before the asynchronous-proxy reads of the shard
                peers_ready |= 1u << fidx;
              }
              tma_load_2d(sA, &p.map_a_peer[peer], &full[s], kb * GEMM_BK, lm * GEMM_BM);
            } else {
              tma_load_2d(sA, &p.map_a, &full[s], kb * GEMM_BK, m0);
            }
          } else if (p.a_mode == OP_MNMAJOR_2D) {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_2d(sA + j * (GEMM_BK * 128), &p.map_a, &full[s], m0 + j * 64, kb * GEMM_BK);
          } else if (p.a_mode == OP_TABLE_5D) {
            const short* e = p.ktable[kb];
            int h = abase[3] + e[3];
            const CUtensorMap* m = &p.map_a;
            if (h < 0 && (p.halo_flags & 1)) {
              m = &p.map_halo_lo;
              h += 1;
            } else if (h >= p.img_h && (p.halo_flags & 2)) {
              m = &p.map_halo_hi;
              h -= p.img_h;
            }
            tma_load_5d(sA, m, &full[s], abase[0] + e[0], abase[1] + e[1], abase[2] + e[2], h, abase[4]);
          } else {  // OP_PIXELS_5D: {channels, 1, w, h, b}
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_5d(sA + j * (GEMM_BK * 128), &p.map_a, &full[s], m0 + j * 64, 0, pw * GEMM_BK, ph_, pb);
          }
          // ---- operand B
          if (p.b_mode == OP_KMAJOR_2D) {
            tma_load_2d(sB, &p.map_b, &full[s], kb * GEMM_BK, n0);
          } else if (p.b_mode == OP_MNMAJOR_2D) {
#pragma unroll
            for (int j = 0; j < Cfg::B_ROWS / 64; ++j)
              tma_load_2d(sB + j * (GEMM_BK * 128), &p.map_b, &full[s], n0 + j * 64, kb * GEMM_BK);
          } else {  // OP_PIXELS_5D with per-group (tap) displacement
            const short* g = p.grp_off[tc.grp];
            int h = ph_ * p.pix_hmul + g[2];
            const CUtensorMap* m = &p.map_b;
            if (h < 0 && (p.halo_flags & 1)) {
              m = &p.map_halo_lo;
              h += 1;
            } else if (h >= p.img_h && (p.halo_flags & 2)) {
              m = &p.map_halo_hi;
              h -= p.img_h;
            }
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_5d(sB + j * (GEMM_BK * 128), m, &full[s], n0 + j * 64, g[0], pw * GEMM_BK + g[1], h, pb);
          }
        }
      }
      atomicAdd(&g_gemm_stalls[3], static_cast<unsigned long long>(clock64() - t_begin));
      atomicAdd(&g_gemm_stalls[4], static_cast<unsigned long long>(t_wait));
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA in pair mode)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(GEMM_BM * CTAS, BN, p.a_mode == OP_MNMAJOR_2D || p.a_mode == OP_PIXELS_5D,
                                             p.b_mode == OP_MNMAJOR_2D || p.b_mode == OP_PIXELS_5D);
      const bool a_mn = (p.a_mode == OP_MNMAJOR_2D || p.a_mode == OP_PIXELS_5D);
      const bool b_mn = (p.b_mode == OP_MNMAJOR_2D || p.b_mode == OP_PIXELS_5D);
      const uint32_t a_lbo = a_mn ? GEMM_BK * 128 : 16, b_lbo = b_mn ? GEMM_BK * 128 : 16;
      const uint32_t a_kstep = a_mn ? (16 * 128) >> 4 : 32 >> 4;   // descriptor units of 16 bytes
      const uint32_t b_kstep = b_mn ? (16 * 128) >> 4 : 32 >> 4;
      const uint32_t idesc_sums = make_idesc_bf16(GEMM_BM, 16, a_mn, 0);
      const uint64_t d_ones = make_smem_desc_plain(smem_u32(bias_slots), 128, 256);
      int s = 0;
      uint32_t ph = 0, tcount = 0;
      const long long t_begin = clock64();
      long long t_acc = 0, t_ops = 0;
      for (int tile = unit; tile < total_tiles && !*abort_flag; tile += units, ++tcount) {
        const TileCoord tc = decode_tile(p, tile, CTAS, rank);
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1u;
        const long long w0 = clock64();
        if (!mbar_wait<PAIR>(&tempty[acc], aph ^ 1u, abort_flag, p.status, 0x200u + acc, mbar_budget)) break;
        t_acc += clock64() - w0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const bool sums = Cfg::CAN_COLSUM && p.colsum != nullptr && tc.n_blk == 0 && tc.grp == 0;
        const uint32_t d_sums = tmem_base + Cfg::SUM_COL0 + acc * 32;
        bool ok = true;
        for (int kb = tc.kb_begin; kb < tc.kb_end; ++kb, ph ^= (s + 1 == stages), s = (s + 1 == stages) ? 0 : s + 1) {
          const long long w1 = clock64();
          if (!mbar_wait<PAIR>(&full[s], ph, abort_flag, p.status, 0x300u + s, mbar_budget)) { ok = false; break; }
          if (PAIR && !mbar_wait<PAIR>(&pfull[s], ph, abort_flag, p.status, 0x380u + s, mbar_budget)) { ok = false; break; }
          t_ops += clock64() - w1;
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint64_t da = make_smem_desc(sA, a_lbo, 1024);
          const uint64_t db = make_smem_desc(sB, b_lbo, 1024);
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            umma_bf16<CTAS>(d_tmem, da + kk * a_kstep, db + kk * b_kstep, idesc, (kb > tc.kb_begin || kk > 0) ? 1u : 0u);
          }
          if (sums) {   // column sums of A: the same A tiles against 16 columns of ones
#pragma unroll
            for (int kk = 0; kk < GEMM_BK / 16; ++kk)
              umma_bf16<CTAS>(d_sums, da + kk * a_kstep, d_ones, idesc_sums, (kb > tc.kb_begin || kk > 0) ? 1u : 0u);
          }
          umma_commit<CTAS>(&empty[s]);     // frees stage s (in both CTAs of a pair)
        }
        if (!ok) break;
        umma_commit<CTAS>(&tfull[acc]);     // accumulator complete (in both CTAs of a pair)
      }
      atomicAdd(&g_gemm_stalls[0], static_cast<unsigned long long>(clock64() - t_begin));
      atomicAdd(&g_gemm_stalls[1], static_cast<unsigned long long>(t_acc));
      atomicAdd(&g_gemm_stalls[2], static_cast<unsigned long long>(t_ops));
    } else if (PAIR && rank == 1 && elect_one()) {
      // Peer CTA: its MMA warp has nothing to issue. It forwards "my half of stage s has landed" to the leader, whose
      // MMA thread waits for both halves before it issues.
      int s = 0;
      uint32_t ph = 0;
      for (int tile = unit; tile < total_tiles && !*abort_flag; tile += units) {
        const TileCoord tc = decode_tile(p, tile, CTAS, rank);
        bool ok = true;
        for (int kb = tc.kb_begin; kb < tc.kb_end; ++kb, ph ^= (s + 1 == stages), s = (s + 1 == stages) ? 0 : s + 1) {
          if (!mbar_wait<PAIR>(&full[s], ph, abort_flag, p.status, 0x3c0u + s, mbar_budget)) { ok = false; break; }
          mbar_arrive_remote(map_to_cta(&pfull[s], 0));
        }
        if (!ok) break;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..13)
    // tcgen05.ld hands lane l the 32 columns of accumulator row l. Global memory wants the opposite: neighbouring
    // lanes on neighbouring addresses. Every transfer of a 32 x 32 chunk (output, saved pre-activation, residual,
    // GELU input) therefore goes through the warp's 2 KB exchange buffer: row-per-lane on one side, four lanes per
    // row (eight rows, 64 contiguous bytes each, per instruction) on the global side. 16-byte vectors are XOR
    // swizzled by (row >> 1); the profiler still counts about two wavefronts per ideal one on the row-gathering
    // side (a padded 80-byte pitch measured worse), which costs a few percent of the short-K GEMMs.
    const int q = warp & 3;               // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;     // chunks part, part + 4, ... of the tile's 32-column chunks
    constexpr int CHUNKS = BN / 32;
    float* my_bias = bias_slots + (warp - 2) * 32;
    uint8_t* my_x = xchg + (warp - 2) * 2048;
    const bool has_bias = (p.epi & EPI_BIAS) != 0;
    const int grow = lane >> 2, gvec = lane & 3;      // global side: rows grow + 8 i, vector gvec
    uint32_t tcount = 0;
    const long long e_begin = clock64();
    long long e_wait = 0;
    auto xaddr = [&](int rr, int vec) -> uint4* {
      return reinterpret_cast<uint4*>(my_x + rr * 64 + (((vec ^ (rr >> 1)) & 3) << 4));
    };
    constexpr int CPW = (CHUNKS + GEMM_EPI_WARPS / 4 - 1) / (GEMM_EPI_WARPS / 4);   // chunks per warp
    if (!PAIR && !PEERS && p.epi_tma) {
      // ---- plain row-major bf16 outputs: chunks leave (and the operand the epilogue reads arrives) through TMA.
      // A chunk is 32 rows of 64 bytes in the 64-byte-swizzled layout, which is also conflict-free for the
      // row-per-lane 16-byte accesses of the warp. Buffer 0 of the warp stages outputs: one lane issues the store and,
      // before the next chunk is written, waits until the store has read the buffer. Buffers 1 and 2 receive the
      // input operand two chunks ahead (across tiles), so its latency hides behind the chunks in between.
      uint8_t* my_bufs = xchg + (warp - 2) * p.epi_bufs * Cfg::EPI_BUF;
      uint64_t* my_in = in_bar + (warp - 2) * 2;
      const bool has_in = (p.epi & (EPI_RESIDUAL | EPI_MUL_DGELU)) != 0;
      const uint32_t row_off = static_cast<uint32_t>(lane) * 64u;
      const uint32_t swz = (static_cast<uint32_t>(lane) >> 1) & 3u;
      const uint32_t out_addr = smem_u32(my_bufs);
      uint32_t issued = 0, consumed = 0;
      int pf_tile = unit, pf_ci = 0;
      auto prefetch_next = [&]() {   // issue the load of this warp's next input chunk, if there is one
        while (pf_tile < total_tiles) {
          const TileCoord t = decode_tile(p, pf_tile, 1, 0);
          const int c = part + pf_ci * (GEMM_EPI_WARPS / 4);
          const int col = t.n_blk * BN + c * 32;
          const int row = t.m_blk * GEMM_BM + q * 32;
          const bool ok = c < CHUNKS && col < p.N;
          if (++pf_ci >= CPW) {
            pf_ci = 0;
            pf_tile += units;
          }
          if (ok) {
            if (lane == 0) {
              uint64_t* b = my_in + (issued & 1u);
              mbar_expect_tx(b, Cfg::EPI_BUF);
              tma_load_2d(my_bufs + Cfg::EPI_BUF * (1 + (issued & 1u)), &p.map_in, b, col, row);
            }
            ++issued;
            return;
          }
        }
      };
      auto stage_store = [&](const CUtensorMap* map, const float (&f)[32], int col, int row) {
        if (lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t a = out_addr + row_off + (((static_cast<uint32_t>(j) ^ swz) & 3u) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(pack_bf16x2(f[8 * j], f[8 * j + 1])),
                       "r"(pack_bf16x2(f[8 * j + 2], f[8 * j + 3])), "r"(pack_bf16x2(f[8 * j + 4], f[8 * j + 5])),
                       "r"(pack_bf16x2(f[8 * j + 6], f[8 * j + 7]))
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row < p.M) {
          tma_store_2d(map, out_addr, col, row);
          bulk_commit_group();
        }
      };
      if (has_in) {
        prefetch_next();
        prefetch_next();
      }
      bool failed = false;
      for (int tile = unit; tile < total_tiles && !failed; tile += units, ++tcount) {
        const TileCoord tc = decode_tile(p, tile, 1, 0);
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1u;
        const int n0 = tc.n_blk * BN;
        const int row0 = tc.m_blk * GEMM_BM + q * 32;
        const long long ew0 = clock64();
        const bool tile_ready = mbar_wait<PAIR>(&tfull[acc], aph, abort_flag, p.status, 0x400u + acc, mbar_budget);
        if (!__all_sync(0xffffffffu, tile_ready)) break;
        e_wait += clock64() - ew0;
        tc_fence_after();
        bool released = false;
#pragma unroll
        for (int ci = 0; ci < CPW; ++ci) {
          const int c = part + ci * (GEMM_EPI_WARPS / 4);
          if (c >= CHUNKS || n0 + c * 32 >= p.N) break;   // warp-uniform
          const int nb = n0 + c * 32;
          const bool last = (ci + 1 >= CPW) || (c + GEMM_EPI_WARPS / 4 >= CHUNKS) || (nb + 32 * (GEMM_EPI_WARPS / 4) >= p.N);
          if (has_bias) {
            float b = 0.f;
            if (nb + lane < p.N)
              b = (p.epi & EPI_BIAS_F32) ? __ldg(static_cast<const float*>(p.bias) + nb + lane)
                                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[nb + lane]);
            __syncwarp();
            my_bias[lane] = b;
            __syncwarp();
          }
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
          uint4 u[4];
          if (has_in) {
            const uint32_t b = consumed & 1u;
            const bool in_ready =
                mbar_wait<false>(&my_in[b], (consumed >> 1) & 1u, abort_flag, p.status, 0x600u + b, mbar_budget);
            if (!__all_sync(0xffffffffu, in_ready)) {
              tmem_ld_wait();
              failed = true;
              break;
            }
            const uint32_t src = smem_u32(my_bufs + Cfg::EPI_BUF * (1 + b)) + row_off;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t a = src + (((static_cast<uint32_t>(j) ^ swz) & 3u) << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(u[j].x), "=r"(u[j].y), "=r"(u[j].z), "=r"(u[j].w)
                           : "r"(a)
                           : "memory");
            }
            ++consumed;
          }
          tmem_ld_wait();
          if (last) {   // the accumulator has been read: the MMA thread may start the tile after next
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
            released = true;
          }
          float f[32];
          if (has_bias) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 b4 = *reinterpret_cast<const float4*>(my_bias + j);
              f[j] = fmaf(__uint_as_float(v[j]), p.alpha, b4.x);
              f[j + 1] = fmaf(__uint_as_float(v[j + 1]), p.alpha, b4.y);
              f[j + 2] = fmaf(__uint_as_float(v[j + 2]), p.alpha, b4.z);
              f[j + 3] = fmaf(__uint_as_float(v[j + 3]), p.alpha, b4.w);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * p.alpha;
          }
          if (p.epi & EPI_SAVE_PRE) stage_store(&p.map_c2, f, nb, row0);
          if (p.epi & EPI_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = gelu_erf(f[j]);
          }
          if (has_in) {
            const bool dgelu = (p.epi & EPI_MUL_DGELU) != 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w4[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 x = unpack_bf16x2(w4[k]);
                if (dgelu) {
                  f[8 * j + 2 * k] *= gelu_erf_grad(x.x);
                  f[8 * j + 2 * k + 1] *= gelu_erf_grad(x.y);
                } else {
                  f[8 * j + 2 * k] += x.x;
                  f[8 * j + 2 * k + 1] += x.y;
                }
              }
            }
            __syncwarp();        // every lane holds its part of the input chunk: its buffer may be refilled
            prefetch_next();
          }
          stage_store(&p.map_c, f, nb, row0);
        }
        if (!released && !failed) {   // a warp without a chunk in this tile (narrow last column tile)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
        }
      }
      if (lane == 0) bulk_wait_group_read<0>();
    } else
    for (int tile = unit; tile < total_tiles; tile += units, ++tcount) {
      const TileCoord tc = decode_tile(p, tile, CTAS, rank);
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1u;
      const int n0 = tc.n_blk * BN;
      // ---- tile row -> output row index (-1: outside the output)
      int col0 = n0;
      if (p.epi & EPI_ROW_SHUFFLE) col0 = n0 % p.shuffle_cout;
      auto out_row = [&](int r) -> long long {
        if (p.epi & EPI_ROW_CONV) {
          const int t0 = tc.m_blk % p.tile_n0;
          const int t1 = (tc.m_blk / p.tile_n0) % p.tile_n1;
          const int t2 = tc.m_blk / (p.tile_n0 * p.tile_n1);
          const int w = t0 * GEMM_BM + r;
          return (w < p.out_w) ? (static_cast<long long>(t2) * p.tile_n1 + t1) * p.out_w + w : -1;
        } else if (p.epi & EPI_ROW_SHUFFLE) {
          const long long g = static_cast<long long>(tc.m_blk) * GEMM_BM + r;
          if (g >= p.M) return -1;
          const int w = static_cast<int>(g % p.out_w);
          const long long t = g / p.out_w;
          const int h = static_cast<int>(t % p.out_h);
          const long long b = t / p.out_h;
          const int qd = n0 / p.shuffle_cout;
          return ((b * 2 * p.out_h + 2 * h + (qd >> 1)) * 2 * p.out_w) + 2 * w + (qd & 1);
        } else if (PEERS && p.a_peers > 1) {
          const int slot = p.a_interleave ? tc.m_blk % p.a_peers : tc.m_blk / p.a_tiles;
          const int peer = (slot + p.a_first) % p.a_peers;
          const int lr = (p.a_interleave ? tc.m_blk / p.a_peers : tc.m_blk % p.a_tiles) * GEMM_BM + r;
          return (lr < p.a_rows) ? static_cast<long long>(peer) * p.a_rows + lr : -1;
        } else {
          const long long g = static_cast<long long>(tc.m_blk) * GEMM_BM + r;
          return (g < p.M) ? g : -1;
        }
      };
      int grows[4];   // row indices fit 32 bits (element offsets may not)
#pragma unroll
      for (int i = 0; i < 4; ++i) grows[i] = static_cast<int>(out_row(q * 32 + grow + 8 * i));
      const long long gofs = static_cast<long long>(tc.grp) * p.grp_c_stride;
      const int ncols_out = (p.epi & EPI_ROW_SHUFFLE) ? p.shuffle_cout : p.N;

      // bf16 chunk from global memory, global-side layout (zeros outside the output)
      auto fetch_chunk = [&](const __nv_bfloat16* base, long long ld, int cb, uint4 (&t)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          t[i] = make_uint4(0, 0, 0, 0);
          if (grows[i] >= 0 && cb + gvec * 8 < ncols_out)
            t[i] = *reinterpret_cast<const uint4*>(base + static_cast<long long>(grows[i]) * ld + cb + gvec * 8);
        }
      };
      // global-side registers -> row-per-lane registers
      auto turn_chunk = [&](const uint4 (&t)[4], uint4 (&u)[4]) {
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) *xaddr(grow + 8 * i, gvec) = t[i];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = *xaddr(lane, j);
      };
      // 32 floats of the row-per-lane layout to bf16 global memory
      auto store_chunk = [&](__nv_bfloat16* base, long long ld, int cb, const float (&f)[32]) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *xaddr(lane, j) = make_uint4(pack_bf16x2(f[8 * j], f[8 * j + 1]), pack_bf16x2(f[8 * j + 2], f[8 * j + 3]),
                                       pack_bf16x2(f[8 * j + 4], f[8 * j + 5]), pack_bf16x2(f[8 * j + 6], f[8 * j + 7]));
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 t = *xaddr(grow + 8 * i, gvec);
          if (grows[i] >= 0 && cb + gvec * 8 < ncols_out) {
            __nv_bfloat16* o = base + static_cast<long long>(grows[i]) * ld + cb + gvec * 8;
            if (PEERS && p.c_peers > 1 && base == static_cast<__nv_bfloat16*>(p.C) + gofs)   // the row's owner stages it
              o = static_cast<__nv_bfloat16*>(p.c_peer[grows[i] / p.c_rows]) + gofs +
                  (static_cast<long long>(p.c_slot) * p.c_rows + grows[i] % p.c_rows) * ld + cb + gvec * 8;
            *reinterpret_cast<uint4*>(o) = t;
          }
        }
      };

      // The operand the epilogue reads (GELU input of the backward pass, or the residual) does not depend on the
      // accumulator: pull it into L2 before waiting for the tile, so the DRAM latency hides behind the main loop;
      // the chunk loop then fetches it (an L2 hit) under the latency of its tcgen05.ld.
      const bool pre_aux = (p.epi & EPI_MUL_DGELU) != 0;
      const bool pre_res = !pre_aux && (p.epi & EPI_RESIDUAL) != 0;
      const __nv_bfloat16* pre_ptr = pre_aux ? p.aux : p.residual;
      const long long pre_ld = pre_aux ? p.ldaux : p.ldr;
      if (pre_aux || pre_res) {
#pragma unroll
        for (int ci = 0; ci < CPW; ++ci) {
          const int c = part + ci * (GEMM_EPI_WARPS / 4);
          if (c < CHUNKS && n0 + c * 32 < p.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (grows[i] >= 0 && col0 + c * 32 + gvec * 8 < ncols_out)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pre_ptr + static_cast<long long>(grows[i]) * pre_ld + col0 + c * 32 + gvec * 8));
          }
        }
      }
      const long long ew0 = clock64();
      // Every lane polls for itself and may leave the wait in a different iteration; the vote reconverges the warp
      // before the warp-collective tcgen05.ld below (and makes a failed wait leave the loop as one warp).
      const bool tile_ready = mbar_wait<PAIR>(&tfull[acc], aph, abort_flag, p.status, 0x400u + acc, mbar_budget);
      if (!__all_sync(0xffffffffu, tile_ready)) break;
      e_wait += clock64() - ew0;
      tc_fence_after();

#pragma unroll
      for (int ci = 0; ci < CPW; ++ci) {
        const int c = part + ci * (GEMM_EPI_WARPS / 4);
        if (c >= CHUNKS || n0 + c * 32 >= p.N) break;   // warp-uniform
        const int cb = col0 + c * 32;          // first output column of this chunk
        const int nb = n0 + c * 32;            // first logical column (bias index)
        uint4 pre[4];
        if (pre_aux || pre_res) fetch_chunk(pre_ptr, pre_ld, cb, pre);
        if (has_bias) {
          // one coalesced load per warp and chunk; the 32 values are then read back as broadcast float4
          float b = 0.f;
          if (nb + lane < p.N)
            b = (p.epi & EPI_BIAS_F32) ? __ldg(static_cast<const float*>(p.bias) + nb + lane)
                                       : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[nb + lane]);
          __syncwarp();
          my_bias[lane] = b;
          __syncwarp();
        }
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
        tmem_ld_wait();
        float f[32];
        if (has_bias) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 b4 = *reinterpret_cast<const float4*>(my_bias + j);
            f[j] = fmaf(__uint_as_float(v[j]), p.alpha, b4.x);
            f[j + 1] = fmaf(__uint_as_float(v[j + 1]), p.alpha, b4.y);
            f[j + 2] = fmaf(__uint_as_float(v[j + 2]), p.alpha, b4.z);
            f[j + 3] = fmaf(__uint_as_float(v[j + 3]), p.alpha, b4.w);
          }
        } else if (p.alpha != 1.0f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * p.alpha;
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        }
        if (p.epi & EPI_SAVE_PRE) store_chunk(static_cast<__nv_bfloat16*>(p.C2), p.ldc2, cb, f);
        if (p.epi & EPI_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = gelu_erf(f[j]);
        }
        if (p.epi & EPI_MUL_DGELU) {
          uint4 u[4];
          turn_chunk(pre, u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w4[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 x = unpack_bf16x2(w4[k]);
              f[8 * j + 2 * k] *= gelu_erf_grad(x.x);
              f[8 * j + 2 * k + 1] *= gelu_erf_grad(x.y);
            }
          }
        }
        if (p.epi & EPI_RESIDUAL) {
          uint4 u[4];
          if (pre_res) {
            turn_chunk(pre, u);
          } else {
            uint4 t[4];
            fetch_chunk(p.residual, p.ldr, cb, t);
            turn_chunk(t, u);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w4[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 x = unpack_bf16x2(w4[k]);
              f[8 * j + 2 * k] += x.x;
              f[8 * j + 2 * k + 1] += x.y;
            }
          }
        }
        if (p.epi & EPI_OUT_F32) {
          // fp32 output: two passes of 16 columns through the exchange buffer (4 floats per 16-byte vector)
          float* obase = static_cast<float*>(p.C) + gofs;
          const bool vec_ok = ((reinterpret_cast<uintptr_t>(obase) & 15) == 0) && ((p.ldc & 3) == 0);
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<float4*>(xaddr(lane, j)) =
                  make_float4(f[16 * hf + 4 * j], f[16 * hf + 4 * j + 1], f[16 * hf + 4 * j + 2], f[16 * hf + 4 * j + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 t = *reinterpret_cast<const float4*>(xaddr(grow + 8 * i, gvec));
              const int col = cb + 16 * hf + gvec * 4;
              if (grows[i] < 0 || col >= ncols_out) continue;
              float* o = obase + static_cast<long long>(grows[i]) * p.ldc + col;
              if (PEERS && p.c_peers > 1)   // the row's owner accumulates it
                o = static_cast<float*>(p.c_peer[grows[i] / p.c_rows]) + gofs +
                    static_cast<long long>(grows[i] % p.c_rows) * p.ldc + col;
              const bool full4 = vec_ok && col + 4 <= ncols_out;
              if (p.epi & EPI_ATOMIC) {
                if (full4) {
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(t.x), "f"(t.y), "f"(t.z),
                               "f"(t.w)
                               : "memory");
                } else {
                  const float tv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    if (col + e < ncols_out) atomicAdd(o + e, tv[e]);
                }
              } else {
                if (full4) {
                  *reinterpret_cast<float4*>(o) = t;
                } else {
                  const float tv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    if (col + e < ncols_out) o[e] = tv[e];
                }
              }
            }
          }
        } else {
          store_chunk(static_cast<__nv_bfloat16*>(p.C) + gofs, p.ldc, cb, f);
        }
      }
      if (Cfg::CAN_COLSUM && p.colsum != nullptr && tc.n_blk == 0 && tc.grp == 0 && part == 0) {
        uint32_t v[32];   // column 0 of the sums accumulator: lane l holds the sum of A's column (row of D) q * 32 + l
        tmem_ld_32x32(tmem_base + Cfg::SUM_COL0 + acc * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
        tmem_ld_wait();
        const int g = tc.m_blk * GEMM_BM + q * 32 + lane;
        if (g < p.M) atomicAdd(p.colsum + g, __uint_as_float(v[0]) * p.alpha);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && rank == 1) mbar_arrive_remote(map_to_cta(&tempty[acc], 0));   // the leader's MMA thread waits
        else mbar_arrive(&tempty[acc]);
      }
    }
    if (warp == 2 && lane == 0) {
      atomicAdd(&g_gemm_stalls[5], static_cast<unsigned long long>(clock64() - e_begin));
      atomicAdd(&g_gemm_stalls[6], static_cast<unsigned long long>(e_wait));
    }
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    // Give copies that are still in flight time to land before shared memory is released.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  // pair mode: neither CTA may leave while the other can still signal its barriers or read its operands
  if (PAIR) cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<Cfg::TMEM_COLS, CTAS>(tmem_base);
  }
}

// ------------------------------------------------------------------------------ host side
template <int BN, int CTAS, bool PEERS = false>
static cudaError_t launch_bn(const GemmParams& p_in, int num_sms, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, CTAS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, CTAS, PEERS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::MAX_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  GemmParams p = p_in;
  if (CTAS != 1 || PEERS) p.epi_tma = 0;
  p.epi_bufs = (p.epi_tma && (p.epi & (EPI_RESIDUAL | EPI_MUL_DGELU))) ? 3 : 1;
  p.stages = p.epi_bufs == 3 ? Cfg::stages_for(3) : Cfg::stages_for(1);
  p.smem_bytes = p.epi_bufs == 3 ? Cfg::smem_bytes(3) : Cfg::smem_bytes(1);
  const int total = p.groups * p.num_m_tiles * p.num_n_tiles * p.split_k;
  const int max_units = num_sms / CTAS;
  const int units = total < max_units ? total : max_units;
  if (units <= 0) return cudaSuccess;
  if (CTAS == 1) {
    gemm_tcgen05_kernel<BN, CTAS, PEERS><<<units, GEMM_THREADS, p.smem_bytes, stream>>>(p);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(units * CTAS);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN, CTAS, PEERS>, p);
}

cudaError_t gemm_read_stalls(unsigned long long* out8, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out8, g_gemm_stalls, 8 * sizeof(unsigned long long));
  if (e != cudaSuccess) return e;
  if (reset) {
    unsigned long long zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    e = cudaMemcpyToSymbol(g_gemm_stalls, zero, sizeof(zero));
  }
  return e;
}

cudaError_t launch_gemm(const GemmParams& p, int bn, int ctas, int num_sms, cudaStream_t stream) {
  if (ctas == 2) {
    switch (bn) {
      case 128: return launch_bn<128, 2>(p, num_sms, stream);
      case 256: return launch_bn<256, 2>(p, num_sms, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  if (p.a_peers > 1 || p.c_peers > 1) {
    switch (bn) {
      case 64: return launch_bn<64, 1, true>(p, num_sms, stream);
      case 128: return launch_bn<128, 1, true>(p, num_sms, stream);
      case 192: return launch_bn<192, 1, true>(p, num_sms, stream);
      case 256: return launch_bn<256, 1, true>(p, num_sms, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (bn) {
    case 64: return launch_bn<64, 1>(p, num_sms, stream);
    case 128: return launch_bn<128, 1>(p, num_sms, stream);
    case 192: return launch_bn<192, 1>(p, num_sms, stream);
    case 256: return launch_bn<256, 1>(p, num_sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace tb
