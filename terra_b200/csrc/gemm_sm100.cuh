// Parameter block shared by the host launcher and the tcgen05 GEMM / implicit-GEMM kernel.
#pragma once
#include "common.cuh"

namespace tb {

// How the producer warp turns (tile, k-block) into TMA coordinates for an operand.
enum : int {
  OP_KMAJOR_2D = 0,    // tensor [rows][K], K contiguous           -> one box {64, rows}
  OP_MNMAJOR_2D = 1,   // tensor [K][rows], rows contiguous        -> rows/64 boxes {64, 64}
  OP_TABLE_5D = 2,     // K-major rows gathered from a 5-D tensor (implicit-GEMM convolution):
                       //   coords = tile base + per-k-block offset table
  OP_PIXELS_5D = 3,    // MN-major, contraction runs over pixels of a 5-D tensor (conv weight grad)
};

enum : int {
  EPI_BIAS = 1 << 0,       // + bias[col]
  EPI_GELU = 1 << 1,       // exact-erf GELU after bias
  EPI_SAVE_PRE = 1 << 2,   // also store the pre-activation (bf16) to C2
  EPI_RESIDUAL = 1 << 3,   // + R[row][col]
  EPI_MUL_DGELU = 1 << 4,  // acc *= gelu'(aux[row][col])      (backward of fc1's GELU)
  EPI_OUT_F32 = 1 << 5,    // C is fp32
  EPI_ATOMIC = 1 << 6,     // fp32 atomic accumulate into C (split-K)
  EPI_ROW_CONV = 1 << 7,   // rows are (w-chunk, h, b) tiles of an image of width out_w
  EPI_ROW_SHUFFLE = 1 << 8,// transposed-conv 2x2/s2 pixel shuffle store
  EPI_BIAS_F32 = 1 << 9,   // bias pointer is fp32
  EPI_SILU_MUL = 1 << 10,  // reserved
};

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_MAX_KTABLE = 128;

struct GemmParams {
  CUtensorMap map_a;
  CUtensorMap map_b;
  // Row-stripe domain parallelism: image rows above / below the local stripe live in separate one-row tensors
  // (received from the neighbours). The image operand (A in OP_TABLE_5D, B in OP_PIXELS_5D) reads row -1 from
  // map_halo_lo and row img_h from map_halo_hi when the corresponding flag is set; otherwise those rows are zero.
  CUtensorMap map_halo_lo;
  CUtensorMap map_halo_hi;
  int halo_flags;              // bit 0: lo valid, bit 1: hi valid
  int img_h;                   // rows of the local image
  int M, N, K;                 // logical output rows, cols, contraction length (elements)
  int num_m_tiles, num_n_tiles;
  int k_blocks;                // total 64-wide k-blocks
  int split_k;                 // >1: tiles are (m, n, split); needs EPI_ATOMIC
  int groups;                  // extra outermost tile dimension (conv taps for the weight gradient); >=1
  int a_mode, b_mode;
  // OP_TABLE_5D: tile decomposition m_tile -> (t0, t1, t2) with extents (n0, n1, *), per-dimension multipliers,
  // and the k-block offset table {c, parity, dw, dh}.
  int tile_n0, tile_n1;
  int a_mul0[5], a_mul1[5], a_mul2[5];
  short ktable[GEMM_MAX_KTABLE][4];
  // OP_PIXELS_5D: k-block -> (wc, h, b) with extents (pix_n0 = chunks per row, pix_n1 = rows).
  int pix_n0, pix_n1;
  int pix_hmul;                // input row = h * pix_hmul + dh   (2 for the stride-2 convolution)
  short grp_off[16][4];        // per group (tap): {parity, dw, dh, unused} applied to operand B
  long long grp_c_stride;      // output offset (elements) between groups
  // epilogue
  int epi;
  void* C;
  void* C2;
  const void* bias;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* aux;
  long long ldc, ldc2, ldr, ldaux;
  int out_w, out_h;            // EPI_ROW_CONV / EPI_ROW_SHUFFLE geometry
  int shuffle_cout;
  float alpha;
  KernelStatus* status;
  // Epilogue through TMA (plain row-major bf16 outputs, single-CTA tiles): every epilogue warp stages its 32 x 32
  // chunk in shared memory in the 64-byte-swizzled layout and one lane stores it through map_c / map_c2; the operand
  // the epilogue reads (residual, or the GELU input of the backward pass) arrives through map_in, loaded two chunks
  // ahead into per-warp buffers. epi_bufs = buffers of 2 KB per epilogue warp (1: output staging; 3: + two inputs).
  // stages / smem_bytes: the launcher sizes the operand ring with what the epilogue buffers leave.
  float* colsum;               // weight-gradient form: += column sums of operand A over the contraction (see GemmEpilogue)
  CUtensorMap map_c, map_c2, map_in;
  int epi_tma;
  int epi_bufs;
  int stages;
  int smem_bytes;
  // Tensor-parallel fusions over peer memory (NVLink), single-CTA mode, 2-D K-major A:
  //  * all-gather -> GEMM: the rows of A live in a_peers buffers of a_rows rows each (one per GPU, one tensor map per
  //    buffer); m tile i reads tile i / a_peers of peer (i % a_peers + a_first) % a_peers: every GPU starts with a
  //    tile of its own rows, and local and remote tiles alternate, so NVLink is busy during the whole kernel rather
  //    than after the local part. Output rows are numbered peer * a_rows + row. With a_flags the TMA
  //    thread itself waits (bounded by a_budget_ns of the global timer) until a_flags[peer] has reached a_epoch
  //    before the first load from that peer: the peers publish "my shard is written" with a one-way signal and no
  //    barrier sits in front of the GEMM.
  //  * GEMM -> reduce-scatter: with c_peers > 1 output row g goes to the buffer of its owner, c_peer[g / c_rows].
  //    fp32 atomic output: vector reductions into row g % c_rows of the owner's accumulation buffer. bf16 output:
  //    plain stores into slot c_slot (this GPU's) of the owner's [c_peers][c_rows] staging, which the owner sums.
  int a_peers, a_rows, a_tiles, a_first;
  int a_interleave;            // 1: local and remote tiles alternate (direct peer loads); 0: own shard first, then peer by peer
  int a_chunks, a_chunk_tiles; // flags per peer: flag [peer * a_chunks + tile / a_chunk_tiles] covers a_chunk_tiles m tiles
  CUtensorMap map_a_peer[8];
  const unsigned int* a_flags;
  unsigned int a_epoch;
  unsigned long long a_budget_ns;
  int c_peers, c_rows, c_slot;
  void* c_peer[8];
};

}  // namespace tb
