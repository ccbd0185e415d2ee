// Host-side construction of TMA tensor maps and GemmParams for the tcgen05 GEMM family.
// No allocation happens here: callers pass every buffer.
#include "gemm_sm100.cuh"
#include "host_api.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace tb {

cudaError_t launch_gemm(const GemmParams& p, int bn, int ctas, int num_sms, cudaStream_t stream);
cudaError_t gemm_read_stalls(unsigned long long* out8, bool reset);

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// rank <= 5, bf16 elements, 128-byte swizzle, zero fill outside the tensor.
// dims/box are innermost first; strides (bytes) are for dims 1..rank-1.
static int make_tensor_map_bf16_swizzled(CUtensorMap* out, const void* base, int rank, const unsigned long long* dims,
                                         const unsigned long long* strides_bytes, const unsigned int* box,
                                         CUtensorMapSwizzle swizzle);

int make_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const unsigned long long* dims,
                         const unsigned long long* strides_bytes, const unsigned int* box) {
  return make_tensor_map_bf16_swizzled(out, base, rank, dims, strides_bytes, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

static int make_tensor_map_bf16_swizzled(CUtensorMap* out, const void* base, int rank, const unsigned long long* dims,
                                         const unsigned long long* strides_bytes, const unsigned int* box,
                                         CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  // cuTensorMapEncodeTiled is a driver call: it needs the primary context bound to THIS thread. A thread that
  // has only queried the device so far (e.g. an autograd worker before its first runtime call) has none, so
  // bind it once per thread through the runtime.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return -2;
  for (int i = 0; i + 1 < rank; ++i)
    if (gstr[i] % 16 != 0) return -3;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                  gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -100 - static_cast<int>(r);
}

static int map_2d(CUtensorMap* out, const void* base, long long inner, long long outer, long long ld_elems,
                  int box_inner, int box_outer) {
  unsigned long long dims[2] = {static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer)};
  unsigned long long str[1] = {static_cast<unsigned long long>(ld_elems) * 2ull};
  unsigned int box[2] = {static_cast<unsigned int>(box_inner), static_cast<unsigned int>(box_outer)};
  return make_tensor_map_bf16(out, base, 2, dims, str, box);
}

// 32 x 32 chunk of a row-major bf16 matrix in the 64-byte-swizzled layout (the epilogue's staging format)
static int map_chunk(CUtensorMap* out, const void* base, long long cols, long long rows, long long ld_elems) {
  unsigned long long dims[2] = {static_cast<unsigned long long>(cols), static_cast<unsigned long long>(rows)};
  unsigned long long str[1] = {static_cast<unsigned long long>(ld_elems) * 2ull};
  unsigned int box[2] = {32u, 32u};
  return make_tensor_map_bf16_swizzled(out, base, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

// Plain row-major bf16 outputs leave through TMA stores (and the residual / GELU-input operand arrives through TMA
// loads) when every matrix qualifies for a tensor map; otherwise the epilogue keeps its per-lane global accesses.
static void try_tma_epilogue(GemmParams& p, long long M, long long N) {
  static const bool enabled = [] {
    const char* e = std::getenv("TERRA_GEMM_TMA_EPILOGUE");
    return e == nullptr || std::atoi(e) != 0;
  }();
  p.epi_tma = 0;
  const int f = p.epi;
  if (!enabled || (f & (EPI_OUT_F32 | EPI_ATOMIC | EPI_ROW_CONV | EPI_ROW_SHUFFLE))) return;
  if ((f & EPI_RESIDUAL) && (f & EPI_MUL_DGELU)) return;
  // The input buffers cost the operand ring one or two stages. A long contraction hides the epilogue behind its main
  // loop anyway and wants the deeper ring instead (K = 1536 with a residual measured 15 % slower on three stages).
  if ((f & (EPI_RESIDUAL | EPI_MUL_DGELU)) && p.k_blocks > 12) return;
  if (p.a_peers > 1 || p.c_peers > 1 || p.groups != 1 || p.C == nullptr) return;
  if (map_chunk(&p.map_c, p.C, N, M, p.ldc) != 0) return;
  if ((f & EPI_SAVE_PRE) && map_chunk(&p.map_c2, p.C2, N, M, p.ldc2) != 0) return;
  if ((f & EPI_RESIDUAL) && map_chunk(&p.map_in, p.residual, N, M, p.ldr) != 0) return;
  if ((f & EPI_MUL_DGELU) && map_chunk(&p.map_in, p.aux, N, M, p.ldaux) != 0) return;
  p.epi_tma = 1;
}

static int pick_bn(long long N, int requested) {
  if (requested == 64 || requested == 128 || requested == 192 || requested == 256) return requested;
  if (N <= 64) return 64;
  if (N % 256 == 0 && N >= 1024) return 256;
  if (N % 192 == 0) return 192;   // 384, 768, 1152: no partial tile, less operand traffic per flop than 128
  return 128;
}

static void fill_epilogue(GemmParams& p, const GemmEpilogue& e) {
  p.epi = e.flags;
  p.C = e.C;
  p.C2 = e.C2;
  p.bias = e.bias;
  p.residual = static_cast<const __nv_bfloat16*>(e.residual);
  p.aux = static_cast<const __nv_bfloat16*>(e.aux);
  p.ldc = e.ldc;
  p.ldc2 = e.ldc2;
  p.ldr = e.ldr;
  p.ldaux = e.ldaux;
  p.alpha = e.alpha;
  p.status = static_cast<KernelStatus*>(e.status);
  p.colsum = e.colsum;
}

int gemm_bf16(const GemmOperand& A, const GemmOperand& B, long long M, long long N, long long K,
              const GemmEpilogue& epi, int split_k, int bn_request, int num_sms, cudaStream_t stream) {
  GemmPeers none;
  std::memset(&none, 0, sizeof(none));
  return gemm_bf16_peers(A, B, M, N, K, epi, none, split_k, bn_request, num_sms, stream);
}

int gemm_bf16_peers(const GemmOperand& A, const GemmOperand& B, long long M, long long N, long long K,
                    const GemmEpilogue& epi, const GemmPeers& peers, int split_k, int bn_request, int num_sms,
                    cudaStream_t stream) {
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  const bool gather_a = peers.a_peers > 1;
  const bool scatter_c = peers.c_peers > 1;
  if (gather_a && (A.mn_major || peers.a_peers > 8 || peers.a_rows <= 0 || M != peers.a_rows * peers.a_peers)) return -12;
  if (scatter_c && (peers.c_peers > 8 || peers.c_rows <= 0 || M != peers.c_rows * peers.c_peers)) return -13;
  // scattered output is either the fp32 atomic form or the plain bf16 form (one staging slot per source GPU)
  if (scatter_c && (epi.flags & EPI_OUT_F32) && !(epi.flags & EPI_ATOMIC)) return -13;
  if ((gather_a || scatter_c) && bn_request >= 1000) return -14;   // single-CTA tiles only
  // CTA pairs (256-row tiles, one MMA over two SMs): explicit request 1000 + BN, or by policy for the shapes where
  // the main loop dominates (long contraction or wide output) when TERRA_GEMM_2CTA=1.
  int ctas = 1;
  if (bn_request >= 1000) {
    ctas = 2;
    bn_request -= 1000;
    if (bn_request != 128 && bn_request != 256) return -11;
  } else {
    static const int policy = [] {
      const char* e = std::getenv("TERRA_GEMM_2CTA");
      return (e != nullptr) ? std::atoi(e) : 0;
    }();
    if (policy == 1 && !gather_a && !scatter_c && M >= 512 && N >= 128 &&
        (bn_request == 0 || bn_request == 128 || bn_request == 256)) {
      ctas = 2;
      if (bn_request == 0) bn_request = (N % 256 == 0 || N >= 1024) ? 256 : 128;
    }
  }
  if (epi.colsum != nullptr) {
    // column sums ride on the weight-gradient form only, and need room for their accumulators behind the tile's
    if (!A.mn_major || (epi.flags & EPI_BIAS) || !(epi.flags & EPI_ATOMIC) || ctas != 1 || gather_a || scatter_c) return -15;
    if (bn_request == 256 || (bn_request == 0 && pick_bn(N, 0) == 256)) bn_request = (N % 192 == 0) ? 192 : 128;
  }
  const int bn = pick_bn(N, bn_request);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.num_m_tiles = static_cast<int>((M + GEMM_BM * ctas - 1) / (GEMM_BM * ctas));
  if (gather_a || scatter_c) ctas = 1;
  if (gather_a) {
    p.a_peers = peers.a_peers;
    p.a_rows = static_cast<int>(peers.a_rows);
    p.a_tiles = static_cast<int>((peers.a_rows + GEMM_BM - 1) / GEMM_BM);
    p.a_first = peers.rank % peers.a_peers;
    p.a_flags = static_cast<const unsigned int*>(peers.a_flags);
    p.a_epoch = peers.a_epoch;
    p.a_budget_ns = peers.a_budget_ns > 0 ? peers.a_budget_ns : 2000000000ull;
    p.a_interleave = peers.a_interleave;
    p.a_chunks = peers.a_chunks < 1 ? 1 : (peers.a_chunks > 4 ? 4 : peers.a_chunks);
    p.a_chunk_tiles = (p.a_tiles + p.a_chunks - 1) / p.a_chunks;
    p.num_m_tiles = p.a_tiles * p.a_peers;
    for (int i = 0; i < peers.a_peers; ++i) {
      const int rc_i = map_2d(&p.map_a_peer[i], peers.a_ptr[i], K, peers.a_rows, A.ld, GEMM_BK, GEMM_BM);
      if (rc_i != 0) return rc_i - 3000;
    }
  }
  if (scatter_c) {
    p.c_peers = peers.c_peers;
    p.c_rows = static_cast<int>(peers.c_rows);
    p.c_slot = peers.rank % peers.c_peers;
    for (int i = 0; i < peers.c_peers; ++i) p.c_peer[i] = peers.c_ptr[i];
  }
  p.num_n_tiles = static_cast<int>((N + bn - 1) / bn);
  p.k_blocks = static_cast<int>((K + GEMM_BK - 1) / GEMM_BK);
  p.groups = 1;
  if (split_k < 1) split_k = 1;
  if (split_k > p.k_blocks) split_k = p.k_blocks;
  {
    const int per = (p.k_blocks + split_k - 1) / split_k;
    split_k = (p.k_blocks + per - 1) / per;   // no empty split
  }
  p.split_k = split_k;
  if (split_k > 1 && !((epi.flags & EPI_ATOMIC) && (epi.flags & EPI_OUT_F32))) return -10;
  p.a_mode = A.mn_major ? OP_MNMAJOR_2D : OP_KMAJOR_2D;
  p.b_mode = B.mn_major ? OP_MNMAJOR_2D : OP_KMAJOR_2D;
  int rc;
  if (A.mn_major) rc = map_2d(&p.map_a, A.ptr, M, K, A.ld, 64, GEMM_BK);
  else rc = map_2d(&p.map_a, gather_a ? peers.a_ptr[p.a_first] : A.ptr, K, gather_a ? peers.a_rows : M, A.ld, GEMM_BK, GEMM_BM);
  if (rc != 0) return rc;
  if (B.mn_major) rc = map_2d(&p.map_b, B.ptr, N, K, B.ld, 64, GEMM_BK);
  else rc = map_2d(&p.map_b, B.ptr, K, N, B.ld, GEMM_BK, bn / ctas);   // a CTA of a pair stages half of B's rows
  if (rc != 0) return rc - 1000;
  fill_epilogue(p, epi);
  p.tile_n0 = 1;
  p.tile_n1 = 1;
  p.out_w = epi.out_w;
  p.out_h = epi.out_h;
  p.shuffle_cout = epi.shuffle_cout > 0 ? epi.shuffle_cout : 1;
  if (ctas == 1) try_tma_epilogue(p, M, N);
  cudaError_t e = launch_gemm(p, bn, ctas, num_sms, stream);
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

// 3x3 convolution, padding 1, stride 1 or 2, NHWC bf16, as implicit GEMM.
//   x: [B, H, W, Cin]   w: [Cout, 9 * Cin_pad] (tap-major, Cin padded to a multiple of 64 with zeros)
//   y: [B, Ho, Wo, Cout]
static int image_map(CUtensorMap* out, const void* base, int Cin, int par, int W, int rows, int B, int box_w) {
  unsigned long long dims[5] = {static_cast<unsigned long long>(Cin), static_cast<unsigned long long>(par),
                                static_cast<unsigned long long>(W / par), static_cast<unsigned long long>(rows),
                                static_cast<unsigned long long>(B)};
  unsigned long long str[4] = {static_cast<unsigned long long>(Cin) * 2ull,
                               static_cast<unsigned long long>(Cin) * 2ull * par,
                               static_cast<unsigned long long>(Cin) * 2ull * W,
                               static_cast<unsigned long long>(Cin) * 2ull * W * rows};
  unsigned int box[5] = {64, 1, static_cast<unsigned int>(box_w), 1, 1};
  return make_tensor_map_bf16(out, base, 5, dims, str, box);
}

static int attach_halos(GemmParams& p, const void* halo_lo, const void* halo_hi, int Cin, int par, int W, int H, int B,
                        int box_w) {
  p.img_h = H;
  p.halo_flags = 0;
  if (halo_lo != nullptr) {
    const int rc = image_map(&p.map_halo_lo, halo_lo, Cin, par, W, 1, B, box_w);
    if (rc != 0) return rc - 3000;
    p.halo_flags |= 1;
  }
  if (halo_hi != nullptr) {
    const int rc = image_map(&p.map_halo_hi, halo_hi, Cin, par, W, 1, B, box_w);
    if (rc != 0) return rc - 4000;
    p.halo_flags |= 2;
  }
  return 0;
}

int conv3x3_fwd_bf16(const void* x, const void* w, int B, int H, int W, int Cin, int Cout, int stride,
                     const GemmEpilogue& epi, int num_sms, cudaStream_t stream, const void* halo_lo,
                     const void* halo_hi) {
  if (stride != 1 && stride != 2) return -11;
  if (stride == 2 && (W % 2 != 0)) return -12;
  if (Cin % 8 != 0 || Cout % 8 != 0) return -13;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  const int Ho = (stride == 1) ? H : (H + 1) / 2;
  const int Wo = (stride == 1) ? W : W / 2;
  const int cchunks = (Cin + 63) / 64;
  const int cin_pad = cchunks * 64;
  if (9 * cchunks > GEMM_MAX_KTABLE) return -14;
  const int bn = pick_bn(Cout, 0);
  p.M = B * Ho * Wo;
  p.N = Cout;
  p.K = 9 * cin_pad;
  p.tile_n0 = (Wo + GEMM_BM - 1) / GEMM_BM;
  p.tile_n1 = Ho;
  p.num_m_tiles = p.tile_n0 * Ho * B;
  p.num_n_tiles = (Cout + bn - 1) / bn;
  p.k_blocks = 9 * cchunks;
  p.split_k = 1;
  p.groups = 1;
  p.a_mode = OP_TABLE_5D;
  p.b_mode = OP_KMAJOR_2D;
  // 5-D view of x: {Cin, parity, W / par, H, B}; par = stride.
  const int par = stride;
  unsigned long long dims[5] = {static_cast<unsigned long long>(Cin), static_cast<unsigned long long>(par),
                                static_cast<unsigned long long>(W / par), static_cast<unsigned long long>(H),
                                static_cast<unsigned long long>(B)};
  unsigned long long str[4] = {static_cast<unsigned long long>(Cin) * 2ull,
                               static_cast<unsigned long long>(Cin) * 2ull * par,
                               static_cast<unsigned long long>(Cin) * 2ull * W,
                               static_cast<unsigned long long>(Cin) * 2ull * W * H};
  unsigned int box[5] = {64, 1, GEMM_BM, 1, 1};
  int rc = make_tensor_map_bf16(&p.map_a, x, 5, dims, str, box);
  if (rc != 0) return rc;
  rc = map_2d(&p.map_b, w, p.K, Cout, p.K, GEMM_BK, bn);
  if (rc != 0) return rc - 1000;
  rc = attach_halos(p, halo_lo, halo_hi, Cin, par, W, H, B, GEMM_BM);
  if (rc != 0) return rc;
  // tile (t0, t1, t2) = (w chunk, ho, b): base coordinates
  p.a_mul0[2] = GEMM_BM;          // w (in units of the strided grid)
  p.a_mul1[3] = stride;           // h_in = ho * stride + dh
  p.a_mul2[4] = 1;                // b
  for (int tap = 0; tap < 9; ++tap) {
    const int dy = tap / 3, dx = tap % 3;
    for (int c = 0; c < cchunks; ++c) {
      short* e = p.ktable[tap * cchunks + c];
      e[0] = static_cast<short>(c * 64);
      if (stride == 1) {
        e[1] = 0;
        e[2] = static_cast<short>(dx - 1);
      } else {
        // w_in = 2*wo + dx - 1: dx=0 -> parity 1 of column wo-1; dx=1 -> parity 0 of wo; dx=2 -> parity 1 of wo
        e[1] = static_cast<short>(dx == 1 ? 0 : 1);
        e[2] = static_cast<short>(dx == 0 ? -1 : 0);
      }
      e[3] = static_cast<short>(dy - 1);
    }
  }
  fill_epilogue(p, epi);
  p.epi |= EPI_ROW_CONV;
  p.out_w = Wo;
  p.out_h = Ho;
  p.shuffle_cout = 1;
  cudaError_t e = launch_gemm(p, bn, 1, num_sms, stream);
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

// Weight gradient of the 3x3 convolution: dw[tap][Cout][Cin] (fp32, pre-zeroed, atomically accumulated)
//   = sum over output pixels of dy[pix][Cout]^T * x[pix shifted by tap][Cin].
int conv3x3_wgrad_bf16(const void* x, const void* dy, float* dw, int B, int H, int W, int Cin, int Cout, int stride,
                       int split_k, void* status, int num_sms, cudaStream_t stream, const void* halo_lo,
                       const void* halo_hi, float* bias_grad) {
  if (stride != 1 && stride != 2) return -11;
  if (stride == 2 && (W % 2 != 0)) return -12;
  if (Cin % 8 != 0 || Cout % 8 != 0) return -13;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  const int Ho = (stride == 1) ? H : (H + 1) / 2;
  const int Wo = (stride == 1) ? W : W / 2;
  const int bn = pick_bn(Cin, Cin % 192 == 0 ? 192 : 128);   // 384 input channels: two tiles of 192, a fifth less operand traffic per flop
  p.M = Cout;
  p.N = Cin;
  p.pix_n0 = (Wo + GEMM_BK - 1) / GEMM_BK;
  p.pix_n1 = Ho;
  p.pix_hmul = stride;
  p.k_blocks = p.pix_n0 * Ho * B;
  p.K = p.k_blocks * GEMM_BK;
  p.num_m_tiles = (Cout + GEMM_BM - 1) / GEMM_BM;
  p.num_n_tiles = (Cin + bn - 1) / bn;
  p.groups = 9;
  if (split_k < 1) split_k = 1;
  if (split_k > p.k_blocks) split_k = p.k_blocks;
  {
    const int per = (p.k_blocks + split_k - 1) / split_k;
    split_k = (p.k_blocks + per - 1) / per;
  }
  p.split_k = split_k;
  p.a_mode = OP_PIXELS_5D;
  p.b_mode = OP_PIXELS_5D;
  {
    unsigned long long dims[5] = {static_cast<unsigned long long>(Cout), 1ull, static_cast<unsigned long long>(Wo),
                                  static_cast<unsigned long long>(Ho), static_cast<unsigned long long>(B)};
    unsigned long long str[4] = {static_cast<unsigned long long>(Cout) * 2ull, static_cast<unsigned long long>(Cout) * 2ull,
                                 static_cast<unsigned long long>(Cout) * 2ull * Wo,
                                 static_cast<unsigned long long>(Cout) * 2ull * Wo * Ho};
    unsigned int box[5] = {64, 1, GEMM_BK, 1, 1};
    int rc = make_tensor_map_bf16(&p.map_a, dy, 5, dims, str, box);
    if (rc != 0) return rc;
  }
  {
    const int par = stride;
    unsigned long long dims[5] = {static_cast<unsigned long long>(Cin), static_cast<unsigned long long>(par),
                                  static_cast<unsigned long long>(W / par), static_cast<unsigned long long>(H),
                                  static_cast<unsigned long long>(B)};
    unsigned long long str[4] = {static_cast<unsigned long long>(Cin) * 2ull,
                                 static_cast<unsigned long long>(Cin) * 2ull * par,
                                 static_cast<unsigned long long>(Cin) * 2ull * W,
                                 static_cast<unsigned long long>(Cin) * 2ull * W * H};
    unsigned int box[5] = {64, 1, GEMM_BK, 1, 1};
    int rc = make_tensor_map_bf16(&p.map_b, x, 5, dims, str, box);
    if (rc != 0) return rc - 1000;
  }
  {
    const int rc = attach_halos(p, halo_lo, halo_hi, Cin, stride, W, H, B, GEMM_BK);
    if (rc != 0) return rc;
  }
  for (int tap = 0; tap < 9; ++tap) {
    const int dyy = tap / 3, dxx = tap % 3;
    short* g = p.grp_off[tap];
    if (stride == 1) {
      g[0] = 0;
      g[1] = static_cast<short>(dxx - 1);
    } else {
      g[0] = static_cast<short>(dxx == 1 ? 0 : 1);
      g[1] = static_cast<short>(dxx == 0 ? -1 : 0);
    }
    g[2] = static_cast<short>(dyy - 1);
  }
  p.grp_c_stride = static_cast<long long>(Cout) * Cin;
  p.epi = EPI_OUT_F32 | EPI_ATOMIC;
  p.colsum = bias_grad;
  p.C = dw;
  p.ldc = Cin;
  p.alpha = 1.0f;
  p.status = static_cast<KernelStatus*>(status);
  p.tile_n0 = 1;
  p.tile_n1 = 1;
  p.shuffle_cout = 1;
  cudaError_t e = launch_gemm(p, bn, 1, num_sms, stream);
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

int gemm_stall_counters(unsigned long long* out8, int reset) {
  return gemm_read_stalls(out8, reset != 0) == cudaSuccess ? 0 : -1;
}

}  // namespace tb
