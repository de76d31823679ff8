// Host side of the tcgen05 contractions: tensor-map encoding, kernel
// selection, and the C-ABI entry points for the affine layers.
#include <cstring>
#include <mutex>

#include <cstdlib>

#include "gemm.cuh"
#include "gemm2.cuh"
#include "prepare.cuh"

namespace nb200 {

// ---- driver entry point for tensor-map encoding (no link against libcuda) --
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode_fn(EncodeTiledFn *out) {
  static std::mutex m;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(m);
  if (fn == nullptr) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    NB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    NB_CHECK(q == cudaDriverEntryPointSuccess && p != nullptr, NB200_ECUDA,
             "cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return NB200_OK;
}

static CUtensorMapL2promotion l2_promotion() {
#ifdef NB200_CC_TRACE
  const char *e = std::getenv("NB_PROMO"); // timing experiments only
  if (e)
    return e[0] == '0' ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                       : (e[0] == '1' ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                      : (e[0] == '2' ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
#endif
  return CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
}

// dtype_code: 0 = bf16, 1 = uint8/int8 bytes, 2 = float32
int encode_tiled(CUtensorMap *map, int dtype_code, int rank, const void *base, const uint64_t *dims,
                 const uint64_t *strides_bytes, const uint32_t *box, const uint32_t *elem_strides,
                 int swizzle_bytes) {
  EncodeTiledFn fn;
  NB_TRY(get_encode_fn(&fn));
  NB_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, NB200_EVALUE, "tensor-map base must be 16-byte aligned");
  for (int i = 0; i < rank - 1; ++i)
    NB_CHECK(strides_bytes[i] % 16 == 0, NB200_EVALUE, "tensor-map stride %d (%llu bytes) is not a multiple of 16", i,
             (unsigned long long)strides_bytes[i]);
  cuuint64_t d[5], s[5];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = elem_strides ? elem_strides[i] : 1;
    if (i < rank - 1)
      s[i] = strides_bytes[i];
  }
  const CUtensorMapDataType dt = dtype_code == 0   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype_code == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                   : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUresult r = fn(map, dt,
                        (cuuint32_t)rank, const_cast<void *>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_bytes == 0    ? CU_TENSOR_MAP_SWIZZLE_NONE
                        : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                              : CU_TENSOR_MAP_SWIZZLE_128B,
                        l2_promotion(),
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NB_CHECK(r == CUDA_SUCCESS, NB200_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return NB200_OK;
}

int make_operand_map(CUtensorMap *map, const void *base, bool int8, int64_t k_extent, int64_t pitch_elems,
                     int64_t rows, int planes, int box_rows, int row_bytes) {
  const uint64_t es = int8 ? 1 : 2;
  const uint64_t dims[3] = {(uint64_t)k_extent, (uint64_t)rows, (uint64_t)planes};
  const uint64_t strides[2] = {(uint64_t)pitch_elems * es, (uint64_t)pitch_elems * es * (uint64_t)rows};
  const uint32_t box[3] = {(uint32_t)(row_bytes / es), (uint32_t)box_rows, 1};
  return encode_tiled(map, int8 ? 1 : 0, 3, base, dims, strides, box, nullptr, row_bytes);
}

// ---- per-device status word written by kernels whose bounded waits gave up --
int device_status_word(int **status) {
  static std::mutex m;
  static int *words[64];
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  NB_CHECK(dev >= 0 && dev < 64, NB200_EVALUE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(m);
  if (words[dev] == nullptr) {
    NB_CUDA(cudaMalloc(&words[dev], sizeof(int)));
    NB_CUDA(cudaMemset(words[dev], 0, sizeof(int)));
  }
  *status = words[dev];
  return NB200_OK;
}

// ---- launch -----------------------------------------------------------------
template <bool kInt8, int PA, int PB, int BN, int STAGES, bool kSkip>
static int launch_gemm(const CUtensorMap &ma, const CUtensorMap &mb, int M, int N, int k_blocks,
                       const GemmEpilogue &ep, int64_t ldy, cudaStream_t st) {
  GemmProblem prob;
  prob.M = M;
  prob.N = N;
  prob.kblocks = k_blocks;
  prob.m_tiles = (M + kTileM - 1) / kTileM;
  prob.n_tiles = (N + BN - 1) / BN;
  prob.bn = BN;
  prob.row_bytes = kRowBytes;
  prob.chunk_blocks = kInt8 ? 0 : k_chunk_blocks((kSkip ? 6 : PA * PB) * 4);
  prob.ldy = ldy;
  return launch_contraction<kInt8, PA, PB, BN, STAGES, kSkip, GemmProblem>(ma, mb, prob, prob.m_tiles * prob.n_tiles,
                                                                           ep, st);
}

// A: [planes_a][M][pitch_a], B: [planes_b][N][pitch_b], both K-major.
int run_gemm(bool int8, int planes_a, int planes_b, const void *A, int64_t pitch_a, const void *B, int64_t pitch_b,
             int M, int N, int K, const GemmEpilogue &ep, int64_t ldy, cudaStream_t st) {
  NB_CHECK(M > 0 && N > 0 && K > 0, NB200_EVALUE, "empty contraction (M=%d N=%d K=%d)", M, N, K);
  const int epb = int8 ? 128 : 64;
  const int k_blocks = (K + epb - 1) / epb;
  const int m_tiles = (M + kTileM - 1) / kTileM;
  // Narrower N tiles when wide ones would leave most SMs idle.
  const bool narrow = (int64_t)m_tiles * ((N + 127) / 128) < sm_count();
  CUtensorMap ma, mb;
  NB_TRY(make_operand_map(&ma, A, int8, K, pitch_a, M, planes_a, kTileM));
  // Large problems: two-SM tiles (256 x 256 per CTA pair) halve the B traffic per SM.
  // NNABLA_B200_GEMM_PAIR=0 forces the single-CTA kernel (debugging aid).
  static const bool pair_enabled = []() {
    const char *e = std::getenv("NNABLA_B200_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  const int64_t pair_tiles = (int64_t)((M + kPairTileM - 1) / kPairTileM) * ((N + kPairTileN - 1) / kPairTileN);
  // (the bulk stores of its epilogue need a 16-byte aligned y with a row pitch that is a multiple of 16 bytes)
  const bool y_tma_ok = (reinterpret_cast<uintptr_t>(ep.y) & 15) == 0 && (ldy % 4) == 0;
  // (peer copies of y and accumulation into y need the plain stores of the single-CTA kernel's epilogue)
  if (pair_enabled && y_tma_ok && ep.n_peers == 0 && !ep.accumulate && planes_b == 1 && pair_tiles >= sm_count() / 2) {
    NB_TRY(make_operand_map(&mb, B, int8, K, pitch_b, N, 1, kPairTileN / 2));
    if (int8)
      return launch_pair_gemm<true, 1, 6>(ma, mb, M, N, k_blocks, ep, ldy, st);
    // (the two-SM kernel accumulates a whole tile in tensor memory; long floating-point K loops go to the
    // single-CTA kernel, whose chunked accumulation bounds the truncation error)
    if (planes_a == 3 && k_blocks * 12 <= 384)
      return launch_pair_gemm<false, 3, 3>(ma, mb, M, N, k_blocks, ep, ldy, st);
  }
  if (int8) {
    NB_CHECK(planes_a == 1 && planes_b == 1, NB200_EVALUE, "int8 operands have one plane");
    const bool wide = (int64_t)m_tiles * ((N + 255) / 256) >= sm_count();
    if (wide) {
      NB_TRY(make_operand_map(&mb, B, true, K, pitch_b, N, 1, 256));
      return launch_gemm<true, 1, 1, 256, 4, false>(ma, mb, M, N, k_blocks, ep, ldy, st);
    }
    if (!narrow) {
      NB_TRY(make_operand_map(&mb, B, true, K, pitch_b, N, 1, 128));
      return launch_gemm<true, 1, 1, 128, 6, false>(ma, mb, M, N, k_blocks, ep, ldy, st);
    }
    NB_TRY(make_operand_map(&mb, B, true, K, pitch_b, N, 1, 64));
    return launch_gemm<true, 1, 1, 64, 8, false>(ma, mb, M, N, k_blocks, ep, ldy, st);
  }
  if (planes_a == 3 && planes_b == 1) {
    if (!narrow) {
      NB_TRY(make_operand_map(&mb, B, false, K, pitch_b, N, 1, 128));
      return launch_gemm<false, 3, 1, 128, 3, false>(ma, mb, M, N, k_blocks, ep, ldy, st);
    }
    NB_TRY(make_operand_map(&mb, B, false, K, pitch_b, N, 1, 64));
    return launch_gemm<false, 3, 1, 64, 3, false>(ma, mb, M, N, k_blocks, ep, ldy, st);
  }
  if (planes_a == 3 && planes_b == 3) {
    NB_TRY(make_operand_map(&mb, B, false, K, pitch_b, N, 3, 64));
    return launch_gemm<false, 3, 3, 64, 2, true>(ma, mb, M, N, k_blocks, ep, ldy, st);
  }
  return fail(NB200_ENOTIMPL, "no kernel for %d x %d operand planes", planes_a, planes_b);
}

static inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

static bool bf16_exact(float v) {
  uint32_t b;
  std::memcpy(&b, &v, 4);
  return (b & 0xffffu) == 0;
}

// Shared body of BinaryWeightAffine / BinaryConnectAffine forward.
static int binary_affine(const float *x, const float *w, float *wb, float *alpha, const float *bias, float *y,
                         int64_t M, int64_t K, int64_t N, float zero_to, cudaStream_t st) {
  NB_CHECK(M > 0 && K > 0 && N > 0, NB200_EVALUE, "empty operand (M=%lld K=%lld N=%lld)", (long long)M, (long long)K,
           (long long)N);
  NB_CHECK(M < (1ll << 31) && K < (1ll << 31) && N < (1ll << 31), NB200_EVALUE, "extent exceeds 2^31");
  NB_CHECK(x && w && wb && y, NB200_EVALUE, "null data pointer");
  NB_CHECK(bf16_exact(zero_to), NB200_ENOTIMPL,
           "quantize_zero_to = %g is not representable in bf16; the exact tensor-core path needs it to be", zero_to);
  const int64_t Kp = round_up(K, 64);
  const size_t planes_bytes = (size_t)3 * M * Kp * 2;
  const size_t side_bytes = (size_t)N * Kp * 2;
  const size_t partial_bytes = alpha ? (size_t)((K + 63) / 64) * N * 4 : 0;
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(round_up(planes_bytes, 256) + round_up(side_bytes, 256) + partial_bytes));
  uint8_t *base = static_cast<uint8_t *>(scratch.p);
  void *planes = base;
  void *side = base + round_up(planes_bytes, 256);
  float *partial = reinterpret_cast<float *>(base + round_up(planes_bytes, 256) + round_up(side_bytes, 256));
  NB_TRY(binarize_columns(w, (int)K, (int)N, zero_to, wb, alpha, side, Kp, false, partial, st));
  NB_TRY(split_rows_bf16(x, M, (int)K, Kp, 3, planes, st));
  GemmEpilogue ep{};
  ep.y = y;
  ep.scale = 1.0f;
  ep.col_scale = alpha;
  ep.col_bias = bias;
  return run_gemm(false, 3, 1, planes, Kp, side, Kp, (int)M, (int)N, (int)K, ep, N, st);
}

// Fills the epilogue's destinations for a column slab [col_begin, col_begin + n)
// of row-major [rows, n_total] matrices, one per rank: y_ranks[rank] is this
// GPU's own matrix, the others are peer mappings, taken in ring order starting
// after this rank so that the ranks do not all write to the same peer first.
static int slab_destinations(GemmEpilogue &ep, float *const *y_ranks, int n_ranks, int rank, int64_t n,
                             int64_t n_total, int64_t col_begin) {
  NB_CHECK(y_ranks != nullptr, NB200_EVALUE, "y_ranks is NULL");
  NB_CHECK(n_ranks >= 1 && n_ranks <= kMaxPeers + 1, NB200_EVALUE, "n_ranks = %d outside [1, %d]", n_ranks,
           kMaxPeers + 1);
  NB_CHECK(rank >= 0 && rank < n_ranks, NB200_EVALUE, "rank %d outside [0, %d)", rank, n_ranks);
  NB_CHECK(col_begin >= 0 && n_total < (1ll << 31) && col_begin + n <= n_total, NB200_EVALUE,
           "column slab [%lld, %lld) outside [0, %lld)", (long long)col_begin, (long long)(col_begin + n),
           (long long)n_total);
  for (int r = 0; r < n_ranks; ++r)
    NB_CHECK(y_ranks[r] != nullptr, NB200_EVALUE, "y_ranks[%d] is NULL", r);
  ep.y = y_ranks[rank] + col_begin;
  ep.n_peers = n_ranks - 1;
  for (int j = 1; j < n_ranks; ++j)
    ep.peer_y[j - 1] = y_ranks[(rank + j) % n_ranks] + col_begin;
  return NB200_OK;
}

// w_kmajor: w_codes already holds the K-major layout [w_col][w_pitch] (nb200_transpose_codes_i8), so the
// re-layout pass is skipped (weights are parameters: their codes can be laid out once and reused).
static int affine_codes(const int8_t *x_codes, const int8_t *w_codes, float delta_x, float delta_w, const float *bias,
                        float *const *y_ranks, int n_ranks, int rank, int64_t rows, int64_t w_row, int64_t w_col,
                        int64_t n_total, int64_t col_begin, cudaStream_t st, bool w_kmajor = false,
                        int64_t w_pitch = 0) {
  const int64_t M = rows, K = w_row, N = w_col;
  NB_CHECK(M > 0 && K > 0 && N > 0, NB200_EVALUE, "empty operand");
  NB_CHECK(M < (1ll << 31) && K < (1ll << 31) && N < (1ll << 31), NB200_EVALUE, "extent exceeds 2^31");
  NB_CHECK(x_codes && w_codes, NB200_EVALUE, "null data pointer");
  // |acc| <= K * 127 * 127 must fit int32
  NB_CHECK(K <= 133000, NB200_ENOTIMPL, "K = %lld could overflow the int32 accumulator", (long long)K);
  GemmEpilogue ep{};
  NB_TRY(slab_destinations(ep, y_ranks, n_ranks, rank, N, n_total, col_begin));
  const int64_t Kp = round_up(K, 128);
  const bool x_direct = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(x_codes) & 15) == 0);
  if (w_kmajor)
    NB_CHECK(w_pitch >= K && w_pitch % 16 == 0 && (reinterpret_cast<uintptr_t>(w_codes) & 15) == 0, NB200_EVALUE,
             "K-major weight codes need a 16-byte aligned base and a pitch >= w_row that is a multiple of 16 (got %lld)",
             (long long)w_pitch);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc((w_kmajor ? 0 : (size_t)N * Kp) + (x_direct ? 0 : (size_t)M * Kp) + 16));
  int8_t *wt = static_cast<int8_t *>(scratch.p);
  const int8_t *wk = w_codes;
  int64_t pitch_b = w_pitch;
  if (!w_kmajor) {
    NB_TRY(transpose_i8(w_codes, (int)K, (int)N, wt, Kp, st));
    wk = wt;
    pitch_b = Kp;
  }
  const int8_t *xa = x_codes;
  int64_t pitch_a = K;
  if (!x_direct) {
    int8_t *xc = wt + (w_kmajor ? 0 : (size_t)N * Kp);
    NB_CUDA(cudaMemcpy2DAsync(xc, (size_t)Kp, x_codes, (size_t)K, (size_t)K, (size_t)M, cudaMemcpyDeviceToDevice, st));
    xa = xc;
    pitch_a = Kp;
  }
  ep.scale = delta_x * delta_w;
  ep.col_bias = bias;
  return run_gemm(true, 1, 1, xa, pitch_a, wk, pitch_b, (int)M, (int)N, (int)K, ep, n_total, st);
}

static int affine_fxp8(const float *xq, const float *wq, float delta_x, float delta_w, const float *bias,
                       float *const *y_ranks, int n_ranks, int rank, int64_t rows, int64_t w_row, int64_t w_col,
                       int64_t n_total, int64_t col_begin, cudaStream_t st) {
  const int64_t M = rows, K = w_row, N = w_col;
  NB_CHECK(M > 0 && K > 0 && N > 0, NB200_EVALUE, "empty operand");
  NB_CHECK(M < (1ll << 31) && K < (1ll << 31) && N < (1ll << 31), NB200_EVALUE, "extent exceeds 2^31");
  NB_CHECK(xq && wq, NB200_EVALUE, "null data pointer");
  NB_CHECK(delta_x > 0.f && delta_w > 0.f, NB200_EVALUE, "step sizes must be positive");
  NB_CHECK(K <= 133000, NB200_ENOTIMPL, "K = %lld could overflow the int32 accumulator", (long long)K);
  GemmEpilogue ep{};
  NB_TRY(slab_destinations(ep, y_ranks, n_ranks, rank, N, n_total, col_begin));
  const int64_t Kp = round_up(K, 128);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc((size_t)(M + N) * Kp + (size_t)K * N));
  int8_t *xc = static_cast<int8_t *>(scratch.p);
  int8_t *wt = xc + (size_t)M * Kp;
  int8_t *wc = wt + (size_t)N * Kp;
  NB_TRY(codes_rows_i8(xq, M, (int)K, Kp, delta_x, xc, st));
  NB_TRY(codes_rows_i8(wq, K, (int)N, N, delta_w, wc, st));
  NB_TRY(transpose_i8(wc, (int)K, (int)N, wt, Kp, st));
  ep.scale = delta_x * delta_w;
  ep.col_bias = bias;
  return run_gemm(true, 1, 1, xc, Kp, wt, Kp, (int)M, (int)N, (int)K, ep, n_total, st);
}

// Backward of y = x . W (+ b) for row-major x [M, K], W [K, N], dy [M, N]
// (Affine::backward_impl, src/nbla/function/generic/affine.cpp:98-138):
//   dx (+)= dy . W^T     A = dy [M][N], B = W [K][N]: both already contraction-major
//   dW (+)= x^T . dy     A = x^T [K][M], B = dy^T [N][M]: two fp32 transposes first
//   db (+)= column sums of dy
// `w_exact_bf16`: W holds values that are exact in bf16 (the +-1 / zero_to
// weights of the binary layers); it is then used as one bf16 plane and
// `w_col_scale` (alpha, per column of W, may be NULL) is folded into dy before
// the split, which reproduces the reference's products dy * (wb * alpha)
// rounding for rounding. Otherwise W is split into three pieces like x.
static int affine_backward(const float *x, const float *w, const float *w_col_scale, bool w_exact_bf16,
                           const float *dy, float *dx, float *dw, float *db, int64_t M, int64_t K, int64_t N,
                           int accum_dx, int accum_dw, int accum_db, cudaStream_t st) {
  NB_CHECK(M > 0 && K > 0 && N > 0, NB200_EVALUE, "empty operand (M=%lld K=%lld N=%lld)", (long long)M, (long long)K,
           (long long)N);
  NB_CHECK(M < (1ll << 31) && K < (1ll << 31) && N < (1ll << 31), NB200_EVALUE, "extent exceeds 2^31");
  NB_CHECK(dy != nullptr, NB200_EVALUE, "dy is NULL");
  if (dx) {
    NB_CHECK(w != nullptr, NB200_EVALUE, "the gradient w.r.t. x needs the weights");
    const int64_t Np = round_up(N, 64);
    const int planes_w = w_exact_bf16 ? 1 : 3;
    const size_t a_bytes = round_up((size_t)3 * M * Np * 2, 256), b_bytes = (size_t)planes_w * K * Np * 2;
    AsyncScratch scratch(st);
    NB_TRY(scratch.alloc(a_bytes + b_bytes));
    uint8_t *base = static_cast<uint8_t *>(scratch.p);
    NB_TRY(split_rows_bf16(dy, M, (int)N, Np, 3, base, st, w_col_scale));
    NB_TRY(split_rows_bf16(w, K, (int)N, Np, planes_w, base + a_bytes, st));
    GemmEpilogue ep{};
    ep.y = dx;
    ep.scale = 1.0f;
    ep.accumulate = accum_dx;
    NB_TRY(run_gemm(false, 3, planes_w, base, Np, base + a_bytes, Np, (int)M, (int)K, (int)N, ep, K, st));
  }
  if (dw) {
    NB_CHECK(x != nullptr, NB200_EVALUE, "the gradient w.r.t. the weights needs x");
    const int64_t Mp = round_up(M, 64);
    const size_t xt_bytes = round_up((size_t)K * M * 4, 256), dyt_bytes = round_up((size_t)N * M * 4, 256);
    const size_t a_bytes = round_up((size_t)3 * K * Mp * 2, 256), b_bytes = round_up((size_t)3 * N * Mp * 2, 256);
    AsyncScratch scratch(st);
    NB_TRY(scratch.alloc(xt_bytes + dyt_bytes + a_bytes + b_bytes));
    uint8_t *base = static_cast<uint8_t *>(scratch.p);
    float *xt = reinterpret_cast<float *>(base), *dyt = reinterpret_cast<float *>(base + xt_bytes);
    uint8_t *pa = base + xt_bytes + dyt_bytes, *pb = pa + a_bytes;
    NB_TRY(transpose_f32(x, (int)M, (int)K, xt, st));
    NB_TRY(transpose_f32(dy, (int)M, (int)N, dyt, st));
    NB_TRY(split_rows_bf16(xt, K, (int)M, Mp, 3, pa, st));
    NB_TRY(split_rows_bf16(dyt, N, (int)M, Mp, 3, pb, st));
    GemmEpilogue ep{};
    ep.y = dw;
    ep.scale = 1.0f;
    ep.accumulate = accum_dw;
    NB_TRY(run_gemm(false, 3, 3, pa, Mp, pb, Mp, (int)K, (int)N, (int)M, ep, N, st));
  }
  if (db) {
    int splits = (int)((M + 255) / 256);
    splits = splits > 64 ? 64 : splits;
    AsyncScratch scratch(st);
    NB_TRY(scratch.alloc((size_t)splits * N * 4));
    NB_TRY(column_sums(dy, M, (int)N, db, accum_db, static_cast<float *>(scratch.p), splits, st));
  }
  return NB200_OK;
}

} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_take_device_status(int *code, void *stream) {
  NB_CHECK(code != nullptr, NB200_EVALUE, "code is NULL");
  int *word = nullptr;
  NB_TRY(device_status_word(&word));
  NB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  NB_CUDA(cudaMemcpy(code, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*code != 0)
    NB_CUDA(cudaMemset(word, 0, sizeof(int)));
  return NB200_OK;
}

int nb200_binary_weight_affine_f32(const float *x, const float *w, float *wb, float *alpha, const float *bias,
                                   float *y, int64_t rows, int64_t w_row, int64_t w_col, float quantize_zero_to,
                                   void *stream) {
  NB_CHECK(alpha != nullptr, NB200_EVALUE, "alpha is NULL");
  return binary_affine(x, w, wb, alpha, bias, y, rows, w_row, w_col, quantize_zero_to, as_stream(stream));
}

int nb200_binary_connect_affine_f32(const float *x, const float *w, float *wb, const float *bias, float *y,
                                    int64_t rows, int64_t w_row, int64_t w_col, float quantize_zero_to,
                                    void *stream) {
  return binary_affine(x, w, wb, nullptr, bias, y, rows, w_row, w_col, quantize_zero_to, as_stream(stream));
}

int nb200_affine_codes_i8_f32(const int8_t *x_codes, const int8_t *w_codes, float delta_x, float delta_w,
                              const float *bias, float *y, int64_t rows, int64_t w_row, int64_t w_col,
                              void *stream) {
  NB_CHECK(y != nullptr, NB200_EVALUE, "null data pointer");
  float *const ys[1] = {y};
  return affine_codes(x_codes, w_codes, delta_x, delta_w, bias, ys, 1, 0, rows, w_row, w_col, w_col, 0,
                      as_stream(stream));
}

int nb200_affine_codes_i8_gather_f32(const int8_t *x_codes, const int8_t *w_codes, float delta_x, float delta_w,
                                     const float *bias, float *const *y_ranks, int n_ranks, int rank, int64_t rows,
                                     int64_t w_row, int64_t w_col, int64_t w_col_total, int64_t col_begin,
                                     void *stream) {
  return affine_codes(x_codes, w_codes, delta_x, delta_w, bias, y_ranks, n_ranks, rank, rows, w_row, w_col,
                      w_col_total, col_begin, as_stream(stream));
}

int nb200_affine_fxp8_f32(const float *xq, const float *wq, float delta_x, float delta_w, const float *bias, float *y,
                          int64_t rows, int64_t w_row, int64_t w_col, void *stream) {
  NB_CHECK(y != nullptr, NB200_EVALUE, "null data pointer");
  float *const ys[1] = {y};
  return affine_fxp8(xq, wq, delta_x, delta_w, bias, ys, 1, 0, rows, w_row, w_col, w_col, 0, as_stream(stream));
}

int nb200_affine_fxp8_gather_f32(const float *xq, const float *wq, float delta_x, float delta_w, const float *bias,
                                 float *const *y_ranks, int n_ranks, int rank, int64_t rows, int64_t w_row,
                                 int64_t w_col, int64_t w_col_total, int64_t col_begin, void *stream) {
  return affine_fxp8(xq, wq, delta_x, delta_w, bias, y_ranks, n_ranks, rank, rows, w_row, w_col, w_col_total,
                     col_begin, as_stream(stream));
}

int nb200_affine_f32(const float *x, const float *w, const float *bias, float *y, int64_t rows, int64_t w_row,
                     int64_t w_col, void *stream) {
  const int64_t M = rows, K = w_row, N = w_col;
  NB_CHECK(M > 0 && K > 0 && N > 0, NB200_EVALUE, "empty operand");
  NB_CHECK(M < (1ll << 31) && K < (1ll << 31) && N < (1ll << 31), NB200_EVALUE, "extent exceeds 2^31");
  NB_CHECK(x && w && y, NB200_EVALUE, "null data pointer");
  cudaStream_t st = as_stream(stream);
  const int64_t Kp = round_up(K, 64);
  // w [K, N] is transposed through a fp32 staging pass into [N][K] planes.
  AsyncScratch scratch(st);
  const size_t xa = round_up((size_t)3 * M * Kp * 2, 256), wa = round_up((size_t)3 * N * Kp * 2, 256);
  NB_TRY(scratch.alloc(xa + wa + (size_t)N * K * 4));
  uint8_t *base = static_cast<uint8_t *>(scratch.p);
  float *wt32 = reinterpret_cast<float *>(base + xa + wa);
  NB_TRY(transpose_f32(w, (int)K, (int)N, wt32, st));
  NB_TRY(split_rows_bf16(x, M, (int)K, Kp, 3, base, st));
  NB_TRY(split_rows_bf16(wt32, N, (int)K, Kp, 3, base + xa, st));
  GemmEpilogue ep{};
  ep.y = y;
  ep.scale = 1.0f;
  ep.col_bias = bias;
  return run_gemm(false, 3, 3, base, Kp, base + xa, Kp, (int)M, (int)N, (int)K, ep, N, st);
}

int nb200_affine_backward_f32(const float *x, const float *w, const float *dy, float *dx, float *dw, float *db,
                              int64_t rows, int64_t w_row, int64_t w_col, int accum_dx, int accum_dw, int accum_db,
                              void *stream) {
  return affine_backward(x, w, nullptr, false, dy, dx, dw, db, rows, w_row, w_col, accum_dx, accum_dw, accum_db,
                         as_stream(stream));
}

int nb200_binary_weight_affine_backward_f32(const float *x, const float *wb, const float *alpha, const float *dy,
                                            float *dx, float *dw, float *db, int64_t rows, int64_t w_row,
                                            int64_t w_col, int accum_dx, int accum_dw, int accum_db, void *stream) {
  NB_CHECK(alpha != nullptr || dx == nullptr, NB200_EVALUE, "alpha is NULL");
  return affine_backward(x, wb, alpha, true, dy, dx, dw, db, rows, w_row, w_col, accum_dx, accum_dw, accum_db,
                         as_stream(stream));
}

int nb200_binary_connect_affine_backward_f32(const float *x, const float *wb, const float *dy, float *dx, float *dw,
                                             float *db, int64_t rows, int64_t w_row, int64_t w_col, int accum_dx,
                                             int accum_dw, int accum_db, void *stream) {
  return affine_backward(x, wb, nullptr, true, dy, dx, dw, db, rows, w_row, w_col, accum_dx, accum_dw, accum_db,
                         as_stream(stream));
}

int nb200_transpose_codes_i8(const int8_t *w_codes, int8_t *w_codes_kmajor, int64_t w_row, int64_t w_col,
                             int64_t pitch, void *stream) {
  NB_CHECK(w_codes && w_codes_kmajor, NB200_EVALUE, "null data pointer");
  NB_CHECK(w_row > 0 && w_col > 0 && w_row < (1ll << 31) && w_col < (1ll << 31), NB200_EVALUE, "bad extents");
  NB_CHECK(pitch >= w_row, NB200_EVALUE, "pitch %lld is smaller than w_row %lld", (long long)pitch, (long long)w_row);
  if (pitch > w_row) // the padding must read as zero codes
    NB_CUDA(cudaMemsetAsync(w_codes_kmajor, 0, (size_t)w_col * pitch, as_stream(stream)));
  return transpose_i8(w_codes, (int)w_row, (int)w_col, w_codes_kmajor, pitch, as_stream(stream));
}

int nb200_affine_codes_i8_kmajor_f32(const int8_t *x_codes, const int8_t *w_codes_kmajor, int64_t w_pitch,
                                     float delta_x, float delta_w, const float *bias, float *y, int64_t rows,
                                     int64_t w_row, int64_t w_col, void *stream) {
  NB_CHECK(y != nullptr, NB200_EVALUE, "null data pointer");
  float *const ys[1] = {y};
  return affine_codes(x_codes, w_codes_kmajor, delta_x, delta_w, bias, ys, 1, 0, rows, w_row, w_col, w_col, 0,
                      as_stream(stream), true, w_pitch);
}
}
