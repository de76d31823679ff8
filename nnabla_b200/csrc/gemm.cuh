// Persistent, warp-specialised tcgen05 contraction kernel for sm_100a.
//
//   D[M, N] = sum over planes (pa, pb) of A_pa[M, K] * B_pb[N, K]^T
//   y       = D * (scale * row_scale[m] * col_scale[n]) + row_bias[m] + col_bias[n]
//
// Both operands are K-major side-band tensors (bf16 or int8) that the prepare
// kernels write; several "planes" of one operand are the bf16 pieces of an
// fp32 tensor (x = hi + mid + lo), all multiplied against the same tile of the
// other operand and accumulated into one fp32 TMEM accumulator, which makes
// products with +-1 (or small-integer) weights exact. int8 operands accumulate
// in int32.
//
// One CTA per SM, static round-robin over output tiles. Warp 0 feeds a
// multi-stage shared-memory ring with TMA tiled loads (128-byte swizzle),
// warp 1 issues tcgen05.mma from one elected thread and owns the TMEM
// allocation, eight epilogue warps drain the double-buffered TMEM accumulator with
// tcgen05.ld and write y. Every mbarrier wait is time-bounded; a wait that
// gives up stores a code in *status, raises the CTA's abort flag and all
// roles fall through to the common teardown (TMEM is always freed).
//
// The tensor core's fp32 accumulation truncates, so a long K loses accuracy
// in proportion to the number of accumulation steps. For floating-point
// operands the K loop can therefore be cut into chunks (Problem::k_chunk() K
// blocks each): every chunk is accumulated in one of the two TMEM buffers and
// the epilogue warps add the chunks in fp32 registers (round to nearest),
// which costs one extra TMEM read per chunk and bounds the error.
//
// A problem policy maps tile indices to operand coordinates and output
// addresses, so that the same kernel serves plain GEMM (GemmProblem) and
// implicit-GEMM convolution (ConvProblem: boxes of an NHWC activation tensor
// shifted by the filter tap).
#pragma once
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace nb200 {

constexpr int kEpilogueWarps = 8;                          // two warps per TMEM lane quarter, alternating column chunks
constexpr int kGemmThreads = 32 * (2 + kEpilogueWarps); // warps: TMA, MMA, epilogue
constexpr int kTileM = 128;
constexpr int kRowBytes = 128; // one swizzle-atom row: 64 bf16 or 128 int8 along K
constexpr int kMaxPeers = 7;   // other ranks of one 8-GPU box
constexpr int kEpilogueStageBytes = kEpilogueWarps * 32 * 33 * 4; // per-warp transpose buffers of the epilogue

// Status codes written by a wait that gave up (low byte = role).
constexpr int kStatusProducerTimeout = 0x101;
constexpr int kStatusMmaTimeout = 0x102;
constexpr int kStatusEpilogueTimeout = 0x103;

// Timing experiments: a build with -DNB200_GEMM_TIMING_KNOBS reads NNABLA_B200_GEMM_DEBUG at launch
// (1 = the epilogue reads TMEM but neither computes nor stores, 2 = no operand loads after the
// first ring fill; both give wrong results on purpose). The default build has neither the variable
// nor the branches: kTimingKnobs is false and the tests on it fold away.
#ifdef NB200_GEMM_TIMING_KNOBS
constexpr bool kTimingKnobs = true;
#else
constexpr bool kTimingKnobs = false;
#endif

struct GemmEpilogue {
  int debug; // timing-knob builds only; always 0 otherwise
  float *y;
  const float *row_scale, *col_scale, *row_bias, *col_bias;
  float scale;
  // Copies of y in other GPUs' memory (peer mappings), addressed exactly like
  // y: every output value is also stored there, so that a column-sharded
  // contraction leaves the gathered result on every rank without a separate
  // collective. Plain stores only; no rank waits on another inside the kernel.
  int n_peers;
  float *peer_y[kMaxPeers];
  int accumulate; // y += value instead of y = value (gradient accumulation); single-CTA kernel only
};

// Per-tile coordinates produced by a problem policy.
struct Tile {
  int m0;      // first row of D (GEMM: row of x; convolution: output map)
  int m_end;   // rows >= m_end are not stored
  int n0;      // GEMM: first column of D; convolution: unused
  int img0;    // convolution: first image of the pixel box
  int oy0;     // convolution: first output row of the pixel box
  int group;   // convolution: group index
  int kb0, kb1; // K blocks [kb0, kb1) of the contraction that this tile accumulates (split K)
  int64_t y_off; // offset of this tile's partial result in y (split K: one staged result per split)
};

// ---- plain GEMM: A [planes][M][K], B [planes][N][K] --------------------------
struct GemmProblem {
  int M, N, kblocks, m_tiles, n_tiles, bn;
  int row_bytes; // bytes of one K block per operand row (128 or 64)
  int chunk_blocks; // K blocks accumulated in tensor memory before the fp32 registers take over (0 = all)
  int64_t ldy;
  __device__ __forceinline__ int k_chunk() const { return chunk_blocks; }
  __device__ __forceinline__ int num_tiles() const { return m_tiles * n_tiles; }
  __device__ __forceinline__ int k_blocks() const { return kblocks; }
  __device__ __forceinline__ uint32_t umma_n() const { return (uint32_t)bn; }
  __device__ __forceinline__ uint32_t b_tx_bytes() const { return (uint32_t)(bn * row_bytes); }
  __device__ __forceinline__ void decode(int tile, Tile &t) const {
    t.m0 = (tile % m_tiles) * kTileM;
    t.m_end = M;
    t.n0 = (tile / m_tiles) * bn;
    t.img0 = t.oy0 = t.group = 0;
    t.kb0 = 0;
    t.kb1 = kblocks;
    t.y_off = 0;
  }
  __device__ __forceinline__ void load_a(const CUtensorMap *map, void *dst, uint64_t *bar, int kb, const Tile &t,
                                         int plane, int epb) const {
    ptx::tma_load_3d(dst, map, bar, kb * epb, t.m0, plane);
  }
  __device__ __forceinline__ void load_b(const CUtensorMap *map, void *dst, uint64_t *bar, int kb, const Tile &t,
                                         int plane, int epb) const {
    ptx::tma_load_3d(dst, map, bar, kb * epb, t.n0, plane);
  }
  // y address of D(row, col) = y + row_offset(row) + column offset; the column
  // part also says whether the column exists and which global column it is
  // (index into col_scale / col_bias).
  __device__ __forceinline__ int64_t row_offset(int row) const { return (int64_t)row * ldy; }
  __device__ __forceinline__ bool col_offset(const Tile &t, int col, int64_t &off, int &gcol) const {
    gcol = t.n0 + col;
    off = gcol;
    return gcol < N;
  }
};

// ---- implicit-GEMM convolution -------------------------------------------------
// A = weight side-band [planes][Ko][taps * cblocks * E] (K ordered tap-major,
// channel-minor), B = activation planes [planes][N][H][W][Ctot] (NHWC), D rows
// = output maps, D columns = a box of n_box images x h_box output rows x Wo
// output columns. One K block = one filter tap x E consecutive channels; its B
// tile is one TMA box shifted by the tap (out-of-range rows/columns read as
// zero = the padding).
struct ConvProblem {
  int Nimg, Ko, Kog, groups, Ho, Wo;
  int h_box, n_box, tiles_h, tiles_n, m_tiles_g;
  int kw, taps, cblocks;
  int sh, sw, ph, pw, dh, dw;
  int c_group_stride; // channel offset between groups in the activation planes
  int row_bytes;      // bytes of one K block per operand row (128, or 64 for few channels)
  int chunk_blocks;   // K blocks accumulated in tensor memory before the fp32 registers take over (0 = all)
  int n_run;          // UMMA N: pixels per box rounded up to 16
  int pixels;         // n_box * h_box * Wo
  int k_splits;       // the K loop is cut into this many tiles, each writing its own partial result
  int64_t split_stride; // elements between the partial results of consecutive splits in y
  __device__ __forceinline__ int k_chunk() const { return chunk_blocks; }
  __device__ __forceinline__ int num_tiles() const { return k_splits * groups * m_tiles_g * tiles_h * tiles_n; }
  __device__ __forceinline__ int k_blocks() const { return taps * cblocks; }
  __device__ __forceinline__ uint32_t umma_n() const { return (uint32_t)n_run; }
  __device__ __forceinline__ uint32_t b_tx_bytes() const { return (uint32_t)(pixels * row_bytes); }
  __device__ __forceinline__ void decode(int tile, Tile &t) const {
    const int split = tile % k_splits;
    tile /= k_splits;
    const int kb_all = taps * cblocks, per = (kb_all + k_splits - 1) / k_splits;
    t.kb0 = split * per;
    t.kb1 = (t.kb0 + per < kb_all) ? t.kb0 + per : kb_all;
    t.y_off = (int64_t)split * split_stride;
    const int mt = tile % m_tiles_g;
    int r = tile / m_tiles_g;
    const int g = r % groups;
    r /= groups;
    t.group = g;
    t.m0 = g * Kog + mt * kTileM;
    t.m_end = (g + 1) * Kog;
    t.oy0 = (r % tiles_h) * h_box;
    t.img0 = (r / tiles_h) * n_box;
    t.n0 = 0;
  }
  __device__ __forceinline__ void load_a(const CUtensorMap *map, void *dst, uint64_t *bar, int kb, const Tile &t,
                                         int plane, int epb) const {
    ptx::tma_load_3d(dst, map, bar, kb * epb, t.m0, plane);
  }
  __device__ __forceinline__ void load_b(const CUtensorMap *map, void *dst, uint64_t *bar, int kb, const Tile &t,
                                         int plane, int epb) const {
    const int tap = kb / cblocks, cb = kb - tap * cblocks;
    const int ky = tap / kw, kx = tap - ky * kw;
    ptx::tma_load_5d(dst, map, bar, t.group * c_group_stride + cb * epb, kx * dw - pw, t.oy0 * sh - ph + ky * dh,
                     t.img0, plane);
  }
  __device__ __forceinline__ int64_t row_offset(int row) const { return (int64_t)row * ((int64_t)Ho * Wo); }
  __device__ __forceinline__ bool col_offset(const Tile &t, int col, int64_t &off, int &gcol) const {
    // Column = (image of the box, pixel inside the image's h_box x Wo slab); slabs are whole output rows.
    gcol = 0;
    const int per_img = h_box * Wo;
    const int nn = col / per_img, q = col - nn * per_img;
    const int img = t.img0 + nn;
    off = (int64_t)img * Ko * ((int64_t)Ho * Wo) + (int64_t)t.oy0 * Wo + q;
    // columns past the box are padding of the MMA shape; rows past Ho belong to no image
    return nn < n_box && img < Nimg && q < (Ho - t.oy0) * Wo;
  }
};

// kResidentA: every tile of the launch uses the same A operand (a convolution
// whose output maps fit one M tile) and all its K blocks fit in shared memory
// beside the ring: A is loaded once per CTA and only the B tiles stream. With
// few channels the copy engine's request rate bounds the kernel (one request
// per 64-byte row), and A was half of the requests.
// kPairs selects the plane products: 0 = all (pa, pb); 1 = those with pa + pb <= 2 (both operands split in
// three bf16 pieces); 2 = all, with operands in fp16 instead of bf16 (two fp16 pieces of scaled activations
// against +-1 weights).
template <bool kInt8, int PA, int PB, int BN, int STAGES, int kPairs, typename Problem, int RB = kRowBytes,
          bool kResidentA = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const Problem prob, const GemmEpilogue ep, int *status) {
  static_assert(RB == 128 || RB == 64, "operand rows are one 128-byte or 64-byte swizzle span");
  constexpr int kElemsPerBlock = kInt8 ? RB : RB / 2; // K elements per operand row of one K block
  constexpr int kUmmaK = kInt8 ? 32 : 16;             // K elements per MMA (32 bytes)
  constexpr int kMmasPerBlock = kElemsPerBlock / kUmmaK;
  constexpr uint32_t kABytes = kTileM * RB;
  constexpr uint32_t kBBytes = BN * RB;
  constexpr uint32_t kStageA = kResidentA ? 0u : PA * kABytes; // bytes of A inside a ring stage
  constexpr uint32_t kStageBytes = kStageA + PB * kBBytes;
  constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N for M = 128");

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atoms.
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // resident A (kResidentA): [k block][plane][kTileM rows] behind the ring
  const uint32_t resident_bytes = kResidentA ? (uint32_t)prob.k_blocks() * PA * kABytes : 0u;
  uint8_t *a_resident = smem + STAGES * kStageBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * kStageBytes + resident_bytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *tmem_full = bars + 2 * STAGES;
  uint64_t *tmem_empty = bars + 2 * STAGES + 2;
  uint64_t *a_full = bars + 2 * STAGES + 4;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 5);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *stage_out = reinterpret_cast<float *>(tmem_slot + 4); // one 32 x 33 float buffer per epilogue warp

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = prob.num_tiles();
  // K blocks per TMEM accumulation (int8 accumulation is exact: never chunked)
  const int chunk_cfg = (!kInt8 && prob.k_chunk() > 0) ? prob.k_chunk() : 0x3fffffff;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tmem_full + b, 1);
      ptx::mbar_init(tmem_empty + b, kEpilogueWarps);
    }
    ptx::mbar_init(a_full, 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t tx_bytes = kStageA + PB * prob.b_tx_bytes();
      if (kResidentA && (int)blockIdx.x < num_tiles) {
        Tile t0;
        prob.decode(blockIdx.x, t0);
        ptx::mbar_expect_tx(a_full, resident_bytes);
        for (int kb = 0; kb < prob.k_blocks(); ++kb)
#pragma unroll
          for (int pa = 0; pa < PA; ++pa)
            prob.load_a(&map_a, a_resident + (size_t)(kb * PA + pa) * kABytes, a_full, kb, t0, pa, kElemsPerBlock);
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        Tile t;
        prob.decode(tile, t);
        for (int kb = t.kb0; kb < t.kb1; ++kb) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusProducerTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t *st = smem + stage * kStageBytes;
          if (kTimingKnobs && (ep.debug & 2) && (tile != (int)blockIdx.x || kb - t.kb0 >= STAGES)) {
            ptx::mbar_arrive(full_bar + stage);
          } else {
            ptx::mbar_expect_tx(full_bar + stage, tx_bytes);
            if (!kResidentA) {
#pragma unroll
              for (int pa = 0; pa < PA; ++pa)
                prob.load_a(&map_a, st + pa * kABytes, full_bar + stage, kb, t, pa, kElemsPerBlock);
            }
#pragma unroll
            for (int pb = 0; pb < PB; ++pb)
              prob.load_b(&map_b, st + kStageA + pb * kBBytes, full_bar + stage, kb, t, pb, kElemsPerBlock);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      const uint32_t idesc = ptx::make_idesc(kInt8 ? 2u : 1u, kPairs == 2 ? 0u : 1u, kTileM,
                                             prob.umma_n()); // operand format: S8 and BF16 encode as 1, F16 as 0
      if (kResidentA && (int)blockIdx.x < num_tiles) {
        if (!ptx::mbar_wait(a_full, 0u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusMmaTimeout);
          *abort_flag = 1;
          ok = false;
        }
        ptx::tc_fence_after_sync();
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        Tile t;
        prob.decode(tile, t);
        const int k_blocks = t.kb1, chunk = chunk_cfg;
        for (int kb0 = t.kb0; kb0 < k_blocks && ok; kb0 += chunk, ++local) {
          const int buf = local & 1;
          const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
          if (!ptx::mbar_wait(tmem_empty + buf, buf_phase ^ 1u, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusMmaTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
          uint32_t accumulate = 0;
          const int kb1 = (k_blocks - kb0 > chunk) ? kb0 + chunk : k_blocks;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!ptx::mbar_wait(full_bar + stage, phase, abort_flag)) {
              if (*abort_flag == 0)
                atomicCAS(status, 0, kStatusMmaTimeout);
              *abort_flag = 1;
              ok = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t st = ptx::smem_u32(smem + stage * kStageBytes);
#pragma unroll
            for (int pa = 0; pa < PA; ++pa) {
#pragma unroll
              for (int pb = 0; pb < PB; ++pb) {
                // With both operands split in three, pieces whose product is below fp32
                // resolution of the leading term (pa + pb > 2) are skipped.
                if (kPairs == 1 && pa + pb > 2)
                  continue;
                const uint64_t adesc =
                    kResidentA ? ptx::smem_desc_k(ptx::smem_u32(a_resident) + (uint32_t)(kb * PA + pa) * kABytes, RB)
                               : ptx::smem_desc_k(st + pa * kABytes, RB);
                const uint64_t bdesc = ptx::smem_desc_k(st + kStageA + pb * kBBytes, RB);
#pragma unroll
                for (int k = 0; k < kMmasPerBlock; ++k) {
                  // advancing 32 bytes along K inside the swizzle atom = +2 in the encoded address
                  if (kInt8)
                    ptx::mma_i8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
                  else
                    ptx::mma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
                  accumulate = 1;
                }
              }
            }
            ptx::mma_commit(empty_bar + stage); // frees the stage once these MMAs have read it
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok)
            ptx::mma_commit(tmem_full + buf);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3; // TMEM lanes [32*quarter, 32*quarter + 32) are visible to this warp
    const int half = (warp - 2) >> 2; // the two warps of a quarter take even / odd 32-column chunks
    const int n_cols = (int)prob.umma_n();
    int local = 0;
    bool ok = true;
    // fp32 sums of the K chunks of this thread's row: one 32-column group per
    // column chunk this warp owns (unused when a tile is a single chunk)
    constexpr int kMyChunks = (BN + 63) / 64;
    constexpr int kUnrollChunks = kInt8 ? 1 : kMyChunks; // the register sums need constant indices; int8 has none
    float acc[kInt8 ? 1 : kMyChunks][kInt8 ? 1 : 32];
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      Tile t;
      prob.decode(tile, t);
      float *stg = stage_out + (warp - 2) * (32 * 33);
      const int row_base = t.m0 + quarter * 32;
      // Row-wise factors are applied by the row's owner before the transpose,
      // column-wise ones by the column's owner after it: no loads in the loops.
      const int my_row = row_base + lane;
      const bool my_row_ok = my_row < t.m_end;
      const float rs = (ep.row_scale && my_row_ok) ? __fmul_rn(ep.row_scale[my_row], ep.scale) : ep.scale;
      const float rb = (ep.row_bias && my_row_ok) ? ep.row_bias[my_row] : 0.0f;
      int rows_here = t.m_end - row_base;
      rows_here = rows_here < 0 ? 0 : (rows_here > 32 ? 32 : rows_here);
      const int64_t row_stride = prob.row_offset(1);
      const int n_kb = t.kb1 - t.kb0;
      const int n_chunks = (n_kb <= chunk_cfg) ? 1 : (n_kb + chunk_cfg - 1) / chunk_cfg;
      for (int kc = 0; kc < n_chunks && ok; ++kc, ++local) {
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        const bool first_chunk = kc == 0, last_chunk = kc == n_chunks - 1;
        // All lanes poll; the verdict is made warp-uniform so that the aligned
        // TMEM loads below always run with the full warp.
        const bool got = ptx::mbar_wait(tmem_full + buf, buf_phase, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusEpilogueTimeout);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        // Each thread holds one row of the accumulator; the chunk is transposed
        // through shared memory so that every store instruction writes one
        // contiguous run of y (lane = column).
#pragma unroll kUnrollChunks
        for (int ci = 0; ci < kMyChunks; ++ci) {
          const int c0 = 32 * half + 64 * ci;
          if (c0 >= n_cols)
            break;
          uint32_t r[32];
          ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), r);
          ptx::tmem_ld_wait();
          if ((kTimingKnobs && (ep.debug & 1)) || rows_here == 0)
            continue;
          if (!kInt8 && n_chunks > 1) {
            // chunk sums in fp32, round to nearest
            if (first_chunk) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                acc[kInt8 ? 0 : ci][j] = __uint_as_float(r[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                acc[kInt8 ? 0 : ci][j] = __fadd_rn(acc[kInt8 ? 0 : ci][j], __uint_as_float(r[j]));
            }
            if (!last_chunk)
              continue;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              r[j] = __float_as_uint(acc[kInt8 ? 0 : ci][j]);
          }
          if (ep.col_scale) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              stg[lane * 33 + j] = kInt8 ? (float)(int)r[j] : __uint_as_float(r[j]);
          } else {
            // y = acc * (scale * row_scale) (+ row_bias): one rounding per operation, like the reference's
            // product followed by its bias addition
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float v = __fmul_rn(kInt8 ? (float)(int)r[j] : __uint_as_float(r[j]), rs);
              if (ep.row_bias)
                v = __fadd_rn(v, rb);
              stg[lane * 33 + j] = v;
            }
          }
          __syncwarp();
          int64_t coff;
          int gcol;
          const bool col_ok = prob.col_offset(t, c0 + lane, coff, gcol);
          const float cb = (ep.col_bias && col_ok) ? ep.col_bias[gcol] : 0.0f;
          const int64_t tile_off = coff + prob.row_offset(row_base) + t.y_off;
          if constexpr (kInt8 && std::is_same<Problem, ConvProblem>::value) {
            // Convolution tiles whose columns are consecutive pixels of y (whole rows of one
            // image): 128-bit stores, four rows of eight column quads per instruction, instead of
            // one 32-column row per instruction.
            if (prob.n_box == 1 && ep.n_peers == 0 && !ep.accumulate && !ep.col_scale && !ep.col_bias) {
              const int rows_left = prob.Ho - t.oy0;
              const int nvalid = (rows_left < prob.h_box ? rows_left : prob.h_box) * prob.Wo - c0;
              const int nv = nvalid < 0 ? 0 : (nvalid > 32 ? 32 : nvalid);
              const int64_t plane = (int64_t)prob.Ho * prob.Wo;
              const int64_t off0 = (int64_t)t.img0 * prob.Ko * plane + (int64_t)t.oy0 * prob.Wo + c0 +
                                   prob.row_offset(row_base) + t.y_off;
              if ((nv & 3) == 0 && (plane & 3) == 0 && (off0 & 3) == 0 &&
                  (reinterpret_cast<uintptr_t>(ep.y) & 15) == 0) {
                const int q4 = 4 * (lane & 7), rr = lane >> 3;
                float *yq = ep.y + off0 + q4;
#pragma unroll 4
                for (int i0 = 0; i0 < rows_here; i0 += 4) {
                  const int i = i0 + rr;
                  if (i < rows_here && q4 < nv) {
                    const float *sp = stg + i * 33 + q4;
                    *reinterpret_cast<float4 *>(yq + (int64_t)i * plane) = make_float4(sp[0], sp[1], sp[2], sp[3]);
                  }
                }
                __syncwarp();
                continue;
              }
            }
          }
          // destination 0 is this GPU's y, the others are the peer copies
#pragma unroll 1
          for (int d = 0; d <= ep.n_peers; ++d) {
            float *yp = ep.y; // (selected with constant indices: a variable index would copy the parameters to the stack)
#pragma unroll
            for (int q = 0; q < kMaxPeers; ++q)
              if (d == q + 1)
                yp = ep.peer_y[q];
            yp += tile_off;
            if (ep.accumulate) {
              // gradient accumulation: y += value (kept out of the plain store loops, whose
              // stores must stay independent of any load from y)
              const float cs = (ep.col_scale && col_ok) ? ep.col_scale[gcol] : 1.0f;
#pragma unroll 4
              for (int i = 0; i < rows_here; ++i, yp += row_stride) {
                const float rsi = __shfl_sync(0xffffffffu, rs, i), rbi = __shfl_sync(0xffffffffu, rb, i);
                float v = stg[i * 33 + lane];
                if (ep.col_scale) {
                  v = __fmul_rn(v, __fmul_rn(rsi, cs));
                  if (ep.row_bias)
                    v = __fadd_rn(v, rbi);
                }
                if (ep.col_bias)
                  v = __fadd_rn(v, cb);
                if (col_ok)
                  *yp = __fadd_rn(*yp, v);
              }
            } else if (ep.col_scale) {
              const float cs = col_ok ? ep.col_scale[gcol] : 1.0f;
#pragma unroll 4
              for (int i = 0; i < rows_here; ++i, yp += row_stride) {
                const float rsi = __shfl_sync(0xffffffffu, rs, i), rbi = __shfl_sync(0xffffffffu, rb, i);
                float v = __fmul_rn(stg[i * 33 + lane], __fmul_rn(rsi, cs));
                if (ep.row_bias)
                  v = __fadd_rn(v, rbi);
                if (ep.col_bias)
                  v = __fadd_rn(v, cb);
                if (col_ok)
                  *yp = v;
              }
            } else {
#pragma unroll 8
              for (int i = 0; i < rows_here; ++i, yp += row_stride) {
                float v = stg[i * 33 + lane];
                if (ep.col_bias)
                  v = __fadd_rn(v, cb);
                if (col_ok)
                  *yp = v;
              }
            }
          }
          __syncwarp();
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          ptx::mbar_arrive(tmem_empty + buf);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // Give copies that may still be in flight time to land before the shared
    // memory and TMEM of this CTA are released.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull)
      __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <bool kInt8, int PA, int PB, int BN, int STAGES, int RB = kRowBytes, bool kResidentA = false>
constexpr size_t gemm_smem_bytes() {
  return (size_t)STAGES * ((kResidentA ? 0 : PA * kTileM * RB) + PB * BN * RB) + (2 * STAGES + 5) * 8 + 16 +
         kEpilogueStageBytes + 1024;
}

// K blocks per TMEM accumulation for a floating-point contraction that issues
// `mmas_per_block` MMAs per K block. Measured on 256 x K x 512 products with
// three bf16 pieces of x against +-1 weights: without chunks the relative RMS
// error grows with K (2.6e-6 at K = 1024, 9.7e-6 at 4096, 3.6e-5 at 16384);
// chunks of 192 steps hold it at 2.6e-6 and chunks of 96 steps at 1.4e-6 for
// every K, at no measurable cost in time. NNABLA_B200_K_CHUNK_MMAS overrides the step count (0 = never chunk).
inline int k_chunk_blocks(int mmas_per_block) {
  static const int steps = []() {
    const char *e = std::getenv("NNABLA_B200_K_CHUNK_MMAS");
    return e ? std::atoi(e) : 96;
  }();
  if (steps <= 0 || mmas_per_block <= 0)
    return 0;
  const int b = steps / mmas_per_block;
  return b < 1 ? 1 : b;
}

// Host helpers (gemm.cu).
// Encodes a tiled tensor map over a K-major side-band tensor viewed as
// (k_extent, rows, planes), rows pitch_elems apart, with a (128 bytes,
// box_rows, 1) box and the 128-byte swizzle. Reads past k_extent or rows are
// zero-filled by the copy engine.
int make_operand_map(CUtensorMap *map, const void *base, bool int8, int64_t k_extent, int64_t pitch_elems,
                     int64_t rows, int planes, int box_rows, int row_bytes = kRowBytes);
int encode_tiled(CUtensorMap *map, int dtype_code, int rank, const void *base, const uint64_t *dims,
                 const uint64_t *strides_bytes, const uint32_t *box, const uint32_t *elem_strides,
                 int swizzle_bytes = 128);
int device_status_word(int **status);
int run_gemm(bool int8, int planes_a, int planes_b, const void *A, int64_t pitch_a, const void *B, int64_t pitch_b,
             int M, int N, int K, const GemmEpilogue &ep, int64_t ldy, cudaStream_t st);


// Launches the contraction kernel for one problem: one persistent CTA per SM
// (or per tile when there are fewer tiles than SMs).
template <bool kInt8, int PA, int PB, int BN, int STAGES, int kSkip, typename Problem, int RB = kRowBytes,
          bool kResidentA = false>
inline int launch_contraction(const CUtensorMap &ma, const CUtensorMap &mb, const Problem &prob, int tiles,
                       const GemmEpilogue &ep, cudaStream_t st, int resident_k_blocks = 0) {
  auto kernel = gemm_tcgen05_kernel<kInt8, PA, PB, BN, STAGES, kSkip, Problem, RB, kResidentA>;
  constexpr size_t smem_fixed = gemm_smem_bytes<kInt8, PA, PB, BN, STAGES, RB, kResidentA>();
  static_assert(smem_fixed <= 227 * 1024, "shared memory budget");
  // a resident A operand adds its K blocks; the attribute is set to the device maximum once
  const size_t smem = smem_fixed + (kResidentA ? (size_t)resident_k_blocks * PA * kTileM * RB : 0);
  NB_CHECK(smem <= 227 * 1024, NB200_EVALUE, "resident operand does not fit in shared memory");
  static bool configured[64];
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    NB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kResidentA ? 227 * 1024 : (int)smem));
    configured[dev & 63] = true;
  }
  int *status = nullptr;
  NB_TRY(device_status_word(&status));
  const int grid = tiles < sm_count() ? tiles : sm_count();
  GemmEpilogue epd = ep;
  epd.debug = 0;
#ifdef NB200_GEMM_TIMING_KNOBS
  {
    static const int dbg = []() {
      const char *e = std::getenv("NNABLA_B200_GEMM_DEBUG");
      return e ? std::atoi(e) : 0;
    }();
    epd.debug = dbg;
  }
#endif
  kernel<<<grid, kGemmThreads, smem, st>>>(ma, mb, prob, epd, status);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}


} // namespace nb200
