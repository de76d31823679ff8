// Full-precision convolution of an input with FEW channels (the 7x7 / stride 2
// stem of a residual network: 3 channels) on the tcgen05 tensor cores.
//
// Convolution<float>::forward_impl (src/nbla/function/generic/convolution.cpp:160-197)
// unfolds every sample to patches and multiplies. Here the product is an
// implicit GEMM whose rows are the pixels of ONE output row (M = 128 >= Wo),
// whose columns are the output maps (64 >= Ko) and whose K axis is the filter
// window laid out as (ky, kx, c) with every filter row padded to 24 values:
// K = 8 x 24 = 192. With c innermost the 24 values of one filter row are
// CONTIGUOUS in a channel-last copy of the input row, so the A operand can be
// built by the SM itself (a TMA box cannot: a 3-channel pixel is 6 bytes):
//
//   1. a pre-pass writes x as three bf16 pieces (x = hi + mid + lo, exact),
//      channel-last, every row padded left and right: xs [piece][n][row][704];
//   2. per output row, one TMA box brings the kh staged rows of the three
//      pieces into shared memory (two tiles ahead);
//   3. ten builder warps copy 48-byte runs from there into the 128-byte-swizzled
//      K-major layout that the tensor core reads, one K chunk (64 values) at a time;
//   4. the weights, three bf16 pieces as well, stay resident in shared memory,
//      the pieces stacked along N: hi x [w_hi; w_mid; w_lo] (N = 192),
//      mid x [w_hi; w_mid] (N = 128), lo x [w_hi] (N = 64) accumulate into three
//      groups of 64 TMEM columns, which the epilogue adds up (smallest first).
//      The six products kept are those above 2^-24 of the leading one.
//
// Shared-memory bandwidth bounds the kernel (operand reads of the tensor core
// plus the builders' copies), which is why the weight pieces are stacked: the
// pixel operand is read once per piece instead of once per product.
//
// Warps: 0-3 epilogue (TMEM lanes = pixels, columns = maps; stores run along
// the pixels of y's rows), 4 MMA issue + TMEM allocation, 5 TMA, 6-15 builders.
// Every mbarrier wait is time-bounded; a wait that gives up stores a code in
// *status and raises the block's abort flag, every role then falls through to
// the common teardown.
#include <cuda_bf16.h>

#include <cstdlib>

#include "common.cuh"
#include "narrow_conv.cuh"
#include "ptx.cuh"

namespace nb200 {

int device_status_word(int **status); // gemm.cu
int encode_tiled(CUtensorMap *map, int dtype_code, int rank, const void *base, const uint64_t *dims,
                 const uint64_t *strides_bytes, const uint32_t *box, const uint32_t *elem_strides, int swizzle_bytes);

namespace {

constexpr int kThreadsNC = 512;
constexpr int kFirstBuilder = 6;  // warps 0-3 epilogue, 4 MMA, 5 TMA, 6-15 builders
constexpr int kBuilderWarps = 10;
constexpr int kSeg = 24;          // K values per filter row (kw * C <= 24)
constexpr int kRowsK = 8;         // filter rows in K (the filter itself has kh <= 7)
constexpr int kK = kSeg * kRowsK; // 192
constexpr int kChunks = 3;        // K chunks of 64 bf16 = one 128-byte swizzled row each
constexpr int kM = 128, kN = 64;
constexpr int kMaxWo = 112;                         // output columns: the A ring holds 112 rows per piece
constexpr int kPieceBytes = kMaxWo * 128;           // one piece of one A chunk (rows past Wo alias what follows)
constexpr int kStageBytesNC = 3 * kPieceBytes;      // A chunk: three pieces
constexpr int kStages = 2;
constexpr int kBPieceBytes = kN * 128;               // one piece of one B chunk
constexpr int kBBytesNC = kChunks * 3 * kBPieceBytes; // resident weights [chunk][piece][64 rows]
constexpr int kMaxKh = 7, kPatchPitch = 704;         // staged rows of 704 bf16 = 11 x 128 bytes
constexpr int kPatchStageBytes = 3 * kMaxKh * kPatchPitch * 2;
constexpr int kPatchStages = 2;
constexpr int kAccCols = 256; // TMEM columns between the two accumulators (192 used)

constexpr int kStatusBuilderTimeout = 0x201;
constexpr int kStatusNcMmaTimeout = 0x202;
constexpr int kStatusNcEpilogueTimeout = 0x203;
constexpr int kStatusNcLoadTimeout = 0x204;

struct NarrowConv {
  int N, C, H, W, Ko, kh, kw, ph, pw, sh, sw, Ho, Wo;
};

// Result as int8 channel-last codes [N][Ho * Wo][slots] instead of fp32 NCHW: the epilogue applies
// ReLU (optional) and FixedPointQuantize (power-of-two step) to conv + bias and stores finished
// codes, 32 consecutive maps of a pixel per thread and chunk. codes == NULL: fp32 result.
struct NarrowCodesOut {
  int8_t *codes;
  int slots, relu, kmax, kmin;
  float two_inv; // 2 / delta
};

// Four codes in [-128, 127] (saturated) -> the four bytes of one word, a in the lowest.
__device__ __forceinline__ uint32_t pack_codes4(int a, int b, int c, int d) {
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
  return out;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void split3(float x, __nv_bfloat16 &h, __nv_bfloat16 &m, __nv_bfloat16 &l) {
  h = __float2bfloat16_rn(x);
  const float r1 = __fsub_rn(x, __bfloat162float(h));
  m = __float2bfloat16_rn(r1);
  const float r2 = __fsub_rn(r1, __bfloat162float(m));
  l = __float2bfloat16_rn(r2);
}

// w [Ko][C][kh][kw] fp32 -> wprep [chunk][piece][kN rows][64] bf16, K index = ky * 24 + kx * C + c, zero elsewhere.
__global__ void narrow_conv_weights_kernel(const float *__restrict__ w, NarrowConv g, __nv_bfloat16 *__restrict__ out) {
  const int total = kN * kK;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int o = i / kK, k = i - o * kK;
    const int ky = k / kSeg, j = k - ky * kSeg;
    const int kx = j / g.C, c = j - kx * g.C;
    float v = 0.0f;
    if (o < g.Ko && ky < g.kh && kx < g.kw)
      v = w[((o * g.C + c) * g.kh + ky) * g.kw + kx];
    __nv_bfloat16 p[3];
    split3(v, p[0], p[1], p[2]);
    const int chunk = k / 64, kk = k - chunk * 64;
#pragma unroll
    for (int q = 0; q < 3; ++q)
      out[((chunk * 3 + q) * kN + o) * 64 + kk] = p[q];
  }
}

// x [N][C][H][W] fp32 -> xs [piece][N][H][704] bf16, channel-last with pw zero pixels in front:
// xs[.., (ix + pw) * C + c]; the rest of the row is zero. One block per (row, sample).
__global__ void __launch_bounds__(256) narrow_conv_split_kernel(const float *__restrict__ x, NarrowConv g,
                                                                __nv_bfloat16 *__restrict__ xs) {
  const int iy = blockIdx.x, n = blockIdx.y;
  const int64_t piece_stride = (int64_t)g.N * g.H * kPatchPitch;
  __nv_bfloat16 *row = xs + ((int64_t)n * g.H + iy) * kPatchPitch;
  const int first = g.pw * g.C, count = g.W * g.C;
  for (int e = threadIdx.x; e < kPatchPitch; e += 256) {
    const int i = e - first;
    float v = 0.0f;
    if (i >= 0 && i < count) {
      const int ix = i / g.C, c = i - ix * g.C;
      v = __ldg(x + (((int64_t)n * g.C + c) * g.H + iy) * g.W + ix);
    }
    __nv_bfloat16 q0, q1, q2;
    split3(v, q0, q1, q2);
    row[e] = q0;
    row[piece_stride + e] = q1;
    row[2 * piece_stride + e] = q2;
  }
}

// Lane 0 polls for its warp; the verdict is shared.
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, volatile int *abort, int lane) {
  int got = 1;
  if (lane == 0)
    got = ptx::mbar_wait(bar, parity, abort) ? 1 : 0;
  return __shfl_sync(0xffffffffu, got, 0) != 0;
}

__global__ void __launch_bounds__(kThreadsNC, 1)
    narrow_conv_tcgen05_kernel(const __grid_constant__ CUtensorMap map_xs, const __nv_bfloat16 *__restrict__ wprep,
                               const float *__restrict__ bias, float *__restrict__ y, NarrowConv g, int *status,
                               NarrowCodesOut co) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *a_ring = smem;                                 // [stage][piece][112 rows][128 B], swizzled
  uint8_t *b_res = smem + kStages * kStageBytesNC;        // [chunk][piece][64 rows][128 B], swizzled
  uint8_t *patch = b_res + kBBytesNC;                     // [stage][piece][kh rows][704] bf16, as the TMA box arrives
  uint64_t *bars = reinterpret_cast<uint64_t *>(patch + kPatchStages * kPatchStageBytes);
  uint64_t *full_bar = bars, *empty_bar = bars + 2, *tmem_full = bars + 4, *tmem_empty = bars + 6,
           *patch_full = bars + 8, *patch_empty = bars + 10;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // bias of every map (0 past Ko or without bias), times 2 / delta when codes are written
  __shared__ float bias_s[kN];
  if (threadIdx.x < kN)
    bias_s[threadIdx.x] = (bias && (int)threadIdx.x < g.Ko)
                              ? (co.codes ? __fmul_rn(bias[threadIdx.x], co.two_inv) : bias[threadIdx.x])
                              : 0.0f;

  // word offsets, inside a staged piece, of the four words of every 16-byte chunk of the K row:
  // K word wk = (filter row ky, word j2 of its 12-word run) -> ky * 352 + j2
  __shared__ uint4 run_offsets[kChunks * 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = g.N * g.Ho;
  constexpr uint32_t kTmemCols = 512; // two accumulators of 192 columns, 256 apart
  if (threadIdx.x < kChunks * 8) {
    uint32_t o[4];
#pragma unroll
    for (int w4 = 0; w4 < 4; ++w4) {
      const int wk = threadIdx.x * 4 + w4;
      int ky = wk / (kSeg / 2);
      const int j2 = wk - ky * (kSeg / 2);
      ky = ky < g.kh ? ky : g.kh - 1; // rows of K past the filter meet zero weights: any finite data
      o[w4] = (uint32_t)(ky * (kPatchPitch / 2) + j2);
    }
    run_offsets[threadIdx.x] = make_uint4(o[0], o[1], o[2], o[3]);
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(full_bar + s, kBuilderWarps);
      ptx::mbar_init(empty_bar + s, 1);
      ptx::mbar_init(tmem_full + s, 1);
      ptx::mbar_init(tmem_empty + s, 4);
      ptx::mbar_init(patch_full + s, 1);
      ptx::mbar_init(patch_empty + s, kBuilderWarps);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&map_xs);
  }
  if (warp == 4) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  // resident weights: plain copy into the swizzled layout (16-byte chunk c of row r sits at chunk c ^ (r & 7))
  {
    const uint4 *src = reinterpret_cast<const uint4 *>(wprep);
    constexpr int kVecs = kBBytesNC / 16;
    for (int i = threadIdx.x; i < kVecs; i += kThreadsNC) {
      const int row_all = i >> 3, c16 = i & 7; // row over [chunk][piece][64]
      *reinterpret_cast<uint4 *>(b_res + (size_t)row_all * 128 + ((c16 ^ (row_all & 7)) << 4)) = __ldg(src + i);
    }
    fence_async_smem();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t piece_bytes = (uint32_t)((g.Wo + 7) >> 3) * 1024u; // whole groups of 8 rows
  const uint32_t patch_piece_words = (uint32_t)(g.kh * kPatchPitch) / 2u;
  const uint32_t patch_bytes = 3u * (uint32_t)g.kh * kPatchPitch * 2u;

  if (warp >= kFirstBuilder) {
    // ------------------------------------------------------------ operand builders
    const int bw = warp - kFirstBuilder;
    int stage = 0, pstage = 0;
    uint32_t phase = 0, pphase = 0;
    const int rows_pad = ((g.Wo + 7) >> 3) << 3;
    const int groups32 = (rows_pad + 31) >> 5;
    const int step = (g.sw * g.C) / 2; // 32-bit words between the runs of neighbouring pixels
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      if (!warp_wait(patch_full + pstage, pphase, abort_flag, lane)) {
        if (lane == 0) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusBuilderTimeout);
          *abort_flag = 1;
        }
        break;
      }
      const uint32_t *pwords = reinterpret_cast<const uint32_t *>(patch + pstage * kPatchStageBytes);
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        if (!warp_wait(empty_bar + stage, phase ^ 1u, abort_flag, lane)) {
          if (lane == 0) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusBuilderTimeout);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        uint8_t *dst = a_ring + stage * kStageBytesNC;
        // item = (piece, group of 32 rows, pair of 16-byte chunks of the K chunk); lane = row. The
        // loads of a warp are 3 words apart (all banks), a quarter warp stores eight rows of one
        // chunk column, whose swizzled positions cover all banks too.
        const int items = 3 * groups32 * 4;
#pragma unroll 2
        for (int it = bw; it < items; it += kBuilderWarps) {
          const int pair = it & 3, prg = it >> 2;
          const int piece = (prg >= groups32 ? 1 : 0) + (prg >= 2 * groups32 ? 1 : 0);
          const int r = (prg - piece * groups32) * 32 + lane;
          if (r < rows_pad) {
            const uint32_t *srow = pwords + piece * patch_piece_words + r * step;
            uint8_t *drow = dst + piece * piece_bytes + r * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int c16 = 2 * pair + h;
              const uint4 off = run_offsets[chunk * 8 + c16];
              uint4 v;
              v.x = srow[off.x];
              v.y = srow[off.y];
              v.z = srow[off.z];
              v.w = srow[off.w];
              *reinterpret_cast<uint4 *>(drow + ((c16 ^ (r & 7)) << 4)) = v;
            }
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0)
          ptx::mbar_arrive(full_bar + stage); // one arrival per warp
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive(patch_empty + pstage); // this warp has read the staged rows
      if (++pstage == kPatchStages) {
        pstage = 0;
        pphase ^= 1u;
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ TMA: staged rows, two tiles ahead
    if (ptx::elect_one()) {
      int pstage = 0;
      uint32_t pphase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (!ptx::mbar_wait(patch_empty + pstage, pphase ^ 1u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusNcLoadTimeout);
          *abort_flag = 1;
          break;
        }
        const int n = tile / g.Ho, oy = tile - n * g.Ho;
        ptx::mbar_expect_tx(patch_full + pstage, patch_bytes);
        // box = (64, 11, kh, 1, 3) at (0, 0, first input row, n, 0); rows outside the image arrive as zeros
        ptx::tma_load_5d(patch + pstage * kPatchStageBytes, &map_xs, patch_full + pstage, 0, 0, oy * g.sh - g.ph, n,
                         0);
        if (++pstage == kPatchStages) {
          pstage = 0;
          pphase ^= 1u;
        }
      }
    }
  } else if (warp == 4) {
    // -------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      const uint32_t idesc192 = ptx::make_idesc(1u, 1u, kM, 192), idesc128 = ptx::make_idesc(1u, 1u, kM, 128),
                     idesc64 = ptx::make_idesc(1u, 1u, kM, 64);
      const uint32_t b_base = ptx::smem_u32(b_res);
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        if (!ptx::mbar_wait(tmem_empty + buf, buf_phase ^ 1u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusNcMmaTimeout);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kAccCols);
        uint32_t accumulate = 0;
        for (int chunk = 0; chunk < kChunks; ++chunk) {
          if (!ptx::mbar_wait(full_bar + stage, phase, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusNcMmaTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_base = ptx::smem_u32(a_ring + stage * kStageBytesNC);
          const uint64_t a0 = ptx::smem_desc_k(a_base, 128u), a1 = ptx::smem_desc_k(a_base + piece_bytes, 128u),
                         a2 = ptx::smem_desc_k(a_base + 2 * piece_bytes, 128u);
          // weight pieces of this chunk, stacked along N: rows [w_hi; w_mid; w_lo]
          const uint64_t bdesc = ptx::smem_desc_k(b_base + chunk * 3 * kBPieceBytes, 128u);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            ptx::mma_bf16(d_tmem, a0 + 2 * k, bdesc + 2 * k, idesc192, accumulate); // hi x (hi, mid, lo) -> columns 0..191
            ptx::mma_bf16(d_tmem, a1 + 2 * k, bdesc + 2 * k, idesc128, 1u);        // mid x (hi, mid)    -> columns 0..127
            ptx::mma_bf16(d_tmem, a2 + 2 * k, bdesc + 2 * k, idesc64, 1u);         // lo x hi            -> columns 0..63
            accumulate = 1;
          }
          ptx::mma_commit(empty_bar + stage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok)
          ptx::mma_commit(tmem_full + buf);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp; // TMEM lanes [32 * warp, 32 * warp + 32)
    int local = 0;
    const int px = quarter * 32 + lane;
    const int64_t plane = (int64_t)g.Ho * g.Wo;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
      const bool got = ptx::mbar_wait_backoff(tmem_full + buf, buf_phase, abort_flag, 100u);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusNcEpilogueTimeout);
          *abort_flag = 1;
        }
        break;
      }
      ptx::tc_fence_after_sync();
      const int n = tile / g.Ho, oy = tile - n * g.Ho;
      float *yrow = y + (int64_t)n * g.Ko * plane + (int64_t)oy * g.Wo + px;
      const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kAccCols);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r0[32], r1[32], r2[32];
        ptx::tmem_ld_32x32(t0 + (uint32_t)(half * 32), r0);       // products with w_hi
        ptx::tmem_ld_32x32(t0 + (uint32_t)(64 + half * 32), r1);  // with w_mid
        ptx::tmem_ld_32x32(t0 + (uint32_t)(128 + half * 32), r2); // with w_lo
        ptx::tmem_ld_wait();
        if (co.codes != nullptr) {
          if (px < g.Wo && half * 32 < co.slots) {
            // u = (conv) * (2 / delta) + bias * (2 / delta), one fused multiply-add; then ReLU and the
            // quantizer of a non-negative value, (floor(u) + 1) >> 1 capped at kmax
            const float cap = (float)(2 * co.kmax) + 0.5f;
            uint32_t wds[8];
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              int c[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int j = 4 * j4 + k;
                const float conv = __fadd_rn(__fadd_rn(__uint_as_float(r2[j]), __uint_as_float(r1[j])), __uint_as_float(r0[j]));
                const float u = __fmaf_rn(conv, co.two_inv, bias_s[half * 32 + j]);
                if (co.relu) {
                  c[k] = (__float2int_rd(fminf(fmaxf(u, 0.0f), cap)) + 1) >> 1; // a NaN becomes 0
                } else {
                  const int m = (__float2int_rd(fminf(fabsf(u), cap)) + 1) >> 1;
                  c[k] = u < 0.0f ? max(-m, co.kmin) : m;
                }
              }
              // maps past Ko have zero weights and zero bias: their code is 0 on its own
              wds[j4] = pack_codes4(c[0], c[1], c[2], c[3]);
            }
            uint4 *cp = reinterpret_cast<uint4 *>(co.codes + ((int64_t)n * plane + (int64_t)oy * g.Wo + px) * co.slots +
                                                  half * 32);
            cp[0] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
            if (half * 32 + 16 < co.slots)
              cp[1] = make_uint4(wds[4], wds[5], wds[6], wds[7]);
          }
        } else if (px < g.Wo) {
          float *yp = yrow + (int64_t)(half * 32) * plane;
#pragma unroll
          for (int j = 0; j < 32; ++j, yp += plane) {
            const int o = half * 32 + j;
            if (o < g.Ko) {
              float v = __fadd_rn(__fadd_rn(__uint_as_float(r2[j]), __uint_as_float(r1[j])), __uint_as_float(r0[j]));
              if (bias)
                v = __fadd_rn(v, bias_s[o]);
              __stcs(yp, v);
            }
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive(tmem_empty + buf);
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // copies that may still be in flight must land before the shared memory is released
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull)
      __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 4) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

constexpr size_t kSmemNC = (size_t)kStages * kStageBytesNC + kBBytesNC + kPatchStages * kPatchStageBytes + 12 * 8 +
                           16 + 1024;

} // namespace

bool narrow_conv_applies(const float *x, int channels, int height, int width, int outmaps, int kernel_h,
                         int kernel_w, int pad_w, int stride_w, int dilation_h, int dilation_w, int group, int Wo) {
  static const bool off = []() {
    const char *e = std::getenv("NNABLA_B200_DIRECT_CONV");
    return e && e[0] == '1';
  }();
  if (off)
    return false;
  (void)x;
  (void)height;
  return group == 1 && dilation_h == 1 && dilation_w == 1 && kernel_w * channels <= kSeg && kernel_h <= kMaxKh &&
         outmaps <= kN && Wo <= kMaxWo && ((stride_w * channels) & 1) == 0 &&
         ((Wo + 7) / 8 * 8 - 1) * stride_w * channels + kSeg <= kPatchPitch &&
         (width + 2 * pad_w) * channels <= kPatchPitch;
}

int narrow_conv_tc(const float *x, const float *w, const float *bias, float *y, int batch, int channels, int height,
                   int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
                   int stride_w, int Ho, int Wo, cudaStream_t st, int8_t *y_codes, int slots, int relu, int kmax,
                   int kmin, float delta) {
  NarrowCodesOut co{y_codes, slots, relu, kmax, kmin, y_codes ? 2.0f / delta : 0.0f};
  NarrowConv g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, Ho, Wo};
  NB_CHECK(batch <= 65535, NB200_ENOTIMPL, "batch larger than 65535");
  const size_t xs_bytes = (size_t)3 * batch * height * kPatchPitch * 2;
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(kBBytesNC + xs_bytes));
  __nv_bfloat16 *wprep = static_cast<__nv_bfloat16 *>(scratch.p);
  __nv_bfloat16 *xs = wprep + kBBytesNC / 2;
  narrow_conv_weights_kernel<<<(kN * kK + 255) / 256, 256, 0, st>>>(w, g, wprep);
  NB_LAUNCH_CHECK();
  narrow_conv_split_kernel<<<dim3((unsigned)height, (unsigned)batch), 256, 0, st>>>(x, g, xs);
  NB_LAUNCH_CHECK();
  // xs as (64, 11, H, N, piece) bf16: a staged row is 11 runs of 128 bytes (a box extent is at most 256);
  // one box = the kh staged rows of an output row, all three pieces
  CUtensorMap map_xs;
  const uint64_t row_b = (uint64_t)kPatchPitch * 2;
  const uint64_t dims[5] = {64, (uint64_t)kPatchPitch / 64, (uint64_t)height, (uint64_t)batch, 3};
  const uint64_t strides[4] = {128, row_b, row_b * height, row_b * height * batch};
  const uint32_t box[5] = {64, (uint32_t)kPatchPitch / 64, (uint32_t)kernel_h, 1, 3};
  NB_TRY(encode_tiled(&map_xs, 0, 5, xs, dims, strides, box, nullptr, 0));
  static bool configured[64];
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    NB_CUDA(cudaFuncSetAttribute(narrow_conv_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemNC));
    configured[dev & 63] = true;
  }
  int *status = nullptr;
  NB_TRY(device_status_word(&status));
  const int tiles = batch * Ho;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  narrow_conv_tcgen05_kernel<<<grid, kThreadsNC, kSmemNC, st>>>(map_xs, wprep, bias, y, g, status, co);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // namespace nb200
