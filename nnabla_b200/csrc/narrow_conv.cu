// Full-precision convolution of an input with FEW channels (the 7x7 / stride 2
// stem of a residual network: 3 channels) on the tcgen05 tensor cores.
//
// Convolution<float>::forward_impl (src/nbla/function/generic/convolution.cpp:160-197)
// unfolds every sample to patches and multiplies. Here the product is an
// implicit GEMM whose rows are the pixels of ONE output row (M = 128 >= Wo),
// whose columns are the output maps (N = 64 >= Ko) and whose K axis is the
// filter window laid out as (ky, kx, c) with every filter row padded to 24
// values: K = 8 x 24 = 192. With c innermost the 24 values of one filter row
// are CONTIGUOUS in a channel-last copy of the input row, so the A operand is
// built by the SM itself: the block stages the kh input rows of its output row
// in shared memory as three bf16 pieces (x = hi + mid + lo, exact), and copies
// 48-byte runs from there into the 128-byte-swizzled K-major layout that the
// tensor core reads. (A TMA box cannot do this: a 3-channel pixel is 6 bytes.)
// The weights, split into three bf16 pieces as well, stay resident in shared
// memory. Six piece products (hi*hi, hi*mid, mid*hi, hi*lo, mid*mid, lo*hi) go
// into one fp32 TMEM accumulator; what is left out is below 2^-24 of a term.
//
// Warps: 0-3 epilogue (TMEM lanes = pixels, columns = maps; stores run along
// the pixels of y's rows), 4 MMA issue + TMEM allocation, 5 TMA (the fp32 input
// rows of a tile arrive as one box, two tiles ahead), 6-15 operand builders. Every mbarrier wait is time-bounded; a wait that gives up stores a
// code in *status and raises the block's abort flag, every role then falls
// through to the common teardown.
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
constexpr int kBuilderWarps = 10, kBuilderThreads = 32 * kBuilderWarps;
constexpr int kSeg = 24;          // K values per filter row (kw * C <= 24)
constexpr int kRowsK = 8;         // filter rows in K (kh <= 8; the patch holds kh <= 7 of them)
constexpr int kK = kSeg * kRowsK; // 192
constexpr int kChunks = 3;        // K chunks of 64 bf16 = one 128-byte swizzled row each
constexpr int kM = 128, kN = 64;
constexpr int kMaxWo = 112;                         // output columns: the A ring holds 112 rows per piece
constexpr int kPieceBytes = kMaxWo * 128;           // one piece of one A chunk (rows past Wo alias what follows)
constexpr int kStageBytesNC = 3 * kPieceBytes;      // A chunk: three pieces
constexpr int kStages = 2;
constexpr int kBPieceBytes = kN * 128;               // one piece of one B chunk
constexpr int kBBytesNC = kChunks * 3 * kBPieceBytes; // resident weights
constexpr int kPatchRows = 7, kPatchPitch = 704;     // staged rows (kh <= 7) of 704 bf16
constexpr int kPatchPieceElems = kPatchRows * kPatchPitch;
constexpr int kPatchBytes = 3 * kPatchPieceElems * 2;
constexpr int kRawBytes = 18816; // one tile's input rows as fp32: C * kh * W * 4 <= 3 * 7 * 224 * 4
constexpr int kRawStages = 2;

constexpr int kStatusBuilderTimeout = 0x201;
constexpr int kStatusNcMmaTimeout = 0x202;
constexpr int kStatusNcEpilogueTimeout = 0x203;
constexpr int kStatusNcLoadTimeout = 0x204;

struct NarrowConv {
  int N, C, H, W, Ko, kh, kw, ph, pw, sh, sw, Ho, Wo;
};

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void builders_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kBuilderThreads) : "memory"); }

__device__ __forceinline__ void split3(float x, __nv_bfloat16 &h, __nv_bfloat16 &m, __nv_bfloat16 &l) {
  h = __float2bfloat16_rn(x);
  const float r1 = __fsub_rn(x, __bfloat162float(h));
  m = __float2bfloat16_rn(r1);
  const float r2 = __fsub_rn(r1, __bfloat162float(m));
  l = __float2bfloat16_rn(r2);
}

// w [Ko][C][kh][kw] fp32 -> wprep [piece][chunk][kN rows][64] bf16, K index = ky * 24 + kx * C + c, zero elsewhere.
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
      out[((q * kChunks + chunk) * kN + o) * 64 + kk] = p[q];
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
    narrow_conv_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __nv_bfloat16 *__restrict__ wprep,
                               const float *__restrict__ bias, float *__restrict__ y, NarrowConv g, int *status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *a_ring = smem;                                 // [stage][piece][112 rows][128 B], swizzled
  uint8_t *b_res = smem + kStages * kStageBytesNC;        // [piece][chunk][64 rows][128 B], swizzled
  uint8_t *patch = b_res + kBBytesNC;                     // [piece][row][kPatchPitch] bf16, channel-last rows
  uint8_t *raw = patch + kPatchBytes;                     // [stage][C][kh][W] fp32, as the TMA box arrives
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw + kRawStages * kRawBytes);
  uint64_t *full_bar = bars, *empty_bar = bars + 2, *tmem_full = bars + 4, *tmem_empty = bars + 6,
           *raw_full = bars + 8, *raw_empty = bars + 10;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = g.N * g.Ho;
  constexpr uint32_t kTmemCols = 128; // two accumulators of 64 columns

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(full_bar + s, kBuilderWarps);
      ptx::mbar_init(empty_bar + s, 1);
      ptx::mbar_init(tmem_full + s, 1);
      ptx::mbar_init(tmem_empty + s, 4);
      ptx::mbar_init(raw_full + s, 1);
      ptx::mbar_init(raw_empty + s, kBuilderWarps);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&map_x);
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
      const int row_all = i >> 3, c16 = i & 7; // row over [piece][chunk][64]
      const int r = row_all & (kN - 1);
      *reinterpret_cast<uint4 *>(b_res + (size_t)row_all * 128 + ((c16 ^ (r & 7)) << 4)) = __ldg(src + i);
    }
    // the staged rows start as zeros: the padding columns and the tail behind the last pixel's
    // run are never written again
    for (int i = threadIdx.x; i < kPatchBytes / 16; i += kThreadsNC)
      reinterpret_cast<uint4 *>(patch)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_async_smem();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t piece_bytes = (uint32_t)((g.Wo + 7) >> 3) * 1024u; // whole groups of 8 rows
  const uint32_t raw_bytes = (uint32_t)(g.C * g.kh * g.W * 4);

  if (warp >= kFirstBuilder) {
    // ------------------------------------------------------------ operand builders
    const int bw = warp - kFirstBuilder;
    int stage = 0, rstage = 0;
    uint32_t phase = 0, rphase = 0;
    bool ok = true;
    __nv_bfloat16 *pt = reinterpret_cast<__nv_bfloat16 *>(patch);
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      builders_sync(); // the previous tile's runs have been copied out of the staged rows
      if (*abort_flag != 0 || !ok)
        break;
      if (!warp_wait(raw_full + rstage, rphase, abort_flag, lane)) {
        if (lane == 0) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusBuilderTimeout);
          *abort_flag = 1;
        }
        ok = false;
      }
      if (ok) {
        // fp32 rows [c][ry][ix] -> three bf16 pieces, channel-last: patch[piece][ry][(ix + pw) * C + c];
        // one (channel, row) pair per warp at a time, lanes along the row
        const float *rw = reinterpret_cast<const float *>(raw + rstage * kRawBytes);
        for (int rc = bw; rc < g.C * g.kh; rc += kBuilderWarps) {
          const int c = rc / g.kh, ry = rc - c * g.kh;
          const float *src = rw + rc * g.W;
          __nv_bfloat16 *d0 = pt + ry * kPatchPitch + g.pw * g.C + c;
#pragma unroll 4
          for (int ix = lane; ix < g.W; ix += 32) {
            __nv_bfloat16 q0, q1, q2;
            split3(src[ix], q0, q1, q2);
            d0[ix * g.C] = q0;
            d0[kPatchPieceElems + ix * g.C] = q1;
            d0[2 * kPatchPieceElems + ix * g.C] = q2;
          }
        }
      }
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive(raw_empty + rstage); // this warp has read the raw rows (or gave up)
      if (++rstage == kRawStages) {
        rstage = 0;
        rphase ^= 1u;
      }
      builders_sync();
      // copy the runs into the three K chunks of this tile
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        if (ok && !warp_wait(empty_bar + stage, phase ^ 1u, abort_flag, lane)) {
          if (lane == 0) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusBuilderTimeout);
            *abort_flag = 1;
          }
          ok = false;
        }
        if (ok) {
          uint8_t *dst = a_ring + stage * kStageBytesNC;
          // A warp copies, for one piece and one group of 8 rows, the eight 16-byte chunks of the
          // K chunk: lane = (chunk pair, row), each lane gathers the four words of a 16-byte chunk
          // and stores it whole. A quarter warp stores eight different rows of one chunk column,
          // whose swizzled positions cover all banks.
          const int r8 = lane & 7, q4 = lane >> 3;
          int src_off[2][4]; // word offset of (filter row, position in the run) of the lane's two chunks
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) {
              const int wk = chunk * 32 + (q4 + 4 * h) * 4 + w4; // 32-bit word of the K row, 0 .. 95
              int ky = wk / (kSeg / 2);
              const int j2 = wk - ky * (kSeg / 2);
              ky = ky < g.kh ? ky : g.kh - 1; // rows of K past the filter meet zero weights: any finite data
              src_off[h][w4] = (ky * kPatchPitch) / 2 + j2;
            }
          const int row_groups = (g.Wo + 7) >> 3;
          const int step = (g.sw * g.C) / 2; // words between the runs of neighbouring pixels
          for (int u = bw; u < 3 * row_groups; u += kBuilderWarps) {
            const int piece = u / row_groups, rg = u - piece * row_groups;
            const int r = rg * 8 + r8;
            const uint32_t *srow = reinterpret_cast<const uint32_t *>(patch) + (piece * kPatchPieceElems) / 2 + r * step;
            uint8_t *drow = dst + piece * piece_bytes + r * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint4 v;
              v.x = srow[src_off[h][0]];
              v.y = srow[src_off[h][1]];
              v.z = srow[src_off[h][2]];
              v.w = srow[src_off[h][3]];
              *reinterpret_cast<uint4 *>(drow + (((q4 + 4 * h) ^ r8) << 4)) = v;
            }
          }
          fence_async_smem();
        }
        // one arrival per warp; it comes even after a give-up so that nobody waits on this warp
        __syncwarp();
        if (lane == 0)
          ptx::mbar_arrive(full_bar + stage);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ TMA: raw input rows, two tiles ahead
    if (ptx::elect_one()) {
      int rstage = 0;
      uint32_t rphase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (!ptx::mbar_wait(raw_empty + rstage, rphase ^ 1u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusNcLoadTimeout);
          *abort_flag = 1;
          break;
        }
        const int n = tile / g.Ho, oy = tile - n * g.Ho;
        ptx::mbar_expect_tx(raw_full + rstage, raw_bytes);
        // box = (W, kh, C, 1) at (0, first input row, 0, n); rows outside the image arrive as zeros
        ptx::tma_load_4d(raw + rstage * kRawBytes, &map_x, raw_full + rstage, 0, oy * g.sh - g.ph, 0, n);
        if (++rstage == kRawStages) {
          rstage = 0;
          rphase ^= 1u;
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
      const uint32_t idesc = ptx::make_idesc(1u, 1u, kM, kN);
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
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kN);
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
#pragma unroll
          for (int pa = 0; pa < 3; ++pa) {
#pragma unroll
            for (int pb = 0; pb < 3; ++pb) {
              if (pa + pb > 2)
                continue; // below fp32 resolution of the leading product
              const uint64_t adesc = ptx::smem_desc_k(a_base + pa * piece_bytes, 128u);
              const uint64_t bdesc = ptx::smem_desc_k(b_base + (pb * kChunks + chunk) * kBPieceBytes, 128u);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                ptx::mma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
                accumulate = 1;
              }
            }
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
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kN + half * 32), r);
        ptx::tmem_ld_wait();
        if (px < g.Wo) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int o = half * 32 + j;
            if (o < g.Ko) {
              float v = __uint_as_float(r[j]);
              if (bias)
                v = __fadd_rn(v, __ldg(bias + o));
              yrow[(int64_t)o * plane] = v;
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

constexpr size_t kSmemNC = (size_t)kStages * kStageBytesNC + kBBytesNC + kPatchBytes + kRawStages * kRawBytes +
                           12 * 8 + 16 + 1024;

} // namespace

bool narrow_conv_applies(const float *x, int channels, int height, int width, int outmaps, int kernel_h,
                         int kernel_w, int pad_w, int stride_w, int dilation_h, int dilation_w, int group, int Wo) {
  static const bool off = []() {
    const char *e = std::getenv("NNABLA_B200_DIRECT_CONV");
    return e && e[0] == '1';
  }();
  if (off)
    return false;
  (void)height;
  return group == 1 && dilation_h == 1 && dilation_w == 1 && kernel_w * channels <= kSeg && kernel_h <= kPatchRows &&
         outmaps <= kN && Wo <= kMaxWo && ((stride_w * channels) & 1) == 0 && width % 4 == 0 && width <= 256 &&
         (reinterpret_cast<uintptr_t>(x) & 15) == 0 && channels * kernel_h * width * 4 <= kRawBytes &&
         ((Wo + 7) / 8 * 8 - 1) * stride_w * channels + kSeg <= kPatchPitch &&
         (width + 2 * pad_w) * channels <= kPatchPitch;
}

int narrow_conv_tc(const float *x, const float *w, const float *bias, float *y, int batch, int channels, int height,
                   int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
                   int stride_w, int Ho, int Wo, cudaStream_t st) {
  NarrowConv g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, Ho, Wo};
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(kBBytesNC));
  __nv_bfloat16 *wprep = static_cast<__nv_bfloat16 *>(scratch.p);
  narrow_conv_weights_kernel<<<(kN * kK + 255) / 256, 256, 0, st>>>(w, g, wprep);
  NB_LAUNCH_CHECK();
  // x as (W, H, C, N) fp32; one box = the kh input rows of an output row, all channels
  CUtensorMap map_x;
  const uint64_t dims[4] = {(uint64_t)width, (uint64_t)height, (uint64_t)channels, (uint64_t)batch};
  const uint64_t strides[3] = {(uint64_t)width * 4, (uint64_t)width * height * 4,
                               (uint64_t)width * height * channels * 4};
  const uint32_t box[4] = {(uint32_t)width, (uint32_t)kernel_h, (uint32_t)channels, 1};
  NB_TRY(encode_tiled(&map_x, 2, 4, x, dims, strides, box, nullptr, 0));
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
  narrow_conv_tcgen05_kernel<<<grid, kThreadsNC, kSmemNC, st>>>(map_x, wprep, bias, y, g, status);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // namespace nb200
