// Full-precision convolution of an input with FEW channels (the 7x7 / stride 2
// stem of a residual network: 3 channels) on the tcgen05 tensor cores.
//
// Convolution<float>::forward_impl (src/nbla/function/generic/convolution.cpp:160-197)
// unfolds every sample to patches and multiplies. Here the product is an
// implicit GEMM whose rows are the pixels of ONE output row (M = 128 >= Wo) and
// whose columns are the output maps (64 >= Ko). No patch matrix is ever built,
// neither in global nor in shared memory:
//
//   1. A pre-pass writes x channel-last in fp16, every pixel in a slot of
//      16 / stride_w bytes (4 channels at stride 2, 8 at stride 1), rows and
//      columns zero-padded. A slot group of 16 bytes then holds the stride_w
//      pixels that separate two neighbouring outputs, so "output pixel m, filter
//      taps kx = c * stride_w .. (c + 1) * stride_w - 1" is the 16-byte unit m + c
//      of the staged input row.
//   2. The tensor core reads that row in place. An un-swizzled K-major operand is
//      addressed as start + (row / 8) * 128 + (row % 8) * 16 + chunk * LBO; with
//      LBO = 16 the second K chunk of row m is the first one of row m + 1: the
//      overlapping windows of a convolution, straight from the staged row. One
//      instruction (K = 16) covers 2 * stride_w filter taps of one filter row;
//      a 7x7 / stride 2 filter takes 7 x 2 of them.
//   3. The staged rows of a persistent block form a ring in shared memory: the
//      next output row needs stride_h new input rows, fetched with one bulk copy
//      each (both pieces of a row are contiguous); the other rows are reused.
//   4. fp32 accuracy from fp16 operands: x * 2^-e = x0 + 2^-11 x1 and
//      w * 2^S = w0 + 2^-11 w1 with fp16 x0, x1, w0, w1 (e per sample from
//      max |x|, S from max |w|, so that every piece is in fp16's normal range and
//      a residual keeps 11 more bits: 22 bits in all). The weights are stacked along
//      N: x0 x [w0; w1] (N = 128) gives the main product in TMEM columns 0..63
//      and one cross product in 64..127; x1 x [w0] (N = 64) accumulates the other
//      cross product there as well. The epilogue forms
//      (main + 2^-11 cross) * 2^(e - S). The product left out, x1 w1, is 2^-22 of
//      the main one, the size of the representation error.
//
// Warps: 0-7 epilogue (TMEM lanes = pixels, columns = maps; warp w takes lanes 32 (w % 4) and
// maps 32 (w / 4)), 8 MMA issue + TMEM allocation, 9 loader. Every mbarrier wait is time-bounded; a wait that gives
// up stores a code in *status and raises the block's abort flag, every role then
// falls through to the common teardown.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "narrow_conv.cuh"
#include "ptx.cuh"

namespace nb200 {

int device_status_word(int **status); // gemm.cu
int encode_tiled(CUtensorMap *map, int dtype_code, int rank, const void *base, const uint64_t *dims,
                 const uint64_t *strides_bytes, const uint32_t *box, const uint32_t *elem_strides, int swizzle_bytes);

namespace {

constexpr int kThreadsNC = 320;
constexpr int kEpilogueWarps = 8, kMmaWarp = 8, kLoadWarp = 9;
constexpr int kM = 128, kN = 64;
constexpr int kMaxSteps = 16;             // K steps of 16 values: kernel_h * ceil(kernel_w / (2 * stride_w))
constexpr int kStepBytes = 2 * kN * 32;   // resident weights of one K step: [w0; w1] x 16 values
constexpr int kRing = 16;                 // staged input rows kept in shared memory
constexpr int kMaxKh = 8;
constexpr int kMaxRowBytes = 2560;        // one piece of one staged row
constexpr int kInFlight = 8;              // tiles between the loader and the completed MMAs (barrier ring)
constexpr size_t kMaxSmemNC = 224 * 1024;
constexpr int kAccCols = 128;             // TMEM columns of one accumulator: main | cross

constexpr int kStatusNcMmaTimeout = 0x202;
constexpr int kStatusNcEpilogueTimeout = 0x203;
constexpr int kStatusNcLoadTimeout = 0x204;

struct NarrowConv {
  int N, C, H, W, Ko, kh, kw, ph, pw, sh, sw, Ho, Wo;
  int Hp;        // staged rows per sample: H + 2 * ph
  int row_bytes; // one piece of one staged row (a multiple of 16)
  int jsteps;    // K steps per filter row
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

// e with max * 2^-e in [2^top, 2^(top + 1)) for the largest magnitude `maxbits` (fp32 bits of a
// non-negative value); 0 for zero, denormal and non-finite maxima.
__device__ __forceinline__ int scale_exponent(uint32_t maxbits, int top) {
  const int E = (int)(maxbits >> 23);
  if (E == 0 || E >= 255)
    return 0;
  const int e = E - 127 - top;
  return e < -120 ? -120 : e;
}
__device__ __forceinline__ float pow2i(int e) { return __int_as_float((127 + e) << 23); } // -126 <= e <= 127

// v = p0 + 2^-11 p1 up to 2^-22 |v| (v within fp16's range)
__device__ __forceinline__ void split2(float v, __half &p0, __half &p1) {
  p0 = __float2half_rn(v);
  p1 = __float2half_rn(__fmul_rn(__fsub_rn(v, __half2float(p0)), 2048.0f));
}

// max |x| of every sample as fp32 bits (non-negative floats order like their bits; a NaN ends above infinity)
__global__ void __launch_bounds__(256) narrow_conv_absmax_kernel(const float *__restrict__ x, int64_t per_sample,
                                                                 uint32_t *__restrict__ maxbits) {
  const int n = blockIdx.y;
  const float *xs = x + (int64_t)n * per_sample;
  uint32_t m = 0;
  const int64_t vecs = ((reinterpret_cast<uintptr_t>(xs) & 15) == 0) ? per_sample / 4 : 0;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < vecs; i += (int64_t)gridDim.x * 256) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(xs) + i);
    m = max(max(m, __float_as_uint(fabsf(v.x))), max(__float_as_uint(fabsf(v.y)), __float_as_uint(fabsf(v.z))));
    m = max(m, __float_as_uint(fabsf(v.w)));
  }
  for (int64_t i = vecs * 4 + (int64_t)blockIdx.x * 256 + threadIdx.x; i < per_sample; i += (int64_t)gridDim.x * 256)
    m = max(m, __float_as_uint(fabsf(__ldg(xs + i))));
  m = __reduce_max_sync(0xffffffffu, m);
  __shared__ uint32_t part[8];
  if ((threadIdx.x & 31) == 0)
    part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i)
      m = max(m, part[i]);
    atomicMax(maxbits + n, m);
  }
}

// x [N][C][H][W] fp32 -> xs [N][Hp][piece][row_bytes] fp16: unit u of a row holds the stride_w pixels
// u * stride_w .. (padded column), 8 / stride_w channel slots each; zero outside the image and past C.
// One block per (kSplitRows staged rows, sample); xscale[n] = 2^e of the sample.
constexpr int kSplitRows = 8;
template <int SW>
__global__ void __launch_bounds__(256) narrow_conv_split_kernel(const float *__restrict__ x, NarrowConv g,
                                                                const uint32_t *__restrict__ maxbits,
                                                                uint8_t *__restrict__ xs, float *__restrict__ xscale) {
  constexpr int cpp = 8 / SW; // channel slots per pixel
  const int n = blockIdx.y;
  const int e = scale_exponent(maxbits[n], 14);
  const float down = pow2i(-e);
  if (blockIdx.x == 0 && threadIdx.x == 0)
    xscale[n] = pow2i(e);
  const int units = g.row_bytes >> 4;
  const int py0 = blockIdx.x * kSplitRows;
  const int rows = min(kSplitRows, g.Hp - py0);
  for (int i = threadIdx.x; i < rows * units; i += 256) {
    const int r = i / units, u = i - r * units;
    const int py = py0 + r, iy = py - g.ph;
    const bool row_in = iy >= 0 && iy < g.H;
    uint8_t *row = xs + ((int64_t)n * g.Hp + py) * 2 * g.row_bytes;
    __align__(16) __half p0[8], p1[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int t = k / cpp, c = k % cpp;
      const int ix = u * SW + t - g.pw;
      float v = 0.0f;
      if (row_in && c < g.C && ix >= 0 && ix < g.W)
        v = __fmul_rn(__ldg(x + (((int64_t)n * g.C + c) * g.H + iy) * g.W + ix), down);
      split2(v, p0[k], p1[k]);
    }
    *reinterpret_cast<uint4 *>(row + (size_t)u * 16) = *reinterpret_cast<const uint4 *>(p0);
    *reinterpret_cast<uint4 *>(row + g.row_bytes + (size_t)u * 16) = *reinterpret_cast<const uint4 *>(p1);
  }
}

// w [Ko][C][kh][kw] fp32 -> wprep [step][group of 8 rows][chunk][row % 8][8] fp16, rows = [w0 (64); w1 (64)]
// of w * 2^S, the layout the tensor core reads without swizzle (8 x 16-byte core matrices contiguous;
// chunk stride 128, group stride 256 bytes). Step = (ky, j); value k of chunk c2 is tap
// kx = (2 j + c2) * stride_w + k / cpp, channel k % cpp. One block per step (every block finds max |w|
// for itself: the filter is a few thousand values); wscale[0] = 2^-S.
__global__ void __launch_bounds__(256) narrow_conv_weights_kernel(const float *__restrict__ w, NarrowConv g,
                                                                  __half *__restrict__ out, float *__restrict__ wscale) {
  __shared__ uint32_t part[8];
  const int count = g.Ko * g.C * g.kh * g.kw;
  uint32_t m = 0;
  for (int i = threadIdx.x; i < count; i += 256)
    m = max(m, __float_as_uint(fabsf(w[i])));
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0)
    part[threadIdx.x >> 5] = m;
  __syncthreads();
  m = part[0];
  for (int i = 1; i < 8; ++i)
    m = max(m, part[i]);
  const int e = scale_exponent(m, 13);
  const float down = pow2i(-e);
  if (threadIdx.x == 0 && blockIdx.x == 0)
    wscale[0] = pow2i(e);
  const int cpp = 8 / g.sw;
  const int s = blockIdx.x;
  for (int rem = threadIdx.x; rem < kN * 16; rem += 256) { // (map, K value); both pieces
    const int o = rem >> 4, kk = rem & 15;
    const int c2 = kk >> 3, k = kk & 7;
    const int ky = s / g.jsteps, j = s - ky * g.jsteps;
    const int t = k / cpp, c = k - t * cpp;
    const int kx = (2 * j + c2) * g.sw + t;
    float v = 0.0f;
    if (o < g.Ko && c < g.C && kx < g.kw)
      v = __fmul_rn(w[((o * g.C + c) * g.kh + ky) * g.kw + kx], down);
    __half p0, p1;
    split2(v, p0, p1);
    __half *base = out + (size_t)s * (kStepBytes / 2);
    base[(((o >> 3) * 2 + c2) * 8 + (o & 7)) * 8 + k] = p0;
    base[((((o + kN) >> 3) * 2 + c2) * 8 + (o & 7)) * 8 + k] = p1;
  }
}

// The staged rows a tile needs and where they sit in the ring. Loader and MMA issuer walk the same
// sequence of tiles and keep one of these each: rows are loaded in increasing order within a sample,
// every loaded row takes the next ring slot (count % kRing).
struct RowWalk {
  int count = 0;       // rows loaded so far by this block
  int sample = -1;     // sample of the previous tile
  int loaded_upto = 0; // first staged row of `sample` that is not in the ring
  // Advances to the tile (n, first row r0, kh rows); returns the number of rows to load, the first of
  // them in `first`, and the load count of row r0 in `s0`.
  __device__ __forceinline__ int next(int n, int r0, int kh, int &first, int &s0) {
    if (n != sample || r0 > loaded_upto) {
      sample = n;
      loaded_upto = r0;
    }
    first = loaded_upto;
    s0 = count - (loaded_upto - r0);
    const int nload = r0 + kh - first;
    count += nload;
    loaded_upto = r0 + kh;
    return nload;
  }
};

__global__ void __launch_bounds__(kThreadsNC, 1)
    narrow_conv_tcgen05_kernel(const __grid_constant__ CUtensorMap map_y, int box_store,
                               const uint8_t *__restrict__ xs, const uint8_t *__restrict__ wprep,
                               const float *__restrict__ xscale, const float *__restrict__ wscale,
                               const float *__restrict__ bias, float *__restrict__ y, NarrowConv g, int *status,
                               NarrowCodesOut co) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int steps = g.kh * g.jsteps;
  const uint32_t slot_bytes = 2u * (uint32_t)g.row_bytes;
  // rows past Wo of the last ring slot read up to (kM + 2 * jsteps) units of its second piece
  const uint32_t tail = (uint32_t)(kM + 2 * g.jsteps) * 16u;
  uint8_t *b_res = smem;                           // [step][16 groups][2 chunks][8 rows][16 B]
  uint8_t *ring = b_res + (size_t)steps * kStepBytes; // [slot][piece][row_bytes]
  // fp32 result: every epilogue warp stages [32 maps][32 pixels] boxes (two, used in turn) for bulk stores
  float *stage = reinterpret_cast<float *>(ring + ((kRing * slot_bytes + tail + 127u) & ~127u));
  uint64_t *bars = reinterpret_cast<uint64_t *>(stage + kEpilogueWarps * 2 * 1024);
  uint64_t *full_bar = bars, *done_bar = bars + kInFlight, *tmem_full = bars + 2 * kInFlight,
           *tmem_empty = bars + 2 * kInFlight + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kInFlight + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // bias of every map (0 past Ko or without bias), times 2 / delta when codes are written
  __shared__ float bias_s[kN];
  if (threadIdx.x < kN)
    bias_s[threadIdx.x] = (bias && (int)threadIdx.x < g.Ko)
                              ? (co.codes ? __fmul_rn(bias[threadIdx.x], co.two_inv) : bias[threadIdx.x])
                              : 0.0f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // consecutive output rows per block, so that a tile finds most of its input rows in the ring
  const int num_tiles = g.N * g.Ho;
  const int tile_first = (int)((int64_t)num_tiles * blockIdx.x / gridDim.x);
  const int tile_last = (int)((int64_t)num_tiles * (blockIdx.x + 1) / gridDim.x);
  constexpr uint32_t kTmemCols = 2 * kAccCols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kInFlight; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(done_bar + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(tmem_full + s, 1);
      ptx::mbar_init(tmem_empty + s, kEpilogueWarps);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  {
    // resident weights (already in the tensor core's layout) and zeros behind the ring
    const uint4 *src = reinterpret_cast<const uint4 *>(wprep);
    const int vecs = steps * (kStepBytes / 16);
    for (int i = threadIdx.x; i < vecs; i += kThreadsNC)
      reinterpret_cast<uint4 *>(b_res)[i] = __ldg(src + i);
    for (uint32_t i = threadIdx.x; i < tail / 16u; i += kThreadsNC)
      reinterpret_cast<uint4 *>(ring + kRing * slot_bytes)[i] = make_uint4(0, 0, 0, 0);
    fence_async_smem();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kLoadWarp) {
    // ------------------------------------------------------------ loader: the new rows of every tile
    if (ptx::elect_one()) {
      RowWalk walk;
      int s0_of[2 * kInFlight];
      int seq = 0, oldest = 0;
      bool ok = true;
      for (int tile = tile_first; tile < tile_last && ok; ++tile, ++seq) {
        const int n = tile / g.Ho, oy = tile - n * g.Ho;
        int first, s0;
        const int count_before = walk.count;
        const int nload = walk.next(n, oy * g.sh, g.kh, first, s0);
        // ring slots about to be overwritten, and the barrier of this tile, must have been released
        // by the tiles that used them
        while (oldest < seq && (s0_of[oldest & (2 * kInFlight - 1)] + kRing < walk.count || seq - oldest >= kInFlight)) {
          if (!ptx::mbar_wait(done_bar + (oldest & (kInFlight - 1)), (uint32_t)(oldest / kInFlight) & 1u, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusNcLoadTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ++oldest;
        }
        if (!ok)
          break;
        s0_of[seq & (2 * kInFlight - 1)] = s0;
        uint64_t *bar = full_bar + (seq & (kInFlight - 1));
        ptx::mbar_expect_tx(bar, (uint32_t)nload * slot_bytes);
        const uint8_t *src = xs + ((int64_t)n * g.Hp + first) * slot_bytes;
        for (int i = 0; i < nload; ++i)
          ptx::bulk_load(ring + (uint32_t)((count_before + i) % kRing) * slot_bytes, src + (int64_t)i * slot_bytes,
                         slot_bytes, bar);
      }
    }
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      RowWalk walk;
      int seq = 0;
      bool ok = true;
      const uint32_t idesc128 = ptx::make_idesc(1u, 0u, kM, 128), idesc64 = ptx::make_idesc(1u, 0u, kM, 64);
      const uint32_t b_base = ptx::smem_u32(b_res), ring_base = ptx::smem_u32(ring);
      for (int tile = tile_first; tile < tile_last && ok; ++tile, ++seq) {
        const int buf = seq & 1;
        const uint32_t buf_phase = (uint32_t)(seq >> 1) & 1u;
        const int n = tile / g.Ho, oy = tile - n * g.Ho;
        int first, s0;
        walk.next(n, oy * g.sh, g.kh, first, s0);
        if (!ptx::mbar_wait(tmem_empty + buf, buf_phase ^ 1u, abort_flag) ||
            !ptx::mbar_wait(full_bar + (seq & (kInFlight - 1)), (uint32_t)(seq / kInFlight) & 1u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusNcMmaTimeout);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kAccCols);
        uint32_t accumulate = 0;
        int step = 0;
        for (int ky = 0; ky < g.kh; ++ky) {
          const uint32_t row = ring_base + (uint32_t)((s0 + ky) % kRing) * slot_bytes;
          for (int j = 0; j < g.jsteps; ++j, ++step) {
            // rows 16 bytes apart, the second K chunk 16 bytes behind the first: sliding windows
            const uint64_t a0 = ptx::smem_desc_k_plain(row + (uint32_t)j * 32u, 16u, 128u);
            const uint64_t a1 = ptx::smem_desc_k_plain(row + (uint32_t)g.row_bytes + (uint32_t)j * 32u, 16u, 128u);
            const uint64_t b = ptx::smem_desc_k_plain(b_base + (uint32_t)step * kStepBytes, 128u, 256u);
            ptx::mma_bf16(d_tmem, a0, b, idesc128, accumulate);  // x0 x [w0; w1] -> columns 0..127
            ptx::mma_bf16(d_tmem + kN, a1, b, idesc64, 1u);      // x1 x [w0]     -> columns 64..127
            accumulate = 1;
          }
        }
        ptx::mma_commit(done_bar + (seq & (kInFlight - 1)));
        ptx::mma_commit(tmem_full + buf);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3; // TMEM lanes [32 * quarter, 32 * quarter + 32)
    const int half = warp >> 2;   // maps [32 * half, 32 * half + 32)
    int local = 0;
    const int px = quarter * 32 + lane;
    const int64_t plane = (int64_t)g.Ho * g.Wo;
    const float ws = __ldg(wscale);
    for (int tile = tile_first; tile < tile_last; ++tile, ++local) {
      const int buf = local & 1;
      const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
      const int n = tile / g.Ho, oy = tile - n * g.Ho;
      const float scale = __fmul_rn(__ldg(xscale + n), ws); // 2^(e - S)
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
      float *yrow = y + (int64_t)n * g.Ko * plane + (int64_t)oy * g.Wo + px;
      const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kAccCols);
      {
        uint32_t r0[32], r1[32];
        ptx::tmem_ld_32x32(t0 + (uint32_t)(half * 32), r0);      // x0 w0
        ptx::tmem_ld_32x32(t0 + (uint32_t)(kN + half * 32), r1); // x0 w1 + x1 w0, times 2^11
        ptx::tmem_ld_wait();
        if (co.codes != nullptr) {
          if (px < g.Wo && half * 32 < co.slots) {
            // u = conv * (2 / delta) + bias * (2 / delta), one fused multiply-add; then ReLU and the
            // quantizer of a non-negative value, (floor(u) + 1) >> 1 capped at kmax
            const float cap = (float)(2 * co.kmax) + 0.5f;
            const float k2 = __fmul_rn(scale, co.two_inv);
            uint32_t wds[8];
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              int c[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int j = 4 * j4 + k;
                const float raw = __fmaf_rn(__uint_as_float(r1[j]), 0.00048828125f, __uint_as_float(r0[j]));
                const float u = __fmaf_rn(raw, k2, bias_s[half * 32 + j]);
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
        } else if (box_store) {
          // the copy engine writes the box: whole lines, clipped at Wo and Ko, while the warp goes on
          float *box = stage + (warp * 2 + (local & 1)) * 1024;
          if (lane == 0)
            ptx::tma_store_wait_read<1>(); // the store before the previous one read this box
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = __fmul_rn(__fmaf_rn(__uint_as_float(r1[j]), 0.00048828125f, __uint_as_float(r0[j])), scale);
            if (bias)
              v = __fadd_rn(v, bias_s[half * 32 + j]);
            box[j * 32 + lane] = v;
          }
          ptx::fence_async_shared();
          __syncwarp();
          if (lane == 0 && quarter * 32 < g.Wo && half * 32 < g.Ko) {
            ptx::tma_store_4d(&map_y, box, quarter * 32, oy, half * 32, n);
            ptx::tma_store_commit();
          }
        } else if (px < g.Wo) {
          float *yp = yrow + (int64_t)(half * 32) * plane;
#pragma unroll
          for (int j = 0; j < 32; ++j, yp += plane) {
            const int o = half * 32 + j;
            if (o < g.Ko) {
              float v = __fmul_rn(__fmaf_rn(__uint_as_float(r1[j]), 0.00048828125f, __uint_as_float(r0[j])), scale);
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
  if (warp < kEpilogueWarps && lane == 0)
    ptx::tma_store_wait_all(); // this thread's bulk stores have been written
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // copies that may still be in flight must land before the shared memory is released
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull)
      __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// K steps per filter row, bytes of one staged piece row, shared memory of the kernel
struct NarrowPlan {
  int jsteps, steps, row_bytes;
  size_t smem;
};

NarrowPlan narrow_plan(int width, int kernel_h, int kernel_w, int pad_w, int stride_w, int Wo) {
  NarrowPlan p;
  p.jsteps = (kernel_w + 2 * stride_w - 1) / (2 * stride_w);
  p.steps = kernel_h * p.jsteps;
  const int units_image = (width + 2 * pad_w + stride_w - 1) / stride_w;
  const int units_read = Wo - 1 + 2 * p.jsteps; // by rows that hold an output pixel
  p.row_bytes = 16 * (units_image > units_read ? units_image : units_read);
  const size_t ring = ((size_t)kRing * 2 * p.row_bytes + (size_t)(kM + 2 * p.jsteps) * 16 + 127) & ~size_t(127);
  p.smem = (size_t)p.steps * kStepBytes + ring + kEpilogueWarps * 2 * 4096 + (2 * kInFlight + 4) * 8 + 16 + 128;
  return p;
}

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
  if (!(group == 1 && dilation_h == 1 && dilation_w == 1 && (stride_w == 1 || stride_w == 2) &&
        channels <= 8 / stride_w && outmaps <= kN && Wo <= kM && kernel_h <= kMaxKh))
    return false;
  const NarrowPlan p = narrow_plan(width, kernel_h, kernel_w, pad_w, stride_w, Wo);
  return p.steps <= kMaxSteps && p.row_bytes <= kMaxRowBytes && p.smem <= kMaxSmemNC;
}

int narrow_conv_tc(const float *x, const float *w, const float *bias, float *y, int batch, int channels, int height,
                   int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
                   int stride_w, int Ho, int Wo, cudaStream_t st, int8_t *y_codes, int slots, int relu, int kmax,
                   int kmin, float delta) {
  NarrowCodesOut co{y_codes, slots, relu, kmax, kmin, y_codes ? 2.0f / delta : 0.0f};
  const NarrowPlan p = narrow_plan(width, kernel_h, kernel_w, pad_w, stride_w, Wo);
  NarrowConv g{batch,    channels, height, width, outmaps, kernel_h,          kernel_w,    pad_h,
               pad_w,    stride_h, stride_w, Ho,  Wo,      height + 2 * pad_h, p.row_bytes, p.jsteps};
  NB_CHECK(batch <= 65535 && g.Hp <= 65535, NB200_ENOTIMPL, "batch or padded height larger than 65535");
  // scratch: weights | staged input | per-sample maxima (bits) | per-sample 2^e | 2^-S
  const size_t w_bytes = (size_t)p.steps * kStepBytes;
  const size_t xs_bytes = (size_t)batch * g.Hp * 2 * p.row_bytes;
  const size_t tail_bytes = ((size_t)batch * 8 + 16 + 255) & ~size_t(255);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(w_bytes + xs_bytes + tail_bytes));
  uint8_t *wprep = static_cast<uint8_t *>(scratch.p);
  uint8_t *xs = wprep + w_bytes;
  uint32_t *maxbits = reinterpret_cast<uint32_t *>(xs + xs_bytes);
  float *xscale = reinterpret_cast<float *>(maxbits + batch);
  float *wscale = xscale + batch;
  NB_CUDA(cudaMemsetAsync(maxbits, 0, (size_t)batch * 4, st));
  const int64_t per_sample = (int64_t)channels * height * width;
  int blocks = (int)((per_sample / 4 + 255) / 256);
  const int cap = (8 * sm_count() + batch - 1) / batch;
  blocks = blocks < 1 ? 1 : (blocks > cap ? (cap < 1 ? 1 : cap) : blocks);
  narrow_conv_absmax_kernel<<<dim3((unsigned)blocks, (unsigned)batch), 256, 0, st>>>(x, per_sample, maxbits);
  NB_LAUNCH_CHECK();
  narrow_conv_weights_kernel<<<p.steps, 256, 0, st>>>(w, g, reinterpret_cast<__half *>(wprep), wscale);
  NB_LAUNCH_CHECK();
  const dim3 split_grid((unsigned)((g.Hp + kSplitRows - 1) / kSplitRows), (unsigned)batch);
  if (stride_w == 2)
    narrow_conv_split_kernel<2><<<split_grid, 256, 0, st>>>(x, g, maxbits, xs, xscale);
  else
    narrow_conv_split_kernel<1><<<split_grid, 256, 0, st>>>(x, g, maxbits, xs, xscale);
  NB_LAUNCH_CHECK();
  static bool configured[64];
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    NB_CUDA(cudaFuncSetAttribute(narrow_conv_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmemNC));
    configured[dev & 63] = true;
  }
  // y as (Wo, Ho, Ko, N) fp32 for the bulk stores of the fp32 result (needs 16-byte row pitch and base)
  CUtensorMap map_y;
  const bool box_store = y_codes == nullptr && (Wo % 4) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
  {
    const bool real = box_store;
    const uint64_t dims[4] = {(uint64_t)(real ? Wo : 32), (uint64_t)(real ? Ho : 1), (uint64_t)(real ? outmaps : 32),
                              (uint64_t)(real ? batch : 1)};
    const uint64_t strides[3] = {dims[0] * 4, dims[0] * dims[1] * 4, dims[0] * dims[1] * dims[2] * 4};
    const uint32_t box[4] = {32, 1, 32, 1};
    // without a usable y the map covers the (16-byte aligned) scratch and is never used
    NB_TRY(encode_tiled(&map_y, 2, 4, real ? static_cast<const void *>(y) : static_cast<const void *>(wprep), dims,
                        strides, box, nullptr, 0));
  }
  int *status = nullptr;
  NB_TRY(device_status_word(&status));
  const int tiles = batch * Ho;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  narrow_conv_tcgen05_kernel<<<grid, kThreadsNC, p.smem, st>>>(map_y, box_store ? 1 : 0, xs, wprep, xscale, wscale, bias, y, g, status, co);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // namespace nb200
