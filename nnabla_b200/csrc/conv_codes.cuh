// Implicit-GEMM convolution of int8 channel-last activation codes with +-1
// (int8) weights on tcgen05, with the layer's whole inference tail in the
// epilogue:
//
//   u      = fma(acc, scale[o] * f, bias[o] * f)    (BN folded into scale / bias; f = 2 / delta, exact)
//   u      = fma(residual, step * f, u)             (codes with their step, or fp32; optional)
//   code   = min((floor(max(u, 0)) + 1) >> 1, kmax) -> int8, channel-last
//
// i.e. code * delta = FixedPointQuantize(ReLU(acc * scale + bias + residual)) with one rounding per
// fused multiply-add (the quantizer rounds |x| / delta + 0.5 down, which is (floor(2x / delta) + 1) >> 1).
//
// The PIXELS of a tile are the rows of the MMA (TMEM lanes), the output maps
// its columns: thread t of an epilogue warp owns one pixel and reads 32
// consecutive maps of it from TMEM, which are 32 consecutive bytes of the
// channel-last result, so the tile leaves as 128-bit stores of finished codes,
// one byte per value, with no transpose through shared memory.
//
//   A (M = 128 rows)  activation box: n_box images x h_box output rows x Wo
//                     pixels, one K block = one filter tap x E channel slots,
//                     fetched by a 5-D TMA box shifted by the tap (stride via
//                     element strides, padding = zero fill)
//   B (N columns)     weights [Ko][taps * c_slots], K-major, as
//                     nb200_binary_weights_prepare_i8 lays them out
//   D (TMEM)          int32, 128 lanes x N columns, double buffered
//
// Warp roles as in the plain contraction kernel: warp 0 TMA producer, warp 1
// MMA issuer and TMEM owner, eight epilogue warps (two per lane quarter,
// alternating 32-column chunks). Every wait is bounded (ptx::mbar_wait); a wait
// that gives up records a status code and all roles fall through to the
// teardown, which always frees TMEM.
#pragma once
#include "gemm.cuh"

namespace nb200 {

struct ConvCodesProblem {
  int Nimg, Ko, Ho, Wo;
  int h_box, n_box, tiles_h, tiles_n, n_tiles; // pixel boxes and column tiles
  int bn;                                      // UMMA N: columns per tile (multiple of 16)
  int kw, taps, cblocks;
  int sh, sw, ph, pw, dh, dw;
  int pixels;    // n_box * h_box * Wo (<= 128)
  int slots_out; // bytes per pixel of the code result / floats per pixel of the fp32 result
  // halo form (stride 1): one box of hp x wp input pixels per tile and channel block
  int wp, hp;          // wp = Wo + (kw - 1) * dw, hp = h_box + (kh - 1) * dh
  int a_tile_bytes;    // bytes of one channel block's pixel tile in shared memory (readable rows included)
  __device__ __forceinline__ int num_tiles() const { return n_tiles * tiles_h * tiles_n; }
  __device__ __forceinline__ int k_blocks() const { return taps * cblocks; }
};

struct ConvCodesEpilogue {
  const float *scale, *bias;   // per output map
  const int8_t *res_codes;     // residual as codes in the result's own layout (or NULL)
  const float *res_f32;        // residual as fp32, channel-last [pixels][slots_out] (or NULL)
  float res_scale;             // factor of the residual: (its step, or 1 for fp32) * out_scale
  int8_t *y_codes;             // result as codes (or NULL)
  float *y_f32;                // result as fp32 channel-last, before ReLU / quantizer (or NULL)
  float *y_nchw;               // result as fp32 [batch][maps][pixels]: acc * scale (+ bias), each operation rounded
                               // on its own like the reference's product followed by its bias addition (or NULL)
  int has_bias;
  int relu;
  float out_scale;             // factor of scale: 2 / delta when codes are written (delta: the quantizer's step, a
                               // power of two), the activations' step for the plain fp32 result, else 1
  float bias_scale;            // factor of bias: 2 / delta when codes are written, else 1
  int kmax, kmin;              // code range
#ifdef NB200_CC_TRACE
  long long *trace; // timing experiments: block 0 writes %globaltimer at its phase boundaries
#endif
};

#ifdef NB200_CC_TRACE
#define NB_CC_STAMP(slot, tile_local)                                                                                 \
  do {                                                                                                                 \
    if (ep.trace && blockIdx.x == 0 && (tile_local) < 64)                                                              \
      ep.trace[(tile_local) * 16 + (slot)] = (long long)ptx::globaltimer_ns();                                         \
  } while (0)
#define NB_CC_WAITED(slot, tile_local, expr)                                                                          \
  do {                                                                                                                 \
    const long long w0_ = (long long)ptx::globaltimer_ns();                                                            \
    expr;                                                                                                              \
    if (ep.trace && blockIdx.x == 0 && (tile_local) < 64)                                                              \
      ep.trace[(tile_local) * 16 + (slot)] += (long long)ptx::globaltimer_ns() - w0_;                                  \
  } while (0)
#else
#define NB_CC_WAITED(slot, tile_local, expr) expr
#define NB_CC_STAMP(slot, tile_local)                                                                                 \
  do {                                                                                                                 \
  } while (0)
#endif

// Exact for |a| < 2^22 (the accumulators of this kernel stay below 2^21 in magnitude for K <= 16384).
__device__ __forceinline__ float int_to_float(int a) {
  return __fsub_rn(__int_as_float(a + 0x4B400000), 12582912.0f);
}

// Four int32 codes -> four int8 lanes of one word (a in the lowest byte), each saturated to [-128, 127].
__device__ __forceinline__ uint32_t pack_s8x4(int a, int b, int c, int d) {
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
  return out;
}

constexpr int kCodesMaxMaps = 512;
constexpr int kCodesKTable = 64; // K blocks whose coordinates are tabulated once per block

// kResidentB: all tiles use the same weights (one column tile) and all their K blocks fit in
// shared memory beside the ring: the weights are loaded once per CTA and only the activation
// boxes stream. The copy engine spends about four cycles on every box row whatever its width,
// so a stage's weight rows (as many as its pixel rows, or more) are the larger part of its cost.
//
// kHalo (stride 1, with kResidentB): the filter taps of a stride-1 convolution read the SAME input
// pixels shifted by whole pixels, so a tile fetches its input once, as one box of hp x wp pixels
// per channel block (rows = pixels in raster order of the padded width wp), instead of once per
// tap. Output pixel (y, x) of the tile is MMA row y * wp + x (rows with x >= Wo are not stored),
// and tap (ky, kx) reads the same tile through a descriptor whose start is moved by
// (ky * dh * wp + kx * dw) rows. That works because the swizzle is a function of the shared-memory
// ADDRESS bits, for the copy engine's writes and the tensor core's reads alike: a start address
// that is a whole number of rows further on reads exactly the rows further on (no base-offset
// field is needed; setting one breaks it). This cuts the copy engine's rows per tile by the number
// of taps.
template <int BN, int STAGES, int RB, bool kResidentB = false, bool kHalo = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
    conv_codes_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                              const ConvCodesProblem prob, const ConvCodesEpilogue ep, int *status) {
  static_assert(RB == 128 || RB == 64, "operand rows are one 128-byte or 64-byte swizzle span");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N for M = 128");
  static_assert(!kHalo || kResidentB, "the halo form streams pixel tiles only");
  constexpr int kElems = RB;              // int8: K elements per operand row of one K block
  constexpr int kMmasPerBlock = RB / 32;  // 32 bytes of K per MMA
  constexpr uint32_t kABytes = kTileM * RB;
  constexpr uint32_t kBBytes = BN * RB;
  constexpr uint32_t kStageBytes = kABytes + (kResidentB ? 0u : kBBytes);
  constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // resident weights (kResidentB): [k block][BN rows] behind the ring
  const uint32_t resident_bytes = kResidentB ? (uint32_t)(prob.taps * prob.cblocks) * kBBytes : 0u;
  // halo form: the ring's place is taken by two buffers of cblocks pixel tiles each
  const uint32_t ring_bytes = kHalo ? 2u * (uint32_t)(prob.cblocks * prob.a_tile_bytes) : (uint32_t)STAGES * kStageBytes;
  uint8_t *b_resident = smem + ring_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + ring_bytes + resident_bytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *tmem_full = bars + 2 * STAGES;
  uint64_t *tmem_empty = bars + 2 * STAGES + 2;
  uint64_t *b_full = bars + 2 * STAGES + 4;
  uint64_t *a_full = bars + 2 * STAGES + 5;  // halo form: two pixel-tile buffers
  uint64_t *a_empty = bars + 2 * STAGES + 7;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 9);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // (scale, bias) of every output map, times out_scale; read as float4 pairs, so 16-byte aligned
  float2 *sb = reinterpret_cast<float2 *>((reinterpret_cast<uintptr_t>(tmem_slot + 4) + 15) & ~uintptr_t(15));
  const float4 *sb2 = reinterpret_cast<const float4 *>(sb);
  // per K block (filter tap x channel block): x = halo form's operand offset in 16-byte units, y = channel
  // coordinate, z / w = the tap's column / row shift. One thread issues all copies and all MMAs of a tile;
  // the two integer divisions per K block that these take cost it more than the instruction they feed.
  int4 *kb_table = reinterpret_cast<int4 *>(sb + kCodesMaxMaps);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = prob.num_tiles();
  const int k_blocks = prob.k_blocks();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tmem_full + b, 1);
      ptx::mbar_init(tmem_empty + b, kEpilogueWarps);
    }
    ptx::mbar_init(b_full, 1);
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(a_full + b, 1);
      ptx::mbar_init(a_empty + b, 1);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&map_x);
    ptx::prefetch_tensormap(&map_w);
  }
  auto kb_entry = [&](int kb) {
    const int tap = kb / prob.cblocks, cb = kb - tap * prob.cblocks;
    const int ky = tap / prob.kw, kx = tap - ky * prob.kw;
    return make_int4((cb * prob.a_tile_bytes + (ky * prob.dh * prob.wp + kx * prob.dw) * RB) >> 4, cb * kElems,
                     kx * prob.dw, ky * prob.dh);
  };
  const bool tabulated = k_blocks <= kCodesKTable;
  for (int kb = threadIdx.x; kb < k_blocks && kb < kCodesKTable; kb += kGemmThreads)
    kb_table[kb] = kb_entry(kb);
  for (int c = threadIdx.x; c < prob.n_tiles * BN; c += kGemmThreads)
    sb[c] = c < prob.Ko ? make_float2(ep.scale ? __fmul_rn(ep.scale[c], ep.out_scale) : ep.out_scale,
                                      ep.bias ? __fmul_rn(ep.bias[c], ep.bias_scale) : 0.0f)
                        : make_float2(0.0f, 0.0f);
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (column tile, pixel box); the column tiles of one box are neighbours in time (the box stays in L2)
  auto decode = [&](int tile, int &n0, int &img0, int &oy0) {
    const int nt = tile % prob.n_tiles;
    const int r = tile / prob.n_tiles;
    n0 = nt * BN;
    oy0 = (r % prob.tiles_h) * prob.h_box;
    img0 = (r / prob.tiles_h) * prob.n_box;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t tx_bytes = (uint32_t)(prob.pixels * RB) + (kResidentB ? 0u : kBBytes);
      if (kResidentB && (int)blockIdx.x < num_tiles) {
        ptx::mbar_expect_tx(b_full, resident_bytes);
        for (int kb = 0; kb < k_blocks; ++kb)
          ptx::tma_load_3d(b_resident + (size_t)kb * kBBytes, &map_w, b_full, kb * kElems, 0, 0);
      }
      int alocal = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++alocal) {
        int n0, img0, oy0;
        decode(tile, n0, img0, oy0);
        NB_CC_STAMP(0, (tile - (int)blockIdx.x) / (int)gridDim.x);
        if constexpr (kHalo) {
          const int ab = alocal & 1;
          if (!ptx::mbar_wait(a_empty + ab, ((uint32_t)(alocal >> 1) & 1u) ^ 1u, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusProducerTimeout);
            *abort_flag = 1;
            break;
          }
          ptx::mbar_expect_tx(a_full + ab, (uint32_t)(prob.cblocks * prob.hp * prob.wp * RB));
          for (int cb = 0; cb < prob.cblocks; ++cb)
            ptx::tma_load_5d(smem + (size_t)(ab * prob.cblocks + cb) * prob.a_tile_bytes, &map_x, a_full + ab,
                             cb * kElems, -prob.pw, oy0 - prob.ph, img0, 0);
        } else {
        for (int kb = 0; kb < k_blocks; ++kb) {
          bool got_slot;
          NB_CC_WAITED(9, (tile - (int)blockIdx.x) / (int)gridDim.x,
                       got_slot = ptx::mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag));
          if (!got_slot) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusProducerTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t *st = smem + stage * kStageBytes;
          ptx::mbar_expect_tx(full_bar + stage, tx_bytes);
          const int4 e = tabulated ? kb_table[kb] : kb_entry(kb);
          ptx::tma_load_5d(st, &map_x, full_bar + stage, e.y, e.z - prob.pw, oy0 * prob.sh - prob.ph + e.w, img0, 0);
          if (!kResidentB)
            ptx::tma_load_3d(st + kABytes, &map_w, full_bar + stage, kb * kElems, n0, 0);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        }
        NB_CC_STAMP(1, (tile - (int)blockIdx.x) / (int)gridDim.x);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      const uint32_t idesc = ptx::make_idesc(2u, 1u, kTileM, BN); // s32 accumulator, s8 operands
      if (kResidentB && (int)blockIdx.x < num_tiles) {
        if (!ptx::mbar_wait(b_full, 0u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusMmaTimeout);
          *abort_flag = 1;
          ok = false;
        }
        ptx::tc_fence_after_sync();
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        NB_CC_STAMP(2, local);
        if (!ptx::mbar_wait(tmem_empty + buf, buf_phase ^ 1u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusMmaTimeout);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        NB_CC_STAMP(3, local);
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        uint32_t accumulate = 0;
        if constexpr (kHalo) {
          const int ab = local & 1;
          if (!ptx::mbar_wait(a_full + ab, (uint32_t)(local >> 1) & 1u, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusMmaTimeout);
            *abort_flag = 1;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_base = ptx::smem_u32(smem) + (uint32_t)(ab * prob.cblocks * prob.a_tile_bytes);
          // (start addresses are 16-byte units in the low 14 bits of a descriptor; shared memory ends below 2^18)
          const uint64_t adesc0 = ptx::smem_desc_k(a_base, RB);
          const uint64_t bdesc0 = ptx::smem_desc_k(ptx::smem_u32(b_resident), RB);
          for (int kb = 0; kb < k_blocks; ++kb) {
            const uint64_t adesc = adesc0 + (uint64_t)(uint32_t)(tabulated ? kb_table[kb].x : kb_entry(kb).x);
            const uint64_t bdesc = bdesc0 + (uint64_t)((uint32_t)kb * (kBBytes >> 4));
#pragma unroll
            for (int k = 0; k < kMmasPerBlock; ++k) {
              ptx::mma_i8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
              accumulate = 1;
            }
          }
          ptx::mma_commit(a_empty + ab); // the pixel tile is free once these MMAs have read it
          ptx::mma_commit(tmem_full + buf);
        } else {
        for (int kb = 0; kb < k_blocks; ++kb) {
          bool got_data;
          NB_CC_WAITED(10, local, got_data = ptx::mbar_wait(full_bar + stage, phase, abort_flag));
          if (!got_data) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusMmaTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t st = ptx::smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = ptx::smem_desc_k(st, RB);
          const uint64_t bdesc = kResidentB ? ptx::smem_desc_k(ptx::smem_u32(b_resident) + (uint32_t)kb * kBBytes, RB)
                                            : ptx::smem_desc_k(st + kABytes, RB);
#pragma unroll
          for (int k = 0; k < kMmasPerBlock; ++k) {
            ptx::mma_i8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
            accumulate = 1;
          }
          ptx::mma_commit(empty_bar + stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok)
          ptx::mma_commit(tmem_full + buf);
        }
        NB_CC_STAMP(4, local);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;      // TMEM lanes [32 * quarter, +32) are visible to this warp
    const int half = (warp - 2) >> 2;  // the two warps of a quarter take even / odd 32-column chunks
    const int per_img = prob.h_box * prob.Wo;
    const float cap = (float)(2 * ep.kmax) + 0.5f;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      int n0, img0, oy0;
      decode(tile, n0, img0, oy0);
      const int buf = local & 1;
      const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
      // this thread's pixel
      const int row = quarter * 32 + lane;
      bool pix_ok;
      int img, in_plane; // image and pixel inside the image's plane
      if (kHalo) {
        const int y = row / prob.wp, x = row - y * prob.wp;
        img = img0;
        pix_ok = x < prob.Wo && y < prob.h_box && oy0 + y < prob.Ho && img0 < prob.Nimg;
        in_plane = (oy0 + y) * prob.Wo + x;
      } else {
        const int nn = row / per_img, q = row - nn * per_img;
        img = img0 + nn;
        pix_ok = nn < prob.n_box && img < prob.Nimg && q < (prob.Ho - oy0) * prob.Wo;
        in_plane = oy0 * prob.Wo + q;
      }
      const int64_t pix = (int64_t)img * prob.Ho * prob.Wo + in_plane;
      // the residual of this warp's first chunk is requested before the accumulator is waited for
      uint4 ra = make_uint4(0, 0, 0, 0), rb = make_uint4(0, 0, 0, 0);
      {
        const int col = n0 + 32 * half;
        if (ep.res_codes && pix_ok && col < prob.slots_out) {
          const int64_t off = pix * prob.slots_out + col;
          ra = __ldg(reinterpret_cast<const uint4 *>(ep.res_codes + off));
          if (col + 16 < prob.slots_out)
            rb = __ldg(reinterpret_cast<const uint4 *>(ep.res_codes + off) + 1);
        }
      }
      if (threadIdx.x == 64)
        NB_CC_STAMP(5, local);
      const bool got = ptx::mbar_wait(tmem_full + buf, buf_phase, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusEpilogueTimeout);
          *abort_flag = 1;
        }
        break;
      }
      ptx::tc_fence_after_sync();
      if (threadIdx.x == 64)
        NB_CC_STAMP(6, local);
#pragma unroll 1
      for (int c0 = 32 * half; c0 < BN; c0 += 64) {
        const int col = n0 + c0; // first output map of the chunk
        const bool live = pix_ok && col < (ep.y_nchw ? prob.Ko : prob.slots_out);
        const int64_t off = pix * prob.slots_out + col;
        const bool upper = col + 16 < prob.slots_out; // the pixel's row ends in the middle of this chunk otherwise
        if (c0 != 32 * half && ep.res_codes && live) { // later chunks: fetched here
          ra = __ldg(reinterpret_cast<const uint4 *>(ep.res_codes + off));
          rb = upper ? __ldg(reinterpret_cast<const uint4 *>(ep.res_codes + off) + 1) : make_uint4(0, 0, 0, 0);
        }
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), r);
        ptx::tmem_ld_wait();
        if (threadIdx.x == 64)
          NB_CC_STAMP(7, local);
        if (!live)
          continue;
        if (ep.y_nchw) {
          // fp32 [batch][maps][pixels]: the 32 lanes of a store are 32 neighbouring pixels of one map
          const int64_t plane = (int64_t)prob.Ho * prob.Wo;
          float *yp = ep.y_nchw + ((int64_t)img * prob.Ko + col) * plane + in_plane;
          // all 32 values first, without branches (maps past Ko have scale = bias = 0), then the stores:
          // with a test per map in between, the maps went through the pipes one after the other
          float val[32];
#pragma unroll
          for (int j2 = 0; j2 < 16; ++j2) {
            const float4 k = sb2[(col >> 1) + j2]; // (scale, bias) of two neighbouring maps
            val[2 * j2] = __fmul_rn((float)(int)r[2 * j2], k.x);
            val[2 * j2 + 1] = __fmul_rn((float)(int)r[2 * j2 + 1], k.z);
            if (ep.has_bias) {
              val[2 * j2] = __fadd_rn(val[2 * j2], k.y);
              val[2 * j2 + 1] = __fadd_rn(val[2 * j2 + 1], k.w);
            }
          }
          if (col + 32 <= prob.Ko) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              yp[(int64_t)j * plane] = val[j];
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < prob.Ko)
                yp[(int64_t)j * plane] = val[j];
          }
          continue;
        }
        // u = acc * scale + bias, one fused multiply-add (scale and bias already carry the factor
        // 2 / delta when codes are written, so u is twice the quantizer's argument)
        // Integers become floats on the add / multiply pipes instead of the (much narrower) conversion
        // pipe: for |a| < 2^22, the bit pattern of 1.5 * 2^23 plus a IS the float 1.5 * 2^23 + a.
        float v[32];
#pragma unroll
        for (int j2 = 0; j2 < 16; ++j2) {
          const float4 k = sb2[(col >> 1) + j2]; // (scale, bias) of two neighbouring maps
          v[2 * j2] = __fmaf_rn(int_to_float((int)r[2 * j2]), k.x, k.y);
          v[2 * j2 + 1] = __fmaf_rn(int_to_float((int)r[2 * j2 + 1]), k.z, k.w);
        }
        if (ep.res_codes) {
          // code + 128 (one XOR per word) lands in the low mantissa byte of 1.5 * 2^23
          const uint32_t w[8] = {ra.x ^ 0x80808080u, ra.y ^ 0x80808080u, ra.z ^ 0x80808080u, ra.w ^ 0x80808080u,
                                 rb.x ^ 0x80808080u, rb.y ^ 0x80808080u, rb.z ^ 0x80808080u, rb.w ^ 0x80808080u};
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float rc = __fsub_rn(__uint_as_float(__byte_perm(w[j >> 2], 0x4B400000u, 0x7650 + (j & 3))),
                                       12582912.0f + 128.0f);
            v[j] = __fmaf_rn(rc, ep.res_scale, v[j]);
          }
        } else if (ep.res_f32) {
          const float4 *rp = reinterpret_cast<const float4 *>(ep.res_f32 + off);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 t = (j4 < 4 || upper) ? __ldg(rp + j4) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[4 * j4 + 0] = __fmaf_rn(t.x, ep.res_scale, v[4 * j4 + 0]);
            v[4 * j4 + 1] = __fmaf_rn(t.y, ep.res_scale, v[4 * j4 + 1]);
            v[4 * j4 + 2] = __fmaf_rn(t.z, ep.res_scale, v[4 * j4 + 2]);
            v[4 * j4 + 3] = __fmaf_rn(t.w, ep.res_scale, v[4 * j4 + 3]);
          }
        }
        if (ep.y_f32) {
          float4 *yp = reinterpret_cast<float4 *>(ep.y_f32 + off);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4)
            if (j4 < 4 || upper)
              yp[j4] = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
          continue;
        }
        uint32_t w[8];
        if (ep.relu && ep.kmax == 127) {
          // ReLU, then the quantizer of a non-negative value: code = (floor(u) + 1) >> 1, capped at 127
          // by the saturating pack (maps past Ko have scale = bias = 0 and give code 0 on their own)
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            int c[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              // floor of 0 <= u < 2^23 without the conversion pipe: u + 2^23 rounded DOWN has it in its mantissa
              const float t = __fadd_rd(fminf(fmaxf(v[4 * j4 + k], 0.0f), cap), 8388608.0f); // a NaN becomes 0
              c[k] = (__float_as_int(t) - 0x4B000000 + 1) >> 1;
            }
            w[j4] = (uint32_t)c[0] | ((uint32_t)c[1] << 8) | ((uint32_t)c[2] << 16) | ((uint32_t)c[3] << 24); // each <= 127
          }
        } else {
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            uint32_t packed = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float x = v[4 * j4 + k];
              int code;
              if (ep.relu) {
                code = (__float2int_rd(fminf(fmaxf(x, 0.0f), cap)) + 1) >> 1;
              } else {
                const int m = (__float2int_rd(fminf(fabsf(x), cap)) + 1) >> 1;
                code = x < 0.0f ? max(-m, ep.kmin) : m;
              }
              packed |= ((uint32_t)code & 0xffu) << (8 * k);
            }
            w[j4] = packed;
          }
        }
        if (ep.y_codes == nullptr)
          continue; // no result configured (the host refuses this; never store through a null pointer)
        uint4 *yp = reinterpret_cast<uint4 *>(ep.y_codes + off);
        yp[0] = make_uint4(w[0], w[1], w[2], w[3]);
        if (upper)
          yp[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive(tmem_empty + buf);
      if (threadIdx.x == 64)
        NB_CC_STAMP(8, local);
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
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

// without the resident weights (k blocks * BN * RB bytes more when kResidentB)
// (in the halo form the ring is replaced by the pixel-tile buffers, counted by the caller)
template <int BN, int STAGES, int RB, bool kResidentB = false, bool kHalo = false>
constexpr size_t conv_codes_smem_bytes() {
  return (kHalo ? 0 : (size_t)STAGES * (kTileM * RB + (kResidentB ? 0 : BN * RB))) + (2 * STAGES + 9) * 8 + 32 +
         kCodesMaxMaps * sizeof(float2) + kCodesKTable * sizeof(int4) + 1024;
}

} // namespace nb200
