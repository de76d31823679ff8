// Implicit-GEMM convolution of int8 channel-last activation codes with +-1
// (int8) weights on tcgen05, with the layer's whole inference tail in the
// epilogue:
//
//   v      = float(acc) * scale[o] + bias[o]        (BN folded into scale / bias)
//   v     += residual                               (codes * step, or fp32, optional)
//   code   = FixedPointQuantize(ReLU(v)) / delta    -> int8, channel-last
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
  __device__ __forceinline__ int num_tiles() const { return n_tiles * tiles_h * tiles_n; }
  __device__ __forceinline__ int k_blocks() const { return taps * cblocks; }
};

struct ConvCodesEpilogue {
  const float *scale, *bias;   // per output map
  const int8_t *res_codes;     // residual as codes in the result's own layout (or NULL)
  float res_delta;
  const float *res_f32;        // residual as fp32, channel-last [pixels][slots_out] (or NULL)
  int8_t *y_codes;             // result as codes (or NULL)
  float *y_f32;                // result as fp32 channel-last, before ReLU / quantizer (or NULL)
  int relu;
  float delta, inv_delta;      // quantizer step (a power of two) and its reciprocal
  int kmax, kmin;              // code range
};

constexpr int kCodesMaxMaps = 512;

template <int BN, int STAGES, int RB>
__global__ void __launch_bounds__(kGemmThreads, 1)
    conv_codes_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                              const ConvCodesProblem prob, const ConvCodesEpilogue ep, int *status) {
  static_assert(RB == 128 || RB == 64, "operand rows are one 128-byte or 64-byte swizzle span");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N for M = 128");
  constexpr int kElems = RB;              // int8: K elements per operand row of one K block
  constexpr int kMmasPerBlock = RB / 32;  // 32 bytes of K per MMA
  constexpr uint32_t kABytes = kTileM * RB;
  constexpr uint32_t kBBytes = BN * RB;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * kStageBytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *tmem_full = bars + 2 * STAGES;
  uint64_t *tmem_empty = bars + 2 * STAGES + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float2 *sb = reinterpret_cast<float2 *>(tmem_slot + 4); // (scale, bias) of every output map

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
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&map_x);
    ptx::prefetch_tensormap(&map_w);
  }
  for (int c = threadIdx.x; c < prob.n_tiles * BN; c += kGemmThreads)
    sb[c] = c < prob.Ko ? make_float2(ep.scale[c], ep.bias ? ep.bias[c] : 0.0f) : make_float2(0.0f, 0.0f);
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
      const uint32_t tx_bytes = (uint32_t)(prob.pixels * RB) + kBBytes;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int n0, img0, oy0;
        decode(tile, n0, img0, oy0);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusProducerTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t *st = smem + stage * kStageBytes;
          ptx::mbar_expect_tx(full_bar + stage, tx_bytes);
          const int tap = kb / prob.cblocks, cb = kb - tap * prob.cblocks;
          const int ky = tap / prob.kw, kx = tap - ky * prob.kw;
          ptx::tma_load_5d(st, &map_x, full_bar + stage, cb * kElems, kx * prob.dw - prob.pw,
                           oy0 * prob.sh - prob.ph + ky * prob.dh, img0, 0);
          ptx::tma_load_3d(st + kABytes, &map_w, full_bar + stage, kb * kElems, n0, 0);
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
      const uint32_t idesc = ptx::make_idesc(2u, 1u, kTileM, BN); // s32 accumulator, s8 operands
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        if (!ptx::mbar_wait(tmem_empty + buf, buf_phase ^ 1u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusMmaTimeout);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        uint32_t accumulate = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait(full_bar + stage, phase, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusMmaTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t st = ptx::smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = ptx::smem_desc_k(st, RB), bdesc = ptx::smem_desc_k(st + kABytes, RB);
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
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;      // TMEM lanes [32 * quarter, +32) are visible to this warp
    const int half = (warp - 2) >> 2;  // the two warps of a quarter take even / odd 32-column chunks
    const int per_img = prob.h_box * prob.Wo;
    const float two_inv = __fmul_rn(ep.inv_delta, 2.0f), cap = (float)(2 * ep.kmax) + 0.5f;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      int n0, img0, oy0;
      decode(tile, n0, img0, oy0);
      const int buf = local & 1;
      const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
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
      // this thread's pixel
      const int row = quarter * 32 + lane;
      const int nn = row / per_img, q = row - nn * per_img;
      const int img = img0 + nn;
      const bool pix_ok = nn < prob.n_box && img < prob.Nimg && q < (prob.Ho - oy0) * prob.Wo;
      const int64_t pix = (int64_t)img * prob.Ho * prob.Wo + (int64_t)oy0 * prob.Wo + q;
#pragma unroll 1
      for (int c0 = 32 * half; c0 < BN; c0 += 64) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), r);
        ptx::tmem_ld_wait();
        const int col = n0 + c0; // first output map of the chunk
        if (!pix_ok || col >= prob.slots_out)
          continue;
        const int64_t off = pix * prob.slots_out + col;
        const bool upper = col + 16 < prob.slots_out; // the pixel's row ends in the middle of this chunk otherwise
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float2 k = sb[col + j];
          v[j] = __fadd_rn(__fmul_rn((float)(int)r[j], k.x), k.y);
        }
        if (ep.res_codes) {
          const uint4 a = __ldg(reinterpret_cast<const uint4 *>(ep.res_codes + off));
          const uint4 b = upper ? __ldg(reinterpret_cast<const uint4 *>(ep.res_codes + off) + 1) : make_uint4(0, 0, 0, 0);
          const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int rc = (int)(int8_t)((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
            v[j] = __fadd_rn(v[j], __fmul_rn((float)rc, ep.res_delta));
          }
        } else if (ep.res_f32) {
          const float4 *rp = reinterpret_cast<const float4 *>(ep.res_f32 + off);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 t = (j4 < 4 || upper) ? __ldg(rp + j4) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[4 * j4 + 0] = __fadd_rn(v[4 * j4 + 0], t.x);
            v[4 * j4 + 1] = __fadd_rn(v[4 * j4 + 1], t.y);
            v[4 * j4 + 2] = __fadd_rn(v[4 * j4 + 2], t.z);
            v[4 * j4 + 3] = __fadd_rn(v[4 * j4 + 3], t.w);
          }
        }
        if (ep.y_f32) {
          float4 *yp = reinterpret_cast<float4 *>(ep.y_f32 + off);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4)
            if (j4 < 4 || upper)
              yp[j4] = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
        }
        if (ep.y_codes) {
          uint32_t w[8];
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            uint32_t packed = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float x = v[4 * j4 + k];
              int code;
              if (ep.relu) {
                // ReLU, then the quantizer of a non-negative value: (floor(2x / delta) + 1) >> 1, capped
                x = fmaxf(x, 0.0f); // a NaN becomes 0
                code = (__float2int_rd(fminf(__fmul_rn(x, two_inv), cap)) + 1) >> 1;
              } else {
                const float a = fminf(__fmul_rn(fabsf(x), two_inv), cap);
                const int m = (__float2int_rd(a) + 1) >> 1;
                code = x < 0.0f ? max(-m, ep.kmin) : m;
              }
              code = (col + 4 * j4 + k < prob.Ko) ? code : 0; // padding slots stay zero
              packed |= ((uint32_t)code & 0xffu) << (8 * k);
            }
            w[j4] = packed;
          }
          uint4 *yp = reinterpret_cast<uint4 *>(ep.y_codes + off);
          yp[0] = make_uint4(w[0], w[1], w[2], w[3]);
          if (upper)
            yp[1] = make_uint4(w[4], w[5], w[6], w[7]);
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

template <int BN, int STAGES, int RB> constexpr size_t conv_codes_smem_bytes() {
  return (size_t)STAGES * (kTileM * RB + BN * RB) + (2 * STAGES + 4) * 8 + 16 + kCodesMaxMaps * sizeof(float2) + 1024;
}

} // namespace nb200
