// Two-SM (cta_group::2) variant of the tcgen05 contraction for large plain
// GEMMs. A cluster of two CTAs computes one 256 x 256 output tile: CTA r of
// the pair TMA-loads its own 128 rows of A and its own 128 rows (output
// columns) of B — operand sharing WITHOUT any multicast copy — and the leader
// CTA issues tcgen05.mma.cta_group::2 instructions that read both halves from
// both shared memories and accumulate 128 x 256 per CTA in tensor memory.
// Per SM this loads 32 KB of operands per K block for the same MMA work that
// costs 48 KB with single-CTA 128 x 256 tiles, which matters because the
// single-CTA kernel is bound by L2 -> shared memory bandwidth.
//
// Barrier protocol (all waits time-bounded, as in gemm.cuh):
//   full[s]      lives in the leader; both CTAs' TMA loads complete_tx on it,
//                the leader's producer posts the expected byte count of both.
//   empty[s]     one per CTA; the leader's MMA thread commits to its own and to
//                the peer's (two plain commits, one per CTA) when the MMAs that
//                read stage s have finished.
//   tmem_full[b] one per CTA, committed the same way after the last K block.
//   tmem_empty[b] lives in the leader, count 16: the eight epilogue warps of both
//                CTAs arrive (the peer's remotely) when they have drained buffer b.
// The two CTAs synchronise as a cluster after barrier initialisation and
// before exit, so neither touches the other's shared memory outside that span.
#pragma once
#include <cstdlib>

#include "gemm.cuh"

namespace nb200 {
namespace ptx {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled load into this CTA's shared memory whose completion is signalled on a
// barrier that may live in the other CTA of the pair (no multicast).
__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const CUtensorMap *m, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2, uint64_t l2_policy) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
               "[%0], [%1, {%3, %4, %5}], [%2], %6;"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1),
               "r"(c2), "l"(l2_policy)
               : "memory");
}
// L2 eviction policies: operands are re-read by many tiles (keep them), the
// output is written once and never read by this kernel (let it go first).
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_pair_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void mma_pair_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}
// Arrives on the barrier at cluster address `bar` once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}


} // namespace ptx

constexpr int kPairEpilogueWarps = 8;                        // two per TMEM lane quarter, alternating column chunks
constexpr int kPairThreads = 32 * (2 + kPairEpilogueWarps); // warps per CTA: TMA, MMA, epilogue
constexpr int kPairTileM = 256; // rows of D per CTA pair
constexpr int kPairTileN = 256; // columns of D per CTA pair
constexpr int kPairEpilogueBytes = kPairEpilogueWarps * 4096; // one swizzled 32 x 32 fp32 box per epilogue warp

struct PairGemmProblem {
  int M, N, kblocks, m_tiles, n_tiles;
  int64_t ldy;
  int debug; // timing-knob builds only (-DNB200_GEMM_TIMING_KNOBS): 1 = no global stores, 2 = no operand loads after the first ring fill; always 0 otherwise
};

template <bool kInt8, int PA, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
    gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                             const __grid_constant__ CUtensorMap map_y, const PairGemmProblem prob,
                             const GemmEpilogue ep, int *status) {
  constexpr int kElemsPerBlock = kInt8 ? 128 : 64;
  constexpr int kUmmaK = kInt8 ? 32 : 16;
  constexpr int kMmasPerBlock = kElemsPerBlock / kUmmaK;
  constexpr uint32_t kABytes = kTileM * kRowBytes;         // this CTA's 128 rows of A
  constexpr uint32_t kBBytes = (kPairTileN / 2) * kRowBytes; // this CTA's 128 rows of B
  constexpr uint32_t kStageBytes = PA * kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 512; // two 256-column accumulators

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Epilogue staging: per warp two 32 x 32 fp32 boxes (4 KB each, 128-byte swizzle, 1024-byte aligned).
  uint8_t *stage_out = smem + STAGES * kStageBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(stage_out + kPairEpilogueBytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *tmem_full = bars + 2 * STAGES;
  uint64_t *tmem_empty = bars + 2 * STAGES + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank(); // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = prob.m_tiles * prob.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tmem_full + b, 1);
      ptx::mbar_init(tmem_empty + b, 2 * kPairEpilogueWarps);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_y);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync(); // the peer's barriers are initialised before anything is signalled remotely
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t keep = ptx::l2_policy_evict_last();
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % prob.m_tiles) * kPairTileM + (int)rank * kTileM;
        const int n0 = (tile / prob.m_tiles) * kPairTileN + (int)rank * (kPairTileN / 2);
        for (int kb = 0; kb < prob.kblocks; ++kb) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag)) {
            if (*abort_flag == 0)
              atomicCAS(status, 0, kStatusProducerTimeout);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t *st = smem + stage * kStageBytes;
          const uint32_t leader_full = ptx::map_to_cta(ptx::smem_u32(full_bar + stage), 0);
          if (kTimingKnobs && (prob.debug & 2) && (tile != pair_id || kb >= STAGES)) {
            if (rank == 0)
              ptx::mbar_arrive(full_bar + stage);
          } else {
          if (rank == 0)
            ptx::mbar_expect_tx(full_bar + stage, 2 * kStageBytes); // bytes of both CTAs
#pragma unroll
          for (int pa = 0; pa < PA; ++pa)
            ptx::tma_load_3d_pair(st + pa * kABytes, &map_a, leader_full, kb * kElemsPerBlock, m0, pa, keep);
          ptx::tma_load_3d_pair(st + PA * kABytes, &map_b, leader_full, kb * kElemsPerBlock, n0, 0, keep);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader only)
    if (rank == 0 && ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      const uint32_t idesc = ptx::make_idesc(kInt8 ? 2u : 1u, 1u, kPairTileM, kPairTileN);
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        if (!ptx::mbar_wait(tmem_empty + buf, buf_phase ^ 1u, abort_flag)) {
          if (*abort_flag == 0)
            atomicCAS(status, 0, kStatusMmaTimeout);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kPairTileN);
        uint32_t accumulate = 0;
        for (int kb = 0; kb < prob.kblocks; ++kb) {
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
            const uint64_t adesc = ptx::smem_desc_k_sw128(st + pa * kABytes);
            const uint64_t bdesc = ptx::smem_desc_k_sw128(st + PA * kABytes);
#pragma unroll
            for (int k = 0; k < kMmasPerBlock; ++k) {
              if (kInt8)
                ptx::mma_pair_i8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
              else
                ptx::mma_pair_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accumulate);
              accumulate = 1;
            }
          }
          // Free the stage in both CTAs once these MMAs have read it.
          ptx::mma_commit_pair(ptx::smem_u32(empty_bar + stage));
          ptx::mma_commit_pair(ptx::map_to_cta(ptx::smem_u32(empty_bar + stage), 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          ptx::mma_commit_pair(ptx::smem_u32(tmem_full + buf));
          ptx::mma_commit_pair(ptx::map_to_cta(ptx::smem_u32(tmem_full + buf), 1));
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    int local = 0;
    bool ok = true;
    const uint64_t stream_out = ptx::l2_policy_evict_first();
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local) {
      const int buf = local & 1;
      const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
      const int m0 = (tile % prob.m_tiles) * kPairTileM + (int)rank * kTileM;
      const int n0 = (tile / prob.m_tiles) * kPairTileN;
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
      // Each thread owns one accumulator row. A chunk of 32 columns is scaled,
      // written to a swizzled 32 x 32 box in shared memory with 128-bit stores
      // and handed to the copy engine, which writes full lines of y and clips
      // at the matrix edges. Column factors are fetched one per lane and
      // broadcast by shuffles, so the inner loop has no memory loads.
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < prob.M;
      const float rs = (ep.row_scale && row_ok) ? __fmul_rn(ep.row_scale[row], ep.scale) : ep.scale;
      const float rb = (ep.row_bias && row_ok) ? ep.row_bias[row] : 0.0f;
      uint8_t *box = stage_out + (warp - 2) * 4096;
      const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll 1
      for (int c0 = 32 * half; c0 < kPairTileN; c0 += 32 * (kPairEpilogueWarps / 4)) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kPairTileN + c0), r);
        ptx::tmem_ld_wait();
        const int col0 = n0 + c0;
        if (col0 >= prob.N || (kTimingKnobs && (prob.debug & 1)))
          continue;
        const bool lane_col_ok = col0 + lane < prob.N;
        const float cs_l = (ep.col_scale && lane_col_ok) ? ep.col_scale[col0 + lane] : 1.0f;
        const float cb_l = (ep.col_bias && lane_col_ok) ? ep.col_bias[col0 + lane] : 0.0f;
        // the previous store from this box must have finished reading it
        if (lane == 0)
          ptx::tma_store_wait_read<0>();
        __syncwarp();
        float4 *rowp = reinterpret_cast<float4 *>(box + lane * 128);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float o[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = 4 * q + u;
            const float acc = kInt8 ? (float)(int)r[j] : __uint_as_float(r[j]);
            float s = rs;
            if (ep.col_scale)
              s = __fmul_rn(rs, __shfl_sync(0xffffffffu, cs_l, j));
            float v = __fmul_rn(acc, s);
            if (ep.row_bias)
              v = __fadd_rn(v, rb);
            if (ep.col_bias)
              v = __fadd_rn(v, __shfl_sync(0xffffffffu, cb_l, j));
            o[u] = v;
          }
          rowp[q ^ sw] = make_float4(o[0], o[1], o[2], o[3]);
        }
        ptx::fence_async_shared();
        __syncwarp();
        if (lane == 0 && !(kTimingKnobs && (prob.debug & 4))) {
          ptx::tma_store_2d(&map_y, box, col0, m0 + quarter * 32, stream_out);
          ptx::tma_store_commit();
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(tmem_empty + buf), 0));
    }
  }

  // ------------------------------------------------------------------ teardown
  if (warp >= 2 && lane == 0)
    ptx::tma_store_wait_all(); // this thread's bulk stores have been written
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull)
      __nanosleep(1000);
    __syncthreads();
  }
  ptx::cluster_sync(); // neither CTA leaves while its peer may still signal its barriers
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <bool kInt8, int PA, int STAGES> constexpr size_t gemm_pair_smem_bytes() {
  return (size_t)STAGES * (PA * kTileM * kRowBytes + (kPairTileN / 2) * kRowBytes) + (2 * STAGES + 4) * 8 + 16 +
         kPairEpilogueBytes + 1024;
}

template <bool kInt8, int PA, int STAGES>
inline int launch_pair_gemm(const CUtensorMap &ma, const CUtensorMap &mb, int M, int N, int k_blocks,
                            const GemmEpilogue &ep, int64_t ldy, cudaStream_t st) {
  // y as a tiled tensor for the bulk stores: (N, M) fp32, 32 x 32 boxes, 128-byte swizzle.
  CUtensorMap my;
  {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)ldy * 4};
    const uint32_t box[2] = {32, 32};
    NB_TRY(encode_tiled(&my, 2, 2, ep.y, dims, strides, box, nullptr));
  }
  auto kernel = gemm_pair_tcgen05_kernel<kInt8, PA, STAGES>;
  constexpr size_t smem = gemm_pair_smem_bytes<kInt8, PA, STAGES>();
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static bool configured[64];
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    NB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev & 63] = true;
  }
  PairGemmProblem prob;
  prob.M = M;
  prob.N = N;
  prob.kblocks = k_blocks;
  prob.m_tiles = (M + kPairTileM - 1) / kPairTileM;
  prob.n_tiles = (N + kPairTileN - 1) / kPairTileN;
  prob.ldy = ldy;
  prob.debug = 0;
#ifdef NB200_GEMM_TIMING_KNOBS
  {
    const char *e = std::getenv("NNABLA_B200_GEMM_DEBUG");
    prob.debug = e ? std::atoi(e) : 0;
  }
#endif
  int *status = nullptr;
  NB_TRY(device_status_word(&status));
  const int tiles = prob.m_tiles * prob.n_tiles;
  int pairs = sm_count() / 2;
  if (pairs > tiles)
    pairs = tiles;
  kernel<<<2 * pairs, kPairThreads, smem, st>>>(ma, mb, my, prob, ep, status);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // namespace nb200
