// The tcgen05 GEMM for M > 128: two CTAs of a cluster work as a pair on 256 x 256 output tiles.
//
//   C[M, N] = A[M, K] * B[N, K]^T      A and B K-major (K contiguous)
//
// In a pair (tcgen05 cta_group::2) each CTA stages its own 128 rows of A and only HALF of the B
// tile (128 of the 256 rows); the hardware feeds both tensor cores from both halves.  Per CTA and
// K step that is 32 KB through shared memory instead of 48 KB, which buys a deeper ring (6 stages)
// and 2-3 % more work per clock than the one-CTA kernel.  Measured at the board's power limit it is
// 2-6 % faster while B (N x K) stays resident in L2, and slower (lower sustained clocks) when B
// streams from HBM, so the launcher picks it only for the first case.
//
// Roles per CTA (192 threads):
//   warp 0   TMA producer of this CTA's A rows and B half; completion bytes of BOTH CTAs are
//            counted on the even CTA's `full` barrier;
//   warp 1   TMEM allocation (collective over the pair); in the even CTA one elected lane issues
//            tcgen05.mma.cta_group::2 (M256 x N256 x 32 bytes of K) and commits stage releases and
//            accumulator completion to the barriers of both CTAs (one commit each, no multicast);
//   warps 2-5 epilogue of this CTA's 128 accumulator rows; they release the accumulator on the even
//            CTA's `tmem_empty` barrier (a remote arrive from the odd CTA).
// Two 256-column accumulators per CTA overlap the epilogue of tile i with the main loop of tile
// i+1.  No TMA multicast.  Every mbarrier wait is bounded; on a timeout the kernel sets bit 1 of
// *status, lets work in flight land, and both CTAs meet at a cluster barrier before they free TMEM.
#include <cuda.h>

#include "gemm_common.cuh"

namespace amct {

constexpr int kPairStages = 6, kPairBN = 256, kPairThreads = 192;
constexpr int kPairBHalfBytes = 128 * kBKBytes;
constexpr int kPairStageBytes = kABytes + kPairBHalfBytes;        // per CTA

struct __align__(1024) PairSmem {
  uint8_t tiles[kPairStages][kPairStageBytes];
  float epi_scale[4][kPairBN];
  float epi_bias[4][kPairBN];
  uint8_t epi_stage[4][kEpiStageBytes];
  uint64_t full[kPairStages], empty[kPairStages], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__global__ void __launch_bounds__(kPairThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmParams p) {
  constexpr int kBN = kPairBN, kStages = kPairStages;
  constexpr int kTmemCols = 512;                                      // two 256-column accumulators
  extern __shared__ uint8_t smem_raw[];
  PairSmem& s = *reinterpret_cast<PairSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc05::cluster_ctarank();                      // 0: issues the MMAs
  const bool leader = rank == 0;
  const int64_t pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  const int esize = p.kind == KIND_I8 ? 1 : 2;
  const int bk = kBKBytes / esize;                                   // K elements per stage
  const int64_t num_kb = (p.k + bk - 1) / bk;
  const int64_t tiles_m = (p.m + 2 * kBM - 1) / (2 * kBM), tiles_n = (p.n + kBN - 1) / kBN;
  const int64_t num_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < kStages; ++i) { tc05::mbar_init(tc05::smem_u32(&s.full[i]), 1); tc05::mbar_init(tc05::smem_u32(&s.empty[i]), 1); }
    // tmem_empty (used in the even CTA): 4 epilogue warps of each CTA
    for (int i = 0; i < 2; ++i) { tc05::mbar_init(tc05::smem_u32(&s.tmem_full[i]), 1); tc05::mbar_init(tc05::smem_u32(&s.tmem_empty[i]), 8); }
    tc05::fence_barrier_init();
    tc05::prefetch_tmap(&tma_a);
    tc05::prefetch_tmap(&tma_b);
  }
  if (warp == 1) {
    tc05::tmem_alloc_pair(tc05::smem_u32(&s.tmem_base), kTmemCols);
    tc05::tmem_relinquish_pair();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::cluster_arrive();            // the other CTA's barriers are initialised before anything signals them
  tc05::cluster_wait();
  tc05::fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (tc05::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool alive = true;
      for (int64_t tile = pair_id; tile < num_tiles && alive; tile += num_pairs) {
        int64_t tm, tn;
        tile_coords(p.group_m, tile, tiles_m, tiles_n, &tm, &tn);
        tm = rotate_tile_m(p, tm, tiles_m, 2 * kBM);
        const int row_a = (int)(tm * 2 * kBM + rank * kBM);
        const int row_b = (int)(tn * kBN + rank * (kBN / 2));
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!tc05::mbar_wait(tc05::smem_u32(&s.empty[stage]), phase ^ 1, abort_flag)) { alive = false; break; }
          const uint32_t bar_local = tc05::smem_u32(&s.full[stage]);
          if (leader) tc05::mbar_expect_tx(bar_local, 2 * kPairStageBytes);     // both CTAs' bytes
          const uint32_t bar = tc05::map_to_cta(bar_local, 0);
          const uint32_t dst = tc05::smem_u32(&s.tiles[stage][0]);
          tc05::tma_load_2d_pair(dst, &tma_a, bar, (int)(kb * bk), row_a);
          tc05::tma_load_2d_pair(dst + kABytes, &tma_b, bar, (int)(kb * bk), row_b);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (leader && tc05::elect_one()) {
      const uint32_t idesc = p.kind == KIND_I8     ? tc05::make_idesc(2, 1, 1, 2 * kBM, kBN)
                             : p.kind == KIND_BF16 ? tc05::make_idesc(1, 1, 1, 2 * kBM, kBN)
                                                   : tc05::make_idesc(1, 0, 0, 2 * kBM, kBN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool alive = true;
      for (int64_t tile = pair_id; tile < num_tiles && alive; tile += num_pairs) {
        if (!tc05::mbar_wait(tc05::smem_u32(&s.tmem_empty[acc]), acc_phase ^ 1, abort_flag)) break;
        tc05::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!tc05::mbar_wait(tc05::smem_u32(&s.full[stage]), phase, abort_flag)) { alive = false; break; }
          tc05::fence_after_sync();
          const uint32_t a0 = tc05::smem_u32(&s.tiles[stage][0]);
          const uint32_t b0 = a0 + kABytes;
#pragma unroll
          for (int ks = 0; ks < kBKBytes / 32; ++ks) {
            const uint64_t adesc = tc05::smem_desc_sw128(a0 + ks * 32);
            const uint64_t bdesc = tc05::smem_desc_sw128(b0 + ks * 32);
            const uint32_t accumulate = (kb > 0 || ks > 0) ? 1u : 0u;
            if (p.kind == KIND_I8) tc05::umma_i8_pair(d_tmem, adesc, bdesc, idesc, accumulate);
            else tc05::umma_f16_pair(d_tmem, adesc, bdesc, idesc, accumulate);
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t e = tc05::smem_u32(&s.empty[stage]);
          tc05::umma_commit_pair(tc05::map_to_cta(e, 0));
          tc05::umma_commit_pair(tc05::map_to_cta(e, 1));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!alive) break;
        const uint32_t f = tc05::smem_u32(&s.tmem_full[acc]);         // accumulator complete, in both CTAs
        tc05::umma_commit_pair(tc05::map_to_cta(f, 0));
        tc05::umma_commit_pair(tc05::map_to_cta(f, 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;                                    // TMEM lane quarter this warp may read
    const int ew = warp - 2;
    float* sc = s.epi_scale[ew];
    float* sb = s.epi_bias[ew];
    uint32_t acc = 0, acc_phase = 0;
    for (int64_t tile = pair_id; tile < num_tiles; tile += num_pairs) {
      int64_t tm, tn;
      tile_coords(p.group_m, tile, tiles_m, tiles_n, &tm, &tn);
      tm = rotate_tile_m(p, tm, tiles_m, 2 * kBM);
      const int64_t n0 = tn * kBN;
      const int64_t row = tm * 2 * kBM + rank * kBM + quarter * 32 + lane;
      for (int c = lane; c < kBN; c += 32) {
        const int64_t n = n0 + c;
        sc[c] = (p.deq && n < p.n) ? p.deq[n] : 1.f;
        sb[c] = staged_bias(p, n);
      }
      const float pt = (p.pertoken && row < p.m) ? p.pertoken[row] : 1.f;
      __syncwarp();
      if (!tc05::mbar_wait(tc05::smem_u32(&s.tmem_full[acc]), acc_phase, abort_flag)) break;
      tc05::fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBN;
      if (p.scatter_world > 0)
        epilogue_rows_scatter<kBN>(p, t_row, tm * 2 * kBM + rank * kBM + quarter * 32, lane, n0, sc, sb, pt, s.epi_stage[ew]);
      else epilogue_rows<kBN>(p, t_row, row, n0, tn, sc, sb, pt);
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive_cluster(tc05::map_to_cta(tc05::smem_u32(&s.tmem_empty[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, 2);
    // let copies and MMAs already in flight land before the shared memory and TMEM go away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA may leave while the other can still read its shared memory or signal its barriers;
  // every wait above is bounded, so both CTAs get here
  tc05::cluster_arrive();
  tc05::cluster_wait();
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

int gemm_cta_budget();         // gemm_tcgen05.cu: SM count of the current device
bool gemm_pair_attr_needed();  // gemm_tcgen05.cu: true once per device

static int max_pairs() {
  const int n = gemm_cta_budget() / 2;
  return n > 0 ? n : 1;
}

// tma_a: box of 128 rows of A; tma_b: box of 128 rows of B (half a tile).
int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t st) {
  const size_t smem = sizeof(PairSmem) + 1024;
  if (gemm_pair_attr_needed()) {
    if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return AMCT_ERR_CUDA;
  }
  const int64_t tiles = ((p.m + 2 * kBM - 1) / (2 * kBM)) * ((p.n + kPairBN - 1) / kPairBN);
  const int pairs = (int)(tiles < max_pairs() ? tiles : max_pairs());
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel, ma, mb, p) != cudaSuccess) return AMCT_ERR_CUDA;
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct
