// Block-scaled MX GEMM on tcgen05 (sm_100a):
//
//   C[m, n] = sum over 32-element K blocks of 2^(sa[m,blk]-127) * 2^(sb[n,blk]-127) * (a_blk . b_blk)
//
// A [M, K] and B [N, K] are MXFP8-E4M3 bytes or packed MXFP4-E2M1 nibbles, K contiguous;
// the E8M0 scales arrive in the 128-row x 4-block tiling amct_mx_quant writes.  The
// reference has no such op; this is the GEMM stage of the MX configuration.
//
// Same skeleton as the INT8 GEMM (persistent 192-thread CTA per SM, TMA producer warp,
// single-thread MMA issuer, four epilogue warps, two accumulators in tensor memory) with
// 128 x 224 tiles: two 224-column fp32 accumulators leave 64 of the 512 TMEM columns for
// the scale factors.  Per 128-byte K slice the producer also bulk-copies the scale atoms
// (512 bytes per 128 rows per 4 K blocks) into shared memory; the MMA thread moves them
// into tensor memory with tcgen05.cp (in order with the MMAs that use them) and issues
// tcgen05.mma.kind::mxf8f6f4.block_scale (K = 32 per instruction, one scale byte per row)
// or kind::mxf4.block_scale.block32 (K = 64, two scale bytes per row).
// 224 is not a multiple of the 128-row scale atom and the scale address of the MMA must
// stay aligned, so B's scales are tiled per 224-row GEMM tile by the quantizer (two atoms
// per tile, the last 32 rows of the second one unused).
#include <cuda.h>

#include "common.cuh"
#include "tc05.cuh"

namespace amct {
namespace mx {

constexpr int kBM = 128, kBN = 224, kBKBytes = 128, kStages = 4;
constexpr int kABytes = kBM * kBKBytes, kBBytes = kBN * kBKBytes, kTileBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kAcc0 = 0, kAcc1 = kBN, kSfaCol = 2 * kBN, kSfbCol = 2 * kBN + 8;   // 448, 456 (.. 480)
constexpr int kGroupM = 16;
constexpr int kThreads = 192;

struct Params {
  int64_t m, n, k;             // k in elements
  int fp4;                     // 0: E4M3 bytes, 1: packed E2M1
  const uint8_t* sfa;          // tiled scales of A and B
  const uint8_t* sfb;
  const void* bias;
  int bias_kind;               // 0 none, 2 f32, 3 f16, 4 bf16
  void* out;
  int out_kind;                // 0 f32, 1 f16, 2 bf16
  int64_t ld_out;
  int* status;
};

struct __align__(1024) Smem {
  uint8_t tiles[kStages][kTileBytes];
  uint8_t sfa[kStages][1024];          // up to 2 atoms (fp4) of A's 128 rows
  uint8_t sfb[kStages][2][1024];       // 2 row atoms x up to 2 K atoms of B
  float epi_bias[4][kBN];
  uint64_t full[kStages], empty[kStages], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t* tm, int64_t* tn) {
  const int64_t per_group = (int64_t)kGroupM * tiles_n;
  const int64_t g = tile / per_group, r = tile - g * per_group;
  const int64_t m0 = g * kGroupM;
  const int64_t gm = (tiles_m - m0) < kGroupM ? (tiles_m - m0) : kGroupM;
  *tn = r / gm;
  *tm = m0 + r % gm;
}

__device__ __forceinline__ float bias_at(const void* bias, int kind, int64_t n) {
  if (kind == 2) return reinterpret_cast<const float*>(bias)[n];
  if (kind == 3) return __half2float(reinterpret_cast<const __half*>(bias)[n]);
  if (kind == 4) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n]);
  return 0.f;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int elems_per_stage = p.fp4 ? 256 : 128;                  // K elements in a 128-byte slice
  const int katoms = p.fp4 ? 2 : 1;                               // 4-block scale atoms per slice
  const int64_t num_kb = p.k / elems_per_stage;
  const int64_t kb4_total = (p.k / 32 + 3) / 4;                   // scale atoms along K
  const int64_t tiles_m = (p.m + kBM - 1) / kBM, tiles_n = (p.n + kBN - 1) / kBN;
  const int64_t num_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < kStages; ++i) { tc05::mbar_init(tc05::smem_u32(&s.full[i]), 1); tc05::mbar_init(tc05::smem_u32(&s.empty[i]), 1); }
    for (int i = 0; i < 2; ++i) { tc05::mbar_init(tc05::smem_u32(&s.tmem_full[i]), 1); tc05::mbar_init(tc05::smem_u32(&s.tmem_empty[i]), 4); }
    tc05::fence_barrier_init();
    tc05::prefetch_tmap(&tma_a);
    tc05::prefetch_tmap(&tma_b);
  }
  if (warp == 1) {
    tc05::tmem_alloc(tc05::smem_u32(&s.tmem_base), kTmemCols);
    tc05::tmem_relinquish();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (tc05::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        int64_t tm, tn;
        tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        const int64_t atom0 = tn * 2;                                             // B's scales: two atoms per 224-row tile
        const int natoms = 2;
        const uint32_t sf_bytes = 512u * katoms;
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!tc05::mbar_wait(tc05::smem_u32(&s.empty[stage]), phase ^ 1, abort_flag)) { alive = false; break; }
          const uint32_t bar = tc05::smem_u32(&s.full[stage]);
          tc05::mbar_expect_tx(bar, kTileBytes + sf_bytes * (1 + natoms));
          const uint32_t dst = tc05::smem_u32(&s.tiles[stage][0]);
          tc05::tma_load_2d(dst, &tma_a, bar, (int)(kb * kBKBytes), (int)(tm * kBM));
          tc05::tma_load_2d(dst + kABytes, &tma_b, bar, (int)(kb * kBKBytes), (int)(tn * kBN));
          const int64_t katom0 = kb * katoms;
          tc05::bulk_load_1d(tc05::smem_u32(&s.sfa[stage][0]), p.sfa + (tm * kb4_total + katom0) * 512, sf_bytes, bar);
          for (int a = 0; a < natoms; ++a)
            tc05::bulk_load_1d(tc05::smem_u32(&s.sfb[stage][a][0]), p.sfb + ((atom0 + a) * kb4_total + katom0) * 512, sf_bytes, bar);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (tc05::elect_one()) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        int64_t tm, tn;
        tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        if (!tc05::mbar_wait(tc05::smem_u32(&s.tmem_empty[acc]), acc_phase ^ 1, abort_flag)) break;
        tc05::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (acc ? kAcc1 : kAcc0);
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!tc05::mbar_wait(tc05::smem_u32(&s.full[stage]), phase, abort_flag)) { alive = false; break; }
          tc05::fence_after_sync();
          // scale atoms: shared -> tensor memory (4 columns per atom)
          for (int j = 0; j < katoms; ++j) {
            tc05::tmem_cp_32x128b_warpx4(tmem_base + kSfaCol + 4 * j, tc05::smem_desc_sf(tc05::smem_u32(&s.sfa[stage][512 * j])));
#pragma unroll
            for (int a = 0; a < 2; ++a)
              tc05::tmem_cp_32x128b_warpx4(tmem_base + kSfbCol + 8 * j + 4 * a,
                                           tc05::smem_desc_sf(tc05::smem_u32(&s.sfb[stage][a][512 * j])));
          }
          const uint32_t a0 = tc05::smem_u32(&s.tiles[stage][0]);
          const uint32_t b0 = a0 + kABytes;
#pragma unroll
          for (int ks = 0; ks < kBKBytes / 32; ++ks) {
            const uint64_t adesc = tc05::smem_desc_sw128(a0 + ks * 32);
            const uint64_t bdesc = tc05::smem_desc_sw128(b0 + ks * 32);
            const uint32_t accumulate = (kb > 0 || ks > 0) ? 1u : 0u;
            if (p.fp4) {
              const int j = ks >> 1;
              const uint32_t idesc = tc05::make_idesc_mx(1, kBM, kBN, (ks & 1) * 2);
              tc05::umma_mxf4(d_tmem, adesc, bdesc, idesc, tmem_base + kSfaCol + 4 * j, tmem_base + kSfbCol + 8 * j, accumulate);
            } else {
              const uint32_t idesc = tc05::make_idesc_mx(0, kBM, kBN, ks);
              tc05::umma_mxf8(d_tmem, adesc, bdesc, idesc, tmem_base + kSfaCol, tmem_base + kSfbCol, accumulate);
            }
          }
          tc05::umma_commit(tc05::smem_u32(&s.empty[stage]));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!alive) break;
        tc05::umma_commit(tc05::smem_u32(&s.tmem_full[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    float* sb = s.epi_bias[warp - 2];
    uint32_t acc = 0, acc_phase = 0;
    for (int64_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int64_t tm, tn;
      tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
      const int64_t n0 = tn * kBN;
      const int64_t row = tm * kBM + quarter * 32 + lane;
      // no bias is staged as -0.0f: x + (-0.0f) is x for every x, so the loop below adds unconditionally (an epilogue
      // warp is alone on its scheduler: a branch per element would cost its full latency each time)
      for (int c = lane; c < kBN; c += 32) sb[c] = (p.bias_kind && n0 + c < p.n) ? bias_at(p.bias, p.bias_kind, n0 + c) : -0.f;
      __syncwarp();
      if (!tc05::mbar_wait(tc05::smem_u32(&s.tmem_full[acc]), acc_phase, abort_flag)) break;
      tc05::fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (acc ? kAcc1 : kAcc0);
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t r[32];
        tc05::tmem_ld_32x32(t_row + c0, r);
        tc05::tmem_ld_wait();
        if (row < p.m && n0 + c0 < p.n) {
          float y[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) y[j] = __fadd_rn(__uint_as_float(r[j]), sb[c0 + j]);
          const int64_t nleft = p.n - (n0 + c0);
          const int64_t off = row * p.ld_out + n0 + c0;
          if (p.out_kind == 0) {
            float* o = reinterpret_cast<float*>(p.out) + off;
            if (nleft >= 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < nleft) o[j] = y[j];
            }
          } else {
            uint32_t h[16];
            epi_pack16(y, p.out_kind == 2, h);
            uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + off;
            if (nleft >= 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 16; j += 4) *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(h[j], h[j + 1], h[j + 2], h[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < nleft) o[j] = (uint16_t)(h[j >> 1] >> (16 * (j & 1)));
            }
          }
        }
      }
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(tc05::smem_u32(&s.tmem_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, 2);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace mx
}  // namespace amct

// ---------------------------------------------------------------------------- host side
namespace amct {
namespace mx {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, row_bytes] byte matrix -> tensor map with a 128-byte x box_rows box, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int64_t ld_bytes, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return AMCT_ERR_CUDA;
  if (!aligned16(base) || ld_bytes % 16 != 0) return AMCT_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
  cuuint32_t box[2] = {(cuuint32_t)kBKBytes, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? AMCT_OK : AMCT_ERR_CUDA;
}

}  // namespace mx
}  // namespace amct

extern "C" int amct_gemm_mx(const void* a, const void* sfa_tiled, const void* b, const void* sfb_tiled, int elem_bits,
                            int64_t m, int64_t n, int64_t k, int64_t ld_a_bytes, int64_t ld_b_bytes, const void* bias,
                            int bias_kind, void* out, int out_kind, int64_t ld_out, int* status, void* stream) {
  using namespace amct::mx;
  if (m < 0 || n < 0 || k <= 0 || (elem_bits != 8 && elem_bits != 4) || ld_out < n) return AMCT_ERR_ARG;
  if (m == 0 || n == 0) return AMCT_OK;
  if (!a || !b || !sfa_tiled || !sfb_tiled || !out) return AMCT_ERR_ARG;
  if (bias_kind != 0 && (bias_kind < 2 || bias_kind > 4 || !bias)) return AMCT_ERR_ARG;
  if (out_kind < 0 || out_kind > 2) return AMCT_ERR_ARG;
  const int fp4 = elem_bits == 4;
  if (k % (fp4 ? 256 : 128) != 0) return AMCT_ERR_UNSUPPORTED;          // whole 128-byte K slices only
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return AMCT_ERR_UNSUPPORTED;
  const int64_t row_bytes = fp4 ? k / 2 : k;
  if (ld_a_bytes < row_bytes || ld_b_bytes < row_bytes) return AMCT_ERR_ARG;
  if (!amct::aligned16(sfa_tiled) || !amct::aligned16(sfb_tiled)) return AMCT_ERR_ALIGN;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, row_bytes, ld_a_bytes, kBM);
  if (rc != AMCT_OK) return rc;
  rc = make_map(&mb, b, n, row_bytes, ld_b_bytes, kBN);
  if (rc != AMCT_OK) return rc;
  Params p{};
  p.m = m; p.n = n; p.k = k; p.fp4 = fp4;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa_tiled); p.sfb = reinterpret_cast<const uint8_t*>(sfb_tiled);
  p.bias = bias; p.bias_kind = bias_kind; p.out = out; p.out_kind = out_kind; p.ld_out = ld_out; p.status = status;
  const size_t smem = sizeof(Smem) + 1024;
  static amct::OncePerDevice attr_set;
  if (attr_set.first()) {
    if (cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return AMCT_ERR_CUDA;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = ((m + kBM - 1) / kBM) * ((n + kBN - 1) / kBN);
  const int grid = (int)(tiles < sms ? tiles : sms);
  gemm_mx_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(ma, mb, p);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}
