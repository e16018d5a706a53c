// Quantized GEMMs on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   C[M, N] = A[M, K] * B[N, K]^T      A and B K-major (K contiguous)
//
// This file: the one-CTA kernel (M <= 128, and M > 128 when asked for) and the C entry points;
// M > 128 normally runs the CTA-pair kernel of gemm_tcgen05_pair.cu.
// One persistent CTA per SM walks 128 x 256 output tiles.  Warp roles:
//   warp 0   TMA producer: cp.async.bulk.tensor tiles of A (128 x 128 B) and
//            B (256 x 128 B) into a 4-stage, 128-byte-swizzled shared-memory ring;
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma (M128 x N256 x 32 B of K
//            per instruction) from shared-memory descriptors into TMEM; owns the
//            TMEM allocation (512 columns = two 128 x 256 fp32/int32 accumulators);
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (each warp its own
//            32-lane quarter), apply the dequant epilogue, store to global.
// The two accumulators let the epilogue of tile i overlap the main loop of tile
// i+1.  No cluster launch, no multicast.  Every mbarrier wait is bounded; on a
// timeout the kernel sets bit 1 of *status, drains and returns.
//
// Epilogues (fp32, each step separately rounded, in this order):
//   W8A8 per-token : y = float(acc) * deq[n] * pertoken[m] + bias_f[n]
//   W8A8 per-tensor: y = float(acc + bias_i32[n]) * deq[n]
//   (the operand construction of amct_pytorch/deploy_op/npu_quantization_linear.py:61-68,
//    :105-130 fixes where each bias is added; the call is
//    torch_npu.npu_quant_matmul at :100-102)
//   raw            : int32 accumulators as they are
//   float kinds    : y = acc + bias_f[n]
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "gemm_common.cuh"

namespace amct {

// two tile shapes: 128 x 256 with a 4-stage ring (large M), and 128 x 64 with an 8-stage ring for
// M <= 128, where the job is to stream the weight once: more, smaller tiles keep every SM loading
constexpr int kBNLarge = 256, kStagesLarge = 4, kBNSmall = 64, kStagesSmall = 8;
constexpr int kThreads = 192;

template <int BN, int STAGES>
struct __align__(1024) GemmSmem {
  uint8_t tiles[STAGES][kABytes + BN * kBKBytes];
  float epi_scale[4][BN];
  float epi_bias[4][BN];
  uint8_t epi_stage[4][kEpiStageBytes];
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmParams p) {
  constexpr int kBN = BN, kStages = STAGES;
  constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;       // two accumulators; a power of two >= 32
  using Smem = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int esize = p.kind == KIND_I8 ? 1 : 2;
  const int bk = kBKBytes / esize;                                   // K elements per stage
  const int64_t num_kb = (p.k + bk - 1) / bk;
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
    // ------------------------------------------------------------ TMA producer
    if (tc05::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        int64_t tm, tn;
        tile_coords(p.group_m, tile, tiles_m, tiles_n, &tm, &tn);
        tm = rotate_tile_m(p, tm, tiles_m, kBM);
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!tc05::mbar_wait(tc05::smem_u32(&s.empty[stage]), phase ^ 1, abort_flag)) { alive = false; break; }
          const uint32_t bar = tc05::smem_u32(&s.full[stage]);
          tc05::mbar_expect_tx(bar, (uint32_t)(p.a_box_rows * kBKBytes + BN * kBKBytes));
          const uint32_t dst = tc05::smem_u32(&s.tiles[stage][0]);
          tc05::tma_load_2d(dst, &tma_a, bar, (int)(kb * bk), (int)(tm * kBM));
          tc05::tma_load_2d(dst + kABytes, &tma_b, bar, (int)(kb * bk), (int)(tn * kBN));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (tc05::elect_one()) {
      const uint32_t idesc = p.kind == KIND_I8     ? tc05::make_idesc(2, 1, 1, kBM, kBN)
                             : p.kind == KIND_BF16 ? tc05::make_idesc(1, 1, 1, kBM, kBN)
                                                   : tc05::make_idesc(1, 0, 0, kBM, kBN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
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
            if (p.kind == KIND_I8) tc05::umma_i8(d_tmem, adesc, bdesc, idesc, accumulate);
            else tc05::umma_f16(d_tmem, adesc, bdesc, idesc, accumulate);
          }
          tc05::umma_commit(tc05::smem_u32(&s.empty[stage]));        // frees the stage when these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!alive) break;
        tc05::umma_commit(tc05::smem_u32(&s.tmem_full[acc]));        // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;                                    // TMEM lane quarter this warp may read
    const int ew = warp - 2;
    float* sc = s.epi_scale[ew];
    float* sb = s.epi_bias[ew];
    uint32_t acc = 0, acc_phase = 0;
    for (int64_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int64_t tm, tn;
      tile_coords(p.group_m, tile, tiles_m, tiles_n, &tm, &tn);
      tm = rotate_tile_m(p, tm, tiles_m, kBM);
      const int64_t n0 = tn * kBN;
      const int64_t row = tm * kBM + quarter * 32 + lane;
      // stage the per-column factors of this tile (per warp, so only __syncwarp is needed)
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
      if (p.scatter_world > 0) epilogue_rows_scatter<kBN>(p, t_row, tm * kBM + quarter * 32, lane, n0, sc, sb, pt, s.epi_stage[ew]);
      else epilogue_rows<kBN>(p, t_row, row, n0, tn, sc, sb, pt);
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(tc05::smem_u32(&s.tmem_empty[acc]));
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
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------- host side
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

// [rows, k] K-major matrix -> tensor map with a (128 bytes of K) x box_rows box, 128-byte swizzle.  A tensor map
// depends only on (base, element size, rows, k, ld, box rows), not on the matrix's contents, and a deployed model
// calls with the same weights (and usually the same activation buffers) again and again: the last maps are kept
// in a small table per host thread, so the steady state encodes nothing.
struct MapKey {
  const void* base;
  int64_t rows, k, ld;
  int esize, box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && k == o.k && ld == o.ld && esize == o.esize && box_rows == o.box_rows;
  }
};
constexpr int kMapCacheSlots = 64;
struct MapCache {
  MapKey key[kMapCacheSlots];
  CUtensorMap map[kMapCacheSlots];
  bool used[kMapCacheSlots] = {};
};

static int make_map(CUtensorMap* map, const void* base, int esize, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  if (!aligned16(base) || (ld * esize) % 16 != 0) return AMCT_ERR_ALIGN;
  static thread_local MapCache cache;
  const MapKey key{base, rows, k, ld, esize, box_rows};
  const uint64_t hsh = (reinterpret_cast<uintptr_t>(base) >> 4) * 0x9E3779B97F4A7C15ull + (uint64_t)rows * 31 + (uint64_t)box_rows;
  const int slot = (int)((hsh >> 32) % kMapCacheSlots);
  if (cache.used[slot] && cache.key[slot] == key) { *map = cache.map[slot]; return AMCT_OK; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return AMCT_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * esize)};
  cuuint32_t box[2] = {(cuuint32_t)(kBKBytes / esize), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return AMCT_ERR_CUDA;
  cache.key[slot] = key; cache.map[slot] = *map; cache.used[slot] = true;
  return AMCT_OK;
}

// Per-device facts, looked up once per device: the SM count and whether each kernel's shared-memory attribute has
// been raised there (the attribute belongs to the device's context, not to the process).
constexpr int kMaxGemmDevices = 64;
struct DeviceFacts {
  int sms = 0;
  bool attr_small = false, attr_large = false, attr_pair = false;
};
static DeviceFacts g_dev[kMaxGemmDevices];
static std::mutex g_dev_mutex;

static DeviceFacts* device_facts() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxGemmDevices) return nullptr;
  DeviceFacts* f = &g_dev[dev];
  if (!f->sms) {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return nullptr;
    f->sms = n;
  }
  return f;
}

// Persistent CTAs of a GEMM on the current device: one per SM.
int gemm_cta_budget() {
  DeviceFacts* f = device_facts();
  return f ? f->sms : 1;
}

// Raises the dynamic shared-memory limit of the pair kernel once per device (used by gemm_tcgen05_pair.cu).
bool gemm_pair_attr_needed() {
  DeviceFacts* f = device_facts();
  if (!f || f->attr_pair) return false;
  f->attr_pair = true;
  return true;
}

int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t st);

// Which kernel takes M > 128.  The CTA-pair kernel does more work per clock; at the power limit it
// wins while the B operand stays in L2 and loses when B streams from HBM (measured on B200), hence
// the size rule.  amct_gemm_set_variant pins one of the two (tests, comparisons).
constexpr int64_t kPairMaxBBytes = 96LL << 20;
static std::atomic<int> g_variant{AMCT_GEMM_VARIANT_AUTO};
static bool use_pair_kernel(const GemmParams& p, int esize) {
  if (p.m <= 128) return false;
  const int v = g_variant.load(std::memory_order_relaxed);
  if (v == AMCT_GEMM_VARIANT_SINGLE) return false;
  if (v == AMCT_GEMM_VARIANT_PAIR) return true;
  return p.n * p.k * esize <= kPairMaxBBytes;
}

static int launch_gemm(const void* a, const void* b, int64_t ld_a, int64_t ld_b, const GemmParams& params, cudaStream_t st) {
  GemmParams p = params;
  if (p.m == 0 || p.n == 0) return AMCT_OK;
  if (p.k <= 0) return AMCT_ERR_ARG;
  if (p.m > 0x7fffffffLL || p.n > 0x7fffffffLL || p.k > 0x7fffffffLL) return AMCT_ERR_UNSUPPORTED;
  DeviceFacts* dev = device_facts();
  if (!dev) return AMCT_ERR_CUDA;
  const int esize = p.kind == KIND_I8 ? 1 : 2;
  CUtensorMap ma, mb;
  p.a_box_rows = p.m <= 64 ? 64 : kBM;
  int rc = make_map(&ma, a, esize, p.m, p.k, ld_a, p.a_box_rows);
  if (rc != AMCT_OK) return rc;
  if (use_pair_kernel(p, esize)) {
    // CTA pairs on 256 x 256 tiles: each CTA loads 128 rows of A and 128 rows (half a tile) of B
    rc = make_map(&mb, b, esize, p.n, p.k, ld_b, 128);
    if (rc != AMCT_OK) return rc;
    p.group_m = group_m_tiles(p.k * esize, 2 * kBM);
    return launch_gemm_pair(ma, mb, p, st);
  }
  const bool small = p.m <= 128 && p.act == 0;
  const int bn = small ? kBNSmall : kBNLarge;
  rc = make_map(&mb, b, esize, p.n, p.k, ld_b, bn);
  if (rc != AMCT_OK) return rc;
  p.group_m = group_m_tiles(p.k * esize, kBM);
  const int64_t tiles = ((p.m + kBM - 1) / kBM) * ((p.n + bn - 1) / bn);
  const int grid = (int)(tiles < dev->sms ? tiles : dev->sms);
  if (small) {
    const size_t smem = sizeof(GemmSmem<kBNSmall, kStagesSmall>) + 1024;
    if (!dev->attr_small) {
      if (cudaFuncSetAttribute(gemm_tcgen05_kernel<kBNSmall, kStagesSmall>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AMCT_ERR_CUDA;
      dev->attr_small = true;
    }
    gemm_tcgen05_kernel<kBNSmall, kStagesSmall><<<grid, kThreads, smem, st>>>(ma, mb, p);
  } else {
    const size_t smem = sizeof(GemmSmem<kBNLarge, kStagesLarge>) + 1024;
    if (!dev->attr_large) {
      if (cudaFuncSetAttribute(gemm_tcgen05_kernel<kBNLarge, kStagesLarge>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AMCT_ERR_CUDA;
      dev->attr_large = true;
    }
    gemm_tcgen05_kernel<kBNLarge, kStagesLarge><<<grid, kThreads, smem, st>>>(ma, mb, p);
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

extern "C" int amct_gemm_w8a8(const int8_t* a, const int8_t* b, int64_t m, int64_t n, int64_t k, int64_t ld_a, int64_t ld_b,
                              const float* deq_scale, const float* pertoken_scale, const void* bias, int bias_kind,
                              void* out, int out_kind, int64_t ld_out, int* status, void* stream) {
  if (m < 0 || n < 0 || k < 0 || ld_a < k || ld_b < k || ld_out < n) return AMCT_ERR_ARG;
  if (m && n && (!a || !b || !out)) return AMCT_ERR_ARG;
  if (bias_kind < amct::BIAS_NONE || bias_kind > amct::BIAS_BF16 || (bias_kind != amct::BIAS_NONE && !bias)) return AMCT_ERR_ARG;
  if (out_kind < amct::OUT_F32 || out_kind > amct::OUT_I32) return AMCT_ERR_ARG;
  if (out_kind != amct::OUT_I32 && !deq_scale) return AMCT_ERR_ARG;
  if (bias_kind == amct::BIAS_I32 && pertoken_scale) return AMCT_ERR_ARG;   // int32 bias belongs to the per-tensor mode
  amct::GemmParams p{};
  p.m = m; p.n = n; p.k = k; p.kind = amct::KIND_I8;
  p.deq = deq_scale; p.pertoken = pertoken_scale; p.bias = bias; p.bias_kind = bias_kind;
  p.out = out; p.out_kind = out_kind; p.ld_out = ld_out; p.status = status;
  return amct::launch_gemm(a, b, ld_a, ld_b, p, (cudaStream_t)stream);
}

extern "C" int amct_gemm_w8a8_swiglu(const int8_t* a, const int8_t* b, int64_t m, int64_t n, int64_t k, int64_t ld_a,
                                     int64_t ld_b, const float* deq_scale, const float* pertoken_scale, const void* bias,
                                     int bias_kind, void* out, int64_t ld_out, int* status, void* stream) {
  if (m < 0 || n < 0 || k < 0 || ld_a < k || ld_b < k || ld_out < n / 2) return AMCT_ERR_ARG;
  if (m && n && (!a || !b || !out || !deq_scale)) return AMCT_ERR_ARG;
  if (n % amct::kBNLarge != 0) return AMCT_ERR_UNSUPPORTED;                 // whole [128 gate | 128 up] blocks only
  if (bias_kind == amct::BIAS_I32 || bias_kind < amct::BIAS_NONE || bias_kind > amct::BIAS_BF16 || (bias_kind && !bias))
    return AMCT_ERR_ARG;
  if (!amct::aligned16(out) || (ld_out * 2) % 16 != 0) return AMCT_ERR_ALIGN;
  amct::GemmParams p{};
  p.m = m; p.n = n; p.k = k; p.kind = amct::KIND_I8;
  p.deq = deq_scale; p.pertoken = pertoken_scale; p.bias = bias; p.bias_kind = bias_kind;
  p.out = out; p.out_kind = amct::OUT_BF16; p.ld_out = ld_out; p.status = status; p.act = 1;
  return amct::launch_gemm(a, b, ld_a, ld_b, p, (cudaStream_t)stream);
}

extern "C" int amct_gemm_f16(const void* a, const void* b, int dtype, int64_t m, int64_t n, int64_t k, int64_t ld_a,
                             int64_t ld_b, const void* bias, int bias_kind, void* out, int out_kind, int64_t ld_out,
                             int* status, void* stream) {
  if (m < 0 || n < 0 || k < 0 || ld_a < k || ld_b < k || ld_out < n) return AMCT_ERR_ARG;
  if (m && n && (!a || !b || !out)) return AMCT_ERR_ARG;
  if (dtype != AMCT_DTYPE_F16 && dtype != AMCT_DTYPE_BF16) return AMCT_ERR_ARG;
  if (bias_kind == amct::BIAS_I32 || bias_kind < 0 || bias_kind > amct::BIAS_BF16 || (bias_kind && !bias)) return AMCT_ERR_ARG;
  if (out_kind < amct::OUT_F32 || out_kind > amct::OUT_BF16) return AMCT_ERR_ARG;
  amct::GemmParams p{};
  p.m = m; p.n = n; p.k = k; p.kind = dtype == AMCT_DTYPE_BF16 ? amct::KIND_BF16 : amct::KIND_F16;
  p.bias = bias; p.bias_kind = bias_kind; p.out = out; p.out_kind = out_kind; p.ld_out = ld_out; p.status = status;
  return amct::launch_gemm(a, b, ld_a, ld_b, p, (cudaStream_t)stream);
}

extern "C" int amct_gemm_w8a8_scatter(const int8_t* a, const int8_t* b, int64_t m, int64_t n, int64_t k, int64_t ld_a,
                                      int64_t ld_b, const float* deq_scale, const float* pertoken_scale,
                                      void* const* out_ptrs, int world, int slot, int64_t rows_per_rank, int out_kind,
                                      int64_t ld_out, int* status, void* stream) {
  if (m < 0 || n < 0 || k < 0 || ld_a < k || ld_b < k || ld_out < n) return AMCT_ERR_ARG;
  if (!out_ptrs || world < 1 || world > amct::kMaxScatterRanks || slot < 0 || slot >= world || rows_per_rank <= 0)
    return AMCT_ERR_ARG;
  if (m > rows_per_rank * world) return AMCT_ERR_ARG;
  if (m && n && (!a || !b || !deq_scale)) return AMCT_ERR_ARG;
  if (out_kind != amct::OUT_BF16 && out_kind != amct::OUT_F16) return AMCT_ERR_UNSUPPORTED;
  if (n % 64 != 0) return AMCT_ERR_UNSUPPORTED;
  if ((ld_out * 2) % 16 != 0) return AMCT_ERR_ALIGN;
  amct::GemmParams p{};
  p.m = m; p.n = n; p.k = k; p.kind = amct::KIND_I8;
  p.deq = deq_scale; p.pertoken = pertoken_scale; p.bias_kind = amct::BIAS_NONE;
  p.out_kind = out_kind; p.ld_out = ld_out; p.status = status;
  p.scatter_world = world; p.scatter_slot = slot; p.scatter_rows = rows_per_rank;
  p.row_rot = ((int64_t)(slot + 1) % world) * rows_per_rank;
  for (int r = 0; r < world; ++r) {
    if (!out_ptrs[r]) return AMCT_ERR_ARG;
    if (!amct::aligned16(out_ptrs[r])) return AMCT_ERR_ALIGN;
    p.scatter_out[r] = out_ptrs[r];
  }
  return amct::launch_gemm(a, b, ld_a, ld_b, p, (cudaStream_t)stream);
}

extern "C" int amct_gemm_set_variant(int variant) {
  if (variant != AMCT_GEMM_VARIANT_AUTO && variant != AMCT_GEMM_VARIANT_SINGLE && variant != AMCT_GEMM_VARIANT_PAIR)
    return AMCT_ERR_ARG;
  amct::g_variant.store(variant, std::memory_order_relaxed);
  return AMCT_OK;
}
