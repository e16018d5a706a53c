// Weight-only quantized Linear as ONE kernel: the weight codes are dequantized in shared memory
// ahead of the tensor-core MMA, the 16-bit weight never exists in HBM.
//
//   y[m, n] = sum_k x[m, k] * w[n, k] + bias[n],   w[n, k] = (q[n, k] + aoff[g(k), n]) * ascale[g(k), n]
//
// the product torch_npu.npu_weight_quant_batchmatmul computes (call site
// amct_pytorch/deploy_op/weight_npu_quant_module.py:116-117; ascale / aoff = scale_w and the
// negated offset_w buffers built at :59-64, laid out [K/group, N], or [1, N] when group == 0).
// w is rounded to the activation dtype exactly as the separate dequant kernel (w4a16.cu) rounds
// it, so both routes feed the MMA the same operand bits.
//
// The kernel computes the TRANSPOSE, y^T[n, m] = w[n, :] . x[m, :]: the 128-row MMA operand is the
// weight tile (always full), the N-side operand is a tile of BN = 32 / 64 / 128 tokens.  A decode
// call (few tokens) then streams each weight byte once and wastes no MMA rows on padding.
// Warp roles (736 threads, one CTA per SM, persistent over tiles):
//   warp 0     TMA of the codes: slots of 128 rows x 128 bytes (256 INT4 or 128 byte codes of K per row), a ring of
//              its own that runs several K steps ahead of the MMA stages;
//   warp 6     TMA of the x tile (BN x 128 bytes) of each 64-element K step;
//   warp 1     TMEM allocation; one elected lane issues tcgen05.mma (M128 x N BN x K16, kind::f16);
//   warps 2-5  epilogue: tcgen05.ld of the accumulator (lane = output channel n), bias, transposed store;
//   warps 7-22 dequant, four groups of four warps, group g on the K steps g (mod 4): one thread per weight row turns
//              the raw codes of a K step into 16-bit values
//              and write them into the stage's A tile in the swizzled layout the MMA descriptor
//              expects (packed arithmetic for INT4: nibble | 0x4300 is the bf16 number 128 + nibble),
//              then fence.proxy.async and arrive on the stage's `ready` barrier.
// Every mbarrier wait is bounded; on a timeout the kernel sets bit 1 of *status, drains and returns.
#include <cuda.h>

#include "gemm_common.cuh"

namespace amct {

constexpr int kDqWarpsDequant = 16;
constexpr int kDqThreads = (7 + kDqWarpsDequant) * 32;      // codes TMA, MMA, 4 epilogue warps, x TMA, dequant warps
constexpr int kDqBK = 64;                                   // K elements per MMA stage (128 bytes of 16-bit values)
constexpr int kDqRawRowBytes = 128;                         // bytes per weight row in one raw slot
constexpr int kDqRawSlotBytes = kBM * kDqRawRowBytes;       // 16 KB

struct DqParams {
  int64_t m, n, k;             // tokens, output channels, K
  int f16;                     // 1: fp16, 0: bf16
  int bits;                    // 4 (two codes per byte, code + 8, even k in the low nibble), 8 (int8 codes) or
                               // 1 (one code byte per weight, decoded through `lut`: HiFloat8)
  int group;                   // 0: one scale per channel
  const void* scale;           // [K/group or 1, n] in the activation dtype
  const void* offset;          // same layout, or null
  const void* lut;             // BITS == 1 (table mode): 256 values of the activation dtype, one per code byte
  const void* bias;
  int bias_kind;
  void* out;                   // [m, n]
  int out_kind;
  int64_t ld_out;
  int* status;
};

// Three rings of different depth: the A tiles (filled on chip by the dequant warps) need few slots, the x tiles and
// the codes come from memory and need enough slots in flight to cover a TMA round trip of a microsecond or more.
template <int BN, int STAGES, int XSLOTS, int RSLOTS>
struct __align__(1024) DqSmem {
  uint8_t a_tile[STAGES][kABytes];                // dequantized weights, 128 rows x 128 bytes, swizzled
  uint8_t b_tile[XSLOTS][BN * kBKBytes];          // x tiles
  uint8_t raw[RSLOTS][kDqRawSlotBytes];           // codes: 128 rows x 128 bytes (256 INT4 or 128 byte codes of K), swizzled
  uint64_t full_x[XSLOTS], empty_x[XSLOTS], ready[STAGES], empty[STAGES], full_raw[RSLOTS], empty_raw[RSLOTS], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  uint16_t lut[256];
};

// One 32-bit word of 8 nibbles (k0 .. k7, low nibble first) -> 8 values of T as four packed words in
// k order.  nibble | magic is the number 128 + u (bf16) or 1024 + u (fp16); `addc` holds
// (aoff - 8 - magic) twice, so the packed add gives code + aoff exactly, the packed multiply rounds
// (code + aoff) * scale once, as the separate dequant kernel does.
template <bool F16>
__device__ __forceinline__ void dq_int4_word(uint32_t w, uint32_t addc, uint32_t scl, uint32_t (&out)[4]) {
  constexpr uint32_t kMagic = F16 ? 0x64006400u : 0x43004300u;
  uint32_t v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t e = ((w >> (4 * i)) & 0x000F000Fu) | kMagic;        // (k_i, k_{i+4})
    if constexpr (F16) {
      const __half2 r = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&e), *reinterpret_cast<const __half2*>(&addc)),
                                *reinterpret_cast<const __half2*>(&scl));
      v[i] = *reinterpret_cast<const uint32_t*>(&r);
    } else {
      const __nv_bfloat162 r = __hmul2(__hadd2(*reinterpret_cast<const __nv_bfloat162*>(&e), *reinterpret_cast<const __nv_bfloat162*>(&addc)),
                                       *reinterpret_cast<const __nv_bfloat162*>(&scl));
      v[i] = *reinterpret_cast<const uint32_t*>(&r);
    }
  }
  out[0] = __byte_perm(v[0], v[1], 0x5410);      // (k0, k1)
  out[1] = __byte_perm(v[2], v[3], 0x5410);      // (k2, k3)
  out[2] = __byte_perm(v[0], v[1], 0x7632);      // (k4, k5)
  out[3] = __byte_perm(v[2], v[3], 0x7632);      // (k6, k7)
}

template <bool F16> __device__ __forceinline__ uint32_t dq_pack2(float a, float b) {
  if constexpr (F16) { const __half2 v = __floats2half2_rn(a, b); return *reinterpret_cast<const uint32_t*>(&v); }
  else { const __nv_bfloat162 v = __floats2bfloat162_rn(a, b); return *reinterpret_cast<const uint32_t*>(&v); }
}
template <bool F16> __device__ __forceinline__ float dq_to_f(uint16_t bits) {
  if constexpr (F16) return __half2float(*reinterpret_cast<const __half*>(&bits));
  else return __uint_as_float((uint32_t)bits << 16);
}

// byte offset `o` (a multiple of 8) of row `row` inside a 128-byte-swizzled tile of 128-byte rows
__device__ __forceinline__ uint32_t sw128(int row, int o) { return (uint32_t)(row * 128 + ((((o >> 4) ^ (row & 7)) << 4) | (o & 15))); }

template <int BN, int STAGES, int XSLOTS, int RSLOTS, int BITS>
__global__ void __launch_bounds__(kDqThreads, 1)
gemm_dq_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_codes, const __grid_constant__ CUtensorMap tma_x, DqParams p) {
  constexpr int SUB = BITS == 4 ? 4 : 2;                           // MMA stages (64 K elements) per raw slot
  constexpr int SUBB = kDqRawRowBytes / SUB;                       // raw bytes per row and MMA stage: 32 or 64
  // MMAs that accumulate into the same TMEM tile are serialised by that dependency, and with BN this small one MMA is
  // far shorter than the pipeline's latency: the four K-16 MMAs of a stage go to NACC separate accumulators instead,
  // which the epilogue adds up (fp32).
  constexpr int NACC = BN <= 64 ? 4 : 2;
  constexpr int kAccCols = NACC * BN;                              // columns of one (double-buffered) accumulator set
  constexpr int kTmemCols = 2 * kAccCols;                          // 256 or 512: a power of two
  using Smem = DqSmem<BN, STAGES, XSLOTS, RSLOTS>;
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int64_t num_kb = p.k / kDqBK;
  const int64_t tiles_w = (p.n + kBM - 1) / kBM, tiles_t = (p.m + BN - 1) / BN;
  const int64_t num_tiles = tiles_w * tiles_t;                    // weight tile fastest: the x tile stays hot in L2

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      tc05::mbar_init(tc05::smem_u32(&s.ready[i]), kDqWarpsDequant / 4);     // the four warps of one dequant group
      tc05::mbar_init(tc05::smem_u32(&s.empty[i]), 1);
    }
    for (int i = 0; i < XSLOTS; ++i) {
      tc05::mbar_init(tc05::smem_u32(&s.full_x[i]), 1);
      tc05::mbar_init(tc05::smem_u32(&s.empty_x[i]), 1);
    }
    for (int i = 0; i < RSLOTS; ++i) {
      tc05::mbar_init(tc05::smem_u32(&s.full_raw[i]), 1);
      tc05::mbar_init(tc05::smem_u32(&s.empty_raw[i]), (kDqWarpsDequant / 4) * SUB);   // each of the slot's SUB steps is one group's
    }
    for (int i = 0; i < 2; ++i) { tc05::mbar_init(tc05::smem_u32(&s.tmem_full[i]), 1); tc05::mbar_init(tc05::smem_u32(&s.tmem_empty[i]), 4); }
    tc05::fence_barrier_init();
    tc05::prefetch_tmap(&tma_codes);
    tc05::prefetch_tmap(&tma_x);
  }
  if (BITS == 1 && threadIdx.x < 256) s.lut[threadIdx.x] = reinterpret_cast<const uint16_t*>(p.lut)[threadIdx.x];
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
    // ------------------------------------------------------------ TMA producer of the codes: runs ahead by the whole raw ring,
    // independent of the (shorter) ring of MMA stages, so that enough bytes are in flight to cover the HBM latency
    if (tc05::elect_one()) {
      uint32_t rslot = 0, rphase = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        const int64_t tw = tile % tiles_w;
        for (int64_t kr = 0; kr * SUB < num_kb; ++kr) {              // one raw slot: 128 bytes of every weight row
          if (!tc05::mbar_wait(tc05::smem_u32(&s.empty_raw[rslot]), rphase ^ 1, abort_flag)) { alive = false; break; }
          const uint32_t rb = tc05::smem_u32(&s.full_raw[rslot]);
          tc05::mbar_expect_tx(rb, kDqRawSlotBytes);
          tc05::tma_load_2d(tc05::smem_u32(&s.raw[rslot][0]), &tma_codes, rb, (int)(kr * kDqRawRowBytes), (int)(tw * kBM));
          if (++rslot == RSLOTS) { rslot = 0; rphase ^= 1; }
        }
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ TMA producer of the x tiles, one per K step, in a ring of its own
    if (tc05::elect_one()) {
      uint32_t xs = 0, xphase = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        const int64_t tt = tile / tiles_w;
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!tc05::mbar_wait(tc05::smem_u32(&s.empty_x[xs]), xphase ^ 1, abort_flag)) { alive = false; break; }
          const uint32_t bar = tc05::smem_u32(&s.full_x[xs]);
          tc05::mbar_expect_tx(bar, BN * kBKBytes);
          tc05::tma_load_2d(tc05::smem_u32(&s.b_tile[xs][0]), &tma_x, bar, (int)(kb * kDqBK), (int)(tt * BN));
          if (++xs == XSLOTS) { xs = 0; xphase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (tc05::elect_one()) {
      const uint32_t idesc = p.f16 ? tc05::make_idesc(1, 0, 0, kBM, BN) : tc05::make_idesc(1, 1, 1, kBM, BN);
      uint32_t stage = 0, phase = 0, xs = 0, xphase = 0, acc = 0, acc_phase = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        if (!tc05::mbar_wait(tc05::smem_u32(&s.tmem_empty[acc]), acc_phase ^ 1, abort_flag)) break;
        tc05::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!tc05::mbar_wait(tc05::smem_u32(&s.full_x[xs]), xphase, abort_flag) ||
              !tc05::mbar_wait(tc05::smem_u32(&s.ready[stage]), phase, abort_flag)) { alive = false; break; }
          tc05::fence_after_sync();
          const uint32_t a0 = tc05::smem_u32(&s.a_tile[stage][0]);
          const uint32_t b0 = tc05::smem_u32(&s.b_tile[xs][0]);
#pragma unroll
          for (int ks = 0; ks < kBKBytes / 32; ++ks) {
            const uint64_t adesc = tc05::smem_desc_sw128(a0 + ks * 32);
            const uint64_t bdesc = tc05::smem_desc_sw128(b0 + ks * 32);
            // K-16 step ks of every stage goes to accumulator ks % NACC; its first use overwrites
            tc05::umma_f16(d_tmem + (ks % NACC) * BN, adesc, bdesc, idesc, (kb > 0 || ks >= NACC) ? 1u : 0u);
          }
          tc05::umma_commit(tc05::smem_u32(&s.empty[stage]));        // the A tile may be overwritten
          tc05::umma_commit(tc05::smem_u32(&s.empty_x[xs]));         // and the x slot refilled
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++xs == XSLOTS) { xs = 0; xphase ^= 1; }
        }
        if (!alive) break;
        tc05::umma_commit(tc05::smem_u32(&s.tmem_full[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5): y[m, n] = acc[n, m] + bias[n]
    const int quarter = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    for (int64_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int64_t tw = tile % tiles_w, tt = tile / tiles_w;
      const int64_t n = tw * kBM + quarter * 32 + lane;            // this lane's output channel
      const int64_t m0 = tt * BN;
      const float bias = (p.bias_kind != BIAS_NONE && n < p.n) ? bias_at(p.bias, p.bias_kind, n) : 0.f;
      if (!tc05::mbar_wait(tc05::smem_u32(&s.tmem_full[acc]), acc_phase, abort_flag)) break;
      tc05::fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kAccCols;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tc05::tmem_ld_32x32(t_row + c0, r);
        tc05::tmem_ld_wait();
#pragma unroll 1
        for (int a = 1; a < NACC; ++a) {                             // add the other partial accumulators
          uint32_t r2[32];
          tc05::tmem_ld_32x32(t_row + a * BN + c0, r2);
          tc05::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(r2[j])));
        }
        if (n < p.n) {
          // a warp writes 32 adjacent channels of one token per store
          const int64_t mleft = p.m - (m0 + c0);
          const int64_t off0 = (m0 + c0) * p.ld_out + n;
          if (p.out_kind == OUT_F32) {
            float* o = reinterpret_cast<float*>(p.out) + off0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < mleft) o[j * p.ld_out] = __fadd_rn(__uint_as_float(r[j]), bias);
          } else if (p.out_kind == OUT_BF16) {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + off0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < mleft) o[j * p.ld_out] = __float2bfloat16_rn(__fadd_rn(__uint_as_float(r[j]), bias));
          } else {
            __half* o = reinterpret_cast<__half*>(p.out) + off0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < mleft) o[j * p.ld_out] = __float2half_rn(__fadd_rn(__uint_as_float(r[j]), bias));
          }
        }
      }
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(tc05::smem_u32(&s.tmem_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------------------------------------ dequant (warps 7..): four groups of four warps.  Group g
    // owns the K steps kb = g (mod 4) and one thread of it owns one weight row (64 values per step): a step costs a warp
    // several hundred cycles of latency (shared-memory round trips, the barrier hand-offs), and four groups working on
    // four consecutive steps at once hide that.
    const int dt = threadIdx.x - 7 * 32;
    const int grp = dt >> 7, row = dt & 127;
    const int steps_per_group = p.group ? p.group / kDqBK : 0;
    const uint32_t kb_pad = (uint32_t)((num_kb + SUB - 1) / SUB * SUB);     // K steps rounded up to whole raw slots
    const uint32_t slots_per_tile = kb_pad / SUB;
    uint32_t t_ord = 0;                                             // tiles this CTA has started
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++t_ord) {
      const int64_t tw = tile % tiles_w;
      const int64_t n = tw * kBM + row;
      const bool valid = n < p.n;
      int64_t cur_g = -1;
      uint32_t addc = 0, scl = 0;                                  // packed (offset constant, scale), both halves equal
      float fs = 0.f, fo = 0.f;
      for (uint32_t kb = grp; kb < kb_pad; kb += 4) {
        const uint32_t slot_seq = t_ord * slots_per_tile + kb / SUB;
        const uint32_t rslot = slot_seq % RSLOTS, rphase = (slot_seq / RSLOTS) & 1;
        if (kb >= (uint32_t)num_kb) {                              // padding step of the last raw slot: only release it
          __syncwarp();
          if (lane == 0) tc05::mbar_arrive(tc05::smem_u32(&s.empty_raw[rslot]));
          continue;
        }
        const uint32_t seq = t_ord * (uint32_t)num_kb + kb;
        const uint32_t stage = seq % STAGES, phase = (seq / STAGES) & 1;
        const int64_t g = steps_per_group ? kb / steps_per_group : 0;
        if (g != cur_g) {                                          // this row's scale / offset for the group of this step
          cur_g = g;
          uint16_t sb = 0, ob = 0;
          if (valid && BITS != 1) {
            sb = reinterpret_cast<const uint16_t*>(p.scale)[g * p.n + n];
            if (p.offset) ob = reinterpret_cast<const uint16_t*>(p.offset)[g * p.n + n];
          }
          fs = p.f16 ? dq_to_f<true>(sb) : dq_to_f<false>(sb);
          fo = p.f16 ? dq_to_f<true>(ob) : dq_to_f<false>(ob);
          // INT4: value = magic + u with u = code + 8, so code + aoff = (magic + u) + (aoff - 8 - magic)
          const float c = fo - 8.f - (p.f16 ? 1024.f : 128.f);
          addc = p.f16 ? dq_pack2<true>(c, c) : dq_pack2<false>(c, c);
          scl = (uint32_t)sb | ((uint32_t)sb << 16);
        }
        if (!tc05::mbar_wait(tc05::smem_u32(&s.full_raw[rslot]), rphase, abort_flag)) { alive = false; break; }
        // the MMAs that read this stage's previous contents are done
        if (!tc05::mbar_wait(tc05::smem_u32(&s.empty[stage]), phase ^ 1, abort_flag)) { alive = false; break; }
        const uint8_t* rawp = &s.raw[rslot][0];
        uint8_t* a_tile = &s.a_tile[stage][0];
        const int sub = (int)(kb % SUB);
        if constexpr (BITS == 4) {
          const uint4 r0 = *reinterpret_cast<const uint4*>(rawp + sw128(row, sub * SUBB));
          const uint4 r1 = *reinterpret_cast<const uint4*>(rawp + sw128(row, sub * SUBB + 16));
          const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
          for (int c = 0; c < 8; ++c) {                            // word c = 8 nibbles = 16-byte chunk c of the A row
            uint32_t o[4];
            if (p.f16) dq_int4_word<true>(w[c], addc, scl, o);
            else dq_int4_word<false>(w[c], addc, scl, o);
            *reinterpret_cast<uint4*>(a_tile + sw128(row, c * 16)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
#pragma unroll
          for (int h = 0; h < 4; ++h) {                            // 16 code bytes -> two 16-byte chunks
            const uint4 raw = *reinterpret_cast<const uint4*>(rawp + sw128(row, sub * SUBB + h * 16));
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {                          // two code bytes -> two values
              const uint32_t ww = w[j >> 1] >> (16 * (j & 1));
              if constexpr (BITS == 1) {
                o[j] = (uint32_t)s.lut[ww & 0xFF] | ((uint32_t)s.lut[(ww >> 8) & 0xFF] << 16);
              } else {                                             // (q + aoff) * scale, rounded once
                const float q0 = (float)(int)(int8_t)(ww & 0xFF), q1 = (float)(int)(int8_t)((ww >> 8) & 0xFF);
                const float v0 = __fmul_rn(__fadd_rn(q0, fo), fs), v1 = __fmul_rn(__fadd_rn(q1, fo), fs);
                o[j] = p.f16 ? dq_pack2<true>(v0, v1) : dq_pack2<false>(v0, v1);
              }
            }
            *reinterpret_cast<uint4*>(a_tile + sw128(row, h * 32)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(a_tile + sw128(row, h * 32 + 16)) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
        tc05::fence_proxy_async();                                 // these generic-proxy stores are read by the MMA (async proxy)
        __syncwarp();
        if (lane == 0) {
          tc05::mbar_arrive(tc05::smem_u32(&s.ready[stage]));
          tc05::mbar_arrive(tc05::smem_u32(&s.empty_raw[rslot]));
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
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

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFnDq)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnDq encode_fn_dq() {
  static EncodeTiledFnDq fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnDq>(p);
  }
  return fn;
}

static int map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int esize, int64_t inner, int64_t rows, int64_t ld_bytes,
                  int box_inner, int box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFnDq fn = encode_fn_dq();
  if (!fn) return AMCT_ERR_CUDA;
  if (!aligned16(base) || ld_bytes % 16 != 0) return AMCT_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  (void)esize;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? AMCT_OK : AMCT_ERR_CUDA;
}

template <int BN, int STAGES, int XSLOTS, int RSLOTS, int BITS>
static int launch_dq(const CUtensorMap& mc, const CUtensorMap& mx, const DqParams& p, int grid, cudaStream_t st) {
  const size_t smem = sizeof(DqSmem<BN, STAGES, XSLOTS, RSLOTS>) + 1024;
  static OncePerDevice attr;
  if (attr.first()) {
    if (cudaFuncSetAttribute(gemm_dq_tcgen05_kernel<BN, STAGES, XSLOTS, RSLOTS, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return AMCT_ERR_CUDA;
  }
  gemm_dq_tcgen05_kernel<BN, STAGES, XSLOTS, RSLOTS, BITS><<<grid, kDqThreads, smem, st>>>(mc, mx, p);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

namespace amct {
// w4a16_stream.cu; returns 1 when the shape does not fit it
int w4a16_stream_try(const void* x, int dtype, const void* codes, int64_t m, int64_t n, int64_t k, int64_t ld_x,
                     int64_t ld_codes, const void* scale, const void* offset, int group, const void* bias, int bias_kind,
                     void* out, int out_kind, int64_t ld_out, cudaStream_t st);
}  // namespace amct

static int run_dq(const void* x, int dtype, const void* codes, int bits, int64_t m, int64_t n, int64_t k, int64_t ld_x,
                  int64_t ld_codes, const void* scale, const void* offset, const void* lut, int group, const void* bias,
                  int bias_kind, void* out, int out_kind, int64_t ld_out, int* status, cudaStream_t st) {
  using namespace amct;
  if (m < 0 || n < 0 || k < 0 || group < 0) return AMCT_ERR_ARG;
  if (dtype != AMCT_DTYPE_F16 && dtype != AMCT_DTYPE_BF16) return AMCT_ERR_ARG;
  if (m == 0 || n == 0) return AMCT_OK;
  if (!x || !codes || !out || k == 0) return AMCT_ERR_ARG;
  if (ld_x < k || ld_out < n || ld_codes < (bits == 4 ? k / 2 : k)) return AMCT_ERR_ARG;
  if (bias_kind == BIAS_I32 || bias_kind < 0 || bias_kind > BIAS_BF16 || (bias_kind && !bias)) return AMCT_ERR_ARG;
  if (out_kind < OUT_F32 || out_kind > OUT_BF16) return AMCT_ERR_ARG;
  // whole 64-element K steps, each inside one group
  if (k % kDqBK != 0 || (group && group % kDqBK != 0) || (group && k % group != 0)) return AMCT_ERR_UNSUPPORTED;
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return AMCT_ERR_UNSUPPORTED;
  CUtensorMap mc, mx;
  // raw slots: 128 bytes of every weight row, with the 128-byte swizzle so that the dequant threads' reads are conflict-free
  int rc = map_2d(&mc, codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, bits == 4 ? k / 2 : k, n, ld_codes, kDqRawRowBytes, kBM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != AMCT_OK) return rc;
  const int bn = m <= 32 ? 32 : (m <= 64 ? 64 : 128);
  rc = map_2d(&mx, x, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, k, m, ld_x * 2, kDqBK, bn, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != AMCT_OK) return rc;
  DqParams p{};
  p.m = m; p.n = n; p.k = k; p.f16 = dtype == AMCT_DTYPE_F16; p.bits = bits; p.group = group;
  p.scale = scale; p.offset = offset; p.lut = lut; p.bias = bias; p.bias_kind = bias_kind; p.out = out; p.out_kind = out_kind;
  p.ld_out = ld_out; p.status = status;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = ((n + kBM - 1) / kBM) * ((m + bn - 1) / bn);
  const int grid = (int)(tiles < sms ? tiles : sms);
  // shared memory: STAGES x 16 KB (A) + XSLOTS x BN x 128 B (x) + RSLOTS x 16 KB (codes).  Each of the four dequant
  // groups needs two A slots of its own (it fills one while the MMAs read the other): STAGES = 8 where that fits.
  if (bits == 4) {
    if (bn == 32) return launch_dq<32, 8, 8, 2, 4>(mc, mx, p, grid, st);
    if (bn == 64) return launch_dq<64, 8, 6, 2, 4>(mc, mx, p, grid, st);
    return launch_dq<128, 6, 4, 2, 4>(mc, mx, p, grid, st);
  }
  if (bits == 8) {
    if (bn == 32) return launch_dq<32, 8, 8, 2, 8>(mc, mx, p, grid, st);
    if (bn == 64) return launch_dq<64, 8, 6, 2, 8>(mc, mx, p, grid, st);
    return launch_dq<128, 6, 4, 2, 8>(mc, mx, p, grid, st);
  }
  if (bn == 32) return launch_dq<32, 8, 8, 2, 1>(mc, mx, p, grid, st);
  if (bn == 64) return launch_dq<64, 8, 6, 2, 1>(mc, mx, p, grid, st);
  return launch_dq<128, 6, 4, 2, 1>(mc, mx, p, grid, st);
}

extern "C" int amct_gemm_w4a16(const void* x, int dtype, const void* codes, int bits, int64_t m, int64_t n, int64_t k,
                               int64_t ld_x, int64_t ld_codes, const void* scale, const void* offset, int group,
                               const void* bias, int bias_kind, void* out, int out_kind, int64_t ld_out, int* status,
                               void* stream) {
  if (bits != 4 && bits != 8) return AMCT_ERR_ARG;
  if (m > 0 && n > 0 && !scale) return AMCT_ERR_ARG;
  // a handful of tokens: the weight-streaming kernel of w4a16_stream.cu (same values, all SMs busy)
  if (bits == 4 && m >= 1 && m <= 16 && n > 0 && k > 0 && x && codes && out && group >= 0 && ld_x >= k && ld_out >= n &&
      ld_codes >= k / 2 && (dtype == AMCT_DTYPE_F16 || dtype == AMCT_DTYPE_BF16) && bias_kind >= amct::BIAS_NONE &&
      bias_kind <= amct::BIAS_BF16 && bias_kind != amct::BIAS_I32 && (!bias_kind || bias) && out_kind >= amct::OUT_F32 &&
      out_kind <= amct::OUT_BF16) {
    const int rc = amct::w4a16_stream_try(x, dtype, codes, m, n, k, ld_x, ld_codes, scale, offset, group, bias, bias_kind, out,
                                          out_kind, ld_out, (cudaStream_t)stream);
    if (rc != 1) return rc;
  }
  return run_dq(x, dtype, codes, bits, m, n, k, ld_x, ld_codes, scale, offset, nullptr, group, bias, bias_kind, out, out_kind,
                ld_out, status, (cudaStream_t)stream);
}

extern "C" int amct_gemm_lut8(const void* x, int dtype, const void* codes, const void* lut, int64_t m, int64_t n, int64_t k,
                              int64_t ld_x, int64_t ld_codes, const void* bias, int bias_kind, void* out, int out_kind,
                              int64_t ld_out, int* status, void* stream) {
  if (m > 0 && n > 0 && !lut) return AMCT_ERR_ARG;
  return run_dq(x, dtype, codes, 1, m, n, k, ld_x, ld_codes, nullptr, nullptr, lut, 0, bias, bias_kind, out, out_kind, ld_out,
                status, (cudaStream_t)stream);
}
