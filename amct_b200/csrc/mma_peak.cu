// Tensor-core peak of one GPU, measured: one CTA per SM issues tcgen05.mma back to back on operands that never
// move -- no global loads, no stores, no epilogue -- so the rate is what the MMA pipe itself sustains for a kind.
// It is the denominator the GEMM rooflines of this repository are quoted against, next to the convention
// "INT8 / FP8 = 2 x, FP4 = 4 x the measured bf16 figure".
//
// Per CTA: warp 0 allocates tensor memory; one elected thread issues, per step, the four K-slices of a 128-byte
// K block exactly as the GEMM kernels do (M128 x N x 32 bytes of K per instruction, 128-byte-swizzled shared
// memory descriptors, accumulating into one of two alternating accumulators) and commits a window of 64 steps to
// one of two mbarriers; a window is awaited before its barrier is used again, and at the end.  The operands
// are pseudo-random bytes, the block scale factors 2^0.
// Every wait is bounded; on a time-out bit 1 of *status is set and the kernel winds down.
#include "tc05.cuh"

#include "../../include/amct_b200.h"
#include "common.cuh"

namespace amct {

constexpr int kPeakBM = 128, kPeakBKBytes = 128;
constexpr int kPeakThreads = 128;

struct __align__(1024) PeakSmem {
  uint8_t a[kPeakBM * kPeakBKBytes];
  uint8_t b[256 * kPeakBKBytes];
  uint8_t sf[1024];
  uint64_t bar[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

// kind: 0 i8, 1 bf16, 2 mxf8 (E4M3, block scale), 3 mxf4 (E2M1, block scale)
__global__ void __launch_bounds__(kPeakThreads, 1) mma_peak_kernel(int kind, int steps, int* status) {
  extern __shared__ uint8_t smem_raw[];
  PeakSmem& s = *reinterpret_cast<PeakSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5;
  // operands: pseudo-random bytes (the tensor pipe's power draw, and with it the clock it sustains at the board's
  // limit, depends on the data; zeros would flatter it), scale factors 2^0
  for (int i = threadIdx.x; i < (int)(sizeof(s.a) + sizeof(s.b)) / 4; i += kPeakThreads) {
    uint32_t v = (uint32_t)(i + 1) * 2654435761u;
    v ^= v >> 15; v *= 2246822519u; v ^= v >> 13;
    reinterpret_cast<uint32_t*>(s.a)[i] = kind >= 1 ? (v & 0x3F3F3F3Fu) : v;          // floats: keep away from NaN / Inf patterns
  }
  for (int i = threadIdx.x; i < (int)sizeof(s.sf) / 4; i += kPeakThreads) reinterpret_cast<uint32_t*>(s.sf)[i] = 0x7F7F7F7Fu;
  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    tc05::mbar_init(tc05::smem_u32(&s.bar[0]), 1);
    tc05::mbar_init(tc05::smem_u32(&s.bar[1]), 1);
    tc05::fence_barrier_init();
  }
  if (warp == 0) {
    tc05::tmem_alloc(tc05::smem_u32(&s.tmem_base), 512);
    tc05::tmem_relinquish();
  }
  // the fill went through the generic proxy; the MMAs read shared memory through the async proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;
  const bool block_scaled = kind >= 2;
  const int bn = block_scaled ? 224 : 256;                  // the tile widths of the GEMM kernels
  const uint32_t sfa = tmem_base + 448, sfb = tmem_base + 456;

  if (warp == 0 && tc05::elect_one()) {
    if (block_scaled) {
      for (int j = 0; j < 2; ++j) {
        tc05::tmem_cp_32x128b_warpx4(sfa + 4 * j, tc05::smem_desc_sf(tc05::smem_u32(&s.sf[512 * j])));
        tc05::tmem_cp_32x128b_warpx4(sfb + 8 * j, tc05::smem_desc_sf(tc05::smem_u32(&s.sf[512 * j])));
        tc05::tmem_cp_32x128b_warpx4(sfb + 8 * j + 4, tc05::smem_desc_sf(tc05::smem_u32(&s.sf[512 * j])));
      }
    }
    const uint32_t a0 = tc05::smem_u32(s.a), b0 = tc05::smem_u32(s.b);
    // Windows of kWindow steps are committed alternately to two mbarriers, and a barrier is awaited before it is
    // committed to again: never more than one commit outstanding per barrier (two completed phases would look like
    // none to a parity wait), one window always in flight behind the one being issued.
    const uint32_t bars[2] = {tc05::smem_u32(&s.bar[0]), tc05::smem_u32(&s.bar[1])};
    constexpr int kWindow = 64;
    uint32_t phase[2] = {0, 0};
    const int windows = (steps + kWindow - 1) / kWindow;
    bool alive = true;
    for (int w = 0; w < windows && alive; ++w) {
      const int b = w & 1;
      if (w >= 2) {
        if (!tc05::mbar_wait(bars[b], phase[b], abort_flag)) { alive = false; break; }
        phase[b] ^= 1;
      }
      const int it_end = (w + 1) * kWindow < steps ? (w + 1) * kWindow : steps;
      for (int it = w * kWindow; it < it_end; ++it) {
        const uint32_t d_tmem = tmem_base + (uint32_t)((it >> 5) & 1) * (uint32_t)bn;    // a "tile" of 32 K blocks, then the other accumulator
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t adesc = tc05::smem_desc_sw128(a0 + ks * 32), bdesc = tc05::smem_desc_sw128(b0 + ks * 32);
          const uint32_t accumulate = ((it & 31) || ks) ? 1u : 0u;
          if (kind == 0) tc05::umma_i8(d_tmem, adesc, bdesc, tc05::make_idesc(2, 1, 1, kPeakBM, 256), accumulate);
          else if (kind == 1) tc05::umma_f16(d_tmem, adesc, bdesc, tc05::make_idesc(1, 1, 1, kPeakBM, 256), accumulate);
          else if (kind == 2) tc05::umma_mxf8(d_tmem, adesc, bdesc, tc05::make_idesc_mx(0, kPeakBM, 224, ks), sfa, sfb, accumulate);
          else tc05::umma_mxf4(d_tmem, adesc, bdesc, tc05::make_idesc_mx(1, kPeakBM, 224, (ks & 1) * 2), sfa + 4 * (ks >> 1),
                               sfb + 8 * (ks >> 1), accumulate);
        }
      }
      tc05::umma_commit(bars[b]);
    }
    // the last two windows (or the only one) are still outstanding
    for (int w = windows >= 2 ? windows - 2 : 0; w < windows && alive; ++w) {
      if (!tc05::mbar_wait(bars[w & 1], phase[w & 1], abort_flag)) alive = false;
      phase[w & 1] ^= 1;
    }
  }
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && status) atomicOr(status, 2);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace amct

// Operations one launch performs on the whole device: steps x 4 MMAs x 2 * 128 * N * K per MMA x CTAs, K = 32 bytes of
// the kind's elements (32 for i8 / fp8, 16 for bf16, 64 for fp4).
extern "C" int64_t amct_mma_peak_ops_per_cta_step(int kind) {
  const int64_t n = kind >= 2 ? 224 : 256;
  const int64_t k = kind == 1 ? 64 : (kind == 3 ? 256 : 128);          // elements in a 128-byte K block
  return 2 * 128 * n * k;
}

extern "C" int amct_mma_peak(int kind, int steps, int ctas, int* status, void* stream) {
  if (kind < 0 || kind > 3 || steps < 1 || ctas < 1) return AMCT_ERR_ARG;
  const size_t smem = sizeof(amct::PeakSmem) + 1024;
  static amct::OncePerDevice attr;
  if (attr.first()) {
    if (cudaFuncSetAttribute(amct::mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return AMCT_ERR_CUDA;
  }
  amct::mma_peak_kernel<<<ctas, amct::kPeakThreads, smem, (cudaStream_t)stream>>>(kind, steps, status);
  return cudaGetLastError() == cudaSuccess ? AMCT_OK : AMCT_ERR_CUDA;
}
