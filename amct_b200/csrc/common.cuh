// Shared device helpers for the quantization kernels (sm_100a).
//
// Numerics contract shared by every kernel in this directory: fp32 arithmetic,
// correctly rounded division (__fdiv_rn, or div_by_recip below, which returns the
// same value), round-half-to-even, no FMA contraction of x*s+z (explicit
// __fmul_rn/__fadd_rn; the quant files are also compiled with -fmad=false).  These choices make integer codes bit-identical to the
// reference's torch arithmetic (amct_pytorch/utils/quant_util.py:57-93).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/amct_b200.h"

#define AMCT_FLT_EPSILON 1.192092896e-7f   // amct_pytorch/quantize_op/utils.py:23

#ifndef AMCT_CHECK_LAUNCH
#define AMCT_CHECK_LAUNCH()                                         \
  do {                                                              \
    cudaError_t e__ = cudaGetLastError();                           \
    if (e__ != cudaSuccess) return AMCT_ERR_CUDA;                   \
  } while (0)
#endif

// Kernel launch written so that a test harness can substitute its own launcher (the newer files use it):
// AMCT_LAUNCH(grid, threads, stream, (arguments), kernel<template arguments>).
#ifndef AMCT_LAUNCH
#define AMCT_LAUNCH(grid, threads, stream, args, ...) __VA_ARGS__<<<(grid), (threads), 0, (stream)>>> args
#endif
// the same with dynamic shared memory, and the declaration of that memory inside the kernel
#ifndef AMCT_LAUNCH_SMEM
#define AMCT_LAUNCH_SMEM(grid, threads, smem_bytes, stream, args, ...) \
  __VA_ARGS__<<<(grid), (threads), (smem_bytes), (stream)>>> args
#endif
#ifndef AMCT_DYNAMIC_SMEM
#define AMCT_DYNAMIC_SMEM(type, name) extern __shared__ type name[]
#endif

namespace amct {

template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  static constexpr int kPerVec = 4;
  __device__ static float to_f(float v) { return v; }
  __device__ static float from_f(float v) { return v; }
};
template <> struct ElemTraits<__half> {
  static constexpr int kPerVec = 8;
  __device__ static float to_f(__half v) { return __half2float(v); }
  __device__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Round an fp32 value to T and back: the value a torch op on T tensors would hold.
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return ElemTraits<T>::to_f(ElemTraits<T>::from_f(v));
}
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }

// 16-byte vector of T.
template <typename T> struct alignas(16) Vec16 {
  T v[ElemTraits<T>::kPerVec];
};

template <typename T> __device__ __forceinline__ Vec16<T> ld_vec(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
  return r;
}
// Streaming variant: data that is read once (evict-first).
template <typename T> __device__ __forceinline__ Vec16<T> ld_vec_stream(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// NaN-propagating fp32 min / max (one instruction; fminf / fmaxf return the other operand instead).
__device__ __forceinline__ float fmin_nan(float a, float b) {
#ifdef AMCT_CUDA_EMU
  return (a != a || b != b) ? NAN : fminf(a, b);
#else
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
#endif
}
__device__ __forceinline__ float fmax_nan(float a, float b) {
#ifdef AMCT_CUDA_EMU
  return (a != a || b != b) ? NAN : fmaxf(a, b);
#else
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
#endif
}

// Monotonic float <-> int mapping, so integer atomicMin/Max order floats.
__device__ __forceinline__ int f2ord(float f) {
  int b = __float_as_int(f);
  return b >= 0 ? b : b ^ 0x7fffffff;
}
__device__ __forceinline__ float ord2f(int b) {
  return __int_as_float(b >= 0 ? b : b ^ 0x7fffffff);
}

// Scale/offset rule of the reference (amct_pytorch/quantize_op/utils.py:75-108).
// Returns false when the scale is not finite (the reference raises there).
__device__ __forceinline__ bool qparams_from_minmax(float mx, float mn, int bits, bool symmetric,
                                                    float* scale, int* offset) {
  float s, o = 0.f;
  if (symmetric) {
    float amx = fabsf(mx), amn = fabsf(mn);
    float div = (float)((1 << (bits - 1)) - 1 + (amx < amn ? 1 : 0));
    float bound = amx > amn ? amx : amn;
    s = __fdiv_rn(bound, div);
    if (s < AMCT_FLT_EPSILON) s = 1.f;
  } else {
    mx = fmaxf(mx, 0.f);
    mn = fminf(mn, 0.f);
    float span = (float)((1 << bits) - 1);
    float half = (float)(1 << (bits - 1));                 // ceil(span / 2)
    s = __fdiv_rn(__fsub_rn(mx, mn), span);
    o = (mx != mn) ? __fsub_rn(-half, __fdiv_rn(mn, s)) : -half;
    if (s < AMCT_FLT_EPSILON) { o = -half; s = 1.f; }
    o = rintf(o);
  }
  *scale = s;
  *offset = (int)o;
  return isfinite(s) && isfinite(o);
}

// Correctly rounded x / s computed from y = rn(1 / s) (__frcp_rn) with two FMA correction steps
// (Markstein): q0 = rn(x y) is within 2 ulp of the quotient; q1 = rn(q0 + (x - s q0) y) is within
// one; and for such a q1 and a correctly rounded reciprocal, rn(q1 + (x - s q1) y) IS the correctly
// rounded quotient, i.e. the value of __fdiv_rn(x, s).  Five FMA-pipe instructions, no branch.
// Valid for normal, finite s and y and a quotient in the normal range; a quotient that underflows
// may differ in its last subnormal bits (it rounds to the integer 0 either way).
__device__ __forceinline__ float div_by_recip(float x, float s, float y) {
  const float q0 = __fmul_rn(x, y);
  const float q1 = __fmaf_rn(__fmaf_rn(-s, q0, x), y, q0);
  return __fmaf_rn(__fmaf_rn(-s, q1, x), y, q1);
}

// cvt.pack.sat: two signed integers saturated to 4 (8) bits each and packed under what `carry` already holds,
//   d = (carry << 8 | sat4(hi) << 4 | sat4(lo))      resp.      d = (carry << 16 | sat8(hi) << 8 | sat8(lo))
// one instruction for the clamp and the packing of two codes.
__device__ __forceinline__ uint32_t pack_sat_s4(int hi, int lo, uint32_t carry) {
#ifdef AMCT_CUDA_EMU
  const int h = hi < -8 ? -8 : hi > 7 ? 7 : hi, l = lo < -8 ? -8 : lo > 7 ? 7 : lo;
  return (carry << 8) | ((uint32_t)(h & 0xF) << 4) | (uint32_t)(l & 0xF);
#else
  uint32_t d;
  asm("cvt.pack.sat.s4.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(carry));
  return d;
#endif
}
__device__ __forceinline__ uint32_t pack_sat_s8(int hi, int lo, uint32_t carry) {
#ifdef AMCT_CUDA_EMU
  const int h = hi < -128 ? -128 : hi > 127 ? 127 : hi, l = lo < -128 ? -128 : lo > 127 ? 127 : lo;
  return (carry << 16) | ((uint32_t)(h & 0xFF) << 8) | (uint32_t)(l & 0xFF);
#else
  uint32_t d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(carry));
  return d;
#endif
}

// 32 values -> 16 words of packed 16-bit outputs
__device__ __forceinline__ void epi_pack16(const float (&y)[32], bool to_bf16, uint32_t (&h)[16]) {
  if (to_bf16) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __nv_bfloat162 v = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
      h[j] = *reinterpret_cast<uint32_t*>(&v);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __half2 v = __floats2half2_rn(y[2 * j], y[2 * j + 1]);
      h[j] = *reinterpret_cast<uint32_t*>(&v);
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// "Done once per device": kernel attributes such as the dynamic shared-memory limit belong to a device's context, so a
// process that drives several GPUs has to set them on each.  first() returns true the first time it is called with a
// given device current (a benign race between threads only repeats the idempotent call it guards).
struct OncePerDevice {
  bool done[64] = {};
  bool first() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
  }
};

}  // namespace amct
