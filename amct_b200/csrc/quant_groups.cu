// Group-wise weight quantization without shared memory or block barriers.
//
// Same arithmetic as the per-group branch of the row kernel in quant_rows.cu -- group min / max
// (amct_pytorch/quantize_op/utils.py:111-136), scale rule (utils.py:75-108), codes
// (amct_pytorch/utils/quant_util.py:57-93), nibble pack, and both fake-quant variants
// (quant_util.py:162-188; amct_pytorch/algorithm/awq.py:129-170) -- for the common case of a
// group that fits inside a warp: group / (elements per 16-byte vector) lanes, a power of two,
// K a multiple of the group.  Every thread owns one 16-byte vector, reduces min / max over its
// lane group with shuffles, derives the group's scale and offset itself, and quantizes its own
// elements.  blockIdx.x covers the columns, blockIdx.y strides over rows: no index division.
//
// Quotients come from rn(1/scale) and two FMA correction steps (div_by_recip in common.cuh: the
// correctly rounded quotient, i.e. the value of the IEEE division), the rounding is done by adding
// 1.5 * 2^23.  Threads whose scale or reciprocal is not a normal number, or that meet a non-finite
// quotient, take the plain IEEE division instead.
//
// Algorithmic HBM traffic per element: sizeof(T) read + the output bytes (+ 8 bytes per group of
// scale and offset).
#include <type_traits>

#include "common.cuh"

namespace amct {

struct GroupParams {
  const void* x;
  int64_t rows, k, ld;
  const void* pre;
  int pre_op;
  int compute;
  int lanes_log2;              // log2(group / elements per vector)
  int bits, symmetric;
  float* scale;
  int* offset;
  int out_mode;
  void* out;
  int64_t ld_out;
  int* status;
};

constexpr float kMagicG = 12582912.0f;

// reference order with the IEEE division, four values at a time (out of line, by value: rare, and
// the caller's arrays stay in registers)
template <typename T>
__device__ __noinline__ float4 levels_exact4(float a, float b, float c, float d, float s, float o, int flags, float qmin, float qmax) {
  const bool has_off = flags & 1, awq = flags & 2;
  float v[4] = {a, b, c, d};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float t = __fdiv_rn(v[e], s);
    if (has_off) t = __fadd_rn(t, o);
    if (awq) t = round_to<T>(t);
    v[e] = fminf(fmaxf(rintf(t), qmin), qmax);
  }
  return make_float4(v[0], v[1], v[2], v[3]);
}

// 16-bit inputs: min / max of a 16-byte vector with the packed instructions (NaN is tracked
// separately by the caller, so the NaN-dropping variants are fine here)
__device__ __forceinline__ void vec_minmax(const Vec16<__nv_bfloat16>& v, float& mn, float& mx) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  const __nv_bfloat162 a = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
  const __nv_bfloat162 b = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
  mn = fminf(mn, fminf(__low2float(a), __high2float(a)));
  mx = fmaxf(mx, fmaxf(__low2float(b), __high2float(b)));
}
__device__ __forceinline__ void vec_minmax(const Vec16<__half>& v, float& mn, float& mx) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  const __half2 a = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
  const __half2 b = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
  mn = fminf(mn, fminf(__low2float(a), __high2float(a)));
  mx = fmaxf(mx, fmaxf(__low2float(b), __high2float(b)));
}
__device__ __forceinline__ void vec_minmax(const Vec16<float>& v, float& mn, float& mx) {
#pragma unroll
  for (int e = 0; e < 4; ++e) { mn = fminf(mn, v.v[e]); mx = fmaxf(mx, v.v[e]); }
}

// Two adjacent 16-byte vectors per thread; a group spans (1 << lanes_log2) threads of a warp.
// OUT is the AMCT_OUT_* mode.  In every mode the rounded level is carried as u = level + 1.5 * 2^23,
// whose low mantissa bits are the level in two's complement.
template <typename T, int OUT>
__global__ void __launch_bounds__(256) quant_groups_kernel(GroupParams p) {
  constexpr int E = ElemTraits<T>::kPerVec;
  constexpr int VPT = 2, EP = E * VPT;              // vectors / elements per thread
  constexpr bool kAwq = OUT == AMCT_OUT_FAKE_AWQ;
  constexpr bool kAwqRounds = kAwq && sizeof(T) == 2;              // the AWQ variant rounds to T before rint()
  constexpr bool kFake = OUT == AMCT_OUT_FAKE || OUT == AMCT_OUT_FAKE_AWQ;
  const int nthr_row = (int)(p.k / EP);             // threads that own part of a row
  const int tcol = blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = tcol < nthr_row;
  const int lanes = 1 << p.lanes_log2;
  const int lane = threadIdx.x & 31;
  const int unit = tcol >> p.lanes_log2;
  const int nunits = nthr_row >> p.lanes_log2;
  const bool has_off = p.offset != nullptr;
  const float qmax = (float)((1 << (p.bits - 1)) - 1), qmin = -qmax - 1.f;
  const T* __restrict__ pre = reinterpret_cast<const T*>(p.pre);
  const int64_t j0 = (int64_t)tcol * EP;

  float pre_f[EP];
  if (p.pre_op != AMCT_PRE_NONE && active) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const Vec16<T> pv = ld_vec(pre + j0 + i * E);
#pragma unroll
      for (int e = 0; e < E; ++e) pre_f[i * E + e] = ElemTraits<T>::to_f(pv.v[e]);
    }
  }

  for (int64_t row = blockIdx.y; row < p.rows; row += gridDim.y) {
    float x[EP];
    float mn = INFINITY, mx = -INFINITY;
    bool bad = false;
    if (active) {
      Vec16<T> raw[VPT];
#pragma unroll
      for (int i = 0; i < VPT; ++i) raw[i] = ld_vec_stream(reinterpret_cast<const T*>(p.x) + row * p.ld + j0 + i * E);
      // one decision per row, not per element: runtime tests inside unrolled loops cost a branch each
      if (p.pre_op == AMCT_PRE_NONE) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
#pragma unroll
          for (int e = 0; e < E; ++e) x[i * E + e] = ElemTraits<T>::to_f(raw[i].v[e]);
          if (p.compute) vec_minmax(raw[i], mn, mx);
        }
      } else {
        if (p.pre_op == AMCT_PRE_MUL) {
#pragma unroll
          for (int e = 0; e < EP; ++e) x[e] = round_to<T>(__fmul_rn(ElemTraits<T>::to_f(raw[e / E].v[e % E]), pre_f[e]));
        } else {
#pragma unroll
          for (int e = 0; e < EP; ++e) x[e] = round_to<T>(__fdiv_rn(ElemTraits<T>::to_f(raw[e / E].v[e % E]), pre_f[e]));
        }
#pragma unroll
        for (int e = 0; e < EP; ++e) { mn = fminf(mn, x[e]); mx = fmaxf(mx, x[e]); }
      }
      // x * 0 is NaN exactly for NaN and Inf: one FMA per element finds a NaN anywhere; an Inf
      // alone is told apart below (it does not raise in the reference when scales are given)
      float poison = 0.f;
#pragma unroll
      for (int e = 0; e < EP; ++e) poison = __fmaf_rn(x[e], 0.f, poison);
      if (poison != poison) {
#pragma unroll
        for (int e = 0; e < EP; ++e) bad |= (x[e] != x[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < EP; ++e) x[e] = 0.f;
      mn = mx = 0.f;
    }
    float s, o = 0.f;
    const int64_t uidx = row * nunits + unit;
    if (p.compute) {
      for (int w = 1; w < lanes; w <<= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, w));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));
      }
      int oi;
      const bool ok = qparams_from_minmax(mx, mn, p.bits, p.symmetric != 0, &s, &oi);
      o = (float)oi;
      if (active && (lane & (lanes - 1)) == 0) {
        p.scale[uidx] = s;
        if (has_off) p.offset[uidx] = oi;
        if (!ok && p.status) atomicOr(p.status, 1);
      }
    } else if (active) {
      s = p.scale[uidx];
      if (has_off) o = (float)p.offset[uidx];
    } else {
      s = 1.f;
    }
    // fminf / fmaxf drop NaN; the reference raises on it
    if (bad && p.status) atomicOr(p.status, 1);
    if (OUT == AMCT_OUT_NONE || !active) continue;

    // ---- levels, in the reference's order: t = x / s, + offset, (AWQ variant: round to T,) rint, clamp.
    // The clamp is applied before the rounding: same result, the bounds are integers.  (Even with
    // scales derived from the group itself it is needed: the largest element can land exactly on
    // qmax + 0.5, which rounds to the even qmax + 1.)
    float u[EP];                                   // level + 1.5 * 2^23
    float sg[kFake ? EP : 1];                      // fake-quant shows the sign of a zero level: rint(-0.3) = -0
    const float y = __frcp_rn(s);
    const float o_add = has_off ? o : -0.f;         // adding -0 keeps the sign of a zero quotient
    bool fast = fabsf(s) >= 1.17549435e-38f && fabsf(y) >= 1.17549435e-38f && isfinite(y) && isfinite(s);
    if (fast) {
      float poison = 0.f;
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        float q = div_by_recip(x[e], s, y);
        if (kFake) q = x[e] == 0.f ? __fmul_rn(x[e], y) : q;    // -0.0 / s is -0.0 (the FMA corrections give +0.0)
        float t = __fadd_rn(q, o_add);
        poison = __fmaf_rn(t, 0.f, poison);
        if (kAwqRounds) t = round_to<T>(t);
        t = fminf(fmaxf(t, qmin), qmax);
        u[e] = __fadd_rn(t, kMagicG);               // round half to even
        if (kFake) sg[e] = t;
      }
      if (poison != poison) fast = false;            // a NaN or infinite quotient: let the IEEE division decide
    }
    if (!fast) {
      const int flags = (has_off ? 1 : 0) | (kAwq ? 2 : 0);
#pragma unroll
      for (int e = 0; e < EP; e += 4) {
        const float4 r = levels_exact4<T>(x[e], x[e + 1], x[e + 2], x[e + 3], s, o, flags, qmin, qmax);
        u[e] = __fadd_rn(r.x, kMagicG); u[e + 1] = __fadd_rn(r.y, kMagicG);
        u[e + 2] = __fadd_rn(r.z, kMagicG); u[e + 3] = __fadd_rn(r.w, kMagicG);
        if (kFake) { sg[e] = r.x; sg[e + 1] = r.y; sg[e + 2] = r.z; sg[e + 3] = r.w; }
      }
    }

    // ---- outputs
    if (OUT == AMCT_OUT_I8) {
      int8_t* dst = reinterpret_cast<int8_t*>(p.out) + row * p.ld_out + j0;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        uint32_t w[E / 4];
#pragma unroll
        for (int g = 0; g < E / 4; ++g) {
          const float* q = &u[i * E + 4 * g];
          w[g] = __byte_perm(__byte_perm(__float_as_uint(q[0]), __float_as_uint(q[1]), 0x0040),
                             __byte_perm(__float_as_uint(q[2]), __float_as_uint(q[3]), 0x0040), 0x5410);
        }
        if constexpr (E == 8) *reinterpret_cast<uint2*>(dst + i * E) = make_uint2(w[0], w[1]);
        else *reinterpret_cast<uint32_t*>(dst + i * E) = w[0];
      }
    } else if (OUT == AMCT_OUT_I32) {
      int* dst = reinterpret_cast<int*>(p.out) + row * p.ld_out + j0;
      // sign-extend the 9 low bits that hold the level
#pragma unroll
      for (int e = 0; e < EP; e += 4)
        *reinterpret_cast<int4*>(dst + e) = make_int4(((int)__float_as_uint(u[e]) << 23) >> 23, ((int)__float_as_uint(u[e + 1]) << 23) >> 23,
                                                      ((int)__float_as_uint(u[e + 2]) << 23) >> 23, ((int)__float_as_uint(u[e + 3]) << 23) >> 23);
    } else if (OUT == AMCT_OUT_PACK4) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + row * p.ld_out + j0 / 2;
      // nibble = level + 8 in [0, 15]; four nibbles are combined as an exact fp32 sum below 2^16
      // (FMA pipe), whose integer value again sits in the low mantissa bits after adding 1.5 * 2^23
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        uint32_t h[E / 4];
#pragma unroll
        for (int g = 0; g < E / 4; ++g) {
          const float* q = &u[i * E + 4 * g];
          const float c0 = __fsub_rn(q[0], kMagicG - 8.f), c1 = __fsub_rn(q[1], kMagicG - 8.f);
          const float c2 = __fsub_rn(q[2], kMagicG - 8.f), c3 = __fsub_rn(q[3], kMagicG - 8.f);
          const float v4 = __fmaf_rn(__fmaf_rn(__fmaf_rn(c3, 16.f, c2), 16.f, c1), 16.f, c0);
          h[g] = __float_as_uint(__fadd_rn(v4, kMagicG));
        }
        if constexpr (E == 8) *reinterpret_cast<uint32_t*>(dst + i * (E / 2)) = __byte_perm(h[0], h[1], 0x5410);
        else *reinterpret_cast<uint16_t*>(dst + i * (E / 2)) = (uint16_t)h[0];
      }
    } else if (kFake) {  // (level - offset) * scale, rounded once to T
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        Vec16<T> r;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          float d = copysignf(__fsub_rn(u[i * E + e], kMagicG), sg[i * E + e]);
          if (has_off) d = __fsub_rn(d, o);
          r.v[e] = ElemTraits<T>::from_f(__fmul_rn(d, s));
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + row * p.ld_out + j0 + i * E) = *reinterpret_cast<const uint4*>(&r);
      }
    }
  }
}

template <typename T>
static int launch_groups(GroupParams p, int group, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  if (group % (2 * E) || p.k % group) return 1;
  const int lanes = group / (2 * E);
  if (lanes > 32 || (lanes & (lanes - 1))) return 1;
  if (!aligned16(p.x) || (p.ld * (int64_t)sizeof(T)) % 16 || (p.pre && !aligned16(p.pre))) return 1;
  if (p.k / E > 0x3fffffff || p.rows > 0x7fffffffLL) return 1;
  if (p.out_mode != AMCT_OUT_NONE) {
    const uintptr_t o = reinterpret_cast<uintptr_t>(p.out);
    switch (p.out_mode) {
      case AMCT_OUT_I8: if (o % E || p.ld_out % E) return 1; break;
      case AMCT_OUT_I32: if (o % 16 || (p.ld_out * 4) % 16) return 1; break;
      case AMCT_OUT_PACK4: if (o % (E / 2) || p.ld_out % (E / 2)) return 1; break;
      default: if (o % 16 || (p.ld_out * (int64_t)sizeof(T)) % 16) return 1; break;
    }
  }
  int l2 = 0;
  while ((1 << l2) < lanes) ++l2;
  p.lanes_log2 = l2;
  const int64_t nthr_row = p.k / (2 * E);
  dim3 grid((unsigned)((nthr_row + 255) / 256), 1);
  int64_t gy = (148LL * 4 + grid.x - 1) / grid.x;      // 4 resident blocks per SM (register use)
  if (gy > p.rows) gy = p.rows;
  if (gy > 65535) gy = 65535;
  grid.y = (unsigned)(gy < 1 ? 1 : gy);
  switch (p.out_mode) {
    case AMCT_OUT_NONE: AMCT_LAUNCH(grid, 256, st, (p), quant_groups_kernel<T, AMCT_OUT_NONE>); break;
    case AMCT_OUT_I8: AMCT_LAUNCH(grid, 256, st, (p), quant_groups_kernel<T, AMCT_OUT_I8>); break;
    case AMCT_OUT_I32: AMCT_LAUNCH(grid, 256, st, (p), quant_groups_kernel<T, AMCT_OUT_I32>); break;
    case AMCT_OUT_PACK4: AMCT_LAUNCH(grid, 256, st, (p), quant_groups_kernel<T, AMCT_OUT_PACK4>); break;
    case AMCT_OUT_FAKE: AMCT_LAUNCH(grid, 256, st, (p), quant_groups_kernel<T, AMCT_OUT_FAKE>); break;
    case AMCT_OUT_FAKE_AWQ: AMCT_LAUNCH(grid, 256, st, (p), quant_groups_kernel<T, AMCT_OUT_FAKE_AWQ>); break;
    default: return AMCT_ERR_ARG;
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

// Returns AMCT_OK when this kernel took the call, 1 when the shape does not fit it (the caller
// then uses the general row kernel), or an error code.
int quant_groups_try(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld, const void* pre, int pre_op, int compute,
                     int group, int bits, int symmetric, float* scale, int* offset, int out_mode, void* out, int64_t ld_out,
                     int* status, cudaStream_t st) {
  GroupParams p{};
  p.x = x; p.rows = rows; p.k = k; p.ld = ld; p.pre = pre; p.pre_op = pre_op; p.compute = compute;
  p.bits = bits; p.symmetric = symmetric; p.scale = scale; p.offset = symmetric ? nullptr : offset;
  p.out_mode = out_mode; p.out = out; p.ld_out = ld_out; p.status = status;
  switch (dtype) {
    case AMCT_DTYPE_F32: return launch_groups<float>(p, group, st);
    case AMCT_DTYPE_F16: return launch_groups<__half>(p, group, st);
    case AMCT_DTYPE_BF16: return launch_groups<__nv_bfloat16>(p, group, st);
  }
  return 1;
}

}  // namespace amct
