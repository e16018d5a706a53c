// Group-wise weight quantization without shared memory or block barriers.
//
// Same arithmetic as the per-group branch of the row kernel in quant_rows.cu -- group min / max
// (amct_pytorch/quantize_op/utils.py:111-136), scale rule (utils.py:75-108), codes
// (amct_pytorch/utils/quant_util.py:57-93), nibble pack, and both fake-quant variants
// (quant_util.py:162-188; amct_pytorch/algorithm/awq.py:129-170) -- for the common case of a
// group that fits inside a warp: a power-of-two number of lanes, each owning four adjacent 16-byte
// vectors (32 elements of a 16-bit type), K a multiple of the group.  Every thread reduces min / max
// over its lane group with shuffles, derives the group's scale and offset itself, and quantizes its
// own elements.  blockIdx.x covers the columns, blockIdx.y strides over rows: no index division.
// The kernel is bound by instruction issue, not by HBM, unless it stays near a dozen instructions
// per element; hence the packed min / max, the scale rule on the FMA pipe, the saturating packs.
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

// NaN-propagating min / max of a 16-byte vector (torch.amin / amax return NaN for a group that holds one, and the
// scale rule then refuses the group): packed instructions for the 16-bit types, min.NaN / max.NaN for fp32.
__device__ __forceinline__ void vec_minmax(const Vec16<__nv_bfloat16>& v, __nv_bfloat162& mn, __nv_bfloat162& mx) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  mn = __hmin2_nan(mn, __hmin2_nan(__hmin2_nan(h[0], h[1]), __hmin2_nan(h[2], h[3])));
  mx = __hmax2_nan(mx, __hmax2_nan(__hmax2_nan(h[0], h[1]), __hmax2_nan(h[2], h[3])));
}
__device__ __forceinline__ void vec_minmax(const Vec16<__half>& v, __half2& mn, __half2& mx) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  mn = __hmin2_nan(mn, __hmin2_nan(__hmin2_nan(h[0], h[1]), __hmin2_nan(h[2], h[3])));
  mx = __hmax2_nan(mx, __hmax2_nan(__hmax2_nan(h[0], h[1]), __hmax2_nan(h[2], h[3])));
}
template <typename T> struct GroupAcc;          // the per-thread min / max accumulator of a type
template <> struct GroupAcc<__nv_bfloat16> {
  using type = __nv_bfloat162;
  __device__ static type init(float v) { return __floats2bfloat162_rn(v, v); }
  __device__ static float lo(type v) { return __low2float(v); }
  __device__ static float hi(type v) { return __high2float(v); }
};
template <> struct GroupAcc<__half> {
  using type = __half2;
  __device__ static type init(float v) { return __floats2half2_rn(v, v); }
  __device__ static float lo(type v) { return __low2float(v); }
  __device__ static float hi(type v) { return __high2float(v); }
};
template <> struct GroupAcc<float> {
  using type = float2;                          // x: running min or max, y unused
  __device__ static type init(float v) { return make_float2(v, v); }
  __device__ static float lo(type v) { return v.x; }
  __device__ static float hi(type v) { return v.y; }
};
__device__ __forceinline__ void vec_minmax(const Vec16<float>& v, float2& mn, float2& mx) {
#pragma unroll
  for (int e = 0; e < 4; e += 2) {
    mn.x = fmin_nan(mn.x, v.v[e]); mn.y = fmin_nan(mn.y, v.v[e + 1]);
    mx.x = fmax_nan(mx.x, v.v[e]); mx.y = fmax_nan(mx.y, v.v[e + 1]);
  }
}

// The scale rule (amct_pytorch/quantize_op/utils.py:75-108) for a group whose bounds are finite, with the two IEEE
// divisions replaced by the exact FMA sequence of div_by_recip: bound / (a small integer constant) and mn / scale.
// Both are valid uses: a quotient that is too small to be a normal number only occurs below the rule's epsilon, where
// the scale is replaced by 1 and the offset by -2^(bits-1) whatever the quotient was; the scale that divides mn is
// then at least that epsilon, so it and its reciprocal are normal.  Returns the scale; *offset as a float.
__device__ __forceinline__ float group_qparams(float mx, float mn, int bits, bool symmetric, float* offset) {
  if (symmetric) {
    const float amx = fabsf(mx), amn = fabsf(mn);
    const bool neg_dom = amx < amn;
    const float bound = neg_dom ? amn : amx;
    float s;
    if (neg_dom) {
      s = __fmul_rn(bound, bits == 8 ? 0.0078125f : 0.125f);                   // / 128 or / 8: exact scaling
      if (s < 1.17549435e-38f) s = 0.f;                                       // (a subnormal result is below epsilon anyway)
    } else {
      const float div = bits == 8 ? 127.f : 7.f;
      s = div_by_recip(bound, div, bits == 8 ? (1.f / 127.f) : (1.f / 7.f));
    }
    if (!(s >= AMCT_FLT_EPSILON)) s = 1.f;
    *offset = 0.f;
    return s;
  }
  mx = fmaxf(mx, 0.f);
  mn = fminf(mn, 0.f);
  const float span = bits == 8 ? 255.f : 15.f, half = bits == 8 ? 128.f : 8.f;
  float s = div_by_recip(__fsub_rn(mx, mn), span, bits == 8 ? (1.f / 255.f) : (1.f / 15.f));
  float o = -half;
  if (s >= AMCT_FLT_EPSILON) {
    // + 0: the reference's offset is an integer tensor, so a zero offset is +0 (rint(-0.3) is -0, and level - (-0)
    // would flip the sign of a zero level in the fake-quant outputs)
    if (mx != mn) o = __fadd_rn(rintf(__fsub_rn(-half, div_by_recip(mn, s, __frcp_rn(s)))), 0.f);
  } else {
    s = 1.f;
  }
  *offset = o;
  return s;
}

// Four adjacent 16-byte vectors per thread (32 elements of a 16-bit type: the scale rule, which every thread of a
// group evaluates, is spread over that many elements); a group spans (1 << lanes_log2) threads of a warp.  The row
// stays packed in T; one vector at a time is unpacked, divided and written.  In every mode the rounded level is
// carried as u = level + 1.5 * 2^23, whose low mantissa bits are the level in two's complement.
// COMPUTE: scales and offsets are derived from the data (then |level| <= 2^(bits-1) + 1 before the clamp, no quotient
// can overflow, and a NaN shows in the group's bounds); otherwise they are given and the levels can be anything.
template <typename T, int OUT, bool COMPUTE, bool HAS_OFF, bool PRE>
__global__ void __launch_bounds__(256, 4) quant_groups_kernel(GroupParams p) {
  constexpr int E = ElemTraits<T>::kPerVec;
  constexpr int VPT = 4, EP = E * VPT;              // vectors / elements per thread
  constexpr bool kAwq = OUT == AMCT_OUT_FAKE_AWQ;
  constexpr bool kAwqRounds = kAwq && sizeof(T) == 2;              // the AWQ variant rounds to T before rint()
  constexpr bool kFake = OUT == AMCT_OUT_FAKE || OUT == AMCT_OUT_FAKE_AWQ;
  constexpr bool kSign = kFake;     // a zero level keeps its sign: rint(-0.3) = -0, and (-0 - 0) * s = -0 (an offset can be 0)
  using Acc = GroupAcc<T>;
  const int nthr_row = (int)(p.k / EP);             // threads that own part of a row
  const int tcol = blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = tcol < nthr_row;
  const int lanes = 1 << p.lanes_log2;
  const int lane = threadIdx.x & 31;
  const int unit = tcol >> p.lanes_log2;
  const int nunits = nthr_row >> p.lanes_log2;
  const float qmax = (float)((1 << (p.bits - 1)) - 1), qmin = -qmax - 1.f;
  const T* __restrict__ pre = reinterpret_cast<const T*>(p.pre);
  const int64_t j0 = (int64_t)tcol * EP;

  Vec16<T> pre_v[PRE ? VPT : 1];
  if (PRE && active) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) pre_v[i] = ld_vec(pre + j0 + i * E);
  }

  for (int64_t row = blockIdx.y; row < p.rows; row += gridDim.y) {
    Vec16<T> raw[VPT];
    if (active) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) raw[i] = ld_vec_stream(reinterpret_cast<const T*>(p.x) + row * p.ld + j0 + i * E);
      if constexpr (PRE) {
        // the product / quotient by the SmoothQuant or AWQ factor is a separate torch op in the reference: rounded to T
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
#pragma unroll
          for (int e = 0; e < E; ++e) {
            const float a = ElemTraits<T>::to_f(raw[i].v[e]), f = ElemTraits<T>::to_f(pre_v[i].v[e]);
            raw[i].v[e] = ElemTraits<T>::from_f(p.pre_op == AMCT_PRE_MUL ? __fmul_rn(a, f) : __fdiv_rn(a, f));
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i) *reinterpret_cast<uint4*>(&raw[i]) = make_uint4(0, 0, 0, 0);
    }
    float s, o = 0.f;
    bool bad = false;
    const int64_t uidx = row * nunits + unit;
    if constexpr (COMPUTE) {
      typename Acc::type vmn = Acc::init(INFINITY), vmx = Acc::init(-INFINITY);
#pragma unroll
      for (int i = 0; i < VPT; ++i) vec_minmax(raw[i], vmn, vmx);
      float mn = fmin_nan(Acc::lo(vmn), Acc::hi(vmn)), mx = fmax_nan(Acc::lo(vmx), Acc::hi(vmx));
      for (int w = 1; w < lanes; w <<= 1) {
        mn = fmin_nan(mn, __shfl_xor_sync(0xffffffffu, mn, w));
        mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, w));
      }
      bool ok;
      if (isfinite(__fsub_rn(mx, mn))) {
        s = group_qparams(mx, mn, p.bits, !HAS_OFF, &o);
        ok = true;
      } else {
        // a NaN or an infinite bound: the rule as the other kernels state it (it ends in a refusal either way)
        int oi;
        ok = qparams_from_minmax(mx, mn, p.bits, !HAS_OFF, &s, &oi) && mx == mx && mn == mn;
        o = (float)oi;
      }
      if (active && (lane & (lanes - 1)) == 0) {
        p.scale[uidx] = s;
        if (HAS_OFF) p.offset[uidx] = (int)o;
        if (!ok && p.status) atomicOr(p.status, 1);
      }
    } else {
      if (active) {
        s = p.scale[uidx];
        if (HAS_OFF) o = (float)p.offset[uidx];
      } else {
        s = 1.f;
      }
    }
    if (OUT == AMCT_OUT_NONE || !active) {
      if (!COMPUTE && active && p.status) {
        // scales given, nothing to write: the input is still checked for NaN like the other paths
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
#pragma unroll
          for (int e = 0; e < E; ++e) { const float a = ElemTraits<T>::to_f(raw[i].v[e]); bad |= (a != a); }
        }
        if (bad) atomicOr(p.status, 1);
      }
      continue;
    }

    // ---- levels, in the reference's order: t = x / s, + offset, (AWQ variant: round to T,) rint, clamp.
    // The clamp is applied before the rounding where it is a float clamp (same result, the bounds are integers), or
    // after it by the saturating pack.  Even with scales derived from the group itself it is needed: the largest
    // element can land exactly on qmax + 0.5, which rounds to the even qmax + 1.
    const float y = __frcp_rn(s);
    const float o_add = HAS_OFF ? o : -0.f;         // adding -0 keeps the sign of a zero quotient
    const bool fast = fabsf(s) >= 1.17549435e-38f && fabsf(y) >= 1.17549435e-38f && isfinite(y) && isfinite(s);
    uint32_t words[VPT * (OUT == AMCT_OUT_I8 ? 2 : 1)];               // PACK4: one word per vector, I8: two
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float x[E], u[E];
      float sg[kSign ? E : 1];
#pragma unroll
      for (int e = 0; e < E; ++e) x[e] = ElemTraits<T>::to_f(raw[i].v[e]);
      bool vec_fast = fast;
      if (vec_fast) {
        float poison = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          float q = div_by_recip(x[e], s, y);
          if (kSign) q = x[e] == 0.f ? __fmul_rn(x[e], y) : q;    // -0.0 / s is -0.0 (the FMA corrections give +0.0)
          float t = __fadd_rn(q, o_add);
          if (!COMPUTE) poison = __fmaf_rn(t, 0.f, poison);        // a NaN or infinite level (x itself, or x / s overflowing)
          if (kAwqRounds) t = round_to<T>(t);
          if (!COMPUTE || kFake || OUT == AMCT_OUT_I32) t = fminf(fmaxf(t, qmin), qmax);
          u[e] = __fadd_rn(t, kMagicG);               // round half to even
          if (kSign) sg[e] = t;
        }
        if (!COMPUTE && poison != poison) vec_fast = false;        // let the IEEE division decide
      }
      if (!vec_fast) {
        const int flags = (HAS_OFF ? 1 : 0) | (kAwq ? 2 : 0);
#pragma unroll
        for (int e = 0; e < E; e += 4) {
          const float4 r = levels_exact4<T>(x[e], x[e + 1], x[e + 2], x[e + 3], s, o, flags, qmin, qmax);
          u[e] = __fadd_rn(r.x, kMagicG); u[e + 1] = __fadd_rn(r.y, kMagicG);
          u[e + 2] = __fadd_rn(r.z, kMagicG); u[e + 3] = __fadd_rn(r.w, kMagicG);
          if (kSign) { sg[e] = r.x; sg[e + 1] = r.y; sg[e + 2] = r.z; sg[e + 3] = r.w; }
        }
        if (!COMPUTE) {
#pragma unroll
          for (int e = 0; e < E; ++e) bad |= (x[e] != x[e]);
        }
      }
      // ---- this vector's output
      constexpr int kMagicBits = 0x4B400000;            // 1.5 * 2^23 as an integer: u's bits minus this is the level
      if constexpr (OUT == AMCT_OUT_PACK4) {
        // nibble = level + 8; the pack saturates to [-8, 7] in two's complement, flipping bit 3 adds the 8
        uint32_t w = 0;
#pragma unroll
        for (int e = E - 2; e >= 0; e -= 2)
          w = pack_sat_s4(__float_as_int(u[e + 1]) - kMagicBits, __float_as_int(u[e]) - kMagicBits, w);
        words[i] = w ^ (E == 8 ? 0x88888888u : 0x8888u);
      } else if constexpr (OUT == AMCT_OUT_I8) {
#pragma unroll
        for (int g = 0; g < E / 4; ++g) {
          uint32_t w = pack_sat_s8(__float_as_int(u[4 * g + 3]) - kMagicBits, __float_as_int(u[4 * g + 2]) - kMagicBits, 0);
          words[i * 2 + g] = pack_sat_s8(__float_as_int(u[4 * g + 1]) - kMagicBits, __float_as_int(u[4 * g]) - kMagicBits, w);
        }
      } else if constexpr (OUT == AMCT_OUT_I32) {
        int* dst = reinterpret_cast<int*>(p.out) + row * p.ld_out + j0 + i * E;
#pragma unroll
        for (int e = 0; e < E; e += 4)
          *reinterpret_cast<int4*>(dst + e) = make_int4(__float_as_int(u[e]) - kMagicBits, __float_as_int(u[e + 1]) - kMagicBits,
                                                        __float_as_int(u[e + 2]) - kMagicBits, __float_as_int(u[e + 3]) - kMagicBits);
      } else if constexpr (kFake) {  // (level - offset) * scale, rounded once to T
        Vec16<T> r;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          float d = __fsub_rn(u[e], kMagicG);
          if (kSign) d = copysignf(d, sg[e]);
          if (HAS_OFF) d = __fsub_rn(d, o);
          r.v[e] = ElemTraits<T>::from_f(__fmul_rn(d, s));
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + row * p.ld_out + j0 + i * E) = *reinterpret_cast<const uint4*>(&r);
      }
    }
    if constexpr (OUT == AMCT_OUT_PACK4) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + row * p.ld_out + j0 / 2;
      if constexpr (E == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
      else *reinterpret_cast<uint2*>(dst) = make_uint2(words[0] | (words[1] << 16), words[2] | (words[3] << 16));
    } else if constexpr (OUT == AMCT_OUT_I8) {
      int8_t* dst = reinterpret_cast<int8_t*>(p.out) + row * p.ld_out + j0;
      if constexpr (E == 8) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(words[4], words[5], words[6], words[7]);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[2], words[4], words[6]);
      }
    }
    // fminf / fmaxf drop NaN; the reference raises on it
    if (!COMPUTE && bad && p.status) atomicOr(p.status, 1);
  }
}

template <typename T, int OUT>
static void launch_groups_mode(const GroupParams& p, dim3 grid, int threads, cudaStream_t st) {
  const bool has_off = p.offset != nullptr, pre = p.pre_op != AMCT_PRE_NONE;
#define AMCT_GROUPS_CASE(C, O, P) \
  if ((p.compute != 0) == C && has_off == O && pre == P) AMCT_LAUNCH(grid, threads, st, (p), quant_groups_kernel<T, OUT, C, O, P>)
  AMCT_GROUPS_CASE(true, true, false); AMCT_GROUPS_CASE(true, false, false);
  AMCT_GROUPS_CASE(false, true, false); AMCT_GROUPS_CASE(false, false, false);
  AMCT_GROUPS_CASE(true, true, true); AMCT_GROUPS_CASE(true, false, true);
  AMCT_GROUPS_CASE(false, true, true); AMCT_GROUPS_CASE(false, false, true);
#undef AMCT_GROUPS_CASE
}

template <typename T>
static int launch_groups(GroupParams p, int group, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  constexpr int EP = 4 * E;                          // elements per thread
  if (group % EP || p.k % group) return 1;
  const int lanes = group / EP;
  if (lanes > 32 || (lanes & (lanes - 1))) return 1;
  if (!aligned16(p.x) || (p.ld * (int64_t)sizeof(T)) % 16 || (p.pre && !aligned16(p.pre))) return 1;
  if (p.k / E > 0x3fffffff || p.rows > 0x7fffffffLL) return 1;
  if (p.out_mode != AMCT_OUT_NONE) {
    const uintptr_t o = reinterpret_cast<uintptr_t>(p.out);
    switch (p.out_mode) {
      case AMCT_OUT_I8: if (o % 16 || p.ld_out % 16) return 1; break;
      case AMCT_OUT_I32: if (o % 16 || (p.ld_out * 4) % 16) return 1; break;
      case AMCT_OUT_PACK4: if (o % (EP / 2) || p.ld_out % (EP / 2)) return 1; break;
      default: if (o % 16 || (p.ld_out * (int64_t)sizeof(T)) % 16) return 1; break;
    }
  }
  int l2 = 0;
  while ((1 << l2) < lanes) ++l2;
  p.lanes_log2 = l2;
  const int64_t nthr_row = p.k / EP;
  // whole warps; a row shorter than a block's worth of threads gets a smaller block instead of idle warps
  int threads = (int)(nthr_row >= 256 ? 256 : ((nthr_row + 31) / 32) * 32);
  dim3 grid((unsigned)((nthr_row + threads - 1) / threads), 1);
  int64_t gy = (148LL * 2048 / threads + grid.x - 1) / grid.x;      // as many blocks as can be resident
  if (gy > p.rows) gy = p.rows;
  if (gy > 65535) gy = 65535;
  grid.y = (unsigned)(gy < 1 ? 1 : gy);
  switch (p.out_mode) {
    case AMCT_OUT_NONE: launch_groups_mode<T, AMCT_OUT_NONE>(p, grid, threads, st); break;
    case AMCT_OUT_I8: launch_groups_mode<T, AMCT_OUT_I8>(p, grid, threads, st); break;
    case AMCT_OUT_I32: launch_groups_mode<T, AMCT_OUT_I32>(p, grid, threads, st); break;
    case AMCT_OUT_PACK4: launch_groups_mode<T, AMCT_OUT_PACK4>(p, grid, threads, st); break;
    case AMCT_OUT_FAKE: launch_groups_mode<T, AMCT_OUT_FAKE>(p, grid, threads, st); break;
    case AMCT_OUT_FAKE_AWQ: launch_groups_mode<T, AMCT_OUT_FAKE_AWQ>(p, grid, threads, st); break;
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
