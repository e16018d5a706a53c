// KV-cache / indexer activation path of the reference's DeepSeek-V3.2 tree
// (amct_pytorch/experimental/quantization/DeepSeekV3.2/cores/...):
//   * rotate_activation: x @ (H / sqrt(d)) over the last axis in fp32, H the Sylvester Hadamard matrix
//     (models/deepseek_v3_2/indexer.py:140-151), here a fast Walsh-Hadamard transform inside one warp;
//   * ActivationQuantizer.fake_quant, per token, dynamic (quantization/node.py:140-215 with :39-66):
//     symmetric without learned clipping (the attention module's afq1 / afq2 / afq_rot_q / afq_rot_k,
//     models/deepseek_v3_2/quant_dsa.py:46-49, :121-124), symmetric or asymmetric with it (k_cache_quantizer,
//     quant_dsa.py:118-119);
//   * the indexer's chain rotate -> .half() -> fake_quant (quant_dsa.py:75-82) in one pass over the row.
//
// One warp owns one row (a token) of the plain fake quantization; a rotated row (a token-head of the indexer) lies on
// k / 16 lanes.  Arithmetic follows torch's dtypes: without
// learned clipping every step is rounded to the activation dtype; with it the fp32 clip parameter promotes the
// bounds and all later steps to fp32 and only the result is cast back.  round_ste(t) = (round(t) - t) + t is
// exact except that it turns a zero into +0, which the symmetric path reproduces.  A NaN quotient stays NaN through the
// clamp as in torch, and a NaN INPUT makes its row's bounds, scale and outputs NaN as torch's amax does.  Compiled
// without FMA contraction.
//
// Algorithmic HBM bytes per element: sizeof(in) read + sizeof(out) written.
#include <type_traits>

#include "common.cuh"

namespace amct {

struct DsaParams {
  const void* x;
  int64_t rows, k, ld_x;
  int bits;            // 16: no quantization (rotation / cast only)
  int symmetric;
  int mode;            // AMCT_DSA_*
  float a, b;          // LEARNED_CLIP: sigmoid of the max / min clip parameter; CLIP_RATIO: a = ratio; STATIC*: scale, zero
  float had_entry;     // fl32(1 / fl32(sqrt(k))) when rotating
  void* out;
  int64_t ld_out;
};

struct DsaRow {
  float scale, recip, zero, qlo, qhi;
  bool fast;     // the scale a normal number and every quotient of the row finite and below 2^21: no NaN, no overflow to handle
};

// torch promotes to fp32 when the bounds or the scale meet a one-element fp32 tensor (the clip parameter, a loaded
// scale buffer); otherwise every step stays in the activation dtype
__device__ __forceinline__ bool dsa_fp32_math(const DsaParams& p) {
  return p.mode == AMCT_DSA_LEARNED_CLIP || p.mode == AMCT_DSA_STATIC_F32;
}
__device__ __forceinline__ bool dsa_static(const DsaParams& p) {
  return p.mode == AMCT_DSA_STATIC || p.mode == AMCT_DSA_STATIC_F32;
}

// rounding to the dtype torch computes in: fp32 with learned clipping, else the output dtype
template <typename T>
__device__ __forceinline__ float round_c(float v, bool fp32_math) {
  return fp32_math ? v : round_to<T>(v);
}

// row bounds (values of the output dtype) -> scale, zero point and code range          node.py:181-215
template <typename T>
__device__ __forceinline__ DsaRow dsa_row_params(float row_max, float row_min, const DsaParams& p) {
  const bool f32 = dsa_fp32_math(p);
  const bool clip = p.mode == AMCT_DSA_LEARNED_CLIP;
  float hi = fmax_nan(row_max, 0.f), lo = fmin_nan(row_min, 0.f);          // torch.clamp keeps a NaN bound
  if (p.mode == AMCT_DSA_CLIP_RATIO) {                          // node.py:198-200, in the activation dtype
    hi = round_to<T>(__fmul_rn(hi, p.a));
    lo = round_to<T>(__fmul_rn(lo, p.a));
  }
  DsaRow r;
  if (p.symmetric) {
    const float qmax = (float)((1 << (p.bits - 1)) - 1);
    r.zero = 0.f;
    r.qlo = -(qmax + 1.f);
    r.qhi = qmax;
    if (dsa_static(p)) {
      r.scale = p.a;
    } else {
      const float bound = clip ? __fmul_rn(fmaxf(fabsf(lo), hi), p.a) : hi;
      r.scale = round_c<T>(__fdiv_rn(bound, qmax), f32);
      if (bound == 0.f) r.scale = 1.f;
    }
  } else {
    const float qmax = (float)((1 << p.bits) - 1);
    r.qlo = 0.f;
    r.qhi = qmax;
    if (dsa_static(p)) {
      r.scale = p.a;
      r.zero = p.b;
    } else {
      if (clip) {
        hi = __fmul_rn(hi, p.a);
        lo = __fmul_rn(lo, p.b);
      }
      if (hi == 0.f && lo == 0.f) {
        hi = 1.f;
        lo = -1.f;
      }
      r.scale = round_c<T>(__fdiv_rn(round_c<T>(__fsub_rn(hi, lo), f32), qmax), f32);
      r.zero = rintf(round_c<T>(__fdiv_rn(-lo, r.scale), f32));
    }
  }
  const float y = __frcp_rn(r.scale);
  const bool ok = fabsf(r.scale) >= 1.17549435e-38f && fabsf(y) >= 1.17549435e-38f && isfinite(y) && isfinite(r.scale);
  r.recip = ok ? y : 0.f;
  // |v / scale| <= max|v| * |1 / scale| (1 + 2^-22) for every value of the row; with a given (static) scale the row's
  // extrema are not known here
  const float reach = __fmul_rn(fmaxf(fabsf(row_max), fabsf(row_min)), fabsf(y));
  r.fast = ok && !dsa_static(p) && reach < 2097152.f;
  return r;
}

// one value of the output dtype -> its fake-quantized value (as fp32, representable in T)   node.py:39-66
template <typename T>
__device__ __forceinline__ float dsa_fake_quant(float v, const DsaRow& r, const DsaParams& p) {
  const bool f32 = dsa_fp32_math(p);
  if (r.fast) {
    // No quotient of this row is NaN, infinite or beyond 2^21: the exact FMA division, no NaN to carry through the clamp.
    const float t = round_c<T>(div_by_recip(v, r.scale, r.recip), f32);
    if (p.symmetric) {
      // clamp before rounding (the bounds are integers, so the order does not matter); round half to even by adding and
      // subtracting 1.5 * 2^23, which also turns a -0 level into +0 as round_ste does; one rounding of scale * level to
      // T (rounding a value of T to T again changes nothing)
      const float level = __fsub_rn(__fadd_rn(fminf(fmaxf(t, r.qlo), r.qhi), 12582912.f), 12582912.f);
      return round_to<T>(__fmul_rn(r.scale, level));
    }
    const float level = fminf(fmaxf(round_c<T>(__fadd_rn(rintf(t), r.zero), f32), r.qlo), r.qhi);
    return round_to<T>(__fmul_rn(r.scale, round_c<T>(__fsub_rn(level, r.zero), f32)));
  }
  float q;
  if (r.recip != 0.f) {
    q = div_by_recip(v, r.scale, r.recip);
    if (!(fabsf(q) <= 3.0e38f)) q = __fdiv_rn(v, r.scale);
  } else {
    q = __fdiv_rn(v, r.scale);
  }
  float level = rintf(round_c<T>(q, f32));
  // torch.clamp keeps a NaN (0 / 0 when a tiny 16-bit scale underflows to zero); fminf / fmaxf would drop it
  const bool is_nan = level != level;
  if (p.symmetric) {
    level = fminf(fmaxf(__fadd_rn(level, 0.f), r.qlo), r.qhi);           // -0 -> +0 like round_ste
    if (is_nan) level = __int_as_float(0x7fc00000);
    return round_to<T>(round_c<T>(__fmul_rn(r.scale, level), f32));
  }
  level = fminf(fmaxf(round_c<T>(__fadd_rn(level, r.zero), f32), r.qlo), r.qhi);
  if (is_nan) level = __int_as_float(0x7fc00000);
  return round_to<T>(round_c<T>(__fmul_rn(r.scale, round_c<T>(__fsub_rn(level, r.zero), f32)), f32));
}

constexpr int kDsaWarps = 4;

// an input element as a value of the output dtype (what `.to(dtype)` of the caller leaves): no rounding to do when the
// two are the same type
template <typename TIN, typename TOUT>
__device__ __forceinline__ float as_out(TIN v) {
  if constexpr (std::is_same<TIN, TOUT>::value) return ElemTraits<TIN>::to_f(v);
  else return round_to<TOUT>(ElemTraits<TIN>::to_f(v));
}

// EPL consecutive elements of T <-> floats, with the widest naturally aligned accesses when `wide` is set
// (the caller has checked that every row starts on a multiple of EPL * sizeof(T) bytes, up to 16).
template <typename T, int EPL>
__device__ __forceinline__ void load_run(const T* p, float* v, bool wide) {
  constexpr int kBytes = EPL * (int)sizeof(T);
  if (wide && kBytes >= 4) {
    constexpr int kWord = kBytes >= 16 ? 16 : kBytes;            // 4, 8 or 16 bytes per access
    constexpr int kPerWord = kWord / (int)sizeof(T);
#pragma unroll
    for (int i = 0; i < kBytes / kWord; ++i) {
      alignas(16) T tmp[kPerWord];
      if (kWord == 16) *reinterpret_cast<uint4*>(tmp) = __ldcs(reinterpret_cast<const uint4*>(p + i * kPerWord));
      else if (kWord == 8) *reinterpret_cast<uint2*>(tmp) = __ldcs(reinterpret_cast<const uint2*>(p + i * kPerWord));
      else *reinterpret_cast<uint32_t*>(tmp) = __ldcs(reinterpret_cast<const uint32_t*>(p + i * kPerWord));
#pragma unroll
      for (int e = 0; e < kPerWord; ++e) v[i * kPerWord + e] = ElemTraits<T>::to_f(tmp[e]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = ElemTraits<T>::to_f(p[e]);
  }
}
template <typename T, int EPL>
__device__ __forceinline__ void store_run(T* p, const float* v, bool wide) {
  constexpr int kBytes = EPL * (int)sizeof(T);
  if (wide && kBytes >= 4) {
    constexpr int kWord = kBytes >= 16 ? 16 : kBytes;
    constexpr int kPerWord = kWord / (int)sizeof(T);
#pragma unroll
    for (int i = 0; i < kBytes / kWord; ++i) {
      alignas(16) T tmp[kPerWord];
#pragma unroll
      for (int e = 0; e < kPerWord; ++e) tmp[e] = ElemTraits<T>::from_f(v[i * kPerWord + e]);
      if (kWord == 16) *reinterpret_cast<uint4*>(p + i * kPerWord) = *reinterpret_cast<const uint4*>(tmp);
      else if (kWord == 8) *reinterpret_cast<uint2*>(p + i * kPerWord) = *reinterpret_cast<const uint2*>(tmp);
      else *reinterpret_cast<uint32_t*>(p + i * kPerWord) = *reinterpret_cast<const uint32_t*>(tmp);
    }
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) p[e] = ElemTraits<T>::from_f(v[e]);
  }
}

// Rotation (+ cast + fake quantization): a row of k = LPR * EPL elements lies on LPR lanes of a warp, lane l of the
// row holding the EPL consecutive elements from l * EPL, and a warp works on 32 / LPR rows side by side.  Sixteen
// elements per lane wherever k allows: the per-row work (bounds, scale rule) and the shuffle stages are then shared by
// 16 elements, and 32 bytes per lane are in flight.  The transform is the same whichever index bits sit in the lane
// number: every bit gets its butterfly, lowest bit first.
template <typename TIN, typename TOUT, int EPL, int LPR>
__global__ void __launch_bounds__(kDsaWarps * 32) dsa_rotate_quant_kernel(DsaParams p, int wide_in, int wide_out) {
  constexpr int RPW = 32 / LPR;                                 // rows per warp
  const int lane = threadIdx.x & 31;
  const int sub = lane & (LPR - 1);                             // lane within its row
  const int64_t row = ((int64_t)blockIdx.x * kDsaWarps + (threadIdx.x >> 5)) * RPW + lane / LPR;
  const bool live = row < p.rows;                               // dead rows compute on zeros: the shuffles need every lane
  float v[EPL];
  if (live) {
    load_run<TIN, EPL>(reinterpret_cast<const TIN*>(p.x) + row * p.ld_x + sub * EPL, v, wide_in != 0);
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = 0.f;
  }
  // butterflies over the index bits held in the register number ...
#pragma unroll
  for (int m = 1; m < EPL; m <<= 1) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      if ((e & m) == 0) {
        const float a = v[e], c = v[e | m];
        v[e] = __fadd_rn(a, c);
        v[e | m] = __fsub_rn(a, c);
      }
    }
  }
  // ... and over the bits held in the lane number (the partners stay inside the row's LPR lanes)
#pragma unroll
  for (int m = 1; m < LPR; m <<= 1) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, v[e], m);
      v[e] = (sub & m) ? __fsub_rn(other, v[e]) : __fadd_rn(v[e], other);
    }
  }
  // scale, round to the input dtype (the rotation's result), then to the output dtype (.half() of the caller)
  float hi = -INFINITY, lo = INFINITY;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    v[e] = round_to<TOUT>(round_to<TIN>(__fmul_rn(v[e], p.had_entry)));
    hi = fmax_nan(hi, v[e]);
    lo = fmin_nan(lo, v[e]);
  }
  if (p.bits != 16) {
#pragma unroll
    for (int m = 1; m < LPR; m <<= 1) {
      hi = fmax_nan(hi, __shfl_xor_sync(0xffffffffu, hi, m));
      lo = fmin_nan(lo, __shfl_xor_sync(0xffffffffu, lo, m));
    }
    const DsaRow q = dsa_row_params<TOUT>(hi, lo, p);
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = dsa_fake_quant<TOUT>(v[e], q, p);
  }
  if (live) store_run<TOUT, EPL>(reinterpret_cast<TOUT*>(p.out) + row * p.ld_out + sub * EPL, v, wide_out != 0);
}

// Fake quantization alone (any k): pass 1 takes the bounds, pass 2 re-reads the row (an L1 / L2 hit).
// VEC: 16-byte loads and stores, possible when input and output elements have the same size.
template <typename TIN, typename TOUT, bool VEC>
__global__ void __launch_bounds__(kDsaWarps * 32) dsa_fakequant_kernel(DsaParams p) {
  constexpr int E = ElemTraits<TIN>::kPerVec;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kDsaWarps + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const TIN* x = reinterpret_cast<const TIN*>(p.x) + row * p.ld_x;
  TOUT* out = reinterpret_cast<TOUT*>(p.out) + row * p.ld_out;
  const int64_t nvec = VEC ? p.k / E : 0;

  float hi = -INFINITY, lo = INFINITY;
  if (dsa_static(p)) {
    hi = lo = 0.f;                                             // given scale: no pass over the row for its bounds
  } else if (VEC) {
    for (int64_t i = lane; i < nvec; i += 32) {
      const Vec16<TIN> raw = ld_vec(x + i * E);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float f = as_out<TIN, TOUT>(raw.v[e]);
        hi = fmax_nan(hi, f);
        lo = fmin_nan(lo, f);
      }
    }
  } else {
    for (int64_t j = lane; j < p.k; j += 32) {
      const float f = round_to<TOUT>(ElemTraits<TIN>::to_f(x[j]));
      hi = fmax_nan(hi, f);
      lo = fmin_nan(lo, f);
    }
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {                           // a NaN anywhere in the row reaches its bounds, as in torch.amax
    hi = fmax_nan(hi, __shfl_xor_sync(0xffffffffu, hi, m));
    lo = fmin_nan(lo, __shfl_xor_sync(0xffffffffu, lo, m));
  }
  const DsaRow r = dsa_row_params<TOUT>(hi, lo, p);

  if (VEC) {
    for (int64_t i = lane; i < nvec; i += 32) {
      const Vec16<TIN> raw = ld_vec_stream(x + i * E);
      Vec16<TOUT> o;
#pragma unroll
      for (int e = 0; e < E; ++e) o.v[e] = ElemTraits<TOUT>::from_f(dsa_fake_quant<TOUT>(as_out<TIN, TOUT>(raw.v[e]), r, p));
      *reinterpret_cast<uint4*>(out + i * E) = *reinterpret_cast<const uint4*>(&o);
    }
  } else {
    for (int64_t j = lane; j < p.k; j += 32) {
      const float f = round_to<TOUT>(ElemTraits<TIN>::to_f(x[j]));
      out[j] = ElemTraits<TOUT>::from_f(dsa_fake_quant<TOUT>(f, r, p));
    }
  }
}

template <typename TIN, typename TOUT>
static int launch_dsa(const DsaParams& p, int rotate, cudaStream_t st) {
  const unsigned grid = (unsigned)((p.rows + kDsaWarps - 1) / kDsaWarps);
  const int threads = kDsaWarps * 32;
  if (rotate) {
    // a lane's run of EPL elements can be moved with wide accesses when every run starts on a multiple of its size
    const int epl = p.k >= 128 ? 16 : (int)(p.k / 8);            // 16 elements per lane from k = 128 on; 8 lanes per row below
    auto run_aligned = [&](const void* base, int64_t ld, size_t elem) {
      const int64_t run = epl * (int64_t)elem;
      const int64_t need = run >= 16 ? 16 : run;
      return need >= 4 && reinterpret_cast<uintptr_t>(base) % need == 0 && (ld * (int64_t)elem) % need == 0;
    };
    const int wi = run_aligned(p.x, p.ld_x, sizeof(TIN)) ? 1 : 0;
    const int wo = run_aligned(p.out, p.ld_out, sizeof(TOUT)) ? 1 : 0;
    auto blocks = [&](int lpr) {
      const int64_t rows_per_block = (int64_t)kDsaWarps * (32 / lpr);
      return (unsigned)((p.rows + rows_per_block - 1) / rows_per_block);
    };
    switch (p.k) {
      case 32: AMCT_LAUNCH(blocks(8), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 4, 8>); break;
      case 64: AMCT_LAUNCH(blocks(8), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 8, 8>); break;
      case 128: AMCT_LAUNCH(blocks(8), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 16, 8>); break;
      case 256: AMCT_LAUNCH(blocks(16), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 16, 16>); break;
      case 512: AMCT_LAUNCH(blocks(32), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 16, 32>); break;
      default: return AMCT_ERR_UNSUPPORTED;
    }
  } else {
    constexpr int E = ElemTraits<TIN>::kPerVec;
    const bool vec = sizeof(TIN) == sizeof(TOUT) && p.k % E == 0 && aligned16(p.x) && aligned16(p.out) &&
                     (p.ld_x * (int64_t)sizeof(TIN)) % 16 == 0 && (p.ld_out * (int64_t)sizeof(TOUT)) % 16 == 0;
    if (vec) AMCT_LAUNCH(grid, threads, st, (p), dsa_fakequant_kernel<TIN, TOUT, sizeof(TIN) == sizeof(TOUT)>);
    else AMCT_LAUNCH(grid, threads, st, (p), dsa_fakequant_kernel<TIN, TOUT, false>);
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

template <typename TIN>
static int dispatch_dsa_out(const DsaParams& p, int rotate, int out_dtype, cudaStream_t st) {
  switch (out_dtype) {
    case AMCT_DTYPE_F32: return launch_dsa<TIN, float>(p, rotate, st);
    case AMCT_DTYPE_F16: return launch_dsa<TIN, __half>(p, rotate, st);
    case AMCT_DTYPE_BF16: return launch_dsa<TIN, __nv_bfloat16>(p, rotate, st);
  }
  return AMCT_ERR_ARG;
}

}  // namespace amct

using namespace amct;

extern "C" int amct_dsa_rotate_fakequant(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int rotate,
                                         int out_dtype, int bits, int symmetric, int mode, float a, float b,
                                         void* out, int64_t ld_out, void* stream) {
  if (rows < 0 || k <= 0 || ld_x < k || ld_out < k) return AMCT_ERR_ARG;
  if (bits != 16 && (bits < 2 || bits > 8)) return AMCT_ERR_ARG;
  if (mode < AMCT_DSA_DYNAMIC || mode > AMCT_DSA_STATIC_F32) return AMCT_ERR_ARG;
  if (rotate && (k & (k - 1)) != 0) return AMCT_ERR_ARG;
  if (rotate && (k < 32 || k > 512)) return AMCT_ERR_UNSUPPORTED;
  if (rows == 0) return AMCT_OK;
  if (!x || !out) return AMCT_ERR_ARG;
  if ((rows + kDsaWarps - 1) / kDsaWarps > 0x7fffffff) return AMCT_ERR_UNSUPPORTED;
  DsaParams p;
  p.x = x;
  p.rows = rows;
  p.k = k;
  p.ld_x = ld_x;
  p.bits = bits;
  p.symmetric = symmetric ? 1 : 0;
  p.mode = mode;
  p.a = a;
  p.b = b;
  p.had_entry = rotate ? 1.0f / sqrtf((float)k) : 1.0f;
  p.out = out;
  p.ld_out = ld_out;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case AMCT_DTYPE_F32: return dispatch_dsa_out<float>(p, rotate, out_dtype, st);
    case AMCT_DTYPE_F16: return dispatch_dsa_out<__half>(p, rotate, out_dtype, st);
    case AMCT_DTYPE_BF16: return dispatch_dsa_out<__nv_bfloat16>(p, rotate, out_dtype, st);
  }
  return AMCT_ERR_ARG;
}
