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
// One warp owns one row (a token, or a token-head of the indexer).  Arithmetic follows torch's dtypes: without
// learned clipping every step is rounded to the activation dtype; with it the fp32 clip parameter promotes the
// bounds and all later steps to fp32 and only the result is cast back.  round_ste(t) = (round(t) - t) + t is
// exact except that it turns a zero into +0, which the symmetric path reproduces.  A NaN quotient stays NaN through the
// clamp as in torch; a NaN INPUT is not treated like torch's amax (which makes the whole row NaN).  Compiled without
// FMA contraction.
//
// Algorithmic HBM bytes per element: sizeof(in) read + sizeof(out) written.
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
  float hi = fmaxf(row_max, 0.f), lo = fminf(row_min, 0.f);
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
  return r;
}

// one value of the output dtype -> its fake-quantized value (as fp32, representable in T)   node.py:39-66
template <typename T>
__device__ __forceinline__ float dsa_fake_quant(float v, const DsaRow& r, const DsaParams& p) {
  const bool f32 = dsa_fp32_math(p);
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

// Rotation (+ cast + fake quantization): k = 32 * EPL, lane l holds the EPL consecutive elements from l * EPL, and
// one warp works on RPW rows at a time so that enough loads are in flight (RPW * EPL = 16 values per lane).
// The transform is the same whichever index bits sit in the lane number: every bit gets its butterfly.
template <typename TIN, typename TOUT, int EPL, int RPW>
__global__ void __launch_bounds__(kDsaWarps * 32) dsa_rotate_quant_kernel(DsaParams p, int wide_in, int wide_out) {
  const int lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * kDsaWarps + (threadIdx.x >> 5)) * RPW;
  if (row0 >= p.rows) return;                                 // whole warps leave together
  float v[RPW][EPL];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    if (row0 + r < p.rows) {
      load_run<TIN, EPL>(reinterpret_cast<const TIN*>(p.x) + (row0 + r) * p.ld_x + lane * EPL, v[r], wide_in != 0);
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[r][e] = 0.f;
    }
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    // butterflies over the index bits held in the register number ...
#pragma unroll
    for (int m = 1; m < EPL; m <<= 1) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        if ((e & m) == 0) {
          const float a = v[r][e], c = v[r][e | m];
          v[r][e] = __fadd_rn(a, c);
          v[r][e | m] = __fsub_rn(a, c);
        }
      }
    }
    // ... and over the bits held in the lane number
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, v[r][e], m);
        v[r][e] = (lane & m) ? __fsub_rn(other, v[r][e]) : __fadd_rn(v[r][e], other);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    // scale, round to the input dtype (the rotation's result), then to the output dtype (.half() of the caller)
    float hi = -INFINITY, lo = INFINITY;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      v[r][e] = round_to<TOUT>(round_to<TIN>(__fmul_rn(v[r][e], p.had_entry)));
      hi = fmaxf(hi, v[r][e]);
      lo = fminf(lo, v[r][e]);
    }
    if (p.bits != 16) {
      const DsaRow q = dsa_row_params<TOUT>(warp_max(hi), warp_min(lo), p);
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[r][e] = dsa_fake_quant<TOUT>(v[r][e], q, p);
    }
    if (row0 + r < p.rows)
      store_run<TOUT, EPL>(reinterpret_cast<TOUT*>(p.out) + (row0 + r) * p.ld_out + lane * EPL, v[r], wide_out != 0);
  }
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
        const float f = round_to<TOUT>(ElemTraits<TIN>::to_f(raw.v[e]));
        hi = fmaxf(hi, f);
        lo = fminf(lo, f);
      }
    }
  } else {
    for (int64_t j = lane; j < p.k; j += 32) {
      const float f = round_to<TOUT>(ElemTraits<TIN>::to_f(x[j]));
      hi = fmaxf(hi, f);
      lo = fminf(lo, f);
    }
  }
  const DsaRow r = dsa_row_params<TOUT>(warp_max(hi), warp_min(lo), p);

  if (VEC) {
    for (int64_t i = lane; i < nvec; i += 32) {
      const Vec16<TIN> raw = ld_vec_stream(x + i * E);
      Vec16<TOUT> o;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float f = round_to<TOUT>(ElemTraits<TIN>::to_f(raw.v[e]));
        o.v[e] = ElemTraits<TOUT>::from_f(dsa_fake_quant<TOUT>(f, r, p));
      }
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
    // a lane's run of k / 32 elements can be moved with wide accesses when every run starts on a multiple of its size
    auto run_aligned = [&](const void* base, int64_t ld, size_t elem) {
      const int64_t run = (p.k / 32) * (int64_t)elem;
      const int64_t need = run >= 16 ? 16 : run;
      return need >= 4 && reinterpret_cast<uintptr_t>(base) % need == 0 && (ld * (int64_t)elem) % need == 0;
    };
    const int wi = run_aligned(p.x, p.ld_x, sizeof(TIN)) ? 1 : 0;
    const int wo = run_aligned(p.out, p.ld_out, sizeof(TOUT)) ? 1 : 0;
    auto blocks = [&](int rpw) { return (unsigned)((p.rows + (int64_t)kDsaWarps * rpw - 1) / ((int64_t)kDsaWarps * rpw)); };
    switch (p.k) {
      case 32: AMCT_LAUNCH(blocks(4), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 1, 4>); break;
      case 64: AMCT_LAUNCH(blocks(4), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 2, 4>); break;
      case 128: AMCT_LAUNCH(blocks(4), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 4, 4>); break;
      case 256: AMCT_LAUNCH(blocks(2), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 8, 2>); break;
      case 512: AMCT_LAUNCH(blocks(1), threads, st, (p, wi, wo), dsa_rotate_quant_kernel<TIN, TOUT, 16, 1>); break;
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
