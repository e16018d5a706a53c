// Static activation quantization: q = sat_int8(rne(x * scale + offset)) with a
// calibrated reciprocal scale, per tensor or per token position.
//
// Stands in for torch_npu.npu_quantize(..., div_mode=False) as the deploy module
// calls it (amct_pytorch/deploy_op/npu_quantization_linear.py:98-99); scale and
// offset arrive already rounded to the activation dtype (:42-45).  The
// SmoothQuant multiply (:96-97) is folded into the load, with the intermediate
// rounding to the activation dtype the two-step reference has.
//
// Elementwise and HBM-bound: sizeof(T) bytes read + 1 byte written per element.
#include "common.cuh"

namespace amct {

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) quantize_static_kernel(const T* x, int64_t nrows, int64_t tokens, int64_t k,
                                                              const T* scale, const T* offset, int per_token,
                                                              const T* smooth, int8_t* q) {
  constexpr int E = VEC ? ElemTraits<T>::kPerVec : 1;
  constexpr int U = 4;                                   // vectors in flight per thread
  const int64_t vec_per_row = k / E;
  const int64_t total = nrows * vec_per_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
    float f[U][E];
    int64_t row[U], j0[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        row[u] = i / vec_per_row;
        j0[u] = (i - row[u] * vec_per_row) * E;
        if constexpr (VEC) {
          Vec16<T> raw = ld_vec_stream(x + row[u] * k + j0[u]);
#pragma unroll
          for (int e = 0; e < E; ++e) f[u][e] = ElemTraits<T>::to_f(raw.v[e]);
        } else {
          f[u][0] = ElemTraits<T>::to_f(x[row[u] * k + j0[u]]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= total) break;
      const int64_t t = per_token ? row[u] % tokens : 0;
      const float s = ElemTraits<T>::to_f(scale[t]);
      const float z = offset ? ElemTraits<T>::to_f(offset[t]) : 0.f;
      int8_t out[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        float a = f[u][e];
        if (smooth) a = round_to<T>(__fmul_rn(a, ElemTraits<T>::to_f(smooth[j0[u] + e])));
        float y = __fmul_rn(a, s);
        if (offset) y = __fadd_rn(y, z);
        // round half to even and saturate: clamp first, then add 1.5 * 2^23 (the low byte is the code)
        y = fminf(fmaxf(y, -128.f), 127.f);
        out[e] = (int8_t)(__float_as_uint(__fadd_rn(y, 12582912.0f)) & 0xFF);
      }
      int8_t* dst = q + row[u] * k + j0[u];
      if constexpr (E == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(out);
      else if constexpr (E == 4) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<uint32_t*>(out);
      else dst[0] = out[0];
    }
  }
}

template <typename T>
static int run_static(const T* x, int64_t outer, int64_t tokens, int64_t k, const T* scale, const T* offset,
                      int per_token, const T* smooth, int8_t* q, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  const int64_t nrows = outer * tokens;
  const bool vec = aligned16(x) && k % E == 0 && (reinterpret_cast<uintptr_t>(q) % E == 0);
  const int64_t work = nrows * (vec ? k / E : k);
  int64_t blocks = (work + 256 * 4 - 1) / (256 * 4);
  if (blocks < 1) blocks = 1;
  const int64_t cap = 148LL * 8 * 2;
  if (blocks > cap) blocks = cap;
  if (vec) quantize_static_kernel<T, true><<<(unsigned)blocks, 256, 0, st>>>(x, nrows, tokens, k, scale, offset, per_token, smooth, q);
  else quantize_static_kernel<T, false><<<(unsigned)blocks, 256, 0, st>>>(x, nrows, tokens, k, scale, offset, per_token, smooth, q);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

extern "C" int amct_quantize_static(const void* x, int dtype, int64_t outer, int64_t tokens, int64_t k,
                                    const void* scale, const void* offset, int per_token, const void* smooth,
                                    int8_t* q, void* stream) {
  if (outer < 0 || tokens < 0 || k < 0 || !scale) return AMCT_ERR_ARG;
  if (outer == 0 || tokens == 0 || k == 0) return AMCT_OK;
  if (!x || !q) return AMCT_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case AMCT_DTYPE_F32:
      return amct::run_static<float>((const float*)x, outer, tokens, k, (const float*)scale, (const float*)offset, per_token,
                                     (const float*)smooth, q, st);
    case AMCT_DTYPE_F16:
      return amct::run_static<__half>((const __half*)x, outer, tokens, k, (const __half*)scale, (const __half*)offset, per_token,
                                      (const __half*)smooth, q, st);
    case AMCT_DTYPE_BF16:
      return amct::run_static<__nv_bfloat16>((const __nv_bfloat16*)x, outer, tokens, k, (const __nv_bfloat16*)scale,
                                             (const __nv_bfloat16*)offset, per_token, (const __nv_bfloat16*)smooth, q, st);
  }
  return AMCT_ERR_ARG;
}
