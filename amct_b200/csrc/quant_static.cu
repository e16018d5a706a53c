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

// Row-tiled variant for wide rows: blockIdx.x picks the column span, blockIdx.y strides over
// rows, four rows in flight per thread; no per-element index division.
template <typename T>
__global__ void __launch_bounds__(256) quantize_static_rows_kernel(const T* x, int nrows, int tokens, int k, const T* scale,
                                                                   const T* offset, int per_token, const T* smooth, int8_t* q) {
  constexpr int E = ElemTraits<T>::kPerVec;
  constexpr int U = 4;
  const int vec = blockIdx.x * blockDim.x + threadIdx.x;
  if (vec >= k / E) return;
  const int j0 = vec * E;
  float sm[E];
  if (smooth) {
    Vec16<T> raw = ld_vec(smooth + j0);
#pragma unroll
    for (int e = 0; e < E; ++e) sm[e] = ElemTraits<T>::to_f(raw.v[e]);
  }
  const float s0 = ElemTraits<T>::to_f(scale[0]);
  const float z0 = offset ? ElemTraits<T>::to_f(offset[0]) : 0.f;
  for (int r0 = blockIdx.y * U; r0 < nrows; r0 += gridDim.y * U) {
    Vec16<T> raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (r0 + u < nrows) raw[u] = ld_vec_stream(x + (int64_t)(r0 + u) * k + j0);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int row = r0 + u;
      if (row >= nrows) break;
      float s = s0, z = z0;
      if (per_token) {
        const int t = (int)((uint32_t)row % (uint32_t)tokens);
        s = ElemTraits<T>::to_f(scale[t]);
        if (offset) z = ElemTraits<T>::to_f(offset[t]);
      }
      uint32_t w[E / 4];
#pragma unroll
      for (int g = 0; g < E / 4; ++g) {
        float r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float a = ElemTraits<T>::to_f(raw[u].v[4 * g + e]);
          if (smooth) a = round_to<T>(__fmul_rn(a, sm[4 * g + e]));
          float y = __fmul_rn(a, s);
          if (offset) y = __fadd_rn(y, z);
          r[e] = __fadd_rn(fminf(fmaxf(y, -128.f), 127.f), 12582912.0f);   // low byte = round-half-even code
        }
        const uint32_t w01 = __byte_perm(__float_as_uint(r[0]), __float_as_uint(r[1]), 0x0040);
        const uint32_t w23 = __byte_perm(__float_as_uint(r[2]), __float_as_uint(r[3]), 0x0040);
        w[g] = __byte_perm(w01, w23, 0x5410);
      }
      int8_t* dst = q + (int64_t)row * k + j0;
      if constexpr (E == 8) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
      else *reinterpret_cast<uint32_t*>(dst) = w[0];
    }
  }
}

template <typename T>
static int run_static(const T* x, int64_t outer, int64_t tokens, int64_t k, const T* scale, const T* offset,
                      int per_token, const T* smooth, int8_t* q, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  const int64_t nrows = outer * tokens;
  const bool vec = aligned16(x) && k % E == 0 && (reinterpret_cast<uintptr_t>(q) % E == 0);
  if (vec && k >= 1024 && nrows < (1LL << 30) && k < (1LL << 30) && tokens < (1LL << 30) && (!smooth || aligned16(smooth))) {
    dim3 grid((unsigned)((k / E + 255) / 256), 1);
    int64_t gy = (148LL * 8 + grid.x - 1) / grid.x;
    const int64_t need = (nrows + 3) / 4;
    if (gy > need) gy = need;
    grid.y = (unsigned)(gy < 1 ? 1 : gy);
    AMCT_LAUNCH(grid, 256, st, (x, (int)nrows, (int)tokens, (int)k, scale, offset, per_token, smooth, q), quantize_static_rows_kernel<T>);
    AMCT_CHECK_LAUNCH();
    return AMCT_OK;
  }
  const int64_t work = nrows * (vec ? k / E : k);
  int64_t blocks = (work + 256 * 4 - 1) / (256 * 4);
  if (blocks < 1) blocks = 1;
  const int64_t cap = 148LL * 8 * 2;
  if (blocks > cap) blocks = cap;
  if (vec) AMCT_LAUNCH((unsigned)blocks, 256, st, (x, nrows, tokens, k, scale, offset, per_token, smooth, q), quantize_static_kernel<T, true>);
  else AMCT_LAUNCH((unsigned)blocks, 256, st, (x, nrows, tokens, k, scale, offset, per_token, smooth, q), quantize_static_kernel<T, false>);
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
