// Weight-only quantized Linear: dequantization of INT8 / packed INT4 weight codes.
//
//   w[n, k] = (q[n, k] + aoff[g(k), n]) * ascale[g(k), n]      rounded to the activation dtype
//
// which is the operand torch_npu.npu_weight_quant_batchmatmul multiplies the
// activations with (call site amct_pytorch/deploy_op/weight_npu_quant_module.py:116-117;
// ascale / aoff = scale_w and the negated offset_w buffers built at :59-64, laid
// out [K/group, N], or [1, N] when group == 0).  The result feeds the fp16/bf16
// tensor-core GEMM.  Codes are K-major: int8 [N, K] or two nibbles per byte
// [N, K/2] (code + 8, even k in the low nibble).
//
// HBM traffic per element: 1 or 0.5 byte read + 2 bytes written.
#include "common.cuh"

namespace amct {

// grid.x covers the 8-element chunks of a row, grid.y strides over rows (two in flight).
template <typename T, int BITS>
__global__ void __launch_bounds__(256) dequant_weight_kernel(const uint8_t* codes, int n_rows, int k, int64_t ld_codes,
                                                             const T* scale, const T* offset, int group, T* out, int64_t ld_out) {
  constexpr int U = 2;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= k / 8) return;
  const int k0 = c * 8;
  const int g = group ? k0 / group : 0;
  for (int n0 = blockIdx.y * U; n0 < n_rows; n0 += gridDim.y * U) {
    uint2 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (n0 + u < n_rows) {
        if (BITS == 8) raw[u] = __ldcs(reinterpret_cast<const uint2*>(codes + (int64_t)(n0 + u) * ld_codes + k0));
        else raw[u] = make_uint2(__ldcs(reinterpret_cast<const uint32_t*>(codes + (int64_t)(n0 + u) * ld_codes + k0 / 2)), 0u);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int n = n0 + u;
      if (n >= n_rows) break;
      int q[8];
      if (BITS == 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          q[e] = (int)(int8_t)(raw[u].x >> (8 * e));
          q[4 + e] = (int)(int8_t)(raw[u].y >> (8 * e));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) q[e] = (int)((raw[u].x >> (4 * e)) & 0xF) - 8;
      }
      const float s = ElemTraits<T>::to_f(scale[(int64_t)g * n_rows + n]);
      const float o = offset ? ElemTraits<T>::to_f(offset[(int64_t)g * n_rows + n]) : 0.f;
      Vec16<T> r;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float v = (float)q[e];
        if (offset) v = __fadd_rn(v, o);
        r.v[e] = ElemTraits<T>::from_f(__fmul_rn(v, s));
      }
      *reinterpret_cast<uint4*>(out + (int64_t)n * ld_out + k0) = *reinterpret_cast<uint4*>(&r);
    }
  }
}

template <typename T>
static int run_dequant(const uint8_t* codes, int bits, int64_t n_rows, int64_t k, int64_t ld_codes, const T* scale,
                       const T* offset, int group, T* out, int64_t ld_out, cudaStream_t st) {
  if (n_rows >= (1LL << 30) || k >= (1LL << 30)) return AMCT_ERR_UNSUPPORTED;
  dim3 grid((unsigned)((k / 8 + 255) / 256), 1);
  int64_t gy = (148LL * 8 + grid.x - 1) / grid.x;
  const int64_t need = (n_rows + 1) / 2;
  if (gy > need) gy = need;
  grid.y = (unsigned)(gy < 1 ? 1 : gy);
  if (bits == 8) AMCT_LAUNCH(grid, 256, st, (codes, (int)n_rows, (int)k, ld_codes, scale, offset, group, out, ld_out), dequant_weight_kernel<T, 8>);
  else AMCT_LAUNCH(grid, 256, st, (codes, (int)n_rows, (int)k, ld_codes, scale, offset, group, out, ld_out), dequant_weight_kernel<T, 4>);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

extern "C" int amct_dequant_weight(const void* codes, int bits, int64_t n_rows, int64_t k, int64_t ld_codes,
                                   const void* scale, const void* offset, int group, int dtype, void* out,
                                   int64_t ld_out, void* stream) {
  if (n_rows < 0 || k < 0 || (bits != 8 && bits != 4) || group < 0) return AMCT_ERR_ARG;
  if (n_rows == 0 || k == 0) return AMCT_OK;
  if (!codes || !scale || !out || ld_out < k || ld_codes < (bits == 8 ? k : k / 2)) return AMCT_ERR_ARG;
  if (k % 8 != 0 || (group && group % 8 != 0)) return AMCT_ERR_UNSUPPORTED;
  if (!amct::aligned16(out) || (ld_out * 2) % 16 != 0 || reinterpret_cast<uintptr_t>(codes) % 8 != 0 ||
      ld_codes % (bits == 8 ? 8 : 4) != 0)
    return AMCT_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const uint8_t* c = reinterpret_cast<const uint8_t*>(codes);
  if (dtype == AMCT_DTYPE_BF16)
    return amct::run_dequant<__nv_bfloat16>(c, bits, n_rows, k, ld_codes, (const __nv_bfloat16*)scale, (const __nv_bfloat16*)offset,
                                            group, (__nv_bfloat16*)out, ld_out, st);
  if (dtype == AMCT_DTYPE_F16)
    return amct::run_dequant<__half>(c, bits, n_rows, k, ld_codes, (const __half*)scale, (const __half*)offset, group,
                                     (__half*)out, ld_out, st);
  return AMCT_ERR_ARG;
}
