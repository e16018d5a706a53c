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

template <typename T, int BITS>
__global__ void __launch_bounds__(256) dequant_weight_kernel(const uint8_t* codes, int64_t n_rows, int64_t k, int64_t ld_codes,
                                                             const T* scale, const T* offset, int group, T* out, int64_t ld_out) {
  const int64_t chunks = k / 8;
  const int64_t total = n_rows * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / chunks, c = i - n * chunks;
    const int64_t k0 = c * 8;
    int q[8];
    if (BITS == 8) {
      uint2 raw = *reinterpret_cast<const uint2*>(codes + n * ld_codes + k0);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        q[e] = (int)(int8_t)(raw.x >> (8 * e));
        q[4 + e] = (int)(int8_t)(raw.y >> (8 * e));
      }
    } else {
      uint32_t raw = *reinterpret_cast<const uint32_t*>(codes + n * ld_codes + k0 / 2);
#pragma unroll
      for (int e = 0; e < 8; ++e) q[e] = (int)((raw >> (4 * e)) & 0xF) - 8;
    }
    const int64_t g = group ? k0 / group : 0;
    const float s = ElemTraits<T>::to_f(scale[g * n_rows + n]);
    const float o = offset ? ElemTraits<T>::to_f(offset[g * n_rows + n]) : 0.f;
    Vec16<T> r;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = (float)q[e];
      if (offset) v = __fadd_rn(v, o);
      r.v[e] = ElemTraits<T>::from_f(__fmul_rn(v, s));
    }
    *reinterpret_cast<uint4*>(out + n * ld_out + k0) = *reinterpret_cast<uint4*>(&r);
  }
}

template <typename T>
static int run_dequant(const uint8_t* codes, int bits, int64_t n_rows, int64_t k, int64_t ld_codes, const T* scale,
                       const T* offset, int group, T* out, int64_t ld_out, cudaStream_t st) {
  const int64_t total = n_rows * (k / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (bits == 8) dequant_weight_kernel<T, 8><<<(unsigned)blocks, 256, 0, st>>>(codes, n_rows, k, ld_codes, scale, offset, group, out, ld_out);
  else dequant_weight_kernel<T, 4><<<(unsigned)blocks, 256, 0, st>>>(codes, n_rows, k, ld_codes, scale, offset, group, out, ld_out);
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
