// GPTQ: the column-by-column update of one block of (up to 128) columns in ONE kernel.
//
// amct_pytorch/quantize_op/gptq_module.py:128-153 walks the columns of a block on the host: quantize-dequantize
// column i (quant_dequant_weight, amct_pytorch/utils/quant_util.py:162-188), err = (w - w_q) / Hinv[i, i], then
// W[:, i:] -= err (x) Hinv[i, i:] -- five small launches per column, 128 times per block.  The rows of W never
// interact inside a block, so here one WARP owns a row: lane l holds columns l, l + 32, l + 64, l + 96 of the block
// in registers, column i's value is broadcast from its owner with a shuffle, every lane computes the quantized
// value and the error (fp32, the reference's operation order: w / s, + offset, rint, clamp, - offset, * s) and
// updates the columns it holds.  The block's corner of the inverse Hessian factor (64 KB at most) is read through L1.  What is
// left for the host per block is the trailing update W[:, i2:] -= Err @ Hinv[i1:i2, i2:], one GEMM.
//
// Each column takes its quant factors from the group of its ORIGINAL column index (the columns are permuted by
// decreasing Hessian diagonal): col_group[i] is that group for block column i.
#include "common.cuh"

namespace amct {

constexpr int kGptqMaxBlock = 128;
constexpr int kGptqWarps = 4;

struct GptqParams {
  float* w;                  // [n, ldw]: the block's columns, updated in place
  float* err;                // [n, lde]: err[:, i] = (w_i - q_i) / hinv[i, i]
  const float* hinv;         // [b, ldh]: upper-triangular factor of the inverse Hessian, the block's corner
  const float* scale;        // [n or 1, factors_ld]
  const int* offset;         // same layout or null
  const int* col_group;      // [b]: column of scale / offset that block column i uses
  int64_t n, ldw, lde, ldh, factors_ld;
  int b, bits, row_factors;  // row_factors: 1 = one row of factors per weight row, 0 = the same factors for every row
};

__global__ void __launch_bounds__(kGptqWarps * 32) gptq_block_kernel(GptqParams p) {
  __shared__ int grp[kGptqMaxBlock];
  for (int i = threadIdx.x; i < p.b; i += blockDim.x) grp[i] = p.col_group[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float qmax = (float)((1 << (p.bits - 1)) - 1), qmin = -qmax - 1.f;
  for (int64_t row = (int64_t)blockIdx.x * kGptqWarps + warp; row < p.n; row += (int64_t)gridDim.x * kGptqWarps) {
    float* wr = p.w + row * p.ldw;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (lane + 32 * j) < p.b ? wr[lane + 32 * j] : 0.f;
    const float* srow = p.scale + (p.row_factors ? row * p.factors_ld : 0);
    const int* orow = p.offset ? p.offset + (p.row_factors ? row * p.factors_ld : 0) : nullptr;
    for (int i = 0; i < p.b; ++i) {
      // column i lives in slot i / 32 of lane i % 32
      float mine = v[0];
      if ((i >> 5) == 1) mine = v[1];
      else if ((i >> 5) == 2) mine = v[2];
      else if ((i >> 5) == 3) mine = v[3];
      const float w = __shfl_sync(0xffffffffu, mine, i & 31);
      const float s = srow[grp[i]];
      float t = __fdiv_rn(w, s);
      float o = 0.f;
      if (orow) { o = (float)orow[grp[i]]; t = __fadd_rn(t, o); }
      t = fminf(fmaxf(rintf(t), qmin), qmax);
      if (orow) t = __fsub_rn(t, o);
      const float q = __fmul_rn(t, s);
      const float* hrow = p.hinv + (int64_t)i * p.ldh;         // 64 KB at most for the block: stays in L1
      const float e = __fdiv_rn(__fsub_rn(w, q), __ldg(hrow + i));
      if (lane == 0) p.err[row * p.lde + i] = e;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = lane + 32 * j;
        if (c >= i && c < p.b) v[j] = __fsub_rn(v[j], __fmul_rn(e, __ldg(hrow + c)));
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if ((lane + 32 * j) < p.b) wr[lane + 32 * j] = v[j];
    }
  }
}

}  // namespace amct

extern "C" int amct_gptq_block(float* w, int64_t n, int64_t ldw, int b, const float* hinv, int64_t ldh, const float* scale,
                               const int* offset, int64_t factors_ld, int row_factors, const int* col_group, int bits,
                               float* err, int64_t lde, void* stream) {
  if (n < 0 || b < 1 || b > amct::kGptqMaxBlock || ldw < b || ldh < b || lde < b || (bits != 4 && bits != 8)) return AMCT_ERR_ARG;
  if (n == 0) return AMCT_OK;
  if (!w || !hinv || !scale || !col_group || !err || factors_ld < 1) return AMCT_ERR_ARG;
  amct::GptqParams p{};
  p.w = w; p.err = err; p.hinv = hinv; p.scale = scale; p.offset = offset; p.col_group = col_group;
  p.n = n; p.ldw = ldw; p.lde = lde; p.ldh = ldh; p.factors_ld = factors_ld; p.b = b; p.bits = bits; p.row_factors = row_factors;
  int64_t blocks = (n + amct::kGptqWarps - 1) / amct::kGptqWarps;
  if (blocks > 148 * 8) blocks = 148 * 8;
  AMCT_LAUNCH((unsigned)blocks, amct::kGptqWarps * 32, (cudaStream_t)stream, (p), amct::gptq_block_kernel);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}
