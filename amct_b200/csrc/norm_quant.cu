// Residual add + RMSNorm + dynamic per-token symmetric INT8 quantization in one pass.
//
// The decoder-layer sequence  h = x + residual;  n = rms_norm(h) * gamma;  q, scale = quant(n)
// reads and writes the hidden state three times when it runs as three kernels.  Here one CTA
// keeps a token row in registers from the add to the codes: x and the residual are read once,
// the new residual and the codes are written once.
//
// The quantizer is the dynamic per-token rule of the deploy Linear (row amax / amin as in
// amct_pytorch/quantize_op/minmax_module.py:99-105, scale rule of
// amct_pytorch/quantize_op/utils.py:75-108, codes of amct_pytorch/utils/quant_util.py:57-73)
// applied to the normalised values after they have been rounded to the tensor dtype, i.e. the
// codes are those the separate quant kernel produces from `norm_out`.  The add rounds once to
// the tensor dtype like a torch add.  The norm is evaluated in fp32:
// rstd = rn(1 / sqrt(mean(h^2) + eps)), n = round_T((h * rstd) * gamma); the order of the fp32
// sum of squares is this kernel's own (torch's differs), so n may differ from torch's
// rms_norm by one unit in the last place of T on a few elements.
//
// Algorithmic HBM traffic per row: 2 K sizeof(T) read (K sizeof(T) without residual),
// K sizeof(T) + K + 4 written (K + 4 without residual output).
#include "common.cuh"

namespace amct {

constexpr float kMagicNQ = 12582912.0f;                  // 1.5 * 2^23
constexpr int kMaxNormRanks = 16;

struct NormQuantParams {
  const void* x;
  const void* residual;       // nullable
  const void* gamma;          // [k]
  void* residual_out;         // nullable
  void* norm_out;             // nullable
  int8_t* q;
  float* scale;
  int* status;
  int64_t rows, k, ld_x, ld_res, ld_res_out, ld_norm, ld_q;
  float eps;
  // Tensor-parallel form (TP kernels only).  Input: x holds `parts` partial sums of this rank's rows, one after the
  // other (part j at x + j * part_stride elements); the row is their fp32 sum in that order, rounded once to T.
  // Output: the codes and the scale of row r go to row (row0 + r) of EVERY rank's buffers, q_all[d] / scale_all[d]
  // (this process's mappings of them), so that each rank ends up with all ranks' rows; q / scale are not used.
  int parts, world, first_dst;
  int64_t part_stride, row0;
  int8_t* q_all[kMaxNormRanks];
  float* scale_all[kMaxNormRanks];
};

__device__ __forceinline__ uint32_t nq_pack4(float ra, float rb, float rc, float rd) {
  const uint32_t w01 = __byte_perm(__float_as_uint(ra), __float_as_uint(rb), 0x0040);
  const uint32_t w23 = __byte_perm(__float_as_uint(rc), __float_as_uint(rd), 0x0040);
  return __byte_perm(w01, w23, 0x5410);
}

// four quotients by the exact FMA sequence (div_by_recip: the value of the IEEE division), the
// upper clamp a negative-dominant row needs, round half to even by the magic add
__device__ __forceinline__ uint32_t nq_quant4(float a, float b, float c, float d, float s, float y) {
  const float ta = fminf(div_by_recip(a, s, y), 127.f), tb = fminf(div_by_recip(b, s, y), 127.f);
  const float tc = fminf(div_by_recip(c, s, y), 127.f), td = fminf(div_by_recip(d, s, y), 127.f);
  return nq_pack4(__fadd_rn(ta, kMagicNQ), __fadd_rn(tb, kMagicNQ), __fadd_rn(tc, kMagicNQ), __fadd_rn(td, kMagicNQ));
}

// block-wide sum; the caller alternates `part` between rows so one barrier per reduction is enough
template <int NW>
__device__ __forceinline__ float block_sum(float v, float* part, int warp, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (lane == 0) part[warp] = v;
  __syncthreads();
  float t = part[0];
#pragma unroll
  for (int w = 1; w < NW; ++w) t = __fadd_rn(t, part[w]);
  return t;
}

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  __device__ static type from_floats(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <> struct Pack2<__half> {
  using type = __half2;
  __device__ static type from_floats(float a, float b) { return __floats2half2_rn(a, b); }
};

// 16-bit T only; NV 16-byte vectors (8 elements each) per thread, NT threads per row.  Values stay
// packed two to a register wherever the arithmetic allows: the residual add is the packed add (the
// exact sum of two 16-bit floats rounded once, which is what an fp32 add followed by the rounding to
// T gives as well), min / max use the packed NaN-propagating instructions, conversions go pairwise.
template <typename T, int NV, int NT, bool TP = false>
__global__ void __launch_bounds__(NT) addnorm_quant_kernel(NormQuantParams p) {
  constexpr int E = 8;
  constexpr int NW = NT / 32;
  using P2 = typename Pack2<T>::type;
  __shared__ float part_sum[2][NW];
  __shared__ float part_mx[2][NW], part_mn[2][NW];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nvec = (int)(p.k / E);
  const T* gamma = reinterpret_cast<const T*>(p.gamma);
  int it = 0;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x, it ^= 1) {
    const T* xr = reinterpret_cast<const T*>(p.x) + row * p.ld_x;
    Vec16<T> h[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = tid + j * NT;
      if (v < nvec) h[j] = ld_vec_stream(xr + v * E);
    }
    if constexpr (TP) {
      // sum of the ranks' partial sums: fp32, in rank order, rounded to T once
      if (p.parts > 1) {
        float acc[NV][E];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const P2* hp = reinterpret_cast<const P2*>(&h[j]);
#pragma unroll
          for (int e = 0; e < E / 2; ++e) { acc[j][2 * e] = __low2float(hp[e]); acc[j][2 * e + 1] = __high2float(hp[e]); }
        }
        for (int part = 1; part < p.parts; ++part) {
          const T* pr = xr + (int64_t)part * p.part_stride;
          Vec16<T> t[NV];
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            const int v = tid + j * NT;
            if (v < nvec) t[j] = ld_vec_stream(pr + v * E);
          }
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            const P2* tp = reinterpret_cast<const P2*>(&t[j]);
#pragma unroll
            for (int e = 0; e < E / 2; ++e) {
              acc[j][2 * e] = __fadd_rn(acc[j][2 * e], __low2float(tp[e]));
              acc[j][2 * e + 1] = __fadd_rn(acc[j][2 * e + 1], __high2float(tp[e]));
            }
          }
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          P2* hp = reinterpret_cast<P2*>(&h[j]);
#pragma unroll
          for (int e = 0; e < E / 2; ++e) hp[e] = Pack2<T>::from_floats(acc[j][2 * e], acc[j][2 * e + 1]);
        }
      }
    }
    if (p.residual) {
      const T* rr = reinterpret_cast<const T*>(p.residual) + row * p.ld_res;
      Vec16<T> r[NV];
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = tid + j * NT;
        if (v < nvec) r[j] = ld_vec_stream(rr + v * E);
      }
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = tid + j * NT;
        if (v < nvec) {
          P2* hp = reinterpret_cast<P2*>(&h[j]);
          const P2* rp = reinterpret_cast<const P2*>(&r[j]);
#pragma unroll
          for (int e = 0; e < E / 2; ++e) hp[e] = __hadd2(hp[e], rp[e]);
          if (p.residual_out)
            *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.residual_out) + row * p.ld_res_out + v * E) =
                *reinterpret_cast<const uint4*>(&h[j]);
        }
      }
    }
    // ---- mean of squares (fp32); the unpacked values are kept for the normalisation
    float f[NV][E];
    float ssq = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (tid + j * NT < nvec) {
        const P2* hp = reinterpret_cast<const P2*>(&h[j]);
#pragma unroll
        for (int e = 0; e < E / 2; ++e) {
          f[j][2 * e] = __low2float(hp[e]);
          f[j][2 * e + 1] = __high2float(hp[e]);
          ssq = __fmaf_rn(f[j][2 * e], f[j][2 * e], ssq);
          ssq = __fmaf_rn(f[j][2 * e + 1], f[j][2 * e + 1], ssq);
        }
      }
    }
    const float total = block_sum<NW>(ssq, part_sum[it], warp, lane);
    const float rstd = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)p.k), p.eps));
    // ---- normalise, round to T (pairwise), packed min / max
    P2 vmx = Pack2<T>::from_floats(-INFINITY, -INFINITY), vmn = Pack2<T>::from_floats(INFINITY, INFINITY);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = tid + j * NT;
      if (v < nvec) {
        const Vec16<T> g = ld_vec(gamma + v * E);
        const P2* gp = reinterpret_cast<const P2*>(&g);
        P2* hp = reinterpret_cast<P2*>(&h[j]);
#pragma unroll
        for (int e = 0; e < E / 2; ++e) {
          hp[e] = Pack2<T>::from_floats(__fmul_rn(__fmul_rn(f[j][2 * e], rstd), __low2float(gp[e])),
                                        __fmul_rn(__fmul_rn(f[j][2 * e + 1], rstd), __high2float(gp[e])));
          vmx = __hmax2_nan(vmx, hp[e]);
          vmn = __hmin2_nan(vmn, hp[e]);
        }
        if (p.norm_out)
          *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.norm_out) + row * p.ld_norm + v * E) = *reinterpret_cast<const uint4*>(&h[j]);
      }
    }
    float mx, mn;
    {
      const float a0 = __low2float(vmx), a1 = __high2float(vmx), b0 = __low2float(vmn), b1 = __high2float(vmn);
      // a NaN in the row: infinite scale, row flagged
      if (a0 != a0 || a1 != a1 || b0 != b0 || b1 != b1) { mx = INFINITY; mn = 0.f; }
      else { mx = fmaxf(a0, a1); mn = fminf(b0, b1); }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    if (lane == 0) { part_mx[it][warp] = mx; part_mn[it][warp] = mn; }
    __syncthreads();
    mx = part_mx[it][0]; mn = part_mn[it][0];
#pragma unroll
    for (int w = 1; w < NW; ++w) { mx = fmaxf(mx, part_mx[it][w]); mn = fminf(mn, part_mn[it][w]); }
    // symmetric INT8 rule: divisor 127, or 128 when the largest magnitude is negative
    const float amx = fabsf(mx), amn = fabsf(mn);
    const bool neg_dom = amx < amn;
    float s = __fdiv_rn(neg_dom ? amn : amx, neg_dom ? 128.f : 127.f);
    if (s < AMCT_FLT_EPSILON) s = 1.f;
    if constexpr (TP) {
      if (tid < p.world) p.scale_all[tid][p.row0 + row] = s;
      if (tid == 0 && !isfinite(s) && p.status) atomicOr(p.status, 1);
    } else {
      if (tid == 0) {
        p.scale[row] = s;
        if (!isfinite(s) && p.status) atomicOr(p.status, 1);
      }
    }
    const float y = __frcp_rn(s);
    int8_t* qrow = TP ? nullptr : p.q + row * p.ld_q;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = tid + j * NT;
      if (v < nvec) {
        const P2* hp = reinterpret_cast<const P2*>(&h[j]);
        const uint32_t w0 = nq_quant4(__low2float(hp[0]), __high2float(hp[0]), __low2float(hp[1]), __high2float(hp[1]), s, y);
        const uint32_t w1 = nq_quant4(__low2float(hp[2]), __high2float(hp[2]), __low2float(hp[3]), __high2float(hp[3]), s, y);
        if constexpr (TP) {
          // a warp writes 256 contiguous bytes per destination: plain stores into every rank's (peer-mapped) buffer
          const int64_t off = (p.row0 + row) * p.ld_q + v * E;
          for (int i = 0; i < p.world; ++i) {
            int d = p.first_dst + i;                          // every rank starts with another destination
            if (d >= p.world) d -= p.world;
            *reinterpret_cast<uint2*>(p.q_all[d] + off) = make_uint2(w0, w1);
          }
        } else {
          *reinterpret_cast<uint2*>(qrow + v * E) = make_uint2(w0, w1);
        }
      }
    }
  }
}

template <typename T, bool TP = false>
static int launch_norm_quant(const NormQuantParams& p, cudaStream_t st) {
  const int64_t nvec = p.k / 8;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // two vectors per thread keep the row within 64 registers, so 1024 threads stay resident per SM
  int64_t grid = (int64_t)sms * 8;
  if (grid > p.rows) grid = p.rows;
  const unsigned g = (unsigned)grid;
  if (nvec <= 128) AMCT_LAUNCH(g, 128, st, (p), addnorm_quant_kernel<T, 1, 128, TP>);
  else if (nvec <= 256) AMCT_LAUNCH(g, 256, st, (p), addnorm_quant_kernel<T, 1, 256, TP>);
  else if (nvec <= 512) AMCT_LAUNCH(g, 256, st, (p), addnorm_quant_kernel<T, 2, 256, TP>);
  else if (nvec <= 1024) AMCT_LAUNCH(g, 512, st, (p), addnorm_quant_kernel<T, 2, 512, TP>);
  else if (nvec <= 2048) AMCT_LAUNCH(g, 512, st, (p), addnorm_quant_kernel<T, 4, 512, TP>);
  else return AMCT_ERR_UNSUPPORTED;
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

extern "C" int amct_addnorm_quant_pertoken(const void* x, const void* residual, int dtype, int64_t rows, int64_t k,
                                           int64_t ld_x, int64_t ld_res, const void* gamma, float eps,
                                           void* residual_out, int64_t ld_res_out, void* norm_out, int64_t ld_norm,
                                           int8_t* q, int64_t ld_q, float* scale, int* status, void* stream) {
  if (rows < 0 || k <= 0 || !gamma) return AMCT_ERR_ARG;
  if (rows == 0) return AMCT_OK;
  if (!x || !q || !scale) return AMCT_ERR_ARG;
  if (dtype != AMCT_DTYPE_F16 && dtype != AMCT_DTYPE_BF16) return AMCT_ERR_UNSUPPORTED;
  if (k % 8 || k > 2048 * 8) return AMCT_ERR_UNSUPPORTED;
  if (ld_x < k || ld_q < k || (residual && ld_res < k) || (residual_out && ld_res_out < k) || (norm_out && ld_norm < k))
    return AMCT_ERR_ARG;
  if (residual_out && !residual) return AMCT_ERR_ARG;
  auto ok16 = [](const void* ptr, int64_t ld_elems) { return amct::aligned16(ptr) && (ld_elems * 2) % 16 == 0; };
  if (!ok16(x, ld_x) || !amct::aligned16(gamma) || (residual && !ok16(residual, ld_res)) ||
      (residual_out && !ok16(residual_out, ld_res_out)) || (norm_out && !ok16(norm_out, ld_norm)) ||
      reinterpret_cast<uintptr_t>(q) % 8 || ld_q % 8)
    return AMCT_ERR_ALIGN;
  amct::NormQuantParams p{};
  p.x = x; p.residual = residual; p.gamma = gamma; p.residual_out = residual_out; p.norm_out = norm_out;
  p.q = q; p.scale = scale; p.status = status;
  p.rows = rows; p.k = k; p.ld_x = ld_x; p.ld_res = ld_res; p.ld_res_out = ld_res_out; p.ld_norm = ld_norm; p.ld_q = ld_q;
  p.eps = eps;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == AMCT_DTYPE_F16) return amct::launch_norm_quant<__half>(p, st);
  return amct::launch_norm_quant<__nv_bfloat16>(p, st);
}

extern "C" int amct_addnorm_quant_pertoken_tp(const void* parts, int n_parts, int64_t part_stride, const void* residual,
                                              int dtype, int64_t rows, int64_t k, int64_t ld_x, int64_t ld_res,
                                              const void* gamma, float eps, void* residual_out, int64_t ld_res_out,
                                              int8_t* const* q_all, float* const* scale_all, int world, int64_t row0,
                                              int64_t ld_q, int* status, void* stream) {
  if (rows < 0 || k <= 0 || !gamma || row0 < 0) return AMCT_ERR_ARG;
  if (n_parts < 1 || n_parts > amct::kMaxNormRanks || world < 1 || world > amct::kMaxNormRanks || !q_all || !scale_all)
    return AMCT_ERR_ARG;
  if (rows == 0) return AMCT_OK;
  if (!parts) return AMCT_ERR_ARG;
  if (dtype != AMCT_DTYPE_F16 && dtype != AMCT_DTYPE_BF16) return AMCT_ERR_UNSUPPORTED;
  if (k % 8 || k > 2048 * 8) return AMCT_ERR_UNSUPPORTED;
  if (ld_x < k || ld_q < k || (residual && ld_res < k) || (residual_out && ld_res_out < k)) return AMCT_ERR_ARG;
  if (residual_out && !residual) return AMCT_ERR_ARG;
  if (n_parts > 1 && part_stride < rows * ld_x) return AMCT_ERR_ARG;
  auto ok16 = [](const void* ptr, int64_t ld_elems) { return amct::aligned16(ptr) && (ld_elems * 2) % 16 == 0; };
  if (!ok16(parts, ld_x) || (part_stride * 2) % 16 || !amct::aligned16(gamma) || (residual && !ok16(residual, ld_res)) ||
      (residual_out && !ok16(residual_out, ld_res_out)) || ld_q % 8)
    return AMCT_ERR_ALIGN;
  amct::NormQuantParams p{};
  p.x = parts; p.residual = residual; p.gamma = gamma; p.residual_out = residual_out; p.status = status;
  p.rows = rows; p.k = k; p.ld_x = ld_x; p.ld_res = ld_res; p.ld_res_out = ld_res_out; p.ld_q = ld_q; p.eps = eps;
  p.parts = n_parts; p.part_stride = part_stride; p.world = world; p.row0 = row0;
  p.first_dst = (int)((row0 / rows + 1) % world);                 // row0 = rank * rows in the sharded workload
  for (int d = 0; d < world; ++d) {
    if (!q_all[d] || !scale_all[d]) return AMCT_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(q_all[d]) % 8) return AMCT_ERR_ALIGN;
    p.q_all[d] = q_all[d];
    p.scale_all[d] = scale_all[d];
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == AMCT_DTYPE_F16) return amct::launch_norm_quant<__half, true>(p, st);
  return amct::launch_norm_quant<__nv_bfloat16, true>(p, st);
}
