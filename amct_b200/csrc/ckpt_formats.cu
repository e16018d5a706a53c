// Offline checkpoint formats either side of the quantized Linear: what the reference's DeepSeek-V3.2 export
// script (amct_pytorch/experimental/quantization/DeepSeekV3.2/deploy.py, "deploy.py" below) does to every
// weight of a checkpoint on the CPU, as HBM-bound kernels.
//
//   * block dequant   E4M3 weight x one fp32 scale per 128 x 128 tile -> bf16          deploy.py:48-90
//   * row quant       symmetric per-output-channel INT8 / INT4 in the weight's own dtype, INT4 packed along
//                     the output-channel axis, with the fp32-in-uint64 scale and the "assistance bias"
//                     of the W4A8 grouped matmul                                           deploy.py:93-157
//   * Hadamard        Sylvester matrix with the reference's per-doubling rounded 1/sqrt(2)  deploy.py:32-45
//
// The reference computes on tensors of the checkpoint dtype T (bf16 in its main()), so every intermediate is
// one correctly rounded fp32 operation rounded again to T; the kernels keep that order so that codes, scales
// and biases are bit-identical.  This file is compiled without FMA contraction.
//
// Algorithmic HBM bytes per element: block dequant 1 read + sizeof(T) written; row quant sizeof(T) read
// (the second pass over the row hits L2) + 1 (INT8) or 0.5 (INT4) written.
#include "common.cuh"

#include <cuda_fp8.h>

namespace amct {

// ------------------------------------------------------------------------------------------------
// block dequant
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t two_bytes) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two_bytes & 0xffffu), __NV_E4M3);
  return __half22float2(__half2(h));
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}

// grid.x covers the 16-element vectors of a row, grid.y strides over rows
template <typename T>
__global__ void __launch_bounds__(128) ckpt_block_dequant_vec_kernel(
    const uint8_t* __restrict__ w, int64_t rows, int64_t vec_per_row, int64_t ld_w, const float* __restrict__ scale,
    int64_t ld_scale, int block, T* __restrict__ out, int64_t ld_out) {
  constexpr int E = ElemTraits<T>::kPerVec;
  const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= vec_per_row) return;
  const int64_t c0 = v * 16;
  const int64_t sc = c0 / block;
  constexpr int U = 4;                             // rows in flight per thread: 64 bytes of loads
  const int64_t step = gridDim.y;
  for (int64_t r0 = blockIdx.y; r0 < rows; r0 += step * U) {
    uint4 raw[U];
    float s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r = r0 + u * step;
      if (r < rows) {
        s[u] = __ldg(scale + (r / block) * ld_scale + sc);
        raw[u] = __ldcs(reinterpret_cast<const uint4*>(w + r * ld_w + c0));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r = r0 + u * step;
      if (r >= rows) break;
      const uint32_t word[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
      float f[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 lo = e4m3x2_to_float2(word[j]);
        const float2 hi = e4m3x2_to_float2(word[j] >> 16);
        f[4 * j + 0] = __fmul_rn(lo.x, s[u]);
        f[4 * j + 1] = __fmul_rn(lo.y, s[u]);
        f[4 * j + 2] = __fmul_rn(hi.x, s[u]);
        f[4 * j + 3] = __fmul_rn(hi.y, s[u]);
      }
      T* dst = out + r * ld_out + c0;
#pragma unroll
      for (int j = 0; j < 16 / E; ++j) {
        Vec16<T> o;
#pragma unroll
        for (int e = 0; e < E; ++e) o.v[e] = ElemTraits<T>::from_f(f[j * E + e]);
        __stcs(reinterpret_cast<uint4*>(dst + j * E), *reinterpret_cast<const uint4*>(&o));
      }
    }
  }
}

// any shape and alignment: one element per thread and row step
template <typename T>
__global__ void __launch_bounds__(128) ckpt_block_dequant_scalar_kernel(
    const uint8_t* __restrict__ w, int64_t rows, int64_t cols, int64_t ld_w, const float* __restrict__ scale,
    int64_t ld_scale, int block, T* __restrict__ out, int64_t ld_out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t sc = c / block;
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
    const float s = __ldg(scale + (r / block) * ld_scale + sc);
    out[r * ld_out + c] = ElemTraits<T>::from_f(__fmul_rn(e4m3_to_float(w[r * ld_w + c]), s));
  }
}

template <typename T>
static int launch_block_dequant(const uint8_t* w, int64_t rows, int64_t cols, int64_t ld_w, const float* scale,
                                int64_t ld_scale, int block, void* out, int64_t ld_out, cudaStream_t st) {
  T* o = reinterpret_cast<T*>(out);
  const bool vec = cols % 16 == 0 && block % 16 == 0 && ld_w % 16 == 0 && aligned16(w) && aligned16(out) &&
                   (ld_out * (int64_t)sizeof(T)) % 16 == 0;
  if (vec) {
    const int64_t quarter = (rows + 3) / 4;                       // the kernel keeps four rows in flight per thread
    const unsigned gy = (unsigned)(quarter < 16384 ? quarter : 16384);
    const int64_t vpr = cols / 16;
    dim3 grid((unsigned)((vpr + 127) / 128), gy);
    AMCT_LAUNCH(grid, 128, st, (w, rows, vpr, ld_w, scale, ld_scale, block, o, ld_out), ckpt_block_dequant_vec_kernel<T>);
  } else {
    const unsigned gy = (unsigned)(rows < 16384 ? rows : 16384);
    dim3 grid((unsigned)((cols + 127) / 128), gy);
    AMCT_LAUNCH(grid, 128, st, (w, rows, cols, ld_w, scale, ld_scale, block, o, ld_out), ckpt_block_dequant_scalar_kernel<T>);
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

// ------------------------------------------------------------------------------------------------
// row quant
// ------------------------------------------------------------------------------------------------
struct CkptRowParams {
  const void* w;
  int64_t rows, k, ld;
  int bits;
  int use_clip;
  float clip;
  int8_t* codes;
  int64_t ld_codes;
  void* scale;      // fp32 [rows] (INT8) or uint64 [rows] (INT4)
  float* bias;      // fp32 [rows] (INT4 only)
};

constexpr int kRowThreads = 256;

// every thread returns the reduction over the block; `red` holds one float per warp
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < kRowThreads / 32; ++i) r = fmaxf(r, red[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < kRowThreads / 32; ++i) r = __fadd_rn(r, red[i]);
  __syncthreads();
  return r;
}

struct CkptScale {
  float s, recip;
};
__device__ __forceinline__ CkptScale make_scale(float s) {
  const float y = __frcp_rn(s);
  const bool ok = fabsf(s) >= 1.17549435e-38f && fabsf(y) >= 1.17549435e-38f && isfinite(y) && isfinite(s);
  return CkptScale{s, ok ? y : 0.f};
}
// round(T(x / s)) clamped to +-qmax; NaN (0 / 0 of an all-zero row, NaN input) gives 0 like the reference's
// float -> int8 cast on x86
template <typename T>
__device__ __forceinline__ float ckpt_level(float x, const CkptScale& u, float qmax) {
  float q;
  if (u.recip != 0.f) {
    q = div_by_recip(x, u.s, u.recip);
    if (!(fabsf(q) <= 3.0e38f)) q = __fdiv_rn(x, u.s);
  } else {
    q = __fdiv_rn(x, u.s);
  }
  const float t = round_to<T>(q);
  return (t != t) ? 0.f : fminf(fmaxf(rintf(t), -qmax), qmax);
}
// one term of the assistance bias: T(T(scale * level) * 8)                       deploy.py:149-157
template <typename T>
__device__ __forceinline__ float ckpt_bias_term(float level, float s) {
  return round_to<T>(__fmul_rn(round_to<T>(__fmul_rn(s, level)), 8.f));
}

// Where the rows come from: values of T as they are, or an E4M3 matrix with block scales, dequantized on the fly
// to the value weight_dequant would have stored in T (so the fused path is bit-identical to dequant + quant, and
// the T copy of the weight never goes to HBM).
template <typename T>
struct SrcRows {
  static constexpr int kElems = ElemTraits<T>::kPerVec;      // elements per 16-byte load
  const T* base;
  int64_t ld;
  // the 16 bytes of vector v of a row as loaded, and their values
  __device__ __forceinline__ uint4 load_raw(int64_t row, int64_t v, bool stream) const {
    const uint4* q = reinterpret_cast<const uint4*>(base + row * ld + v * kElems);
    return stream ? __ldcs(q) : __ldg(q);
  }
  __device__ __forceinline__ void expand(const uint4& raw, int64_t, int64_t, float* f) const {
    const Vec16<T>& t = *reinterpret_cast<const Vec16<T>*>(&raw);
#pragma unroll
    for (int e = 0; e < kElems; ++e) f[e] = ElemTraits<T>::to_f(t.v[e]);
  }
  __device__ __forceinline__ void load_vec(int64_t row, int64_t v, float* f, bool stream) const {
    expand(load_raw(row, v, stream), row, v, f);
  }
  __device__ __forceinline__ float load_one(int64_t row, int64_t j) const { return ElemTraits<T>::to_f(base[row * ld + j]); }
};
template <typename T>
struct SrcFp8Blocks {
  static constexpr int kElems = 16;
  const uint8_t* base;
  int64_t ld;
  const float* scale;
  int64_t ld_scale;
  int block;
  __device__ __forceinline__ uint4 load_raw(int64_t row, int64_t v, bool stream) const {
    const uint4* q = reinterpret_cast<const uint4*>(base + row * ld + v * 16);
    return stream ? __ldcs(q) : __ldg(q);
  }
  __device__ __forceinline__ void load_vec(int64_t row, int64_t v, float* f, bool stream) const {
    expand(load_raw(row, v, stream), row, v, f);
  }
  __device__ __forceinline__ void expand(const uint4& raw, int64_t row, int64_t v, float* f) const {
    const float s = __ldg(scale + (row / block) * ld_scale + (v * 16) / block);
    const uint32_t word[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 lo = e4m3x2_to_float2(word[j]);
      const float2 hi = e4m3x2_to_float2(word[j] >> 16);
      f[4 * j + 0] = round_to<T>(__fmul_rn(lo.x, s));
      f[4 * j + 1] = round_to<T>(__fmul_rn(lo.y, s));
      f[4 * j + 2] = round_to<T>(__fmul_rn(hi.x, s));
      f[4 * j + 3] = round_to<T>(__fmul_rn(hi.y, s));
    }
  }
  __device__ __forceinline__ float load_one(int64_t row, int64_t j) const {
    const float s = __ldg(scale + (row / block) * ld_scale + j / block);
    return round_to<T>(__fmul_rn(e4m3_to_float(base[row * ld + j]), s));
  }
};

template <int N>
__device__ __forceinline__ void store_codes(int8_t* dst, const int8_t* bytes) {
  if (N == 16) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(bytes);
  else if (N == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(bytes);
  else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(bytes);
}

// One CTA per row (INT8) or per pair of rows 2j, 2j + 1 (INT4: their codes share the bytes of output row j).
template <typename T, typename SRC, bool VEC, int NROW>
__global__ void __launch_bounds__(kRowThreads) ckpt_rowquant_kernel(CkptRowParams p, SRC src) {
  constexpr int E = SRC::kElems;
  __shared__ float red[kRowThreads / 32];
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * NROW;
  const float qmax = (float)((1 << (p.bits - 1)) - 1);
  const int64_t nvec = VEC ? p.k / E : 0;

  // pass 1: |max| per row
  float amax[NROW], nan_seen[NROW];
#pragma unroll
  for (int r = 0; r < NROW; ++r) {
    float m = 0.f, bad = 0.f;
    if (VEC) {
      for (int64_t v = tid; v < nvec; v += kRowThreads) {
        float f[E];
        src.load_vec(row0 + r, v, f, false);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          m = fmaxf(m, fabsf(f[e]));
          if (f[e] != f[e]) bad = 1.f;
        }
      }
    } else {
      for (int64_t j = tid; j < p.k; j += kRowThreads) {
        const float f = src.load_one(row0 + r, j);
        m = fmaxf(m, fabsf(f));
        if (f != f) bad = 1.f;
      }
    }
    amax[r] = block_max(m, red);
    nan_seen[r] = block_max(bad, red);
  }

  CkptScale u[NROW];
#pragma unroll
  for (int r = 0; r < NROW; ++r) {
    float a = nan_seen[r] != 0.f ? __int_as_float(0x7fc00000) : amax[r];       // torch.max propagates NaN
    if (p.use_clip) a = round_to<T>(__fmul_rn(a, p.clip));                     // deploy.py:132-133
    u[r] = make_scale(round_to<T>(__fdiv_rn(a, qmax)));                        // deploy.py:134
  }

  // pass 2: codes (and the bias terms of INT4); the row comes back from L1 / L2
  float acc[NROW];
#pragma unroll
  for (int r = 0; r < NROW; ++r) acc[r] = 0.f;
  int8_t* out_row = p.codes + (int64_t)blockIdx.x * p.ld_codes;
  if (VEC) {
    for (int64_t v = tid; v < nvec; v += kRowThreads) {
      float lvl[NROW][E];
#pragma unroll
      for (int r = 0; r < NROW; ++r) {
        src.load_vec(row0 + r, v, lvl[r], true);
#pragma unroll
        for (int e = 0; e < E; ++e) lvl[r][e] = ckpt_level<T>(lvl[r][e], u[r], qmax);
      }
      alignas(16) int8_t bytes[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        if (NROW == 1) {
          bytes[e] = (int8_t)(int)lvl[0][e];
        } else {
          const int lo = (int)lvl[0][e], hi = (int)lvl[NROW - 1][e];
          bytes[e] = (int8_t)((lo & 0xF) | ((hi & 0xF) << 4));                 // deploy.py:117-123
#pragma unroll
          for (int r = 0; r < NROW; ++r) acc[r] = __fadd_rn(acc[r], ckpt_bias_term<T>(lvl[r][e], u[r].s));
        }
      }
      store_codes<E>(out_row + v * E, bytes);
    }
  } else {
    for (int64_t j = tid; j < p.k; j += kRowThreads) {
      float lvl[NROW];
#pragma unroll
      for (int r = 0; r < NROW; ++r) lvl[r] = ckpt_level<T>(src.load_one(row0 + r, j), u[r], qmax);
      if (NROW == 1) {
        out_row[j] = (int8_t)(int)lvl[0];
      } else {
        const int lo = (int)lvl[0], hi = (int)lvl[NROW - 1];
        out_row[j] = (int8_t)((lo & 0xF) | ((hi & 0xF) << 4));
#pragma unroll
        for (int r = 0; r < NROW; ++r) acc[r] = __fadd_rn(acc[r], ckpt_bias_term<T>(lvl[r], u[r].s));
      }
    }
  }

  if (NROW == 1) {
    if (tid == 0) reinterpret_cast<float*>(p.scale)[row0] = u[0].s;            // deploy.py:146
  } else {
#pragma unroll
    for (int r = 0; r < NROW; ++r) {
      // every partial sum is exact in fp32 for 16-bit T and k < 8192 (bf16) / k < 1024 (fp16): all terms
      // are multiples of one ulp of the smallest term, so the order of the additions does not matter there
      const float total = block_sum(acc[r], red);
      if (tid == 0) {
        p.bias[row0 + r] = round_to<T>(total);                                  // deploy.py:156
        reinterpret_cast<unsigned long long*>(p.scale)[row0 + r] =
            (unsigned long long)__float_as_uint(u[r].s);                        // deploy.py:93-106
      }
    }
  }
}

// ---- rows short enough to stay in registers -----------------------------------------------------------------------
// Every thread keeps the (up to NV) 16-byte vectors it owns of the row -- of both rows for INT4 -- as loaded: all
// loads are issued before the first use, the row is read from memory once, and the second pass works from
// registers.  A row whose scale is a normal number and whose quotients stay far below 2^22 (every row of a real
// checkpoint) takes a short path per element: the exact FMA division, the rounding to T, a clamp, and the magic-add
// rounding, packed by cvt.pack.  For such a row no quotient is NaN or infinite, and round-then-clamp equals
// clamp-then-round because the bounds are integers, so the levels are those of ckpt_level.  Any other row (all
// zeros, NaN / Inf, a denormal scale, a tiny clip factor) goes through ckpt_level element by element.
constexpr float kCkptMagic = 12582912.f;                      // 1.5 * 2^23
constexpr int kCkptMagicBits = 0x4B400000;

template <int NROW>
__device__ __forceinline__ void block_max_nan(float (&v)[NROW], float (*red)[kRowThreads / 32]) {
#pragma unroll
  for (int r = 0; r < NROW; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[r] = fmax_nan(v[r], __shfl_xor_sync(0xffffffffu, v[r], o));
    if ((threadIdx.x & 31) == 0) red[r][threadIdx.x >> 5] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < NROW; ++r) {
    float m = red[r][0];
#pragma unroll
    for (int i = 1; i < kRowThreads / 32; ++i) m = fmax_nan(m, red[r][i]);
    v[r] = m;
  }
}

template <typename T, typename SRC, int NROW, int NV>
__global__ void __launch_bounds__(kRowThreads) ckpt_rowquant_reg_kernel(CkptRowParams p, SRC src) {
  constexpr int E = SRC::kElems;
  __shared__ float red[NROW][kRowThreads / 32];
  __shared__ float red_sum[kRowThreads / 32];
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * NROW;
  const float qmax = (float)((1 << (p.bits - 1)) - 1);
  const int nvec = (int)(p.k / E);

  uint4 raw[NROW][NV];
#pragma unroll
  for (int r = 0; r < NROW; ++r) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = tid + i * kRowThreads;
      raw[r][i] = v < nvec ? src.load_raw(row0 + r, v, true) : make_uint4(0u, 0u, 0u, 0u);
    }
  }

  // pass 1: max |w| per row; a NaN anywhere makes it NaN, as torch.max does
  float amax[NROW];
#pragma unroll
  for (int r = 0; r < NROW; ++r) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = tid + i * kRowThreads;
      if (v < nvec) {
        float f[E];
        src.expand(raw[r][i], row0 + r, v, f);
#pragma unroll
        for (int e = 0; e < E; ++e) m = fmax_nan(m, fabsf(f[e]));
      }
    }
    amax[r] = m;
  }
  block_max_nan<NROW>(amax, red);

  CkptScale u[NROW];
  bool regular[NROW];
#pragma unroll
  for (int r = 0; r < NROW; ++r) {
    float a = amax[r];
    if (p.use_clip) a = round_to<T>(__fmul_rn(a, p.clip));                     // deploy.py:132-133
    u[r] = make_scale(round_to<T>(__fdiv_rn(a, qmax)));                        // deploy.py:134
    // |x / s| <= amax * |1 / s| (1 + 2^-22) for every x of the row
    regular[r] = u[r].recip != 0.f && __fmul_rn(amax[r], fabsf(u[r].recip)) < 2097152.f;
  }

  // pass 2, from registers
  float acc[NROW];
#pragma unroll
  for (int r = 0; r < NROW; ++r) acc[r] = 0.f;
  int8_t* out_row = p.codes + (int64_t)blockIdx.x * p.ld_codes;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = tid + i * kRowThreads;
    if (v >= nvec) continue;
    int lvl[NROW][E];
#pragma unroll
    for (int r = 0; r < NROW; ++r) {
      float f[E];
      src.expand(raw[r][i], row0 + r, v, f);
      if (regular[r]) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          float t = round_to<T>(div_by_recip(f[e], u[r].s, u[r].recip));
          t = __fadd_rn(fminf(fmaxf(t, -qmax), qmax), kCkptMagic);
          lvl[r][e] = __float_as_int(t) - kCkptMagicBits;
          if (NROW == 2) acc[r] = __fadd_rn(acc[r], ckpt_bias_term<T>(__fsub_rn(t, kCkptMagic), u[r].s));
        }
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float l = ckpt_level<T>(f[e], u[r], qmax);
          lvl[r][e] = (int)l;
          if (NROW == 2) acc[r] = __fadd_rn(acc[r], ckpt_bias_term<T>(l, u[r].s));
        }
      }
    }
    uint32_t words[E / 4];
#pragma unroll
    for (int g = 0; g < E / 4; ++g) {
      uint32_t w = 0;
      if (NROW == 1) {
        w = pack_sat_s8(lvl[0][4 * g + 3], lvl[0][4 * g + 2], 0);
        w = pack_sat_s8(lvl[0][4 * g + 1], lvl[0][4 * g], w);
      } else {
#pragma unroll
        for (int e = 3; e >= 0; --e) w = pack_sat_s4(lvl[NROW - 1][4 * g + e], lvl[0][4 * g + e], w);   // deploy.py:117-123
      }
      words[g] = w;
    }
    store_codes<E>(out_row + (int64_t)v * E, reinterpret_cast<const int8_t*>(words));
  }

  if (NROW == 1) {
    if (tid == 0) reinterpret_cast<float*>(p.scale)[row0] = u[0].s;            // deploy.py:146
  } else {
#pragma unroll
    for (int r = 0; r < NROW; ++r) {
      const float total = block_sum(acc[r], red_sum);     // exact for 16-bit T and the row lengths that fit here
      if (tid == 0) {
        p.bias[row0 + r] = round_to<T>(total);                                  // deploy.py:156
        reinterpret_cast<unsigned long long*>(p.scale)[row0 + r] =
            (unsigned long long)__float_as_uint(u[r].s);                        // deploy.py:93-106
      }
    }
  }
}


template <typename T, typename SRC>
static int launch_rowquant(const CkptRowParams& p, const SRC& src, bool vec, cudaStream_t st) {
  const int64_t nvec = vec ? p.k / SRC::kElems : 0;
  if (vec && nvec <= 4 * kRowThreads) {                 // the row fits the registers of a CTA
    const bool two = nvec <= 2 * kRowThreads;
    if (p.bits == 8) {
      const unsigned grid = (unsigned)p.rows;
      if (two) AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_reg_kernel<T, SRC, 1, 2>);
      else AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_reg_kernel<T, SRC, 1, 4>);
    } else {
      const unsigned grid = (unsigned)(p.rows / 2);
      if (two) AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_reg_kernel<T, SRC, 2, 2>);
      else AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_reg_kernel<T, SRC, 2, 4>);
    }
    AMCT_CHECK_LAUNCH();
    return AMCT_OK;
  }
  if (p.bits == 8) {
    const unsigned grid = (unsigned)p.rows;
    if (vec) AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_kernel<T, SRC, true, 1>);
    else AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_kernel<T, SRC, false, 1>);
  } else {
    const unsigned grid = (unsigned)(p.rows / 2);
    if (vec) AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_kernel<T, SRC, true, 2>);
    else AMCT_LAUNCH(grid, kRowThreads, st, (p, src), ckpt_rowquant_kernel<T, SRC, false, 2>);
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

// rows of T
template <typename T>
static int launch_rowquant_plain(const CkptRowParams& p, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  const bool vec = p.k % E == 0 && aligned16(p.w) && (p.ld * (int64_t)sizeof(T)) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(p.codes) % E) == 0 && p.ld_codes % E == 0;
  SrcRows<T> src{reinterpret_cast<const T*>(p.w), p.ld};
  return launch_rowquant<T, SrcRows<T>>(p, src, vec, st);
}

// E4M3 rows with block scales, dequantized to T on the fly
template <typename T>
static int launch_rowquant_fp8(const CkptRowParams& p, const float* scale, int64_t ld_scale, int block, cudaStream_t st) {
  const bool vec = p.k % 16 == 0 && block % 16 == 0 && aligned16(p.w) && p.ld % 16 == 0 && aligned16(p.codes) &&
                   p.ld_codes % 16 == 0;
  SrcFp8Blocks<T> src{reinterpret_cast<const uint8_t*>(p.w), p.ld, scale, ld_scale, block};
  return launch_rowquant<T, SrcFp8Blocks<T>>(p, src, vec, st);
}

// ------------------------------------------------------------------------------------------------
// stand-alone pieces of the INT4 export
// ------------------------------------------------------------------------------------------------
// out[j, c] = (codes[2j, c] & 15) | (codes[2j + 1, c] << 4)                       deploy.py:109-125
__global__ void __launch_bounds__(128) ckpt_pack4_rows_kernel(const int8_t* __restrict__ codes, int64_t pairs, int64_t k,
                                                              int64_t ld, int8_t* __restrict__ out, int64_t ld_out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= k) return;
  for (int64_t j = blockIdx.y; j < pairs; j += gridDim.y) {
    const int lo = codes[(2 * j) * ld + c], hi = codes[(2 * j + 1) * ld + c];
    out[j * ld_out + c] = (int8_t)((lo & 0xF) | ((hi & 0xF) << 4));
  }
}

// bias[n] = T(sum_k T(T(scale[n, k / repeat] * codes[n, k]) * 8)); one CTA per row     deploy.py:149-157
template <typename T>
__global__ void __launch_bounds__(kRowThreads) ckpt_int4_bias_kernel(const int8_t* __restrict__ codes, int64_t k,
                                                                     int64_t ld, const T* __restrict__ scale,
                                                                     int64_t groups, float* __restrict__ bias) {
  __shared__ float red[kRowThreads / 32];
  const int64_t n = blockIdx.x;
  const int64_t repeat = k / groups;
  float acc = 0.f;
  for (int64_t j = threadIdx.x; j < k; j += kRowThreads) {
    const float s = ElemTraits<T>::to_f(scale[n * groups + j / repeat]);
    acc = __fadd_rn(acc, ckpt_bias_term<T>((float)codes[n * ld + j], s));
  }
  const float total = block_sum(acc, red);
  if (threadIdx.x == 0) bias[n] = round_to<T>(total);
}

// H[i, j] = (-1)^popcount(i & j) * m, m = 1 divided log2(n) times by fp32 sqrt(2) with a rounding to T after
// every division (the reference halves the norm at each doubling, on a tensor of dtype T)   deploy.py:32-45
template <typename T>
__global__ void __launch_bounds__(256) ckpt_hadamard_kernel(int n, int log2n, int norm, T* __restrict__ out) {
  float m = 1.f;
  if (norm)
    for (int i = 0; i < log2n; ++i) m = round_to<T>(__fdiv_rn(m, 1.41421354f));
  const int64_t total = (int64_t)n * n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const unsigned i = (unsigned)(idx / n), j = (unsigned)(idx % n);
    out[idx] = ElemTraits<T>::from_f((__popc(i & j) & 1) ? -m : m);
  }
}

}  // namespace amct

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
using namespace amct;

extern "C" int amct_ckpt_block_dequant(const void* w_fp8, int64_t rows, int64_t cols, int64_t ld_w, const float* scale,
                                       int64_t ld_scale, int block, void* out, int out_dtype, int64_t ld_out,
                                       void* stream) {
  if (rows < 0 || cols < 0 || block <= 0 || ld_w < cols || ld_out < cols) return AMCT_ERR_ARG;
  if (ld_scale < (cols + block - 1) / block) return AMCT_ERR_ARG;
  if (rows == 0 || cols == 0) return AMCT_OK;
  if (!w_fp8 || !scale || !out) return AMCT_ERR_ARG;
  if (cols > (int64_t)128 * 0x7fffffff) return AMCT_ERR_UNSUPPORTED;
  const uint8_t* w = reinterpret_cast<const uint8_t*>(w_fp8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case AMCT_DTYPE_F32: return launch_block_dequant<float>(w, rows, cols, ld_w, scale, ld_scale, block, out, ld_out, st);
    case AMCT_DTYPE_F16: return launch_block_dequant<__half>(w, rows, cols, ld_w, scale, ld_scale, block, out, ld_out, st);
    case AMCT_DTYPE_BF16:
      return launch_block_dequant<__nv_bfloat16>(w, rows, cols, ld_w, scale, ld_scale, block, out, ld_out, st);
  }
  return AMCT_ERR_ARG;
}

extern "C" int amct_ckpt_rowquant(const void* w, int dtype, int64_t rows, int64_t k, int64_t ld, int bits, int use_clip,
                                  float clip_factor, int8_t* codes, int64_t ld_codes, void* scale, float* bias,
                                  void* stream) {
  if (rows < 0 || k < 0 || ld < k || ld_codes < k) return AMCT_ERR_ARG;
  if (bits != 8 && bits != 4) return AMCT_ERR_ARG;
  if (bits == 4 && rows % 2 != 0) return AMCT_ERR_ARG;          // the reference's reshape fails on odd N too
  if (rows == 0) return AMCT_OK;
  if (!w || !codes || !scale || (bits == 4 && !bias)) return AMCT_ERR_ARG;
  if (rows > 0x7fffffff) return AMCT_ERR_UNSUPPORTED;
  CkptRowParams p{w, rows, k, ld, bits, use_clip ? 1 : 0, clip_factor, codes, ld_codes, scale, bias};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case AMCT_DTYPE_F32: return launch_rowquant_plain<float>(p, st);
    case AMCT_DTYPE_F16: return launch_rowquant_plain<__half>(p, st);
    case AMCT_DTYPE_BF16: return launch_rowquant_plain<__nv_bfloat16>(p, st);
  }
  return AMCT_ERR_ARG;
}

extern "C" int amct_ckpt_dequant_rowquant(const void* w_fp8, int64_t rows, int64_t k, int64_t ld_w, const float* block_scale,
                                          int64_t ld_scale, int block, int dtype, int bits, int use_clip,
                                          float clip_factor, int8_t* codes, int64_t ld_codes, void* scale, float* bias,
                                          void* stream) {
  if (rows < 0 || k < 0 || ld_w < k || ld_codes < k || block <= 0) return AMCT_ERR_ARG;
  if (ld_scale < (k + block - 1) / block) return AMCT_ERR_ARG;
  if (bits != 8 && bits != 4) return AMCT_ERR_ARG;
  if (bits == 4 && rows % 2 != 0) return AMCT_ERR_ARG;
  if (rows == 0) return AMCT_OK;
  if (!w_fp8 || !block_scale || !codes || !scale || (bits == 4 && !bias)) return AMCT_ERR_ARG;
  if (rows > 0x7fffffff) return AMCT_ERR_UNSUPPORTED;
  CkptRowParams p{w_fp8, rows, k, ld_w, bits, use_clip ? 1 : 0, clip_factor, codes, ld_codes, scale, bias};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case AMCT_DTYPE_F32: return launch_rowquant_fp8<float>(p, block_scale, ld_scale, block, st);
    case AMCT_DTYPE_F16: return launch_rowquant_fp8<__half>(p, block_scale, ld_scale, block, st);
    case AMCT_DTYPE_BF16: return launch_rowquant_fp8<__nv_bfloat16>(p, block_scale, ld_scale, block, st);
  }
  return AMCT_ERR_ARG;
}

extern "C" int amct_ckpt_pack4_rows(const int8_t* codes, int64_t rows, int64_t k, int64_t ld, int8_t* out,
                                    int64_t ld_out, void* stream) {
  if (rows < 0 || k < 0 || ld < k || ld_out < k || rows % 2 != 0) return AMCT_ERR_ARG;
  if (rows == 0 || k == 0) return AMCT_OK;
  if (!codes || !out) return AMCT_ERR_ARG;
  if (k > (int64_t)128 * 0x7fffffff) return AMCT_ERR_UNSUPPORTED;
  const int64_t pairs = rows / 2;
  dim3 grid((unsigned)((k + 127) / 128), (unsigned)(pairs < 16384 ? pairs : 16384));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  AMCT_LAUNCH(grid, 128, st, (codes, pairs, k, ld, out, ld_out), ckpt_pack4_rows_kernel);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

extern "C" int amct_ckpt_int4_bias(const int8_t* codes, int64_t rows, int64_t k, int64_t ld, const void* scale, int dtype,
                                   int64_t groups, float* bias, void* stream) {
  if (rows < 0 || k < 0 || ld < k || groups <= 0 || k % groups != 0) return AMCT_ERR_ARG;
  if (rows == 0) return AMCT_OK;
  if (!codes || !scale || !bias) return AMCT_ERR_ARG;
  if (rows > 0x7fffffff) return AMCT_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)rows;
  switch (dtype) {
    case AMCT_DTYPE_F32:
      AMCT_LAUNCH(grid, kRowThreads, st, (codes, k, ld, (const float*)scale, groups, bias), ckpt_int4_bias_kernel<float>);
      break;
    case AMCT_DTYPE_F16:
      AMCT_LAUNCH(grid, kRowThreads, st, (codes, k, ld, (const __half*)scale, groups, bias), ckpt_int4_bias_kernel<__half>);
      break;
    case AMCT_DTYPE_BF16:
      AMCT_LAUNCH(grid, kRowThreads, st, (codes, k, ld, (const __nv_bfloat16*)scale,
                                                                          groups, bias), ckpt_int4_bias_kernel<__nv_bfloat16>);
      break;
    default: return AMCT_ERR_ARG;
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

extern "C" int amct_hadamard_pow2(int n, int norm, int dtype, void* out, void* stream) {
  if (n <= 0 || (n & (n - 1)) != 0 || n > 32768 || !out) return AMCT_ERR_ARG;
  int log2n = 0;
  while ((1 << log2n) < n) ++log2n;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t total = (int64_t)n * n;
  const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  switch (dtype) {
    case AMCT_DTYPE_F32: AMCT_LAUNCH(grid, 256, st, (n, log2n, norm, (float*)out), ckpt_hadamard_kernel<float>); break;
    case AMCT_DTYPE_F16: AMCT_LAUNCH(grid, 256, st, (n, log2n, norm, (__half*)out), ckpt_hadamard_kernel<__half>); break;
    case AMCT_DTYPE_BF16:
      AMCT_LAUNCH(grid, 256, st, (n, log2n, norm, (__nv_bfloat16*)out), ckpt_hadamard_kernel<__nv_bfloat16>);
      break;
    default: return AMCT_ERR_ARG;
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}
