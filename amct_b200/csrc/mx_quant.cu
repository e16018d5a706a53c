// MXFP8 (E4M3) / MXFP4 (E2M1) block quantization with E8M0 scales over 32-element
// blocks along K.  The reference has no MX code (amct_pytorch/utils/vars.py:19-20
// admits only int8 / int4); the arithmetic follows the public OCP Microscaling v1.0
// conversion rule:
//     shared_exp = floor(log2(max|v|)) - emax_elem     (emax 8 for E4M3, 2 for E2M1)
//     scale byte = clamp(shared_exp, -127, 127) + 127
//     element    = saturating round-to-nearest-even of v * 2^-shared_exp
// with these choices where the rule is silent: an all-zero block gets scale byte 0; a
// block holding NaN or Inf gets scale byte 0xFF, E4M3 elements 0x7F, and E2M1 elements
// computed from the finite part (NaN -> +0, Inf saturates).
//
// Four adjacent lanes own one block (8 elements each): loads and payload stores are
// fully coalesced 16- / 8- / 4-byte accesses, the block maximum is two shuffles, and
// the 2^-e scaling is an exact multiply by a constructed power of two.  Scales are
// written row-major [rows, K/32] and, optionally, in the 128 x 4 tiling the
// block-scaled tensor-core GEMM copies straight into tensor memory: rows are cut into
// GEMM tiles of `tile_rows` rows (128 for the A operand, 224 for the B operand), each tile
// into atoms of 128 rows, and an atom holds 4 K blocks of its 128 rows in 512 bytes:
//     t = r / tile_rows, q = r % tile_rows, atom = t * ceil(tile_rows/128) + q/128
//     offset(r, kb) = (atom * ceil(K/128) + kb/4) * 512 + (q%32)*16 + ((q%128)/32)*4 + kb%4
//
// HBM traffic per element: sizeof(T) read + 1 (fp8) or 0.5 (fp4) + 1/32 bytes written.
#include <cuda_fp8.h>
#include <cuda_fp4.h>

#include "common.cuh"

namespace amct {

template <typename T>
__device__ __forceinline__ void mx_load8(const T* src, float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    Vec16<T> raw = ld_vec_stream(src);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = ElemTraits<T>::to_f(raw.v[e]);
  } else {
    Vec16<T> r0 = ld_vec_stream(src), r1 = ld_vec_stream(src + 4);
#pragma unroll
    for (int e = 0; e < 4; ++e) { v[e] = ElemTraits<T>::to_f(r0.v[e]); v[4 + e] = ElemTraits<T>::to_f(r1.v[e]); }
  }
}

// One lane's 8 elements of a 32-element block (4 adjacent lanes share the block).
template <int FMT>
__device__ __forceinline__ void mx_block(const float (&v)[8], bool valid, int lane, int64_t row, int64_t oct, int64_t k,
                                         int64_t kb_per_row, int64_t kb4_per_row, bool wide, int tile_rows,
                                         uint8_t* payload, uint8_t* scales_rm, uint8_t* scales_tiled) {
  constexpr int EMAX = FMT == 8 ? 8 : 2;
  // max |v| through the integer order of the magnitude bits: Inf / NaN show up as >= 0x7F800000
  uint32_t amax_bits = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax_bits = max(amax_bits, __float_as_uint(v[e]) & 0x7fffffffu);
  amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 1));
  amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 2));
  const bool bad = amax_bits >= 0x7f800000u;
  if (bad) {                                     // rare: the shared exponent comes from the finite part only
    uint32_t fin = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t b = __float_as_uint(v[e]) & 0x7fffffffu;
      fin = max(fin, b < 0x7f800000u ? b : 0u);
    }
    const unsigned act = __activemask();          // the 4 lanes of a block take this branch together
    fin = max(fin, __shfl_xor_sync(act, fin, 1));
    fin = max(fin, __shfl_xor_sync(act, fin, 2));
    amax_bits = fin;
  }
  // biased exponent of amax minus emax = shared_exp + 127; fp32 denormals and zero land on 0
  int sb = (int)(amax_bits >> 23) - EMAX;
  sb = sb < 0 ? 0 : (sb > 254 ? 254 : sb);
  const int field = 254 - sb;                                            // exponent field of 2^-shared_exp
  const float mult = __uint_as_float(field > 0 ? (uint32_t)field << 23 : 0x00400000u);
  const uint32_t scale_byte = bad ? 0xFFu : (uint32_t)sb;

  if (valid) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = __fmul_rn(v[e], mult);
    if constexpr (FMT == 8) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        lo |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(s[e], s[e + 1]), __NV_SATFINITE, __NV_E4M3) << (8 * e);
        hi |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(s[4 + e], s[5 + e]), __NV_SATFINITE, __NV_E4M3) << (8 * e);
      }
      if (bad) { lo = 0x7F7F7F7Fu; hi = 0x7F7F7F7Fu; }
      *reinterpret_cast<uint2*>(payload + row * k + oct * 8) = make_uint2(lo, hi);
    } else {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        float a = s[e], b = s[e + 1];
        if (bad) { a = a == a ? a : 0.f; b = b == b ? b : 0.f; }         // E2M1 has no NaN
        word |= (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest) << (4 * e);
      }
      *reinterpret_cast<uint32_t*>(payload + row * (k / 2) + oct * 4) = word;
    }
  }

  const int64_t kb = oct / 4;
  const uint32_t r32 = (uint32_t)row;                                  // rows < 2^31 (checked on the host)
  const uint32_t tile = r32 / (uint32_t)tile_rows, tq = r32 - tile * (uint32_t)tile_rows;
  const int64_t atom = (int64_t)tile * ((tile_rows + 127) / 128) + tq / 128;
  const int64_t tiled_off = (atom * kb4_per_row + kb / 4) * 512 + (tq % 32) * 16 + ((tq % 128) / 32) * 4 + (kb % 4);
  if (wide) {
    const int g16 = lane & ~15;
    uint32_t word = __shfl_sync(0xffffffffu, scale_byte, g16) | (__shfl_sync(0xffffffffu, scale_byte, g16 + 4) << 8) |
                    (__shfl_sync(0xffffffffu, scale_byte, g16 + 8) << 16) | (__shfl_sync(0xffffffffu, scale_byte, g16 + 12) << 24);
    if (valid && (lane & 15) == 0) {
      if (scales_rm) *reinterpret_cast<uint32_t*>(scales_rm + row * kb_per_row + kb) = word;
      if (scales_tiled) *reinterpret_cast<uint32_t*>(scales_tiled + tiled_off) = word;
    }
  } else if (valid && (lane & 3) == 0) {
    if (scales_rm) scales_rm[row * kb_per_row + kb] = (uint8_t)scale_byte;
    if (scales_tiled) scales_tiled[tiled_off] = (uint8_t)scale_byte;
  }
}

template <typename T, int FMT>
__global__ void __launch_bounds__(256) mx_quant_kernel(const T* x, int64_t rows, int64_t k, int64_t ld, uint8_t* payload,
                                                       uint8_t* scales_rm, uint8_t* scales_tiled, int tile_rows) {
  constexpr int U = 2;                                      // blocks in flight per thread
  const int lane = threadIdx.x & 31;
  const int64_t oct_per_row = k / 8;
  const int64_t total = rows * oct_per_row;
  const int64_t kb_per_row = k / 32;
  const int64_t kb4_per_row = (kb_per_row + 3) / 4;
  const bool wide = (kb_per_row % 4) == 0;                  // 4 scale bytes of a row go out as one word
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x; base < total; base += stride * U) {
    float v[U][8];
    int64_t row[U], oct[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t w = base + u * stride + threadIdx.x;
      valid[u] = w < total;
      row[u] = valid[u] ? w / oct_per_row : 0;
      oct[u] = valid[u] ? w - row[u] * oct_per_row : 0;
      if (valid[u]) mx_load8<T>(x + row[u] * ld + oct[u] * 8, v[u]);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (base + u * stride >= total) break;                // uniform across the block
      mx_block<FMT>(v[u], valid[u], lane, row[u], oct[u], k, kb_per_row, kb4_per_row, wide, tile_rows, payload, scales_rm,
                    scales_tiled);
    }
  }
}

// Row-tiled variant for K >= 1024: blockIdx.x picks a 2048-element span of the row,
// blockIdx.y strides over rows, so no thread ever divides to find its row, and the tile /
// atom position of the scale layout advances incrementally.
template <typename T, int FMT>
__global__ void __launch_bounds__(256) mx_quant_rows_kernel(const T* x, int rows, int k, int64_t ld, uint8_t* payload,
                                                            uint8_t* scales_rm, uint8_t* scales_tiled, int tile_rows) {
  constexpr int U = 2;                                      // rows in flight per thread
  const int lane = threadIdx.x & 31;
  const int oct_per_row = k / 8;
  const int oct = blockIdx.x * blockDim.x + threadIdx.x;
  const bool in_row = oct < oct_per_row;
  const int kb_per_row = k / 32;
  const int kb4_per_row = (kb_per_row + 3) / 4;
  const bool wide = (kb_per_row % 4) == 0;
  for (int r0 = blockIdx.y * U; r0 < rows; r0 += gridDim.y * U) {
    float v[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (in_row && r0 + u < rows) mx_load8<T>(x + (int64_t)(r0 + u) * ld + (int64_t)oct * 8, v[u]);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (r0 + u >= rows) break;                            // uniform across the block
      mx_block<FMT>(v[u], in_row, lane, r0 + u, in_row ? oct : 0, k, kb_per_row, kb4_per_row, wide, tile_rows, payload,
                    scales_rm, scales_tiled);
    }
  }
}

template <typename T>
static int run_mx(const T* x, int64_t rows, int64_t k, int64_t ld, int fmt, uint8_t* payload, uint8_t* srm, uint8_t* st,
                  int tile_rows, cudaStream_t stream) {
  if (k >= 1024 && rows < (1LL << 30) && k < (1LL << 30)) {
    dim3 grid((unsigned)((k / 8 + 255) / 256), 1);
    int64_t gy = (148LL * 8 + grid.x - 1) / grid.x;        // about 8 CTAs per SM
    const int64_t need = (rows + 1) / 2;
    if (gy > need) gy = need;
    grid.y = (unsigned)(gy < 1 ? 1 : gy);
    if (fmt == 8) AMCT_LAUNCH(grid, 256, stream, (x, (int)rows, (int)k, ld, payload, srm, st, tile_rows), mx_quant_rows_kernel<T, 8>);
    else AMCT_LAUNCH(grid, 256, stream, (x, (int)rows, (int)k, ld, payload, srm, st, tile_rows), mx_quant_rows_kernel<T, 4>);
    AMCT_CHECK_LAUNCH();
    return AMCT_OK;
  }
  const int64_t total = rows * (k / 8);
  int64_t blocks = (total + 511) / 512;
  if (blocks < 1) blocks = 1;
  const int64_t cap = 148LL * 8 * 4;
  if (blocks > cap) blocks = cap;
  if (fmt == 8) AMCT_LAUNCH((unsigned)blocks, 256, stream, (x, rows, k, ld, payload, srm, st, tile_rows), mx_quant_kernel<T, 8>);
  else AMCT_LAUNCH((unsigned)blocks, 256, stream, (x, rows, k, ld, payload, srm, st, tile_rows), mx_quant_kernel<T, 4>);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

extern "C" int64_t amct_mx_tiled_scale_bytes(int64_t rows, int64_t k, int tile_rows) {
  if (rows < 0 || k < 0 || tile_rows < 32 || tile_rows % 32) return 0;
  const int64_t tiles = (rows + tile_rows - 1) / tile_rows;
  return tiles * ((tile_rows + 127) / 128) * ((k / 32 + 3) / 4) * 512;
}

extern "C" int amct_mx_quant(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int elem_bits, void* payload,
                             void* scales_rowmajor, void* scales_tiled, int scale_tile_rows, void* stream) {
  if (rows < 0 || k < 0 || ld_x < k || (elem_bits != 8 && elem_bits != 4)) return AMCT_ERR_ARG;
  if (rows == 0 || k == 0) return AMCT_OK;
  if (!x || !payload || (!scales_rowmajor && !scales_tiled)) return AMCT_ERR_ARG;
  if (k % 32 != 0 || rows > 0x7fffffffLL) return AMCT_ERR_UNSUPPORTED;
  if (scales_tiled && (scale_tile_rows < 32 || scale_tile_rows % 32 != 0)) return AMCT_ERR_ARG;
  const int tr = scales_tiled ? scale_tile_rows : 128;
  const int esize = dtype == AMCT_DTYPE_F32 ? 4 : 2;
  if (!amct::aligned16(x) || (ld_x * esize) % 16 != 0 || reinterpret_cast<uintptr_t>(payload) % 8 != 0 ||
      (scales_rowmajor && reinterpret_cast<uintptr_t>(scales_rowmajor) % 4 != 0) ||
      (scales_tiled && reinterpret_cast<uintptr_t>(scales_tiled) % 16 != 0))
    return AMCT_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* p = reinterpret_cast<uint8_t*>(payload);
  uint8_t* srm = reinterpret_cast<uint8_t*>(scales_rowmajor);
  uint8_t* stl = reinterpret_cast<uint8_t*>(scales_tiled);
  switch (dtype) {
    case AMCT_DTYPE_F32: return amct::run_mx<float>((const float*)x, rows, k, ld_x, elem_bits, p, srm, stl, tr, st);
    case AMCT_DTYPE_F16: return amct::run_mx<__half>((const __half*)x, rows, k, ld_x, elem_bits, p, srm, stl, tr, st);
    case AMCT_DTYPE_BF16: return amct::run_mx<__nv_bfloat16>((const __nv_bfloat16*)x, rows, k, ld_x, elem_bits, p, srm, stl, tr, st);
  }
  return AMCT_ERR_ARG;
}
