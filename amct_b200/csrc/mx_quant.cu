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
// One thread owns one 32-element block: 64 (16-bit input) or 128 contiguous bytes are loaded as 16-byte vectors, the
// block maximum needs no shuffle (packed |x| / max instructions on the 16-bit types), the per-block work (exponent
// arithmetic, scale addresses) is paid once per 32 elements, the payload leaves as 32 (E4M3) or 16 (E2M1) contiguous
// bytes, and the 2^-e scaling is an exact multiply by a constructed power of two.  blockIdx.x covers the K blocks of
// a row, blockIdx.y strides over rows: no thread divides to find its row.  Scales are
// written row-major [rows, K/32] and, optionally, in the 128 x 4 tiling the
// block-scaled tensor-core GEMM copies straight into tensor memory: rows are cut into
// GEMM tiles of `tile_rows` rows (128 for the A operand, 224 for the B operand), each tile
// into atoms of 128 rows, and an atom holds 4 K blocks of its 128 rows in 512 bytes:
//     t = r / tile_rows, q = r % tile_rows, atom = t * ceil(tile_rows/128) + q/128
//     offset(r, kb) = (atom * ceil(K/128) + kb/4) * 512 + (q%32)*16 + ((q%128)/32)*4 + kb%4
// The padding of that layout (rows of the last atom of a tile that no row maps to, K blocks beyond K/32 in the last
// group of four) is written as zero by this kernel: the buffer needs no clearing beforehand.
//
// HBM traffic per element: sizeof(T) read + 1 (fp8) or 0.5 (fp4) + 1/32 bytes written.
#include <cuda_fp8.h>
#include <cuda_fp4.h>

#include "common.cuh"

namespace amct {

constexpr int kMxBlock = 32;

// |amax| of a 32-element block as fp32 bits (NaN / Inf show as >= 0x7F800000), from the packed vectors.
template <typename T> struct MxMax;
template <> struct MxMax<__nv_bfloat16> {
  __device__ static uint32_t of(const Vec16<__nv_bfloat16> (&raw)[4]) {
    __nv_bfloat162 m = __habs2(reinterpret_cast<const __nv_bfloat162*>(&raw[0])[0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) m = __hmax2_nan(m, __habs2(h[e]));
    }
    const float a = __low2float(m), b = __high2float(m);
    return max(__float_as_uint(a) & 0x7fffffffu, __float_as_uint(b) & 0x7fffffffu);   // a NaN's bits exceed every number's
  }
};
template <> struct MxMax<__half> {
  __device__ static uint32_t of(const Vec16<__half> (&raw)[4]) {
    __half2 m = __habs2(reinterpret_cast<const __half2*>(&raw[0])[0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) m = __hmax2_nan(m, __habs2(h[e]));
    }
    const float a = __low2float(m), b = __high2float(m);
    return max(__float_as_uint(a) & 0x7fffffffu, __float_as_uint(b) & 0x7fffffffu);
  }
};
template <> struct MxMax<float> {
  __device__ static uint32_t of(const Vec16<float> (&raw)[8]) {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) m = max(m, __float_as_uint(raw[i].v[e]) & 0x7fffffffu);
    }
    return m;
  }
};

// 8 scaled values -> 8 E4M3 bytes (two words) or 8 E2M1 nibbles (one word)
__device__ __forceinline__ uint2 mx_e4m3x8(const float (&s)[8]) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(s[4 * h], s[4 * h + 1]), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(s[4 * h + 2], s[4 * h + 3]), __NV_SATFINITE, __NV_E4M3);
    w[h] = lo | (hi << 16);
  }
  return make_uint2(w[0], w[1]);
}
__device__ __forceinline__ uint32_t mx_e2m1x8(const float (&s)[8], bool bad) {
  uint32_t word = 0;
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    float a = s[e], b = s[e + 1];
    if (bad) { a = a == a ? a : 0.f; b = b == b ? b : 0.f; }         // E2M1 has no NaN
    word |= (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest) << (4 * e);
  }
  return word;
}

// Where a row slot of the loop below lies: its row (or none: padding of the tiled layout) and its tiled-scale offset.
struct MxSlot {
  int row;
  bool is_row;
  int64_t tiled_off;
};
__device__ __forceinline__ MxSlot mx_slot(int slot, bool tiled, int rows, int tile_rows, int atoms_per_tile, int kb4_per_row, int kb) {
  MxSlot r{slot, true, 0};
  if (tiled) {
    const int atom = slot >> 7, q128 = slot & 127;
    const int tile = atom / atoms_per_tile, atom_in_tile = atom - tile * atoms_per_tile;
    const int q = atom_in_tile * 128 + q128;                 // row within the tile
    r.row = tile * tile_rows + q;
    r.is_row = q < tile_rows && r.row < rows;
    r.tiled_off = ((int64_t)atom * kb4_per_row + kb / 4) * 512 + (q128 % 32) * 16 + (q128 / 32) * 4 + (kb % 4);
  }
  return r;
}

// One 32-element block, already loaded: shared exponent, payload, scale byte(s).
template <typename T, int FMT, int NV>
__device__ __forceinline__ void mx_one_block(const Vec16<T> (&raw)[NV], const MxSlot& sl, int k, int kb, int kb_per_row, int pad_kb,
                                             uint8_t* payload, uint8_t* scales_rm, uint8_t* scales_tiled) {
  constexpr int EMAX = FMT == 8 ? 8 : 2;
  constexpr int EV = 16 / (int)sizeof(T);                     // elements per vector
  uint32_t amax_bits = MxMax<T>::of(raw);
  const bool bad = amax_bits >= 0x7f800000u;
  if (bad) {                                     // rare: the shared exponent comes from the finite part only
    uint32_t fin = 0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
      for (int e = 0; e < EV; ++e) {
        const uint32_t b = __float_as_uint(ElemTraits<T>::to_f(raw[i].v[e])) & 0x7fffffffu;
        fin = max(fin, b < 0x7f800000u ? b : 0u);
      }
    }
    amax_bits = fin;
  }
  // biased exponent of amax minus emax = shared_exp + 127; fp32 denormals and zero land on 0
  int sb = (int)(amax_bits >> 23) - EMAX;
  sb = sb < 0 ? 0 : (sb > 254 ? 254 : sb);
  const int field = 254 - sb;                                            // exponent field of 2^-shared_exp
  const float mult = __uint_as_float(field > 0 ? (uint32_t)field << 23 : 0x00400000u);
  const uint8_t scale_byte = bad ? 0xFFu : (uint8_t)sb;

  // ---- payload: 8 elements at a time
  uint32_t words[FMT == 8 ? 8 : 4];
#pragma unroll
  for (int o8 = 0; o8 < 4; ++o8) {
    float sv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int idx = o8 * 8 + e;
      sv[e] = __fmul_rn(ElemTraits<T>::to_f(raw[idx / EV].v[idx % EV]), mult);
    }
    if constexpr (FMT == 8) {
      const uint2 w = mx_e4m3x8(sv);
      words[2 * o8] = bad ? 0x7F7F7F7Fu : w.x;
      words[2 * o8 + 1] = bad ? 0x7F7F7F7Fu : w.y;
    } else {
      words[o8] = mx_e2m1x8(sv, bad);
    }
  }
  if constexpr (FMT == 8) {
    uint4* dst = reinterpret_cast<uint4*>(payload + (int64_t)sl.row * k + (int64_t)kb * kMxBlock);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
  } else {
    *reinterpret_cast<uint4*>(payload + (int64_t)sl.row * (k / 2) + (int64_t)kb * (kMxBlock / 2)) =
        make_uint4(words[0], words[1], words[2], words[3]);
  }
  if (scales_rm) scales_rm[(int64_t)sl.row * kb_per_row + kb] = scale_byte;
  if (scales_tiled) {
    scales_tiled[sl.tiled_off] = scale_byte;
    for (int j = 1; j <= pad_kb; ++j) scales_tiled[sl.tiled_off + j] = 0;
  }
}

// blockIdx.x * blockDim.x + threadIdx.x = the K block of the row this thread owns; blockIdx.y strides over row SLOTS,
// two at a time (both blocks' loads are issued before either is worked on).  Without the tiled layout a slot is a
// row.  With it, slots enumerate the layout's rows -- tiles x atoms x 128 -- so that the slots no row maps to get
// their zero padding from the same loop.
template <typename T, int FMT>
__global__ void __launch_bounds__(256) mx_quant_kernel(const T* x, int rows, int k, int64_t ld, uint8_t* payload,
                                                       uint8_t* scales_rm, uint8_t* scales_tiled, int tile_rows, int slots) {
  constexpr int NV = kMxBlock * (int)sizeof(T) / 16;          // 16-byte vectors per block: 4 or 8
  constexpr int EV = 16 / (int)sizeof(T);
  constexpr int U = 2;
  const int kb_per_row = k / kMxBlock;
  const int kb4_per_row = (kb_per_row + 3) / 4;
  const int kb = blockIdx.x * blockDim.x + threadIdx.x;
  const int atoms_per_tile = (tile_rows + 127) / 128;
  // K blocks this thread zero-fills in the tiled layout besides its own: the rest of the last group of four
  const int pad_kb = (scales_tiled && kb == kb_per_row - 1) ? kb4_per_row * 4 - kb_per_row : 0;
  if (kb >= kb_per_row) return;
  for (int slot0 = blockIdx.y; slot0 < slots; slot0 += U * gridDim.y) {
    MxSlot sl[U];
    Vec16<T> raw[U][NV];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int slot = slot0 + u * gridDim.y;
      live[u] = slot < slots;
      sl[u] = mx_slot(live[u] ? slot : 0, scales_tiled != nullptr, rows, tile_rows, atoms_per_tile, kb4_per_row, kb);
      if (live[u] && sl[u].is_row) {
        const T* src = x + (int64_t)sl[u].row * ld + (int64_t)kb * kMxBlock;
#pragma unroll
        for (int i = 0; i < NV; ++i) raw[u][i] = ld_vec_stream(src + i * EV);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      if (!sl[u].is_row) {
        for (int j = 0; j <= pad_kb; ++j) scales_tiled[sl[u].tiled_off + j] = 0;
        continue;
      }
      mx_one_block<T, FMT, NV>(raw[u], sl[u], k, kb, kb_per_row, pad_kb, payload, scales_rm, scales_tiled);
    }
  }
}

template <typename T>
static int run_mx(const T* x, int64_t rows, int64_t k, int64_t ld, int fmt, uint8_t* payload, uint8_t* srm, uint8_t* st,
                  int tile_rows, cudaStream_t stream) {
  if (k >= (1LL << 30)) return AMCT_ERR_UNSUPPORTED;
  const int kb_per_row = (int)(k / kMxBlock);
  const int threads = kb_per_row >= 256 ? 256 : ((kb_per_row + 31) / 32) * 32;
  dim3 grid((unsigned)((kb_per_row + threads - 1) / threads), 1);
  int64_t slots = rows;
  if (st) slots = ((rows + tile_rows - 1) / tile_rows) * ((tile_rows + 127) / 128) * 128;
  if (slots > 0x7fffffffLL) return AMCT_ERR_UNSUPPORTED;
  int64_t gy = (148LL * 2048 / threads + grid.x - 1) / grid.x;          // every SM full of resident blocks
  if (gy > slots) gy = slots;
  if (gy > 65535) gy = 65535;
  grid.y = (unsigned)(gy < 1 ? 1 : gy);
  if (fmt == 8) AMCT_LAUNCH(grid, threads, stream, (x, (int)rows, (int)k, ld, payload, srm, st, tile_rows, (int)slots), mx_quant_kernel<T, 8>);
  else AMCT_LAUNCH(grid, threads, stream, (x, (int)rows, (int)k, ld, payload, srm, st, tile_rows, (int)slots), mx_quant_kernel<T, 4>);
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
  if (!amct::aligned16(x) || (ld_x * esize) % 16 != 0 || reinterpret_cast<uintptr_t>(payload) % 16 != 0 ||
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
