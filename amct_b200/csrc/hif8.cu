// HiFloat8 (HiF8) encode / decode.  The reference has no HiFloat8 code; the format is
// the published tapered-precision 8-bit float:
//   bit 7 sign | "dot" prefix code selecting the exponent width D (11 -> 4, 10 -> 3,
//   01 -> 2, 001 -> 1, 0001 -> 0, 0000 -> denormal) | D exponent bits (sign + magnitude
//   under an implicit leading one) | mantissa (1 bit for D = 4, 2 for D = 3, else 3)
//   normal (-1)^S 2^E (1 + M/2^mb), E in [-15, 15]; denormal (-1)^S 2^(M-23), M = 1..7;
//   0x00 = +0, 0x80 = NaN, 0x6F / 0xEF = +-Inf (so the largest finite magnitude is 2^15).
// Encoding: nearest representable value, ties away from zero, finite values saturate to
// +-2^15, magnitudes below 2^-23 flush to +0 (build decisions, pinned by the CPU oracle).
//
// Both directions are elementwise and HBM-bound: encode reads sizeof(T) and writes 1 byte
// per element, decode the reverse.  Decoding is exact in fp16, bf16 and fp32.
#include <type_traits>

#include "common.cuh"

namespace amct {

__device__ __forceinline__ uint32_t hif8_pack(uint32_t sign, int e, uint32_t m) {
  const int ae = e < 0 ? -e : e;
  const uint32_t se = e < 0 ? 1u : 0u;
  int d, mb;
  uint32_t dot;
  if (ae >= 8) { d = 4; mb = 1; dot = 3; }
  else if (ae >= 4) { d = 3; mb = 2; dot = 2; }
  else if (ae >= 2) { d = 2; mb = 3; dot = 1; }
  else if (ae >= 1) { d = 1; mb = 3; dot = 1; }
  else { d = 0; mb = 3; dot = 1; }
  uint32_t efield = 0;
  if (d > 0) efield = (se << (d - 1)) | ((uint32_t)ae - (1u << (d - 1)));
  return (sign << 7) | ((((dot << d) | efield) << mb) | m);
}

__device__ __forceinline__ uint32_t hif8_encode(float x) {
  const uint32_t bits = __float_as_uint(x);
  const uint32_t sign = bits >> 31;
  const int e = (int)((bits >> 23) & 0xFF) - 127;
  const uint32_t man = bits & 0x7FFFFF;
  if (e == 128) return man ? 0x80u : (sign ? 0xEFu : 0x6Fu);       // NaN, +-Inf
  if (e < -23) return 0u;                                          // flush (also fp32 zero / denormals)
  if (e < -15) {                                                   // powers of two 2^-22 .. 2^-16 (or 2^-15 after rounding up)
    const int ed = e == -23 ? -22 : e + (man >= 0x400000u ? 1 : 0);
    const int md = ed + 23;
    return md >= 8 ? hif8_pack(sign, -15, 0) : ((sign << 7) | (uint32_t)md);
  }
  if (e > 15) return sign ? 0xEEu : 0x6Eu;                         // saturate
  const int ae = e < 0 ? -e : e;
  const int mb = ae >= 8 ? 1 : (ae >= 4 ? 2 : 3);
  const int shift = 23 - mb;
  const uint32_t r = man + (1u << (shift - 1));                    // ties away: add half, truncate
  const uint32_t carry = r >> 23;
  const uint32_t m = carry ? 0u : ((r >> shift) & ((1u << mb) - 1));
  const int en = e + (int)carry;
  if (en > 15 || (en == 15 && m == 1)) return sign ? 0xEEu : 0x6Eu;
  return hif8_pack(sign, en, m);
}

__device__ __forceinline__ float hif8_decode(uint32_t code) {
  const uint32_t body = code & 0x7F;
  const float sgn = (code & 0x80) ? -1.f : 1.f;
  int d, nrest;
  if ((body >> 5) == 3) { d = 4; nrest = 5; }
  else if ((body >> 5) == 2) { d = 3; nrest = 5; }
  else if ((body >> 5) == 1) { d = 2; nrest = 5; }
  else if ((body >> 4) == 1) { d = 1; nrest = 4; }
  else if ((body >> 3) == 1) { d = 0; nrest = 3; }
  else {
    const uint32_t m = body & 7;
    if (m == 0) return (code & 0x80) ? __uint_as_float(0x7FC00000u) : 0.f;
    return sgn * __uint_as_float((uint32_t)(127 + (int)m - 23) << 23);
  }
  const uint32_t rest = body & ((1u << nrest) - 1);
  const int mb = nrest - d;
  const uint32_t ebits = rest >> mb, m = rest & ((1u << mb) - 1);
  int e = 0;
  if (d > 0) {
    const int mag = (1 << (d - 1)) | (int)(ebits & ((1u << (d - 1)) - 1));
    e = ((ebits >> (d - 1)) & 1) ? -mag : mag;
  }
  if (e == 15 && m == 1) return sgn * __uint_as_float(0x7F800000u);
  return sgn * __uint_as_float(((uint32_t)(127 + e) << 23) | (m << (23 - mb)));
}

// 8 consecutive values -> memory (dst 16-byte aligned for 16-bit T, 32-byte data for fp32)
template <typename T> __device__ __forceinline__ void store8(T* dst, const float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    Vec16<T> r;
#pragma unroll
    for (int e = 0; e < 8; ++e) r.v[e] = ElemTraits<T>::from_f(f[e]);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(&r);
  } else {
    *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
}

// With ties rounded away from zero, the code of x depends only on its sign, its exponent and
// the top four mantissa bits (the deepest rounding position is mantissa bit 19).  So a
// 4096-entry table indexed by bits [30:19] of the fp32 pattern encodes any magnitude; NaN
// payloads hidden in lower mantissa bits are the one case checked separately.
__device__ __forceinline__ uint32_t hif8_lookup(const uint8_t* tab, float x) {
  const uint32_t bits = __float_as_uint(x);
  const uint32_t abits = bits & 0x7fffffffu;
  uint32_t t = tab[abits >> 19];
  t = t ? (t | ((bits >> 24) & 0x80u)) : 0u;            // -0 and flushed negatives are +0 (0x80 means NaN)
  return abits > 0x7f800000u ? 0x80u : t;
}

// The two tables, built once per device by hif8_init_tables and copied into shared memory by every
// CTA (building the 4096 entries in each CTA cost as much as the encoding itself).
static __device__ __align__(16) uint8_t g_hif8_tab[4096];
static __device__ __align__(16) float g_hif8_dec[256];
// bfloat16 input needs no detour through fp32: its top 13 bits (sign, exponent, four mantissa bits) ARE the table
// index.  g_hif8_tab13[i] = code of the bf16 pattern i << 3 (sign included, -0 and flushed negatives are code 0);
// g_hif8_fq13[i] = bf16 pattern of decode(that code): fake quantization bf16 -> bf16 is one lookup.
// Decoded values as 16-bit patterns (decoding is exact in both types): index 0 = bf16, 1 = fp16.
static __device__ __align__(16) uint8_t g_hif8_tab13[8192];
static __device__ __align__(16) uint16_t g_hif8_fq13[8192];
static __device__ __align__(16) uint16_t g_hif8_dec16[2][256];

__global__ void hif8_init_tables() {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < 4096) g_hif8_tab[i] = (uint8_t)hif8_encode(__uint_as_float((uint32_t)i << 19));
  if (i < 8192) {
    const uint32_t code = hif8_encode(__uint_as_float((uint32_t)i << 19));
    g_hif8_tab13[i] = (uint8_t)code;
    const __nv_bfloat16 v = __float2bfloat16_rn(hif8_decode(code));
    g_hif8_fq13[i] = *reinterpret_cast<const uint16_t*>(&v);
  }
  if (i < 256) {
    const float d = hif8_decode(i);
    g_hif8_dec[i] = d;
    const __nv_bfloat16 b = __float2bfloat16_rn(d);
    const __half h = __float2half_rn(d);
    g_hif8_dec16[0][i] = *reinterpret_cast<const uint16_t*>(&b);
    g_hif8_dec16[1][i] = *reinterpret_cast<const uint16_t*>(&h);
  }
}

// Launch-ordered on `st` before the first use on each device; repeating it is harmless.
static int ensure_tables(cudaStream_t st) {
  static bool done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return AMCT_ERR_CUDA;
  if (dev >= 0 && dev < 64 && done[dev]) return AMCT_OK;
  // the tables must be complete before any later kernel on any stream reads them
  AMCT_LAUNCH(32, 256, st, (), hif8_init_tables);
  AMCT_CHECK_LAUNCH();
  if (cudaStreamSynchronize(st) != cudaSuccess) return AMCT_ERR_CUDA;
  if (dev >= 0 && dev < 64) done[dev] = true;
  return AMCT_OK;
}

// mode 0: encode x -> codes;  mode 1: fake-quantize x -> decode(encode(x)) in T
template <typename T, int MODE>
__global__ void __launch_bounds__(256) hif8_encode_kernel(const T* x, int64_t n, uint8_t* codes, T* fake) {
  __shared__ __align__(16) uint8_t tab[4096];
  __shared__ float dec[256];
  reinterpret_cast<uint4*>(tab)[threadIdx.x] = reinterpret_cast<const uint4*>(g_hif8_tab)[threadIdx.x];
  if (MODE == 1) dec[threadIdx.x] = g_hif8_dec[threadIdx.x];
  __syncthreads();
  constexpr int U = 2;
  const int64_t nv = n / 8;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nv; v0 += stride * U) {
    float f[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = v0 + u * stride;
      if (v < nv) {
        if constexpr (sizeof(T) == 2) {
          Vec16<T> raw = ld_vec_stream(x + v * 8);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[u][e] = ElemTraits<T>::to_f(raw.v[e]);
        } else {
          Vec16<T> r0 = ld_vec_stream(x + v * 8), r1 = ld_vec_stream(x + v * 8 + 4);
#pragma unroll
          for (int e = 0; e < 4; ++e) { f[u][e] = ElemTraits<T>::to_f(r0.v[e]); f[u][4 + e] = ElemTraits<T>::to_f(r1.v[e]); }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = v0 + u * stride;
      if (v >= nv) break;
      uint32_t c[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) c[e] = hif8_lookup(tab, f[u][e]);
      if constexpr (MODE == 0) {
        uint32_t lo = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24), hi = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
        *reinterpret_cast<uint2*>(codes + v * 8) = make_uint2(lo, hi);
      } else {
        float d[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) d[e] = dec[c[e]];
        store8<T>(fake + v * 8, d);
      }
    }
  }
  // tail (n not a multiple of 8): the first threads of block 0 take one element each
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nv * 8)) {
    const int64_t i = nv * 8 + threadIdx.x;
    const uint32_t c = hif8_lookup(tab, ElemTraits<T>::to_f(x[i]));
    if constexpr (MODE == 0) codes[i] = (uint8_t)c;
    else fake[i] = ElemTraits<T>::from_f(hif8_decode(c));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) hif8_decode_kernel(const uint8_t* codes, int64_t n, T* out) {
  __shared__ float table[256];
  table[threadIdx.x] = g_hif8_dec[threadIdx.x];
  __syncthreads();
  const int64_t nv = n / 8;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += stride) {
    const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(codes + v * 8));
    float d[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) d[e] = table[((e < 4 ? raw.x : raw.y) >> (8 * (e & 3))) & 0xFF];
    store8<T>(out + v * 8, d);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nv * 8)) {
    const int64_t i = nv * 8 + threadIdx.x;
    out[i] = ElemTraits<T>::from_f(table[codes[i]]);
  }
}

// bfloat16 input: the table index is cut straight out of the 16-bit pattern -- (w >> 3) & 0x1FFF and w >> 19 for the two
// halves of a word -- and the entry already carries the sign.  The one case the index cannot tell apart is a NaN
// whose payload sits in the three lowest mantissa bits only (it shares its index with Inf); a vector that holds any
// all-ones exponent, found with three integer instructions per word, is redone element by element.
// MODE 0: codes; MODE 1: fake quantization (bf16 out).
template <int MODE>
__global__ void __launch_bounds__(256) hif8_encode_bf16_kernel(const __nv_bfloat16* x, int64_t n, uint8_t* codes,
                                                               __nv_bfloat16* fake) {
  using Entry = typename std::conditional<MODE == 0, uint8_t, uint16_t>::type;
  __shared__ __align__(16) Entry tab[8192];
  {
    const uint4* src = reinterpret_cast<const uint4*>(MODE == 0 ? reinterpret_cast<const void*>(g_hif8_tab13)
                                                                : reinterpret_cast<const void*>(g_hif8_fq13));
    constexpr int kVecs = 8192 * (int)sizeof(Entry) / 16;
    for (int i = threadIdx.x; i < kVecs; i += blockDim.x) reinterpret_cast<uint4*>(tab)[i] = src[i];
  }
  __syncthreads();
  constexpr int U = 4;                                  // 16-byte vectors in flight per thread
  const int64_t nv = n / 8;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nv; v0 += stride * U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = v0 + u * stride;
      raw[u] = v < nv ? __ldcs(reinterpret_cast<const uint4*>(x) + v) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = v0 + u * stride;
      if (v >= nv) break;
      const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
      uint32_t c[8], special = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        c[2 * j] = tab[(w[j] >> 3) & 0x1FFFu];
        c[2 * j + 1] = tab[w[j] >> 19];
        special |= ((w[j] & 0x7F807F80u) + 0x00800080u) & 0x80008000u;      // a half with exponent 0xFF
      }
      if (special) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t h = (w[e >> 1] >> (16 * (e & 1))) & 0x7FFFu;
          if (h > 0x7F80u) c[e] = MODE == 0 ? 0x80u : 0x7FC0u;                // NaN whatever its payload
        }
      }
      if constexpr (MODE == 0) {
        const uint32_t lo = __byte_perm(__byte_perm(c[0], c[1], 0x0040), __byte_perm(c[2], c[3], 0x0040), 0x5410);
        const uint32_t hi = __byte_perm(__byte_perm(c[4], c[5], 0x0040), __byte_perm(c[6], c[7], 0x0040), 0x5410);
        *reinterpret_cast<uint2*>(codes + v * 8) = make_uint2(lo, hi);
      } else {
        *reinterpret_cast<uint4*>(fake + v * 8) = make_uint4(__byte_perm(c[0], c[1], 0x5410), __byte_perm(c[2], c[3], 0x5410),
                                                             __byte_perm(c[4], c[5], 0x5410), __byte_perm(c[6], c[7], 0x5410));
      }
    }
  }
  // tail (n not a multiple of 8): the first threads of block 0 take one element each
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nv * 8)) {
    const int64_t i = nv * 8 + threadIdx.x;
    const uint32_t h = *reinterpret_cast<const uint16_t*>(x + i);
    uint32_t c = tab[h >> 3];
    if ((h & 0x7FFFu) > 0x7F80u) c = MODE == 0 ? 0x80u : 0x7FC0u;
    if constexpr (MODE == 0) codes[i] = (uint8_t)c;
    else *reinterpret_cast<uint16_t*>(fake + i) = (uint16_t)c;
  }
}

// Decoding into a 16-bit type: 16 codes per thread (one 16-byte load, two 16-byte stores), values taken as 16-bit
// patterns from a 512-byte table.
template <typename T>
__global__ void __launch_bounds__(256) hif8_decode16_kernel(const uint8_t* codes, int64_t n, T* out) {
  __shared__ uint16_t table[256];
  table[threadIdx.x] = g_hif8_dec16[std::is_same<T, __half>::value ? 1 : 0][threadIdx.x];
  __syncthreads();
  const int64_t nv = n / 16;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += stride) {
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(codes) + v);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t d0 = table[w[j] & 0xFFu], d1 = table[(w[j] >> 8) & 0xFFu];
      const uint32_t d2 = table[(w[j] >> 16) & 0xFFu], d3 = table[w[j] >> 24];
      o[2 * j] = __byte_perm(d0, d1, 0x5410);
      o[2 * j + 1] = __byte_perm(d2, d3, 0x5410);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + v * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nv * 16)) {
    const int64_t i = nv * 16 + threadIdx.x;
    *reinterpret_cast<uint16_t*>(out + i) = table[codes[i]];
  }
}

static unsigned grid_for(int64_t n) {
  int64_t blocks = (n / 8 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return (unsigned)blocks;
}

template <typename T>
static int run_encode(const T* x, int64_t n, uint8_t* codes, T* fake, cudaStream_t st) {
  const int rc = ensure_tables(st);
  if (rc != AMCT_OK) return rc;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    if (codes) AMCT_LAUNCH(grid_for(n), 256, st, (x, n, codes, nullptr), hif8_encode_bf16_kernel<0>);
    else AMCT_LAUNCH(grid_for(n), 256, st, (x, n, nullptr, fake), hif8_encode_bf16_kernel<1>);
    AMCT_CHECK_LAUNCH();
    return AMCT_OK;
  }
  if (codes) AMCT_LAUNCH(grid_for(n), 256, st, (x, n, codes, nullptr), hif8_encode_kernel<T, 0>);
  else AMCT_LAUNCH(grid_for(n), 256, st, (x, n, nullptr, fake), hif8_encode_kernel<T, 1>);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

// x [n] contiguous -> HiF8 codes [n] (codes != NULL) or fake-quantized values in x's dtype (fake != NULL).
extern "C" int amct_hif8_encode(const void* x, int dtype, int64_t n, void* codes, void* fake, void* stream) {
  if (n < 0) return AMCT_ERR_ARG;
  if (n == 0) return AMCT_OK;                                 // an empty tensor has no storage: its pointers are null
  if ((!codes) == (!fake) || !x) return AMCT_ERR_ARG;
  if (!amct::aligned16(x) || (codes && reinterpret_cast<uintptr_t>(codes) % 8) || (fake && !amct::aligned16(fake)))
    return AMCT_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* c = reinterpret_cast<uint8_t*>(codes);
  switch (dtype) {
    case AMCT_DTYPE_F32: return amct::run_encode<float>((const float*)x, n, c, (float*)fake, st);
    case AMCT_DTYPE_F16: return amct::run_encode<__half>((const __half*)x, n, c, (__half*)fake, st);
    case AMCT_DTYPE_BF16: return amct::run_encode<__nv_bfloat16>((const __nv_bfloat16*)x, n, c, (__nv_bfloat16*)fake, st);
  }
  return AMCT_ERR_ARG;
}

extern "C" int amct_hif8_decode(const void* codes, int64_t n, int dtype, void* out, void* stream) {
  if (n < 0) return AMCT_ERR_ARG;
  if (n == 0) return AMCT_OK;
  if (!codes || !out) return AMCT_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(codes) % 8 || !amct::aligned16(out)) return AMCT_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const uint8_t* c = reinterpret_cast<const uint8_t*>(codes);
  const int rc = amct::ensure_tables(st);
  if (rc != AMCT_OK) return rc;
  const unsigned grid = amct::grid_for(n);
  const bool wide = amct::aligned16(codes);                  // 16 codes per thread
  switch (dtype) {
    case AMCT_DTYPE_F32: AMCT_LAUNCH(grid, 256, st, (c, n, (float*)out), amct::hif8_decode_kernel<float>); break;
    case AMCT_DTYPE_F16:
      if (wide) AMCT_LAUNCH(amct::grid_for(n / 2), 256, st, (c, n, (__half*)out), amct::hif8_decode16_kernel<__half>);
      else AMCT_LAUNCH(grid, 256, st, (c, n, (__half*)out), amct::hif8_decode_kernel<__half>);
      break;
    case AMCT_DTYPE_BF16:
      if (wide) AMCT_LAUNCH(amct::grid_for(n / 2), 256, st, (c, n, (__nv_bfloat16*)out), amct::hif8_decode16_kernel<__nv_bfloat16>);
      else AMCT_LAUNCH(grid, 256, st, (c, n, (__nv_bfloat16*)out), amct::hif8_decode_kernel<__nv_bfloat16>);
      break;
    default: return AMCT_ERR_ARG;
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}
