// Dynamic per-token symmetric INT8 activation quantization, streaming version.
//
// Same arithmetic as the per-row kernel in quant_rows.cu (row amax/amin as in
// amct_pytorch/quantize_op/minmax_module.py:99-105, scale rule of
// amct_pytorch/quantize_op/utils.py:75-108, codes of amct_pytorch/utils/quant_util.py:57-73,
// optional SmoothQuant multiply of amct_pytorch/deploy_op/npu_quantization_linear.py:96-97),
// restructured so that HBM stays busy:
//   * persistent CTAs; rows are brought into a shared-memory ring by 1-D bulk copies
//     (cp.async.bulk + mbarrier), several rows ahead of the one being processed;
//   * 16-bit inputs stay packed in registers; min / max use the packed NaN-propagating
//     half2 / bfloat162 instructions (one instruction per two elements);
//   * the quotient x / scale is computed from rn(1 / scale) with two FMA correction steps
//     (div_by_recip in common.cuh), which yields the correctly rounded quotient: the value of
//     the IEEE division, without its range checks and without a branch.  (A plain
//     x * rn(1/scale) is not enough: 16-bit inputs make EXACT ties -- x / scale = k + 0.5 --
//     common, and there the product rounds the wrong way a quarter of the time.)
//   * rounding uses the add-1.5*2^23 trick (a full-rate FADD whose low mantissa byte is the
//     two's-complement code) instead of the quarter-rate FRND / F2I conversions; the only
//     clamp this rule can need is the upper one (a negative-dominant row divides by 128).
// Algorithmic HBM traffic per row: K * sizeof(T) read, K + 4 bytes written.
#include "common.cuh"
#include "tc05.cuh"

namespace amct {

struct TokenParams {
  const void* x;
  int64_t rows, k, ld;       // elements
  const void* smooth;        // [k] in T or nullptr
  int8_t* q;
  int64_t ld_q;
  float* scale;
  int* status;
  int slots;                 // ring depth
  int slot_bytes;            // k * sizeof(T), multiple of 16
};

constexpr float kMagic = 12582912.0f;          // 1.5 * 2^23: x + kMagic rounds x to an integer (half to even)

// four quotients (|t| <= 128.0001) -> four int8 codes in one word, little endian
__device__ __forceinline__ uint32_t pack4_s8(float ra, float rb, float rc, float rd) {
  const uint32_t w01 = __byte_perm(__float_as_uint(ra), __float_as_uint(rb), 0x0040);
  const uint32_t w23 = __byte_perm(__float_as_uint(rc), __float_as_uint(rd), 0x0040);
  return __byte_perm(w01, w23, 0x5410);
}

template <typename T> struct Packed;
template <> struct Packed<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  __device__ static V2 vmax(V2 a, V2 b) { return __hmax2_nan(a, b); }
  __device__ static V2 vmin(V2 a, V2 b) { return __hmin2_nan(a, b); }
  __device__ static float lo(V2 a) { return __low2float(a); }
  __device__ static float hi(V2 a) { return __high2float(a); }
  __device__ static V2 mul(V2 a, V2 b) {       // each product rounded once to bf16, like a torch bf16 multiply
    return __floats2bfloat162_rn(__fmul_rn(__low2float(a), __low2float(b)), __fmul_rn(__high2float(a), __high2float(b)));
  }
};
template <> struct Packed<__half> {
  using V2 = __half2;
  __device__ static V2 vmax(V2 a, V2 b) { return __hmax2_nan(a, b); }
  __device__ static V2 vmin(V2 a, V2 b) { return __hmin2_nan(a, b); }
  __device__ static float lo(V2 a) { return __low2float(a); }
  __device__ static float hi(V2 a) { return __high2float(a); }
  __device__ static V2 mul(V2 a, V2 b) {
    return __floats2half2_rn(__fmul_rn(__low2float(a), __low2float(b)), __fmul_rn(__high2float(a), __high2float(b)));
  }
};

__device__ __forceinline__ float max_nan(float a, float b) { return (a != a || b != b) ? NAN : fmaxf(a, b); }
__device__ __forceinline__ float min_nan(float a, float b) { return (a != a || b != b) ? NAN : fminf(a, b); }

// four quotients -> four codes: x / scale by the FMA sequence of div_by_recip (bit-identical to the
// IEEE division), rounded half to even by the magic add
template <bool CLAMP>
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float s, float y) {
  // only a negative-dominant row (divisor 128) can produce a quotient above 127.5
  float ta = div_by_recip(a, s, y), tb = div_by_recip(b, s, y), tc = div_by_recip(c, s, y), td = div_by_recip(d, s, y);
  if (CLAMP) { ta = fminf(ta, 127.f); tb = fminf(tb, 127.f); tc = fminf(tc, 127.f); td = fminf(td, 127.f); }
  return pack4_s8(__fadd_rn(ta, kMagic), __fadd_rn(tb, kMagic), __fadd_rn(tc, kMagic), __fadd_rn(td, kMagic));
}

// second pass over the row held in shared memory: quantize and store
template <typename T, bool CLAMP>
__device__ __forceinline__ void quantize_row(const uint4* src, int8_t* qrow, int nvec, int nthr, int tid, float s, float y) {
#pragma unroll 2
  for (int v = tid; v < nvec; v += nthr) {
    const uint4 raw = src[v];
    if constexpr (sizeof(T) == 2) {
      using P = Packed<T>;
      const typename P::V2* h = reinterpret_cast<const typename P::V2*>(&raw);
      const float f0 = P::lo(h[0]), f1 = P::hi(h[0]), f2 = P::lo(h[1]), f3 = P::hi(h[1]);
      const float f4 = P::lo(h[2]), f5 = P::hi(h[2]), f6 = P::lo(h[3]), f7 = P::hi(h[3]);
      *reinterpret_cast<uint2*>(qrow + (int64_t)v * 8) = make_uint2(quant4<CLAMP>(f0, f1, f2, f3, s, y), quant4<CLAMP>(f4, f5, f6, f7, s, y));
    } else {
      const float* f = reinterpret_cast<const float*>(&raw);
      *reinterpret_cast<uint32_t*>(qrow + (int64_t)v * 4) = quant4<CLAMP>(f[0], f[1], f[2], f[3], s, y);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(512) quant_token_kernel(TokenParams p) {
  constexpr int E = ElemTraits<T>::kPerVec;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full[8];
  __shared__ float part[2][2][16];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;

  const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31, nwarp = nthr >> 5;
  const int nvec = (int)(p.k / E);
  uint8_t* smooth_s = smem + (size_t)p.slots * p.slot_bytes;       // staged smooth vector (if any)
  const int64_t my_rows = p.rows > blockIdx.x ? (p.rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const T* xbase = reinterpret_cast<const T*>(p.x);

  if (tid == 0) {
    abort_word = 0;
    for (int i = 0; i < p.slots; ++i) tc05::mbar_init(tc05::smem_u32(&full[i]), 1);
    tc05::fence_barrier_init();
  }
  if (p.smooth) {
    const uint4* src = reinterpret_cast<const uint4*>(p.smooth);
    for (int v = tid; v < nvec; v += nthr) reinterpret_cast<uint4*>(smooth_s)[v] = __ldg(src + v);
  }
  __syncthreads();
  // rows 0 .. slots-2 are requested up front; row i + slots - 1 is requested during row i
  auto request = [&](int64_t i) {
    const int sl = (int)(i % p.slots);
    const uint32_t bar = tc05::smem_u32(&full[sl]);
    tc05::mbar_expect_tx(bar, (uint32_t)p.slot_bytes);
    tc05::bulk_load_1d(tc05::smem_u32(smem + (size_t)sl * p.slot_bytes), xbase + (blockIdx.x + i * gridDim.x) * p.ld,
                       (uint32_t)p.slot_bytes, bar);
  };
  if (tid == 0)
    for (int64_t i = 0; i < p.slots - 1 && i < my_rows; ++i) request(i);

  int slot = 0;
  uint32_t parity = 0;
  for (int64_t i = 0; i < my_rows; ++i) {
    const int64_t row = blockIdx.x + i * gridDim.x;
    // a timed-out wait does not leave the loop here: every thread goes on to the block barrier
    // below and all of them leave together after it, so no thread is left waiting at a barrier
    tc05::mbar_wait(tc05::smem_u32(&full[slot]), parity, abort_flag);
    uint4* src = reinterpret_cast<uint4*>(smem + (size_t)slot * p.slot_bytes);

    // ---- pass 1: (smooth multiply, written back to shared memory) + min / max
    float mn = INFINITY, mx = -INFINITY;
    if constexpr (sizeof(T) == 2) {
      using P = Packed<T>;
      // every thread owns at least one vector (nvec >= blockDim.x is a launch condition)
      typename P::V2 vmx = reinterpret_cast<const typename P::V2*>(src + tid)[0], vmn = vmx;
      if (p.smooth) vmx = vmn = P::mul(vmx, reinterpret_cast<const typename P::V2*>(reinterpret_cast<const uint4*>(smooth_s) + tid)[0]);
#pragma unroll 4
      for (int v = tid; v < nvec; v += nthr) {
        uint4 raw = src[v];
        typename P::V2* h = reinterpret_cast<typename P::V2*>(&raw);
        if (p.smooth) {
          const uint4 sv = reinterpret_cast<const uint4*>(smooth_s)[v];
          const typename P::V2* sh = reinterpret_cast<const typename P::V2*>(&sv);
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = P::mul(h[e], sh[e]);
          src[v] = raw;
        }
        typename P::V2 a = P::vmax(P::vmax(h[0], h[1]), P::vmax(h[2], h[3]));
        typename P::V2 b = P::vmin(P::vmin(h[0], h[1]), P::vmin(h[2], h[3]));
        vmx = P::vmax(vmx, a);
        vmn = P::vmin(vmn, b);
      }
      mx = max_nan(P::lo(vmx), P::hi(vmx));
      mn = min_nan(P::lo(vmn), P::hi(vmn));
    } else {
      float poison = 0.f;
#pragma unroll 4
      for (int v = tid; v < nvec; v += nthr) {
        uint4 raw = src[v];
        float* f = reinterpret_cast<float*>(&raw);
        if (p.smooth) {
          const float4 sv = reinterpret_cast<const float4*>(smooth_s)[v];
          f[0] = __fmul_rn(f[0], sv.x); f[1] = __fmul_rn(f[1], sv.y); f[2] = __fmul_rn(f[2], sv.z); f[3] = __fmul_rn(f[3], sv.w);
          src[v] = raw;
        }
        mx = fmaxf(mx, fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])));
        mn = fminf(mn, fminf(fminf(f[0], f[1]), fminf(f[2], f[3])));
        // fmaxf / fminf drop NaN: x * 0 is NaN exactly for NaN and Inf inputs, and accumulates
        poison = __fmaf_rn(f[0], 0.f, __fmaf_rn(f[1], 0.f, __fmaf_rn(f[2], 0.f, __fmaf_rn(f[3], 0.f, poison))));
      }
      if (poison != poison) mx = NAN;
    }
    // a NaN anywhere in the row becomes max = +inf: the scale is then infinite and the row is flagged
    if (mx != mx || mn != mn) { mx = INFINITY; mn = 0.f; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    const int buf = (int)(i & 1);
    if (lane == 0) { part[buf][0][warp] = mx; part[buf][1][warp] = mn; }
    __syncthreads();                       // also: every thread has finished pass 2 of the previous row
    if (*abort_flag) break;
    if (tid == 0 && i + p.slots - 1 < my_rows) {
      tc05::fence_proxy_async();           // generic-proxy accesses to that slot are ordered before the bulk copy
      request(i + p.slots - 1);            // into the slot row i-1 just left
    }
    mx = part[buf][0][0]; mn = part[buf][1][0];
    for (int w = 1; w < nwarp; ++w) { mx = fmaxf(mx, part[buf][0][w]); mn = fminf(mn, part[buf][1][w]); }

    // symmetric INT8 rule (amct_pytorch/quantize_op/utils.py:87-91): divisor 127, or 128 when the
    // largest magnitude is negative; a scale below FLT_EPSILON becomes 1
    const float amx = fabsf(mx), amn = fabsf(mn);
    const bool neg_dom = amx < amn;
    float s = __fdiv_rn(neg_dom ? amn : amx, neg_dom ? 128.f : 127.f);
    if (s < AMCT_FLT_EPSILON) s = 1.f;
    if (tid == 0) {
      p.scale[row] = s;
      if (!isfinite(s) && p.status) atomicOr(p.status, 1);
    }
    const float y = __frcp_rn(s);
    int8_t* qrow = p.q + row * p.ld_q;
    // ---- pass 2 (uniform branch per row)
    if (neg_dom) quantize_row<T, true>(src, qrow, nvec, nthr, tid, s, y);
    else quantize_row<T, false>(src, qrow, nvec, nthr, tid, s, y);
    if (++slot == p.slots) { slot = 0; parity ^= 1; }
  }
  if (*abort_flag) {
    if (tid == 0 && p.status) atomicOr(p.status, 2);
    for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let bulk copies already in flight land
  }
}

// Returns AMCT_OK when the streaming kernel took the call, 1 when the shape does not fit
// it (the caller then uses the general row kernel).
template <typename T>
static int launch_token(const TokenParams& p0, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  TokenParams p = p0;
  const int64_t row_bytes = p.k * (int64_t)sizeof(T);
  if (p.k % E || row_bytes % 16 || !aligned16(p.x) || (p.ld * (int64_t)sizeof(T)) % 16) return 1;
  if (reinterpret_cast<uintptr_t>(p.q) % E || p.ld_q % E) return 1;
  if (p.smooth && !aligned16(p.smooth)) return 1;
  if (p.rows < 64 || row_bytes < 2048 || row_bytes > 64 * 1024) return 1;
  const int64_t nvec = p.k / E;
  // up to 8 vectors per thread: more elements per thread amortise the per-row reduction
  const int threads = nvec <= 1024 ? 128 : (nvec <= 2048 ? 256 : 512);
  const int64_t smooth_bytes = p.smooth ? row_bytes : 0;
  // as many CTAs per SM as fit with at least 3 rows in flight each (about 200 KB of shared memory per SM)
  int ctas_per_sm = 2048 / threads > 4 ? 4 : 2048 / threads;
  while (ctas_per_sm > 1 && (200 * 1024 / ctas_per_sm - smooth_bytes - 1024) < 3 * row_bytes) --ctas_per_sm;
  const int64_t budget = 200 * 1024 / ctas_per_sm - smooth_bytes - 1024;
  int slots = (int)(budget / row_bytes);
  if (slots > 8) slots = 8;
  if (slots < 2) return 1;
  p.slots = slots;
  p.slot_bytes = (int)row_bytes;
  const size_t smem = (size_t)slots * row_bytes + smooth_bytes;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t grid = (int64_t)sms * ctas_per_sm;
  if (grid > p.rows) grid = p.rows;
  if (cudaFuncSetAttribute(quant_token_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return AMCT_ERR_CUDA;
  quant_token_kernel<T><<<(unsigned)grid, threads, smem, st>>>(p);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

int quant_token_try(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, const void* smooth, int8_t* q,
                    int64_t ld_q, float* scale, int* status, cudaStream_t st) {
  TokenParams p{};
  p.x = x; p.rows = rows; p.k = k; p.ld = ld_x; p.smooth = smooth; p.q = q; p.ld_q = ld_q; p.scale = scale; p.status = status;
  switch (dtype) {
    case AMCT_DTYPE_F32: return launch_token<float>(p, st);
    case AMCT_DTYPE_F16: return launch_token<__half>(p, st);
    case AMCT_DTYPE_BF16: return launch_token<__nv_bfloat16>(p, st);
  }
  return 1;
}

}  // namespace amct
