// Weight-only INT4 Linear for up to 16 tokens (decode): a weight-streaming kernel.
//
//   out[m, n] = sum_k x[m, k] * w[n, k] + bias[n],   w[n, k] = (code[n, k] + offset[g(k), n]) * scale[g(k), n]
//
// the call torch_npu.npu_weight_quant_batchmatmul at amct_pytorch/deploy_op/weight_npu_quant_module.py:116-117
// serves when the batch is a handful of tokens.  With so few tokens the job is to read the packed weight once, at
// HBM speed, on every SM: the tensor-core tile kernel (gemm_dq_tcgen05.cu) is built around 128-row MMA tiles and one
// CTA per tile and leaves most of the machine idle here.  This kernel instead:
//   * gives every 16 weight rows (one MMA tile) to a CTA of four warps, each warp taking every fourth 128-element
//     step of K: several hundred small CTAs, all resident at once (five per SM), so the whole weight is requested
//     in a single wave and the partial sums of a tile meet in shared memory, in warp order (deterministic; no
//     workspace, no atomics);
//   * streams the codes with 16-byte loads straight into registers, three or four steps ahead of their use (all
//     addresses are per-thread base pointers plus one 32-bit counter that advances by a constant), dequantizes them
//     there with packed 16-bit arithmetic -- (nibble | 0x4300) is the bf16 number 128 + nibble, a packed add of
//     (offset - 8 - 128) is exact, a packed multiply by the scale rounds once: bit for bit the value
//     amct_dequant_weight stores -- and multiplies with mma.sync.m16n8k16 (weights as the 16-row operand, tokens as the
//     8-column one; fp32 accumulation).  With at most 16 tokens the tensor-core work is negligible; what matters is
//     that the dequantization stays near two instructions per weight.
//   * The mask-and-or trick yields the nibbles of a word as the pairs (0,4) (1,5) (2,6) (3,7); a dot product does not
//     care about the order of k, so the activations (a few KB, resident in L1) are loaded 16 bytes at a time and put
//     into that order with four byte permutes.
// 16-bit activations (bf16 / fp16), K % 128 == 0, group a power of two >= 32 (or 0 = one group), 16-byte aligned rows.
#include "common.cuh"

namespace amct {

constexpr int kWsWarps = 4;
constexpr int kWsThreads = kWsWarps * 32;
constexpr int kWsStepK = 128;         // K per warp step: 4 lanes x 32 codes

struct WsParams {
  const void* x;
  const uint8_t* codes;
  const void* scale;
  const void* offset;        // nullable
  const void* bias;          // nullable
  void* out;
  int m, n, k, group_shift;   // log2(group), or 31 for one group over all of K
  int64_t ld_x, ld_codes, ld_out;
  int bias_kind, out_kind;   // AMCT_BIAS_* / AMCT_GEMM_OUT_*
};

template <typename T> struct WsType;
template <> struct WsType<__nv_bfloat16> {
  using P2 = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43004300u;       // bf16 128.0 twice
  static constexpr float kMagicValue = 128.f;
  __device__ static P2 from_float(float v) { return __floats2bfloat162_rn(v, v); }
  __device__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct WsType<__half> {
  using P2 = __half2;
  static constexpr uint32_t kMagic = 0x64006400u;       // fp16 1024.0 twice
  static constexpr float kMagicValue = 1024.f;
  __device__ static P2 from_float(float v) { return __floats2half2_rn(v, v); }
  __device__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

// one 16-bit half of v in both halves of a packed pair
template <typename P2>
__device__ __forceinline__ P2 ws_dup(uint32_t v, uint32_t selector) {
  const uint32_t d = __byte_perm(v, 0u, selector);
  return *reinterpret_cast<const P2*>(&d);
}

// pair s of a word of eight nibbles: codes (s, s + 4) as two 16-bit numbers magic + nibble, then (+ add) * mul
template <typename T>
__device__ __forceinline__ uint32_t ws_pair(uint32_t w, int s, typename WsType<T>::P2 add, typename WsType<T>::P2 mul) {
  using P2 = typename WsType<T>::P2;
  const uint32_t raw = ((w >> (4 * s)) & 0x000F000Fu) | WsType<T>::kMagic;
  const P2 v = __hmul2(__hadd2(*reinterpret_cast<const P2*>(&raw), add), mul);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// NT: token groups of 8 (1: up to 8 tokens, 2: up to 16).
template <typename T, int NT, bool PAIR>
__global__ void __launch_bounds__(kWsThreads, 5) w4a16_stream_kernel(WsParams p) {
  using P2 = typename WsType<T>::P2;
  __shared__ float part[kWsWarps][16][NT * 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  // this CTA's 16 weight rows.  MMA rows r and r + 8 (the two rows a lane holds) are the ADJACENT weight rows
  // n0 + 2r and n0 + 2r + 1, so that their scales (and offsets) are one 4-byte load when n is even and the factor
  // arrays are 4-byte aligned (PAIR; two 2-byte loads otherwise); rows beyond n read the last rows (their
  // results are not stored)
  const int n0 = blockIdx.x * 16;
  const int row_a = min(n0 + 2 * r, PAIR ? p.n - 2 : p.n - 1), row_b = min(row_a + 1, p.n - 1);
  const int b_step = row_b - row_a;
  const T* scale = reinterpret_cast<const T*>(p.scale);
  const T* offset = reinterpret_cast<const T*>(p.offset);
  const T* x = reinterpret_cast<const T*>(p.x);
  const int nsteps = p.k / kWsStepK;                     // this warp takes steps warp, warp + 4, ...
  const int my_steps = nsteps > warp ? (nsteps - warp + kWsWarps - 1) / kWsWarps : 0;
  float acc[NT][4];
#pragma unroll
  for (int g = 0; g < NT; ++g) { acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f; }
  // the activation rows this lane feeds to the MMA as its column (token) lane >> 2 of each group; a token beyond m
  // reads row 0 and is multiplied by nothing (its accumulators are dropped)
  const T* xrow[NT];
#pragma unroll
  for (int gq = 0; gq < NT; ++gq) xrow[gq] = x + (int64_t)((r + 8 * gq) < p.m ? (r + 8 * gq) : 0) * p.ld_x;

  constexpr int DEPTH = NT == 1 ? 4 : 3;                 // steps in flight per warp (32 bytes of codes per thread each); what fits the registers
  uint4 qa[DEPTH], qb[DEPTH];
  uint32_t sc2[DEPTH], of2[DEPTH];                      // the group's scale and offset of both rows travel with the codes
  // Everything that moves from step to step is one 32-bit counter: the first k of this thread's 32 codes (they lie in
  // one group), advancing by kWsWarps * kWsStepK per step.  Code, activation and factor addresses are that counter
  // added to per-thread base pointers fixed here.
  const int k_first = warp * kWsStepK + 32 * c;
  const uint8_t* code_a = p.codes + (int64_t)row_a * p.ld_codes;
  const uint8_t* code_b = p.codes + (int64_t)row_b * p.ld_codes;
  const T* scale_a = scale + row_a;
  const T* offset_a = offset ? offset + row_a : nullptr;
  auto issue = [&](int kk, int slot) {
    qa[slot] = __ldcs(reinterpret_cast<const uint4*>(code_a + (kk >> 1)));
    qb[slot] = __ldcs(reinterpret_cast<const uint4*>(code_b + (kk >> 1)));
    const int g = (kk >> p.group_shift) * p.n;          // fits an int: checked on the host
    if (PAIR) {                                         // rows a (low half) and b
      sc2[slot] = __ldg(reinterpret_cast<const uint32_t*>(scale_a + g));
      if (offset) of2[slot] = __ldg(reinterpret_cast<const uint32_t*>(offset_a + g));
    } else {
      const uint16_t* s16 = reinterpret_cast<const uint16_t*>(scale_a + g);
      sc2[slot] = (uint32_t)__ldg(s16) | ((uint32_t)__ldg(s16 + b_step) << 16);
      if (offset) {
        const uint16_t* o16 = reinterpret_cast<const uint16_t*>(offset_a + g);
        of2[slot] = (uint32_t)__ldg(o16) | ((uint32_t)__ldg(o16 + b_step) << 16);
      }
    }
  };
  // one step: dequantize the 2 x 32 codes of slot d in registers and feed them to the tensor cores
  const P2 bias2 = WsType<T>::from_float(-8.f - WsType<T>::kMagicValue);
  auto step = [&](int kk, int d, bool refill) {
    // offset - 8 - magic is an integer of small magnitude: exact in T, formed with one packed add
    const P2 mul_a = ws_dup<P2>(sc2[d], 0x1010), mul_b = ws_dup<P2>(sc2[d], 0x3232);
    const P2 add_a = offset ? __hadd2(ws_dup<P2>(of2[d], 0x1010), bias2) : bias2;
    const P2 add_b = offset ? __hadd2(ws_dup<P2>(of2[d], 0x3232), bias2) : bias2;
    const uint32_t wa[4] = {qa[d].x, qa[d].y, qa[d].z, qa[d].w};
    const uint32_t wb[4] = {qb[d].x, qb[d].y, qb[d].z, qb[d].w};
    if (refill) issue(kk + DEPTH * kWsWarps * kWsStepK, d);      // the slot just read
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 xv[NT];
#pragma unroll
      for (int gq = 0; gq < NT; ++gq) {
        const uint4 in = __ldg(reinterpret_cast<const uint4*>(xrow[gq] + kk) + j);
        // elements (0,4) (1,5) (2,6) (3,7): the order in which ws_pair hands out the nibbles
        xv[gq] = make_uint4(__byte_perm(in.x, in.z, 0x5410), __byte_perm(in.x, in.z, 0x7632),
                            __byte_perm(in.y, in.w, 0x5410), __byte_perm(in.y, in.w, 0x7632));
      }
      uint32_t a[4];
      a[0] = ws_pair<T>(wa[j], 0, add_a, mul_a); a[1] = ws_pair<T>(wb[j], 0, add_b, mul_b);
      a[2] = ws_pair<T>(wa[j], 1, add_a, mul_a); a[3] = ws_pair<T>(wb[j], 1, add_b, mul_b);
#pragma unroll
      for (int gq = 0; gq < NT; ++gq) WsType<T>::mma(acc[gq], a, xv[gq].x, xv[gq].y);
      a[0] = ws_pair<T>(wa[j], 2, add_a, mul_a); a[1] = ws_pair<T>(wb[j], 2, add_b, mul_b);
      a[2] = ws_pair<T>(wa[j], 3, add_a, mul_a); a[3] = ws_pair<T>(wb[j], 3, add_b, mul_b);
#pragma unroll
      for (int gq = 0; gq < NT; ++gq) WsType<T>::mma(acc[gq], a, xv[gq].z, xv[gq].w);
    }
  };

  constexpr int kStride = kWsWarps * kWsStepK;
#pragma unroll
  for (int i = 0; i < DEPTH; ++i) {
    if (i < my_steps) issue(k_first + i * kStride, i);
  }
  int kk = k_first, left = my_steps;
  // full rounds of DEPTH steps that all refill their slot, then the rounds that run the ring dry
  for (; left >= 2 * DEPTH; left -= DEPTH) {
#pragma unroll
    for (int d = 0; d < DEPTH; ++d, kk += kStride) step(kk, d, true);
  }
  if (left > DEPTH) {                                    // DEPTH < left < 2 DEPTH: the first left - DEPTH steps still refill
#pragma unroll
    for (int d = 0; d < DEPTH; ++d, kk += kStride) step(kk, d, d < left - DEPTH);
    left -= DEPTH;
  }
#pragma unroll
  for (int d = 0; d < DEPTH; ++d, kk += kStride) {
    if (d < left) step(kk, d, false);
  }

  // ---- the four warps' partial sums of the tile meet in shared memory and are added in warp order
#pragma unroll
  for (int gq = 0; gq < NT; ++gq) {
    *reinterpret_cast<float2*>(&part[warp][r][gq * 8 + 2 * c]) = make_float2(acc[gq][0], acc[gq][1]);
    *reinterpret_cast<float2*>(&part[warp][r + 8][gq * 8 + 2 * c]) = make_float2(acc[gq][2], acc[gq][3]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * p.m; i += kWsThreads) {
    const int t = i >> 4, rr = i & 15;                   // consecutive threads: consecutive output channels of one token
    const int n = n0 + rr;
    if (n >= p.n) continue;
    const int mr = (rr >> 1) + 8 * (rr & 1);              // the MMA row that held weight row n0 + rr
    float sum = part[0][mr][t];
#pragma unroll
    for (int w = 1; w < kWsWarps; ++w) sum = __fadd_rn(sum, part[w][mr][t]);
    if (p.bias_kind == AMCT_BIAS_F32) sum = __fadd_rn(sum, reinterpret_cast<const float*>(p.bias)[n]);
    else if (p.bias_kind == AMCT_BIAS_F16) sum = __fadd_rn(sum, __half2float(reinterpret_cast<const __half*>(p.bias)[n]));
    else if (p.bias_kind == AMCT_BIAS_BF16) sum = __fadd_rn(sum, __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]));
    const int64_t o = (int64_t)t * p.ld_out + n;
    if (p.out_kind == AMCT_GEMM_OUT_F32) reinterpret_cast<float*>(p.out)[o] = sum;
    else if (p.out_kind == AMCT_GEMM_OUT_F16) reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(sum);
    else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(sum);
  }
}

template <typename T, int NT>
static int ws_launch(const WsParams& p, bool pair, cudaStream_t st) {
  const unsigned tiles = (unsigned)((p.n + 15) / 16);
  if (pair) w4a16_stream_kernel<T, NT, true><<<tiles, kWsThreads, 0, st>>>(p);
  else w4a16_stream_kernel<T, NT, false><<<tiles, kWsThreads, 0, st>>>(p);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

// Returns AMCT_OK when this kernel took the call, 1 when the shape does not fit it (the caller then uses the
// tensor-core tile kernel), or an error code.
int w4a16_stream_try(const void* x, int dtype, const void* codes, int64_t m, int64_t n, int64_t k, int64_t ld_x,
                     int64_t ld_codes, const void* scale, const void* offset, int group, const void* bias, int bias_kind,
                     void* out, int out_kind, int64_t ld_out, cudaStream_t st) {
  if (m < 1 || m > 16 || n < 1 || k < kWsStepK || k % kWsStepK) return 1;
  if (n > 0x7fffffffLL / 2 || k > 0x3fffffffLL) return 1;
  if (group && (k / group) * n > 0x7fffffffLL) return 1;                        // factor indices are ints in the kernel
  if (group && (group < 32 || (group & (group - 1)) || k % group)) return 1;      // a power of two: the group of a k is a shift
  if (!aligned16(x) || (ld_x * 2) % 16 || !aligned16(codes) || ld_codes % 16) return 1;
  WsParams p{};
  p.x = x; p.codes = reinterpret_cast<const uint8_t*>(codes); p.scale = scale; p.offset = offset; p.bias = bias; p.out = out;
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.group_shift = 31;
  if (group) { p.group_shift = 0; while ((1 << p.group_shift) < group) ++p.group_shift; }
  // both rows' factors with one 4-byte load
  const bool pair = n % 2 == 0 && reinterpret_cast<uintptr_t>(scale) % 4 == 0 && reinterpret_cast<uintptr_t>(offset) % 4 == 0;
  p.ld_x = ld_x; p.ld_codes = ld_codes; p.ld_out = ld_out; p.bias_kind = bias_kind; p.out_kind = out_kind;
  if (dtype == AMCT_DTYPE_BF16) return m <= 8 ? ws_launch<__nv_bfloat16, 1>(p, pair, st) : ws_launch<__nv_bfloat16, 2>(p, pair, st);
  if (dtype == AMCT_DTYPE_F16) return m <= 8 ? ws_launch<__half, 1>(p, pair, st) : ws_launch<__half, 2>(p, pair, st);
  return 1;
}

}  // namespace amct
