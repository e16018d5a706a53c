// Row-wise integer quantization family: one CTA owns one row of a [rows, K]
// matrix, reads it from HBM exactly once into registers, derives (or is given)
// the quantization parameters of each unit of the row -- the whole row
// (per-token / per-channel), each group of `group` elements, or one tensor-wide
// value -- and writes integer codes, packed nibbles or fake-quantized values.
//
// This one kernel covers, in the reference's terms:
//   * dynamic per-token activation quantization: amax/amin per row
//     (amct_pytorch/quantize_op/minmax_module.py:99-105) -> scale rule
//     (amct_pytorch/quantize_op/utils.py:75-108) -> codes
//     (amct_pytorch/utils/quant_util.py:57-73), with the SmoothQuant multiply
//     of the deploy forward (amct_pytorch/deploy_op/npu_quantization_linear.py:96-97)
//     folded into the load;
//   * weight min/max by granularity (amct_pytorch/quantize_op/utils.py:111-136),
//     including the zero padding of a ragged last group
//     (amct_pytorch/utils/quant_util.py:23-53);
//   * weight codes, INT8 and INT4 (amct_pytorch/utils/quant_util.py:76-93,
//     amct_pytorch/deploy_op/npu_quantization_linear.py:72-87) and the nibble
//     pack (low nibble first, as amct_pytorch/experimental/quantization/
//     DeepSeekV3.2/deploy.py:109-125);
//   * fake quantization in both rounding variants
//     (amct_pytorch/utils/quant_util.py:162-188; amct_pytorch/algorithm/awq.py:129-170).
//
// Algorithmic HBM traffic per row: K*sizeof(T) read + the output bytes written
// (+ K*sizeof(T) of the pre-scale vector, which stays in L2).
#include "common.cuh"

namespace amct {

struct RowParams {
  const void* x;
  int64_t rows, k, ld;         // ld in elements
  const void* pre;             // [k] in T, or nullptr
  int pre_op;                  // AMCT_PRE_*
  int compute;                 // 1: derive scale/offset from this row; 0: read them
  int strategy;                // AMCT_STRATEGY_*
  int group;                   // group size (strategy group)
  int bits;
  int symmetric;
  int rule;                    // AMCT_RULE_* (per-row symmetric int8 only)
  float* scale;                // [1] | [rows] | [rows, ngroups]
  int* offset;                 // same layout, or nullptr when symmetric
  int out_mode;                // AMCT_OUT_*
  void* out;
  int64_t ld_out;              // in output elements (bytes for PACK4)
  int* status;                 // device word, bit 0 set on a non-finite scale
};

__device__ __forceinline__ int units_per_row(const RowParams& p) {
  return p.strategy == AMCT_STRATEGY_GROUP ? (int)((p.k + p.group - 1) / p.group) : 1;
}

template <typename T>
__device__ __forceinline__ float apply_pre(float x, const T* pre, int64_t j, int pre_op) {
  if (pre_op == AMCT_PRE_MUL) return round_to<T>(__fmul_rn(x, ElemTraits<T>::to_f(pre[j])));
  if (pre_op == AMCT_PRE_DIV) return round_to<T>(__fdiv_rn(x, ElemTraits<T>::to_f(pre[j])));
  return x;
}

// Parameters of one unit -> one element's output value(s).
struct UnitQ {
  float scale, offset;
  bool has_offset;
  float recip;                 // rn(1 / scale) when the FMA division applies, else 0
};

// the FMA division of common.cuh needs a normal scale and a normal reciprocal
__device__ __forceinline__ float usable_recip(float s) {
  const float y = __frcp_rn(s);
  const bool ok = fabsf(s) >= 1.17549435e-38f && fabsf(y) >= 1.17549435e-38f && isfinite(y) && isfinite(s);
  return ok ? y : 0.f;
}

// x / scale as the reference's torch division gives it: the branch-free FMA sequence where it is
// valid (and the result is finite), the IEEE division otherwise
__device__ __forceinline__ float quotient(float x, const UnitQ& u) {
  if (u.recip != 0.f) {
    // the correction steps of div_by_recip turn the quotient of -0.0 into +0.0; the fake-quant outputs show that
    // sign, so a zero input takes the plain product, whose sign is the IEEE quotient's
    const float q = x == 0.f ? __fmul_rn(x, u.recip) : div_by_recip(x, u.scale, u.recip);
    if (fabsf(q) <= 3.0e38f) return q;
  }
  return __fdiv_rn(x, u.scale);
}

template <typename T>
__device__ __forceinline__ float level_of(float x, const UnitQ& u, const RowParams& p, float qmin, float qmax) {
  if (p.rule == AMCT_RULE_EXPERIMENTAL) {
    // division carried out in the input dtype (node.py:39-43 on T tensors)
    float t = round_to<T>(quotient(x, u));
    // a 16-bit scale that underflowed to zero makes 0 / 0: the reference's level is NaN there, stored as code 0
    return (t != t) ? 0.f : fminf(fmaxf(rintf(t), qmin), qmax);
  }
  if (p.out_mode == AMCT_OUT_FAKE_AWQ) {
    float t = quotient(x, u);
    if (u.has_offset) t = __fadd_rn(t, u.offset);
    t = round_to<T>(t);                               // awq.py:149 casts before rounding
    return fminf(fmaxf(rintf(t), qmin), qmax);
  }
  float t = quotient(x, u);
  if (u.has_offset) t = __fadd_rn(t, u.offset);
  return fminf(fmaxf(rintf(t), qmin), qmax);
}

template <typename T>
__device__ __forceinline__ float dequant_of(float level, const UnitQ& u) {
  float r = level;
  if (u.has_offset) r = __fsub_rn(r, u.offset);
  return __fmul_rn(r, u.scale);
}

// Shared-memory layout (dynamic): [0, nunits) scale, [nunits, 2*nunits) offset,
// then per-vector min and max (group strategy) or per-warp partials.
template <typename T, int NV>
__global__ void __launch_bounds__(512) quant_rows_vec_kernel(RowParams p) {
  constexpr int E = ElemTraits<T>::kPerVec;
  AMCT_DYNAMIC_SMEM(float, smem);
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int64_t row = blockIdx.x;
  const int nvec = (int)(p.k / E);
  const int nunits = units_per_row(p);
  float* s_scale = smem;
  float* s_off = smem + nunits;
  float* s_red = smem + 2 * nunits;

  const T* xrow = reinterpret_cast<const T*>(p.x) + row * p.ld;
  const T* pre = reinterpret_cast<const T*>(p.pre);

  float val[NV][E];
  bool saw_nan = false;                      // fmaxf/fminf drop NaN; the reference raises on it
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int v = i * nthr + tid;
    if (v < nvec) {
      Vec16<T> raw = ld_vec_stream(xrow + (int64_t)v * E);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        float f = ElemTraits<T>::to_f(raw.v[e]);
        val[i][e] = p.pre_op ? apply_pre<T>(f, pre, (int64_t)v * E + e, p.pre_op) : f;
        saw_nan |= (val[i][e] != val[i][e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) val[i][e] = 0.f;
    }
  }

  if (saw_nan && p.status) atomicOr(p.status, 1);

  const float qmax = (float)((1 << (p.bits - 1)) - 1), qmin = -qmax - 1.f;
  const int64_t ubase = p.strategy == AMCT_STRATEGY_TENSOR ? 0 : row * nunits;

  if (p.compute) {
    if (p.strategy == AMCT_STRATEGY_GROUP) {
      float* vmin = s_red;
      float* vmax = s_red + nvec;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        int v = i * nthr + tid;
        if (v < nvec) {
          float mn = val[i][0], mx = val[i][0];
#pragma unroll
          for (int e = 1; e < E; ++e) { mn = fminf(mn, val[i][e]); mx = fmaxf(mx, val[i][e]); }
          vmin[v] = mn; vmax[v] = mx;
        }
      }
      __syncthreads();
      const int vpg = p.group / E;
      for (int u = tid; u < nunits; u += nthr) {
        int v0 = u * vpg, v1 = min(v0 + vpg, nvec);
        float mn = vmin[v0], mx = vmax[v0];
        for (int v = v0 + 1; v < v1; ++v) { mn = fminf(mn, vmin[v]); mx = fmaxf(mx, vmax[v]); }
        if ((int64_t)(u + 1) * p.group > p.k) { mn = fminf(mn, 0.f); mx = fmaxf(mx, 0.f); }  // zero padding
        float s; int o;
        bool ok = qparams_from_minmax(mx, mn, p.bits, p.symmetric != 0, &s, &o);
        if (!ok && p.status) atomicOr(p.status, 1);
        s_scale[u] = s; s_off[u] = (float)o;
        p.scale[ubase + u] = s;
        if (p.offset) p.offset[ubase + u] = o;
      }
    } else {  // one unit per row
      float mn = INFINITY, mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        int v = i * nthr + tid;
        if (v < nvec) {
#pragma unroll
          for (int e = 0; e < E; ++e) { mn = fminf(mn, val[i][e]); mx = fmaxf(mx, val[i][e]); }
        }
      }
      mn = warp_min(mn); mx = warp_max(mx);
      const int warp = tid >> 5, nwarp = (nthr + 31) >> 5;
      if ((tid & 31) == 0) { s_red[warp] = mn; s_red[32 + warp] = mx; }
      __syncthreads();
      if (tid < 32) {
        mn = tid < nwarp ? s_red[tid] : INFINITY;
        mx = tid < nwarp ? s_red[32 + tid] : -INFINITY;
        mn = warp_min(mn); mx = warp_max(mx);
        if (tid == 0) {
          float s; int o = 0; bool ok;
          if (p.rule == AMCT_RULE_EXPERIMENTAL) {
            float bound = fmaxf(mx, 0.f);
            s = round_to<T>(__fdiv_rn(bound, 127.f));
            if (bound == 0.f) s = 1.f;
            ok = isfinite(s);
          } else {
            ok = qparams_from_minmax(mx, mn, p.bits, p.symmetric != 0, &s, &o);
          }
          if (!ok && p.status) atomicOr(p.status, 1);
          s_scale[0] = s; s_off[0] = (float)o;
          p.scale[ubase] = s;
          if (p.offset) p.offset[ubase] = o;
        }
      }
    }
    __syncthreads();
  } else {
    for (int u = tid; u < nunits; u += nthr) {
      s_scale[u] = p.scale[ubase + u];
      s_off[u] = p.offset ? (float)p.offset[ubase + u] : 0.f;
    }
    __syncthreads();
  }

  if (p.out_mode == AMCT_OUT_NONE) return;
  const bool has_off = p.offset != nullptr;

#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int v = i * nthr + tid;
    if (v >= nvec) continue;
    const int64_t j0 = (int64_t)v * E;
    const int u = p.strategy == AMCT_STRATEGY_GROUP ? (int)(j0 / p.group) : 0;
    UnitQ uq{s_scale[u], s_off[u], has_off, usable_recip(s_scale[u])};
    float lv[E];
#pragma unroll
    for (int e = 0; e < E; ++e) lv[e] = level_of<T>(val[i][e], uq, p, qmin, qmax);

    if (p.out_mode == AMCT_OUT_I8) {
      int8_t* o = reinterpret_cast<int8_t*>(p.out) + row * p.ld_out + j0;
      if constexpr (E == 8) {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          w0 |= (uint32_t)(uint8_t)(int8_t)(int)lv[e] << (8 * e);
          w1 |= (uint32_t)(uint8_t)(int8_t)(int)lv[4 + e] << (8 * e);
        }
        *reinterpret_cast<uint2*>(o) = make_uint2(w0, w1);
      } else {
        uint32_t w0 = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) w0 |= (uint32_t)(uint8_t)(int8_t)(int)lv[e] << (8 * e);
        *reinterpret_cast<uint32_t*>(o) = w0;
      }
    } else if (p.out_mode == AMCT_OUT_I32) {
      int* o = reinterpret_cast<int*>(p.out) + row * p.ld_out + j0;
#pragma unroll
      for (int e = 0; e < E; e += 4)
        *reinterpret_cast<int4*>(o + e) = make_int4((int)lv[e], (int)lv[e + 1], (int)lv[e + 2], (int)lv[e + 3]);
    } else if (p.out_mode == AMCT_OUT_PACK4) {
      uint8_t* o = reinterpret_cast<uint8_t*>(p.out) + row * p.ld_out + j0 / 2;
      uint32_t w = 0;
#pragma unroll
      for (int e = 0; e < E; ++e) w |= (uint32_t)(((int)lv[e] + 8) & 0xF) << (4 * e);
      if constexpr (E == 8) *reinterpret_cast<uint32_t*>(o) = w;
      else *reinterpret_cast<uint16_t*>(o) = (uint16_t)w;
    } else {  // FAKE / FAKE_AWQ
      Vec16<T> r;
#pragma unroll
      for (int e = 0; e < E; ++e) r.v[e] = ElemTraits<T>::from_f(dequant_of<T>(lv[e], uq));
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + row * p.ld_out + j0) =
          *reinterpret_cast<uint4*>(&r);
    }
  }
}

// Any K, any alignment: two passes over the row (the second one hits L2),
// scalar accesses.  Used for ragged shapes only.
template <typename T>
__global__ void __launch_bounds__(256) quant_rows_generic_kernel(RowParams p) {
  AMCT_DYNAMIC_SMEM(float, smem);
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int64_t row = blockIdx.x;
  const int nunits = units_per_row(p);
  float* s_scale = smem;
  float* s_off = smem + nunits;
  int* s_min = reinterpret_cast<int*>(smem + 2 * nunits);
  int* s_max = s_min + nunits;
  const T* xrow = reinterpret_cast<const T*>(p.x) + row * p.ld;
  const T* pre = reinterpret_cast<const T*>(p.pre);
  const float qmax = (float)((1 << (p.bits - 1)) - 1), qmin = -qmax - 1.f;
  const int64_t ubase = p.strategy == AMCT_STRATEGY_TENSOR ? 0 : row * nunits;
  const int64_t gsz = p.strategy == AMCT_STRATEGY_GROUP ? p.group : p.k;

  if (p.compute) {
    for (int u = tid; u < nunits; u += nthr) { s_min[u] = f2ord(INFINITY); s_max[u] = f2ord(-INFINITY); }
    __syncthreads();
    for (int64_t j = tid; j < p.k; j += nthr) {
      float f = apply_pre<T>(ElemTraits<T>::to_f(xrow[j]), pre, j, p.pre_op);
      if (f != f && p.status) atomicOr(p.status, 1);
      int u = (int)(j / gsz);
      atomicMin(&s_min[u], f2ord(f));
      atomicMax(&s_max[u], f2ord(f));
    }
    __syncthreads();
    for (int u = tid; u < nunits; u += nthr) {
      float mn = ord2f(s_min[u]), mx = ord2f(s_max[u]);
      if (p.strategy == AMCT_STRATEGY_GROUP && (int64_t)(u + 1) * p.group > p.k) {
        mn = fminf(mn, 0.f); mx = fmaxf(mx, 0.f);
      }
      float s; int o = 0; bool ok;
      if (p.rule == AMCT_RULE_EXPERIMENTAL) {
        float bound = fmaxf(mx, 0.f);
        s = round_to<T>(__fdiv_rn(bound, 127.f));
        if (bound == 0.f) s = 1.f;
        ok = isfinite(s);
      } else {
        ok = qparams_from_minmax(mx, mn, p.bits, p.symmetric != 0, &s, &o);
      }
      if (!ok && p.status) atomicOr(p.status, 1);
      s_scale[u] = s; s_off[u] = (float)o;
      p.scale[ubase + u] = s;
      if (p.offset) p.offset[ubase + u] = o;
    }
  } else {
    for (int u = tid; u < nunits; u += nthr) {
      s_scale[u] = p.scale[ubase + u];
      s_off[u] = p.offset ? (float)p.offset[ubase + u] : 0.f;
    }
  }
  __syncthreads();
  if (p.out_mode == AMCT_OUT_NONE) return;
  const bool has_off = p.offset != nullptr;

  if (p.out_mode == AMCT_OUT_PACK4) {
    uint8_t* o = reinterpret_cast<uint8_t*>(p.out) + row * p.ld_out;
    for (int64_t b = tid; b < (p.k + 1) / 2; b += nthr) {
      uint32_t byte = 0;
      for (int h = 0; h < 2; ++h) {
        int64_t j = 2 * b + h;
        int q = 0;
        if (j < p.k) {
          float f = apply_pre<T>(ElemTraits<T>::to_f(xrow[j]), pre, j, p.pre_op);
          int u = (int)(j / gsz);
          UnitQ uq{s_scale[u], s_off[u], has_off, 0.f};
          q = (int)level_of<T>(f, uq, p, qmin, qmax);
        }
        byte |= (uint32_t)((q + 8) & 0xF) << (4 * h);
      }
      o[b] = (uint8_t)byte;
    }
    return;
  }
  for (int64_t j = tid; j < p.k; j += nthr) {
    float f = apply_pre<T>(ElemTraits<T>::to_f(xrow[j]), pre, j, p.pre_op);
    int u = (int)(j / gsz);
    UnitQ uq{s_scale[u], s_off[u], has_off, 0.f};
    float lv = level_of<T>(f, uq, p, qmin, qmax);
    if (p.out_mode == AMCT_OUT_I8) reinterpret_cast<int8_t*>(p.out)[row * p.ld_out + j] = (int8_t)(int)lv;
    else if (p.out_mode == AMCT_OUT_I32) reinterpret_cast<int*>(p.out)[row * p.ld_out + j] = (int)lv;
    else reinterpret_cast<T*>(p.out)[row * p.ld_out + j] = ElemTraits<T>::from_f(dequant_of<T>(lv, uq));
  }
}

template <typename T>
static int launch_rows(const RowParams& p, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  if (p.rows == 0 || p.k == 0) return AMCT_OK;
  const int nunits = p.strategy == AMCT_STRATEGY_GROUP ? (int)((p.k + p.group - 1) / p.group) : 1;
  const int64_t out_esize = p.out_mode == AMCT_OUT_I32 ? 4 : (p.out_mode == AMCT_OUT_FAKE || p.out_mode == AMCT_OUT_FAKE_AWQ)
                                                                 ? (int64_t)sizeof(T) : 1;
  // vector path needs 16-byte aligned rows and a whole number of vectors per row and per group
  bool vec_ok = aligned16(p.x) && (p.ld * (int64_t)sizeof(T)) % 16 == 0 && p.k % E == 0 &&
                (p.strategy != AMCT_STRATEGY_GROUP || p.group % E == 0);
  if (p.out_mode != AMCT_OUT_NONE) {
    int64_t out_vec_bytes = p.out_mode == AMCT_OUT_PACK4 ? E / 2 : E * out_esize;
    int64_t align = out_vec_bytes > 16 ? 16 : out_vec_bytes;
    int64_t ld_bytes = p.ld_out * (p.out_mode == AMCT_OUT_PACK4 ? 1 : out_esize);
    vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(p.out) % align == 0) && (ld_bytes % align == 0);
  }
  const int64_t nvec = p.k / E;
  // register-resident rows: at most 512 threads x 8 vectors (32768 16-bit or 16384 fp32 elements)
  if (vec_ok && nvec <= 512 * 8) {
    int threads = 64;
    while (threads < 512 && nvec > (int64_t)threads * 4) threads <<= 1;
    int nv = (int)((nvec + threads - 1) / threads);
    size_t smem = (size_t)(2 * nunits + (p.strategy == AMCT_STRATEGY_GROUP && p.compute ? 2 * nvec : 64)) * sizeof(float);
    dim3 grid((unsigned)p.rows);
#define AMCT_ROWS_CASE(NVC)                                                                     \
  if (nv <= NVC) {                                                                              \
    if (smem > 48 * 1024)                                                                       \
      cudaFuncSetAttribute(quant_rows_vec_kernel<T, NVC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    AMCT_LAUNCH_SMEM(grid, threads, smem, st, (p), quant_rows_vec_kernel<T, NVC>);              \
    AMCT_CHECK_LAUNCH();                                                                        \
    return AMCT_OK;                                                                             \
  }
    AMCT_ROWS_CASE(1) AMCT_ROWS_CASE(2) AMCT_ROWS_CASE(4) AMCT_ROWS_CASE(8)
#undef AMCT_ROWS_CASE
  }
  size_t smem = (size_t)(4 * nunits) * sizeof(float);
  if (smem > 200 * 1024) return AMCT_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(quant_rows_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  AMCT_LAUNCH_SMEM((unsigned)p.rows, 256, smem, st, (p), quant_rows_generic_kernel<T>);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

static int dispatch_rows(int dtype, const RowParams& p, cudaStream_t st) {
  switch (dtype) {
    case AMCT_DTYPE_F32: return launch_rows<float>(p, st);
    case AMCT_DTYPE_F16: return launch_rows<__half>(p, st);
    case AMCT_DTYPE_BF16: return launch_rows<__nv_bfloat16>(p, st);
  }
  return AMCT_ERR_ARG;
}

// group-wise kernel of quant_groups.cu; returns 1 when the shape does not fit it
int quant_groups_try(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld, const void* pre, int pre_op, int compute,
                     int group, int bits, int symmetric, float* scale, int* offset, int out_mode, void* out, int64_t ld_out,
                     int* status, cudaStream_t st);

// streaming kernel of quant_token.cu; returns 1 when the shape does not fit it
int quant_token_try(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, const void* smooth, int8_t* q,
                    int64_t ld_q, float* scale, int* status, cudaStream_t st);

}  // namespace amct

using amct::RowParams;

extern "C" int amct_quant_dynamic_pertoken(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x,
                                           const void* smooth, int rule, int8_t* q, int64_t ld_q, float* scale,
                                           int* status, void* stream) {
  if (rows < 0 || k < 0 || (rows && k && (!x || !q || !scale)) || ld_x < k || ld_q < k) return AMCT_ERR_ARG;
  if (rule != AMCT_RULE_RELEASED && rule != AMCT_RULE_EXPERIMENTAL) return AMCT_ERR_ARG;
  if (rows > 0x7fffffffLL) return AMCT_ERR_UNSUPPORTED;
  if (rule == AMCT_RULE_RELEASED && rows > 0 && k > 0) {
    int rc = amct::quant_token_try(x, dtype, rows, k, ld_x, smooth, q, ld_q, scale, status, (cudaStream_t)stream);
    if (rc != 1) return rc;
  }
  RowParams p{};
  p.x = x; p.rows = rows; p.k = k; p.ld = ld_x;
  p.pre = smooth; p.pre_op = smooth ? AMCT_PRE_MUL : AMCT_PRE_NONE;
  p.compute = 1; p.strategy = AMCT_STRATEGY_CHANNEL; p.group = 0; p.bits = 8; p.symmetric = 1; p.rule = rule;
  p.scale = scale; p.offset = nullptr; p.out_mode = AMCT_OUT_I8; p.out = q; p.ld_out = ld_q; p.status = status;
  return amct::dispatch_rows(dtype, p, (cudaStream_t)stream);
}

extern "C" int amct_quant_rows(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x,
                               const void* pre, int pre_op, int compute, int strategy, int group, int bits,
                               int symmetric, float* scale, int* offset, int out_mode, void* out, int64_t ld_out,
                               int* status, void* stream) {
  if (rows < 0 || k < 0 || ld_x < k || !scale) return AMCT_ERR_ARG;
  if (rows && k && !x) return AMCT_ERR_ARG;
  if (bits != 8 && bits != 4) return AMCT_ERR_ARG;
  if (strategy < AMCT_STRATEGY_TENSOR || strategy > AMCT_STRATEGY_GROUP) return AMCT_ERR_ARG;
  if (strategy == AMCT_STRATEGY_GROUP && group <= 0) return AMCT_ERR_ARG;
  if (strategy == AMCT_STRATEGY_TENSOR && compute) return AMCT_ERR_ARG;   // needs the tensor-wide reduction first
  if (!symmetric && !offset) return AMCT_ERR_ARG;
  if (pre_op != AMCT_PRE_NONE && !pre) return AMCT_ERR_ARG;
  if (out_mode < AMCT_OUT_NONE || out_mode > AMCT_OUT_FAKE_AWQ) return AMCT_ERR_ARG;
  if (out_mode != AMCT_OUT_NONE && (!out || ld_out < (out_mode == AMCT_OUT_PACK4 ? (k + 1) / 2 : k))) return AMCT_ERR_ARG;
  if (out_mode == AMCT_OUT_PACK4 && bits != 4) return AMCT_ERR_ARG;
  if (rows > 0x7fffffffLL) return AMCT_ERR_UNSUPPORTED;
  // per-channel symmetric INT8 codes follow exactly the per-token rule: use the streaming kernel
  if (compute && strategy == AMCT_STRATEGY_CHANNEL && bits == 8 && symmetric && out_mode == AMCT_OUT_I8 &&
      (pre_op == AMCT_PRE_NONE || pre_op == AMCT_PRE_MUL) && rows > 0 && k > 0) {
    int rc = amct::quant_token_try(x, dtype, rows, k, ld_x, pre_op == AMCT_PRE_MUL ? pre : nullptr,
                                   reinterpret_cast<int8_t*>(out), ld_out, scale, status, (cudaStream_t)stream);
    if (rc != 1) return rc;
  }
  // groups that fit inside a warp: the shuffle-based kernel of quant_groups.cu
  if (strategy == AMCT_STRATEGY_GROUP && rows > 0 && k > 0) {
    int rc = amct::quant_groups_try(x, dtype, rows, k, ld_x, pre, pre_op, compute, group, bits, symmetric, scale, offset,
                                    out_mode, out, ld_out, status, (cudaStream_t)stream);
    if (rc != 1) return rc;
  }
  RowParams p{};
  p.x = x; p.rows = rows; p.k = k; p.ld = ld_x; p.pre = pre; p.pre_op = pre_op;
  p.compute = compute; p.strategy = strategy; p.group = group; p.bits = bits; p.symmetric = symmetric;
  p.rule = AMCT_RULE_RELEASED;
  p.scale = scale; p.offset = symmetric ? nullptr : offset;
  p.out_mode = out_mode; p.out = out; p.ld_out = ld_out; p.status = status;
  return amct::dispatch_rows(dtype, p, (cudaStream_t)stream);
}
