// Observer reductions and small helpers of the calibration / convert steps.
//
//   amct_minmax        tensor-wide and per-column min/max with running merge
//                      (amct_pytorch/quantize_op/minmax_module.py:96-110,
//                       amct_pytorch/quantize_op/smooth_quant_module.py:79-91)
//   amct_scale_offset  the scale/offset rule on arrays of (max, min)
//                      (amct_pytorch/quantize_op/utils.py:75-108)
//   amct_rowsum_i8     integer row sums of the weight codes, the exact form of the
//                      matmul that builds offset_bias
//                      (amct_pytorch/deploy_op/npu_quantization_linear.py:56-59)
//   amct_transpose_i8  byte-matrix transpose (npu_quantization_linear.py:54)
//
// All of them are HBM-bound single-read reductions: algorithmic traffic is the
// input size; partials live in a caller-provided workspace.
#include <mutex>

#include "common.cuh"

namespace amct {

constexpr int kMaxRowChunks = 64;
constexpr int kTensorBlocks = 1184;          // 148 SMs x 8

// torch.amax / amin / maximum / minimum return NaN when an operand is NaN, fmaxf / fminf return the other
// operand.  The inner loops use the fast instructions and remember that a NaN went by; everything that
// combines partial results uses these, so a NaN reaches the output and the scale rule refuses it as the
// reference does.
__device__ __forceinline__ float nan_max(float a, float b) { return (a != a || b != b) ? NAN : fmaxf(a, b); }
__device__ __forceinline__ float nan_min(float a, float b) { return (a != a || b != b) ? NAN : fminf(a, b); }
// The running merge of the observers is torch.where(batch > running, batch, running)
// (amct_pytorch/quantize_op/minmax_module.py:108-109, smooth_quant_module.py:90-91): a NaN batch value loses the
// comparison and is dropped, a NaN running value stays.
__device__ __forceinline__ float merge_max(float batch, float running) { return batch > running ? batch : running; }
__device__ __forceinline__ float merge_min(float batch, float running) { return batch < running ? batch : running; }
__device__ __forceinline__ float warp_nan_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = nan_max(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_nan_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = nan_min(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) minmax_tensor_kernel(const T* x, int64_t rows, int64_t k, int64_t ld,
                                                            float* part, int* status) {
  constexpr int E = VEC ? ElemTraits<T>::kPerVec : 1;
  float mn = INFINITY, mx = -INFINITY;
  bool nan = false;
  const int64_t nv = k / E;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* row = x + r * ld;
    for (int64_t v = threadIdx.x; v < nv; v += blockDim.x) {
      if constexpr (VEC) {
        Vec16<T> raw = ld_vec_stream(row + v * E);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          float f = ElemTraits<T>::to_f(raw.v[e]);
          mn = fminf(mn, f); mx = fmaxf(mx, f); nan |= (f != f);
        }
      } else {
        float f = ElemTraits<T>::to_f(row[v]);
        mn = fminf(mn, f); mx = fmaxf(mx, f); nan |= (f != f);
      }
    }
  }
  __shared__ float s[64];
  if (nan) { mn = NAN; mx = NAN; }
  mn = warp_nan_min(mn); mx = warp_nan_max(mx);
  int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { s[w] = mn; s[32 + w] = mx; }
  if (nan && status) atomicOr(status, 1);
  __syncthreads();
  if (threadIdx.x < 32) {
    int nw = blockDim.x >> 5;
    mn = threadIdx.x < nw ? s[threadIdx.x] : INFINITY;
    mx = threadIdx.x < nw ? s[32 + threadIdx.x] : -INFINITY;
    mn = warp_nan_min(mn); mx = warp_nan_max(mx);
    if (threadIdx.x == 0) { part[blockIdx.x] = mn; part[gridDim.x + blockIdx.x] = mx; }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) minmax_tensor_final_kernel(const float* part, int nblocks, int merge,
                                                                  T* out_min, T* out_max) {
  float mn = INFINITY, mx = -INFINITY;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) { mn = nan_min(mn, part[i]); mx = nan_max(mx, part[nblocks + i]); }
  __shared__ float s[64];
  mn = warp_nan_min(mn); mx = warp_nan_max(mx);
  int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { s[w] = mn; s[32 + w] = mx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) { mn = nan_min(mn, s[i]); mx = nan_max(mx, s[32 + i]); }
    if (merge) {
      mn = merge_min(mn, ElemTraits<T>::to_f(*out_min));
      mx = merge_max(mx, ElemTraits<T>::to_f(*out_max));
    }
    *out_min = ElemTraits<T>::from_f(mn);       // exact: the extremum is one of the inputs
    *out_max = ElemTraits<T>::from_f(mx);
  }
}

// packed NaN-propagating min / max of two 16-bit values per instruction
__device__ __forceinline__ __nv_bfloat162 pmax2(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmax2_nan(a, b); }
__device__ __forceinline__ __nv_bfloat162 pmin2(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmin2_nan(a, b); }
__device__ __forceinline__ __half2 pmax2(__half2 a, __half2 b) { return __hmax2_nan(a, b); }
__device__ __forceinline__ __half2 pmin2(__half2 a, __half2 b) { return __hmin2_nan(a, b); }
template <typename T> struct Pair2;
template <> struct Pair2<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Pair2<__half> { using type = __half2; };

// grid (column blocks, row chunks); each thread owns E adjacent columns and walks its row chunk
// four rows at a time (four independent 16-byte loads in flight).  16-bit inputs stay packed: one
// NaN-propagating min and max instruction per two elements, a NaN shows in the result.
template <typename T, bool VEC>
__global__ void __launch_bounds__(128) minmax_column_kernel(const T* x, int64_t rows, int64_t k, int64_t ld,
                                                            float* part, int* status) {
  constexpr int E = VEC ? ElemTraits<T>::kPerVec : 1;
  constexpr int U = 4;
  const int64_t c0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * E;
  if (c0 >= k) return;
  const int64_t per = (rows + gridDim.y - 1) / gridDim.y;
  const int64_t r0 = blockIdx.y * per, r1 = min(rows, r0 + per);
  float mn[E], mx[E];
  bool nan = false;
  if constexpr (VEC && sizeof(T) == 2) {
    using P2 = typename Pair2<T>::type;
    P2 pmn[E / 2], pmx[E / 2];
    {
      const Vec16<T> first = ld_vec(x + (r0 < r1 ? r0 : 0) * ld + c0);       // seed with a real row
      const P2* h = reinterpret_cast<const P2*>(&first);
#pragma unroll
      for (int e = 0; e < E / 2; ++e) { pmn[e] = h[e]; pmx[e] = h[e]; }
    }
    int64_t r = r0;
    for (; r + U <= r1; r += U) {
      Vec16<T> raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) raw[u] = ld_vec_stream(x + (r + u) * ld + c0);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const P2* h = reinterpret_cast<const P2*>(&raw[u]);
#pragma unroll
        for (int e = 0; e < E / 2; ++e) { pmn[e] = pmin2(pmn[e], h[e]); pmx[e] = pmax2(pmx[e], h[e]); }
      }
    }
    for (; r < r1; ++r) {
      const Vec16<T> raw = ld_vec_stream(x + r * ld + c0);
      const P2* h = reinterpret_cast<const P2*>(&raw);
#pragma unroll
      for (int e = 0; e < E / 2; ++e) { pmn[e] = pmin2(pmn[e], h[e]); pmx[e] = pmax2(pmx[e], h[e]); }
    }
#pragma unroll
    for (int e = 0; e < E / 2; ++e) {
      mn[2 * e] = __low2float(pmn[e]); mn[2 * e + 1] = __high2float(pmn[e]);
      mx[2 * e] = __low2float(pmx[e]); mx[2 * e + 1] = __high2float(pmx[e]);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      nan |= (mn[e] != mn[e]) || (mx[e] != mx[e]);
      if (r0 >= r1) { mn[e] = INFINITY; mx[e] = -INFINITY; }               // empty chunk
    }
  } else {
    unsigned nan_cols = 0;                                                   // bit e: column c0 + e has seen a NaN
#pragma unroll
    for (int e = 0; e < E; ++e) { mn[e] = INFINITY; mx[e] = -INFINITY; }
    int64_t r = r0;
    if constexpr (VEC) {
      for (; r + U <= r1; r += U) {
        Vec16<T> raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) raw[u] = ld_vec_stream(x + (r + u) * ld + c0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int e = 0; e < E; ++e) {
            const float f = ElemTraits<T>::to_f(raw[u].v[e]);
            mn[e] = fminf(mn[e], f); mx[e] = fmaxf(mx[e], f); nan_cols |= (unsigned)(f != f) << e;
          }
        }
      }
    }
    for (; r < r1; ++r) {
      if constexpr (VEC) {
        const Vec16<T> raw = ld_vec_stream(x + r * ld + c0);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float f = ElemTraits<T>::to_f(raw.v[e]);
          mn[e] = fminf(mn[e], f); mx[e] = fmaxf(mx[e], f); nan_cols |= (unsigned)(f != f) << e;
        }
      } else {
        const float f = ElemTraits<T>::to_f(x[r * ld + c0]);
        mn[0] = fminf(mn[0], f); mx[0] = fmaxf(mx[0], f); nan_cols |= (unsigned)(f != f);
      }
    }
    nan = nan_cols != 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if ((nan_cols >> e) & 1u) { mn[e] = NAN; mx[e] = NAN; }
    }
  }
  if (nan && status) atomicOr(status, 1);
  float* pmin = part + (int64_t)blockIdx.y * k;
  float* pmax = part + (int64_t)(gridDim.y + blockIdx.y) * k;
#pragma unroll
  for (int e = 0; e < E; ++e) { pmin[c0 + e] = mn[e]; pmax[c0 + e] = mx[e]; }
}

template <typename T>
__global__ void minmax_column_final_kernel(const float* part, int chunks, int64_t k, int merge, T* out_min, T* out_max) {
  int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= k) return;
  float mn = INFINITY, mx = -INFINITY;
  for (int i = 0; i < chunks; ++i) {
    mn = nan_min(mn, part[(int64_t)i * k + c]);
    mx = nan_max(mx, part[(int64_t)(chunks + i) * k + c]);
  }
  if (merge) {
    mn = merge_min(mn, ElemTraits<T>::to_f(out_min[c]));
    mx = merge_max(mx, ElemTraits<T>::to_f(out_max[c]));
  }
  out_min[c] = ElemTraits<T>::from_f(mn);
  out_max[c] = ElemTraits<T>::from_f(mx);
}

template <typename T>
static int run_minmax(const T* x, int64_t rows, int64_t k, int64_t ld, int axis, int merge, T* out_min, T* out_max,
                      float* ws, int* status, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  const bool vec = aligned16(x) && (ld * (int64_t)sizeof(T)) % 16 == 0 && k % E == 0;
  if (axis == AMCT_AXIS_TENSOR) {
    int blocks = (int)(rows < kTensorBlocks ? rows : kTensorBlocks);
    if (vec) AMCT_LAUNCH(blocks, 256, st, (x, rows, k, ld, ws, status), minmax_tensor_kernel<T, true>);
    else AMCT_LAUNCH(blocks, 256, st, (x, rows, k, ld, ws, status), minmax_tensor_kernel<T, false>);
    AMCT_CHECK_LAUNCH();
    AMCT_LAUNCH(1, 256, st, (ws, blocks, merge, out_min, out_max), minmax_tensor_final_kernel<T>);
    AMCT_CHECK_LAUNCH();
    return AMCT_OK;
  }
  const int ev = vec ? E : 1;
  const int64_t cols_per_block = 128LL * ev;
  const unsigned cblocks = (unsigned)((k + cols_per_block - 1) / cols_per_block);
  // enough row chunks to fill the GPU, at most kMaxRowChunks, at least 8 rows each
  int chunks = (int)((148 * 8 + cblocks - 1) / cblocks);
  if (chunks > kMaxRowChunks) chunks = kMaxRowChunks;
  if ((int64_t)chunks * 8 > rows) chunks = (int)((rows + 7) / 8);
  if (chunks < 1) chunks = 1;
  dim3 grid(cblocks, (unsigned)chunks);
  if (vec) AMCT_LAUNCH(grid, 128, st, (x, rows, k, ld, ws, status), minmax_column_kernel<T, true>);
  else AMCT_LAUNCH(grid, 128, st, (x, rows, k, ld, ws, status), minmax_column_kernel<T, false>);
  AMCT_CHECK_LAUNCH();
  AMCT_LAUNCH((unsigned)((k + 255) / 256), 256, st, (ws, chunks, k, merge, out_min, out_max), minmax_column_final_kernel<T>);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}


// One CTA per row: min/max of each row, optional element-wise pre-scale in T.
template <typename T, bool VEC>
__global__ void __launch_bounds__(128) minmax_rows_kernel(const T* x, int64_t k, int64_t ld, const T* pre, int pre_op,
                                                          int merge, T* out_min, T* out_max, int* status) {
  constexpr int E = VEC ? ElemTraits<T>::kPerVec : 1;
  const T* row = x + (int64_t)blockIdx.x * ld;
  float mn = INFINITY, mx = -INFINITY;
  bool nan = false;
  for (int64_t v = threadIdx.x; v < k / E; v += blockDim.x) {
    float f[E];
    if constexpr (VEC) {
      Vec16<T> raw = ld_vec_stream(row + v * E);
#pragma unroll
      for (int e = 0; e < E; ++e) f[e] = ElemTraits<T>::to_f(raw.v[e]);
    } else {
      f[0] = ElemTraits<T>::to_f(row[v]);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      float a = f[e];
      if (pre_op == AMCT_PRE_MUL) a = round_to<T>(__fmul_rn(a, ElemTraits<T>::to_f(pre[v * E + e])));
      else if (pre_op == AMCT_PRE_DIV) a = round_to<T>(__fdiv_rn(a, ElemTraits<T>::to_f(pre[v * E + e])));
      mn = fminf(mn, a); mx = fmaxf(mx, a); nan |= (a != a);
    }
  }
  if (nan && status) atomicOr(status, 1);
  if (nan) { mn = NAN; mx = NAN; }
  __shared__ float s[8];
  mn = warp_nan_min(mn); mx = warp_nan_max(mx);
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { s[w] = mn; s[4 + w] = mx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 4; ++i) { mn = nan_min(mn, s[i]); mx = nan_max(mx, s[4 + i]); }
    if (merge) {
      mn = merge_min(mn, ElemTraits<T>::to_f(out_min[blockIdx.x]));
      mx = merge_max(mx, ElemTraits<T>::to_f(out_max[blockIdx.x]));
    }
    out_min[blockIdx.x] = ElemTraits<T>::from_f(mn);
    out_max[blockIdx.x] = ElemTraits<T>::from_f(mx);
  }
}

template <typename T>
static int run_minmax_rows(const T* x, int64_t rows, int64_t k, int64_t ld, const T* pre, int pre_op, int merge,
                           T* out_min, T* out_max, int* status, cudaStream_t st) {
  constexpr int E = ElemTraits<T>::kPerVec;
  const bool vec = aligned16(x) && (ld * (int64_t)sizeof(T)) % 16 == 0 && k % E == 0;
  if (vec) AMCT_LAUNCH((unsigned)rows, 128, st, (x, k, ld, pre, pre_op, merge, out_min, out_max, status), minmax_rows_kernel<T, true>);
  else AMCT_LAUNCH((unsigned)rows, 128, st, (x, k, ld, pre, pre_op, merge, out_min, out_max, status), minmax_rows_kernel<T, false>);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

template <typename T>
__global__ void scale_offset_kernel(const T* vmax, const T* vmin, int64_t n, int bits, int symmetric, float* scale,
                                    int* offset, int* status) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float mx = ElemTraits<T>::to_f(vmax[i]), mn = ElemTraits<T>::to_f(vmin[i]);
  float s; int o;
  bool ok = qparams_from_minmax(mx, mn, bits, symmetric != 0, &s, &o) && mx == mx && mn == mn;
  if (!ok && status) atomicOr(status, 1);
  scale[i] = s;
  if (offset) offset[i] = o;
}

__global__ void __launch_bounds__(256) rowsum_i8_kernel(const int8_t* wq, int64_t n_rows, int64_t k, int64_t ld,
                                                        int32_t* out, int vec) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= n_rows) return;
  const int8_t* p = wq + row * ld;
  int acc = 0;
  if (vec) {
    const int64_t nv = k / 16;
    for (int64_t v = lane; v < nv; v += 32) {
      int4 q = __ldcs(reinterpret_cast<const int4*>(p) + v);
      acc = __dp4a(q.x, 0x01010101, acc);
      acc = __dp4a(q.y, 0x01010101, acc);
      acc = __dp4a(q.z, 0x01010101, acc);
      acc = __dp4a(q.w, 0x01010101, acc);
    }
    for (int64_t j = nv * 16 + lane; j < k; j += 32) acc += p[j];
  } else {
    for (int64_t j = lane; j < k; j += 32) acc += p[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[row] = acc;
}

__global__ void __launch_bounds__(256) transpose_i8_kernel(const int8_t* in, int64_t rows, int64_t cols, int8_t* out) {
  __shared__ int8_t tile[64][65];
  const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;        // 64 x 4
  for (int i = ty; i < 64; i += 4) {
    int64_t r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) tile[i][tx] = in[r * cols + c];
  }
  __syncthreads();
  for (int i = ty; i < 64; i += 4) {
    int64_t c = c0 + i, r = r0 + tx;
    if (r < rows && c < cols) out[c * rows + r] = tile[tx][i];
  }
}


// ---------------------------------------------------------------------------
// Built-in scratch for amct_minmax_noalloc.
//
// Some hosts of this library may not allocate device memory once they are up: a
// serving process that carves its whole memory budget at start-up and treats any
// later cudaMalloc as a fault (it takes a device-wide lock and can stall every
// stream), or a plugin host that only ever hands the library input and output
// buffers and has no way to pass a workspace.  For them the partial results of
// the reduction live in this file-scope array instead of a caller workspace.
// Every GPU that loads the library carries these 8 MiB until the process exits.
//
// `g_minmax_scratch` is a device symbol: in host code the name is only a handle,
// not an address a kernel can use.  The device address is looked up with
// cudaGetSymbolAddress once per device (with that device current) and cached.
constexpr int64_t kStaticScratchBytes = 8LL << 20;
static __device__ __align__(256) unsigned char g_minmax_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

static int static_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return AMCT_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_minmax_scratch) != cudaSuccess || !p) return AMCT_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = reinterpret_cast<float*>(g_scratch_addr[dev]);
  return AMCT_OK;
}

}  // namespace amct

extern "C" int amct_abi_version(void) { return 1; }

extern "C" int64_t amct_minmax_workspace_bytes(int64_t k) {
  int64_t a = 2LL * amct::kMaxRowChunks * (k > 0 ? k : 0) * 4;
  int64_t b = 2LL * amct::kTensorBlocks * 4;
  return a > b ? a : b;
}

extern "C" int amct_minmax(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int axis, int merge,
                           void* out_min, void* out_max, void* workspace, int* status, void* stream) {
  if (rows <= 0 || k <= 0 || !x || !out_min || !out_max || !workspace || ld_x < k) return AMCT_ERR_ARG;
  if (axis != AMCT_AXIS_TENSOR && axis != AMCT_AXIS_COLUMN) return AMCT_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  float* ws = reinterpret_cast<float*>(workspace);
  switch (dtype) {
    case AMCT_DTYPE_F32:
      return amct::run_minmax<float>((const float*)x, rows, k, ld_x, axis, merge, (float*)out_min, (float*)out_max, ws, status, st);
    case AMCT_DTYPE_F16:
      return amct::run_minmax<__half>((const __half*)x, rows, k, ld_x, axis, merge, (__half*)out_min, (__half*)out_max, ws, status, st);
    case AMCT_DTYPE_BF16:
      return amct::run_minmax<__nv_bfloat16>((const __nv_bfloat16*)x, rows, k, ld_x, axis, merge, (__nv_bfloat16*)out_min,
                                             (__nv_bfloat16*)out_max, ws, status, st);
  }
  return AMCT_ERR_ARG;
}

extern "C" int64_t amct_minmax_noalloc_max_k(void) { return amct::kStaticScratchBytes / (2LL * amct::kMaxRowChunks * 4); }

extern "C" int amct_minmax_noalloc(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int axis, int merge,
                                   void* out_min, void* out_max, int* status, void* stream) {
  if (rows <= 0 || k <= 0 || !x || !out_min || !out_max || ld_x < k) return AMCT_ERR_ARG;
  if (axis != AMCT_AXIS_TENSOR && axis != AMCT_AXIS_COLUMN) return AMCT_ERR_ARG;
  // the column reduction keeps 2 x 64 partial rows of k floats: refuse what the built-in array cannot hold
  if (axis == AMCT_AXIS_COLUMN && amct_minmax_workspace_bytes(k) > amct::kStaticScratchBytes) return AMCT_ERR_TOO_LARGE;
  float* ws = nullptr;
  int rc = amct::static_scratch(&ws);
  if (rc != AMCT_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // Nothing in the scratch has to start at zero: every partial that the second
  // stage reads is written by the first stage of the same call.
  switch (dtype) {
    case AMCT_DTYPE_F32:
      return amct::run_minmax<float>((const float*)x, rows, k, ld_x, axis, merge, (float*)out_min, (float*)out_max, ws, status, st);
    case AMCT_DTYPE_F16:
      return amct::run_minmax<__half>((const __half*)x, rows, k, ld_x, axis, merge, (__half*)out_min, (__half*)out_max, ws, status, st);
    case AMCT_DTYPE_BF16:
      return amct::run_minmax<__nv_bfloat16>((const __nv_bfloat16*)x, rows, k, ld_x, axis, merge, (__nv_bfloat16*)out_min,
                                             (__nv_bfloat16*)out_max, ws, status, st);
  }
  return AMCT_ERR_ARG;
}

extern "C" int amct_minmax_rows(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, const void* pre,
                                int pre_op, int merge, void* out_min, void* out_max, int* status, void* stream) {
  if (rows <= 0 || k <= 0 || !x || !out_min || !out_max || ld_x < k || rows > 0x7fffffffLL) return AMCT_ERR_ARG;
  if (pre_op != AMCT_PRE_NONE && !pre) return AMCT_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case AMCT_DTYPE_F32:
      return amct::run_minmax_rows<float>((const float*)x, rows, k, ld_x, (const float*)pre, pre_op, merge, (float*)out_min,
                                          (float*)out_max, status, st);
    case AMCT_DTYPE_F16:
      return amct::run_minmax_rows<__half>((const __half*)x, rows, k, ld_x, (const __half*)pre, pre_op, merge, (__half*)out_min,
                                           (__half*)out_max, status, st);
    case AMCT_DTYPE_BF16:
      return amct::run_minmax_rows<__nv_bfloat16>((const __nv_bfloat16*)x, rows, k, ld_x, (const __nv_bfloat16*)pre, pre_op, merge,
                                                  (__nv_bfloat16*)out_min, (__nv_bfloat16*)out_max, status, st);
  }
  return AMCT_ERR_ARG;
}

extern "C" int amct_scale_offset(const void* vmax, const void* vmin, int dtype, int64_t n, int bits, int symmetric,
                                 float* scale, int* offset, int* status, void* stream) {
  if (n < 0 || (n && (!vmax || !vmin || !scale)) || (bits != 8 && bits != 4)) return AMCT_ERR_ARG;
  if (!symmetric && !offset) return AMCT_ERR_ARG;
  if (n == 0) return AMCT_OK;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned blocks = (unsigned)((n + 255) / 256);
  int* off = symmetric ? nullptr : offset;
  switch (dtype) {
    case AMCT_DTYPE_F32:
      AMCT_LAUNCH(blocks, 256, st, ((const float*)vmax, (const float*)vmin, n, bits, symmetric, scale, off, status), amct::scale_offset_kernel<float>);
      break;
    case AMCT_DTYPE_F16:
      AMCT_LAUNCH(blocks, 256, st, ((const __half*)vmax, (const __half*)vmin, n, bits, symmetric, scale, off, status), amct::scale_offset_kernel<__half>);
      break;
    case AMCT_DTYPE_BF16:
      AMCT_LAUNCH(blocks, 256, st, ((const __nv_bfloat16*)vmax, (const __nv_bfloat16*)vmin, n, bits,
                                                                       symmetric, scale, off, status), amct::scale_offset_kernel<__nv_bfloat16>);
      break;
    default:
      return AMCT_ERR_ARG;
  }
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

extern "C" int amct_rowsum_i8(const int8_t* wq, int64_t n_rows, int64_t k, int64_t ld, int32_t* out, void* stream) {
  if (n_rows < 0 || k < 0 || ld < k || (n_rows && (!wq || !out))) return AMCT_ERR_ARG;
  if (n_rows == 0) return AMCT_OK;
  int vec = amct::aligned16(wq) && ld % 16 == 0;
  unsigned blocks = (unsigned)((n_rows + 7) / 8);
  AMCT_LAUNCH(blocks, 256, (cudaStream_t)stream, (wq, n_rows, k, ld, out, vec), amct::rowsum_i8_kernel);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

extern "C" int amct_transpose_i8(const int8_t* in, int64_t rows, int64_t cols, int8_t* out, void* stream) {
  if (rows < 0 || cols < 0 || (rows && cols && (!in || !out))) return AMCT_ERR_ARG;
  if (rows == 0 || cols == 0) return AMCT_OK;
  dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
  if (grid.y > 65535) return AMCT_ERR_UNSUPPORTED;
  AMCT_LAUNCH(grid, 256, (cudaStream_t)stream, (in, rows, cols, out), amct::transpose_i8_kernel);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}
