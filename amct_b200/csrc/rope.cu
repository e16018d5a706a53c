// Rotary position embedding applied in place to the query and key heads of a fused q/k/v
// projection output (the tensor the sharded deploy workload's attention reads next).
//
// Rotate-half convention: for a head of D values, x1 = x[:D/2], x2 = x[D/2:],
//   out1 = x1 * cos - x2 * sin,   out2 = x2 * cos + x1 * sin.
// Every product and every sum is rounded to the tensor dtype separately, which is what the
// same expression written with torch ops on 16-bit tensors produces, so fused and unfused
// results are bit-identical.  The reference has no counterpart; this kernel only removes the
// seven strided elementwise launches the torch expression costs per decoder layer.
//
// HBM traffic per token: 2 * heads * D * sizeof(T) (read and written once), cos / sin from L2.
#include "common.cuh"

namespace amct {

template <typename T>
__global__ void __launch_bounds__(256) rope_inplace_kernel(T* x, uint32_t tokens, int64_t ld, int heads, int head_dim,
                                                           const T* cos_t, const T* sin_t, uint32_t seq) {
  constexpr int E = 8;
  const int half = head_dim / 2;
  const int vec_per_head = half / E;                 // 16-byte vectors in one half head
  const int work = blockIdx.x * blockDim.x + threadIdx.x;
  if (work >= heads * vec_per_head) return;
  const int head = work / vec_per_head;
  const int d0 = (work - head * vec_per_head) * E;
  const int64_t col = (int64_t)head * head_dim + d0;
  for (uint32_t t = blockIdx.y; t < tokens; t += gridDim.y) {
    T* p1 = x + (int64_t)t * ld + col;
    T* p2 = p1 + half;
    const int64_t pos = t % seq;
    const Vec16<T> a = ld_vec_stream(p1), b = ld_vec_stream(p2);
    const Vec16<T> c = ld_vec(cos_t + pos * half + d0), s = ld_vec(sin_t + pos * half + d0);
    Vec16<T> o1, o2;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float x1 = ElemTraits<T>::to_f(a.v[e]), x2 = ElemTraits<T>::to_f(b.v[e]);
      const float cf = ElemTraits<T>::to_f(c.v[e]), sf = ElemTraits<T>::to_f(s.v[e]);
      o1.v[e] = ElemTraits<T>::from_f(__fsub_rn(round_to<T>(__fmul_rn(x1, cf)), round_to<T>(__fmul_rn(x2, sf))));
      o2.v[e] = ElemTraits<T>::from_f(__fadd_rn(round_to<T>(__fmul_rn(x2, cf)), round_to<T>(__fmul_rn(x1, sf))));
    }
    *reinterpret_cast<uint4*>(p1) = *reinterpret_cast<const uint4*>(&o1);
    *reinterpret_cast<uint4*>(p2) = *reinterpret_cast<const uint4*>(&o2);
  }
}

template <typename T>
static int run_rope(T* x, int64_t tokens, int64_t ld, int heads, int head_dim, const T* c, const T* s, int64_t seq,
                    cudaStream_t st) {
  const int work = heads * (head_dim / 16);
  dim3 grid((unsigned)((work + 255) / 256), 1);
  int64_t gy = (148LL * 8 + grid.x - 1) / grid.x;
  if (gy > tokens) gy = tokens;
  if (gy > 65535) gy = 65535;
  grid.y = (unsigned)gy;
  AMCT_LAUNCH(grid, 256, st, (x, (uint32_t)tokens, ld, heads, head_dim, c, s, (uint32_t)seq), rope_inplace_kernel<T>);
  AMCT_CHECK_LAUNCH();
  return AMCT_OK;
}

}  // namespace amct

extern "C" int amct_rope_inplace(void* x, int dtype, int64_t tokens, int64_t ld, int heads, int head_dim,
                                 const void* cos_table, const void* sin_table, int64_t seq, void* stream) {
  if (tokens < 0 || heads < 0 || head_dim <= 0 || seq <= 0 || tokens >= (1LL << 31) || seq >= (1LL << 31)) return AMCT_ERR_ARG;
  if (tokens == 0 || heads == 0) return AMCT_OK;
  if (!x || !cos_table || !sin_table || ld < (int64_t)heads * head_dim) return AMCT_ERR_ARG;
  if (dtype != AMCT_DTYPE_F16 && dtype != AMCT_DTYPE_BF16) return AMCT_ERR_UNSUPPORTED;
  if (head_dim % 16) return AMCT_ERR_UNSUPPORTED;
  if (!amct::aligned16(x) || (ld * 2) % 16 || !amct::aligned16(cos_table) || !amct::aligned16(sin_table)) return AMCT_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == AMCT_DTYPE_F16)
    return amct::run_rope<__half>((__half*)x, tokens, ld, heads, head_dim, (const __half*)cos_table, (const __half*)sin_table, seq, st);
  return amct::run_rope<__nv_bfloat16>((__nv_bfloat16*)x, tokens, ld, heads, head_dim, (const __nv_bfloat16*)cos_table,
                                       (const __nv_bfloat16*)sin_table, seq, st);
}
