// Pieces shared by the tcgen05 GEMM kernels: parameters, tile rasterisation and the
// epilogue that turns one 128-row accumulator tile in tensor memory into output values.
//
// Epilogues (fp32, each step separately rounded, in this order):
//   W8A8 per-token : y = float(acc) * deq[n] * pertoken[m] + bias_f[n]
//   W8A8 per-tensor: y = float(acc + bias_i32[n]) * deq[n]
//   (the operand construction of amct_pytorch/deploy_op/npu_quantization_linear.py:61-68,
//    :105-130 fixes where each bias is added; the call is
//    torch_npu.npu_quant_matmul at :100-102)
//   raw            : int32 accumulators as they are
//   float kinds    : y = acc + bias_f[n]
#pragma once
#include "common.cuh"
#include "tc05.cuh"

namespace amct {

constexpr int kBM = 128, kBKBytes = 128;
constexpr int kABytes = kBM * kBKBytes;
constexpr int kMaxScatterRanks = 16;
constexpr int kEpiStageBytes = 32 * 128;       // per epilogue warp: 32 rows x 64 16-bit columns, for the scatter mode

enum { KIND_I8 = 0, KIND_BF16 = 1, KIND_F16 = 2 };
enum { BIAS_NONE = 0, BIAS_I32 = 1, BIAS_F32 = 2, BIAS_F16 = 3, BIAS_BF16 = 4 };
enum { OUT_F32 = 0, OUT_F16 = 1, OUT_BF16 = 2, OUT_I32 = 3 };

struct GemmParams {
  int64_t m, n, k;             // k in elements
  int kind;
  const float* deq;            // [n] or null
  const float* pertoken;       // [m] or null
  const void* bias;            // [n] or null
  int bias_kind;
  void* out;
  int out_kind;
  int64_t ld_out;              // elements
  int* status;
  int act;                     // 0 none, 1 SwiGLU over interleaved [128 gate | 128 up] column blocks
  // Scatter mode of a row-parallel (K-sharded) Linear under tensor parallelism, scatter_world > 0: output
  // row r belongs to rank r / scatter_rows and goes to row (scatter_slot * scatter_rows + r % scatter_rows) of
  // scatter_out[that rank] (this process's mapping of that rank's buffer, ld_out elements per row); `out` is
  // not used.  16-bit outputs, n a multiple of 64.
  int scatter_world, scatter_slot;
  int64_t scatter_rows;
  void* scatter_out[kMaxScatterRanks];
  // Rows by which the walk over the m-tiles starts later (scatter mode: rank s starts with the rows of rank s + 1,
  // so that at any moment the ranks write to DIFFERENT owners; all starting at row 0 would aim every rank's
  // stores at one GPU at a time and the transfer would run at one GPU's ingress bandwidth, not at everybody's).
  int64_t row_rot;
  // Rasterisation: m-tiles per group (set by the launcher from the bytes of an A row block, see group_m_tiles).
  int group_m;
  // Rows of A a tile load brings in: 128, or 64 when the whole problem has at most 64 rows (a decode batch).  The MMA
  // still works on 128 rows; rows 64..127 of the shared-memory tile then hold whatever was there, which only reaches
  // accumulator rows that are never stored, and every CTA's A traffic is halved (set by the launcher).
  int a_box_rows;
};

// m-tiles per rasterisation group: as many as keep the group's A panel (group x tile_rows x K bytes) near 32 MB,
// a quarter of L2.  Within a group the kernel walks all n-tiles with m fastest, so the panel is read from HBM once
// and the B operand streams past it once per group: bigger groups mean fewer passes over B (measured on the
// 57344 x 8192 INT8 weight: 32 tiles of 128 rows instead of 16 halve the DRAM reads and are 1 % faster at the power
// limit; 64 tiles thrash L2 and are 10 % slower).
inline int group_m_tiles(int64_t k_bytes, int tile_rows) {
  const int64_t g = (32LL << 20) / (k_bytes * tile_rows > 0 ? k_bytes * tile_rows : 1);
  return (int)(g < 4 ? 4 : g > 64 ? 64 : g);
}

// the m-tile a kernel works on for the rasterised index tm, with the start of the walk rotated by p.row_rot rows
__device__ __forceinline__ int64_t rotate_tile_m(const GemmParams& p, int64_t tm, int64_t tiles_m, int tile_rows) {
  if (p.row_rot == 0) return tm;
  const int64_t r = (tm + p.row_rot / tile_rows) % tiles_m;
  return r;
}

// Rasterisation: GROUP m-tiles x all n-tiles per group, m fastest, so that the tiles in flight
// at one time share a few A row blocks and a few B row blocks in L2.
__device__ __forceinline__ void tile_coords(int GROUP, int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t* tm, int64_t* tn) {
  const int64_t per_group = (int64_t)GROUP * tiles_n;
  const int64_t g = tile / per_group, r = tile - g * per_group;
  const int64_t m0 = g * GROUP;
  const int64_t gm = (tiles_m - m0) < GROUP ? (tiles_m - m0) : GROUP;
  *tn = r / gm;
  *tm = m0 + r % gm;
}

__device__ __forceinline__ float bias_at(const void* bias, int kind, int64_t n) {
  switch (kind) {
    case BIAS_F32: return reinterpret_cast<const float*>(bias)[n];
    case BIAS_F16: return __half2float(reinterpret_cast<const __half*>(bias)[n]);
    case BIAS_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n]);
    case BIAS_I32: return __int_as_float(reinterpret_cast<const int*>(bias)[n]);   // carried as raw bits
  }
  return 0.f;
}

// Per-column bias as the epilogue loops want it when a tile's factors are staged: the int32 bias as raw bits, a
// float bias as its value, and NO bias as -0.0f -- x + (-0.0f) is x for every x, signed zeros and NaN included, so
// the loops add it unconditionally.
__device__ __forceinline__ float staged_bias(const GemmParams& p, int64_t n) {
  if (p.bias_kind == BIAS_NONE || n >= p.n) return p.bias_kind == BIAS_I32 ? 0.f : -0.f;
  return bias_at(p.bias, p.bias_kind, n);
}

// Output values of 32 consecutive accumulator columns of one row.  Which formula applies is decided ONCE per call,
// outside the loops: an epilogue warp is alone on its scheduler, so every branch inside a per-element loop costs its
// full latency (the per-element form of this function took 24 K cycles per 128 x 256 tile, this one takes a third).
//   INT8, int32 bias : y = float(acc + bias_i32[n]) * deq[n]
//   INT8 otherwise   : y = float(acc) * deq[n] * pt + bias_f[n]      (pt = 1.0f without per-token scales: exact)
//   float kinds      : y = acc + bias_f[n]
// sc / sb point at the 32 columns' staged factors (16-byte aligned); sb as staged_bias leaves it.
__device__ __forceinline__ void epi_values32(const GemmParams& p, const uint32_t (&r)[32], const float* sc, const float* sb,
                                             float pt, float (&y)[32]) {
  float s[32], b[32];
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 s4 = *reinterpret_cast<const float4*>(sc + j), b4 = *reinterpret_cast<const float4*>(sb + j);
    s[j] = s4.x; s[j + 1] = s4.y; s[j + 2] = s4.z; s[j + 3] = s4.w;
    b[j] = b4.x; b[j + 1] = b4.y; b[j + 2] = b4.z; b[j + 3] = b4.w;
  }
  if (p.kind == KIND_I8) {
    if (p.bias_kind == BIAS_I32) {
#pragma unroll
      for (int j = 0; j < 32; ++j) y[j] = __fmul_rn((float)((int)r[j] + __float_as_int(b[j])), s[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) y[j] = __fadd_rn(__fmul_rn(__fmul_rn((float)(int)r[j], s[j]), pt), b[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = __fadd_rn(__uint_as_float(r[j]), b[j]);
  }
}

// One warp's share of an accumulator tile: the 32 rows starting at TMEM address t_row (lane =
// row), kBN columns.  `row` is this lane's output row, n0 the tile's first output column, tn the
// tile's column index; sc / sb hold the tile's per-column scale and bias (staged_bias), pt the row's scale
// (1.0f without per-token scales).
template <int kBN>
__device__ __forceinline__ void epilogue_rows(const GemmParams& p, uint32_t t_row, int64_t row, int64_t n0, int64_t tn,
                                              const float* sc, const float* sb, float pt) {
  if (p.act == 1) {
    // SwiGLU: the tile holds 128 gate columns followed by their 128 up columns.  Both are
    // dequantized and rounded to bf16 as the unfused Linear would output them, then
    // out = bf16(bf16(silu(gate)) * up); the output has N/2 columns.
#pragma unroll 1
    for (int c0 = 0; c0 < kBN / 2; c0 += 32) {
      uint32_t rg[32], ru[32];
      tc05::tmem_ld_32x32(t_row + c0, rg);
      tc05::tmem_ld_32x32(t_row + kBN / 2 + c0, ru);
      tc05::tmem_ld_wait();
      if (row < p.m) {
        float g[32], u[32];
        epi_values32(p, rg, sc + c0, sb + c0, pt, g);
        epi_values32(p, ru, sc + kBN / 2 + c0, sb + kBN / 2 + c0, pt, u);
        float sg[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          g[j] = __bfloat162float(__float2bfloat16_rn(g[j]));
          u[j] = __bfloat162float(__float2bfloat16_rn(u[j]));
          sg[j] = __fdiv_rn(g[j], __fadd_rn(1.f, expf(-g[j])));
        }
        uint32_t h[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float o0 = __fmul_rn(__bfloat162float(__float2bfloat16_rn(sg[j])), u[j]);
          const float o1 = __fmul_rn(__bfloat162float(__float2bfloat16_rn(sg[j + 1])), u[j + 1]);
          __nv_bfloat162 v = __floats2bfloat162_rn(o0, o1);
          h[j >> 1] = *reinterpret_cast<uint32_t*>(&v);
        }
        uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + row * p.ld_out + tn * (kBN / 2) + c0;
#pragma unroll
        for (int j = 0; j < 16; j += 4) *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(h[j], h[j + 1], h[j + 2], h[j + 3]);
      }
    }
    return;
  }
#pragma unroll 1
  for (int c0 = 0; c0 < kBN; c0 += 32) {
    uint32_t r[32];
    tc05::tmem_ld_32x32(t_row + c0, r);
    tc05::tmem_ld_wait();
    if (row < p.m && n0 + c0 < p.n) {
      const int64_t nleft = p.n - (n0 + c0);
      const int64_t off = row * p.ld_out + n0 + c0;
      if (p.out_kind == OUT_I32) {
        int* o = reinterpret_cast<int*>(p.out) + off;
        if (nleft >= 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (j < nleft) o[j] = (int)r[j];
        }
        continue;
      }
      float y[32];
      epi_values32(p, r, sc + c0, sb + c0, pt, y);
      if (p.out_kind == OUT_F32) {
        float* o = reinterpret_cast<float*>(p.out) + off;
        if (nleft >= 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (j < nleft) o[j] = y[j];
        }
      } else {
        uint32_t h[16];
        epi_pack16(y, p.out_kind == OUT_BF16, h);
        uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + off;
        if (nleft >= 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(h[j], h[j + 1], h[j + 2], h[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (j < nleft) o[j] = (uint16_t)(h[j >> 1] >> (16 * (j & 1)));
        }
      }
    }
  }
}

// The same values as epilogue_rows' 16-bit store, written for links instead of local memory.  In epilogue_rows a
// lane owns a row, so one store instruction touches 32 rows with 16 bytes each: fine for the local L2, wasteful as
// 32 small packets on NVLink.  Here 64 columns at a time go through a swizzled 4 KB staging tile in shared memory
// (`stage`, this warp's own) and leave as whole 128-byte row segments: 8 lanes per row, 4 rows per instruction.
// Plain st.global to peer-mapped memory; no TMA store, no multicast.  warp_row0 = first of the warp's 32 rows.
template <int kBN>
__device__ __forceinline__ void epilogue_rows_scatter(const GemmParams& p, uint32_t t_row, int64_t warp_row0, int lane,
                                                      int64_t n0, const float* sc, const float* sb, float pt,
                                                      uint8_t* stage) {
  static_assert(kBN % 64 == 0, "scatter epilogue works on 64-column chunks");
  // where the warp's rows go: worked out once per tile (a 64-bit division), not once per store
  const int64_t owner0 = warp_row0 / p.scatter_rows, local0 = warp_row0 - owner0 * p.scatter_rows;
  const bool one_owner = local0 + 32 <= p.scatter_rows && owner0 < p.scatter_world;
  uint16_t* owner_base = one_owner ? reinterpret_cast<uint16_t*>(p.scatter_out[owner0]) +
                                         ((int64_t)p.scatter_slot * p.scatter_rows + local0) * p.ld_out
                                   : nullptr;
#pragma unroll 1
  for (int c0 = 0; c0 < kBN; c0 += 64) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t r[32];
      tc05::tmem_ld_32x32(t_row + c0 + half * 32, r);
      tc05::tmem_ld_wait();
      float y[32];
      epi_values32(p, r, sc + c0 + half * 32, sb + c0 + half * 32, pt, y);
      uint32_t h[16];
      epi_pack16(y, p.out_kind == OUT_BF16, h);
      // lane = row: four 16-byte chunks of this half, chunk index XOR (row & 7) so that neither side conflicts
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int chunk = (half * 4 + i) ^ (lane & 7);
        *reinterpret_cast<uint4*>(stage + lane * 128 + chunk * 16) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
      }
    }
    __syncwarp();
    const int chunk = lane & 7;
    const int64_t col = n0 + c0 + chunk * 8;
    if (col < p.n) {
      if (one_owner) {
        // the warp's 32 rows belong to one rank: one base pointer, no division per row
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r_in = it * 4 + (lane >> 3);
          const uint4 v = *reinterpret_cast<const uint4*>(stage + r_in * 128 + ((chunk ^ (r_in & 7)) * 16));
          if (warp_row0 + r_in < p.m) *reinterpret_cast<uint4*>(owner_base + (int64_t)r_in * p.ld_out + col) = v;
        }
      } else {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r_in = it * 4 + (lane >> 3);
          const uint4 v = *reinterpret_cast<const uint4*>(stage + r_in * 128 + ((chunk ^ (r_in & 7)) * 16));
          const int64_t row = warp_row0 + r_in;
          if (row < p.m) {
            const int64_t owner = row / p.scatter_rows;
            const int64_t local = row - owner * p.scatter_rows;
            uint16_t* o = reinterpret_cast<uint16_t*>(p.scatter_out[owner]) +
                          ((int64_t)p.scatter_slot * p.scatter_rows + local) * p.ld_out + col;
            *reinterpret_cast<uint4*>(o) = v;
          }
        }
      }
    }
    __syncwarp();
  }
}

}  // namespace amct
