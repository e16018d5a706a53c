/* C ABI of the B200 (sm_100a) implementation of AMCT's quantization hot path.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless it is named host_*; the caller
 *     owns all memory, nothing here allocates persistent device memory;
 *   - `stream` is a cudaStream_t; calls enqueue work and return, they do not
 *     synchronise;
 *   - the return value is AMCT_OK or a negative AMCT_ERR_* code; arguments are
 *     validated on the host before anything is launched;
 *   - `status` (optional, may be NULL) is a device int; bit 0 is OR-ed in when a
 *     kernel meets a non-finite value where the reference raises
 *     "Param scale has invalid value inf, nan or zeros!"
 *     (amct_pytorch/quantize_op/utils.py:54-72);
 *   - `dtype` is AMCT_DTYPE_*; leading dimensions are in elements.
 *
 * Each entry point names the reference interface it stands in for (paths
 * relative to the reference project root).
 */
#ifndef AMCT_B200_H_
#define AMCT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { AMCT_OK = 0, AMCT_ERR_ARG = -1, AMCT_ERR_ALIGN = -2, AMCT_ERR_CUDA = -3, AMCT_ERR_UNSUPPORTED = -4,
       AMCT_ERR_TIMEOUT = -5, AMCT_ERR_TOO_LARGE = -6 };
enum { AMCT_DTYPE_F32 = 0, AMCT_DTYPE_F16 = 1, AMCT_DTYPE_BF16 = 2 };
enum { AMCT_STRATEGY_TENSOR = 0, AMCT_STRATEGY_CHANNEL = 1, AMCT_STRATEGY_GROUP = 2 };
enum { AMCT_RULE_RELEASED = 0, AMCT_RULE_EXPERIMENTAL = 1 };
enum { AMCT_PRE_NONE = 0, AMCT_PRE_MUL = 1, AMCT_PRE_DIV = 2 };
enum { AMCT_OUT_NONE = 0, AMCT_OUT_I8 = 1, AMCT_OUT_I32 = 2, AMCT_OUT_PACK4 = 3, AMCT_OUT_FAKE = 4,
       AMCT_OUT_FAKE_AWQ = 5 };
enum { AMCT_AXIS_TENSOR = 0, AMCT_AXIS_COLUMN = 1 };
enum { AMCT_DSA_DYNAMIC = 0, AMCT_DSA_LEARNED_CLIP = 1, AMCT_DSA_CLIP_RATIO = 2, AMCT_DSA_STATIC = 3,
       AMCT_DSA_STATIC_F32 = 4 };

/* Version of this ABI; bumped when a signature changes. */
int amct_abi_version(void);

/* Dynamic per-token symmetric INT8 activation quantization, one scale per row.
 * Replaces the eager sequence amax/amin over K
 * (amct_pytorch/quantize_op/minmax_module.py:99-105) -> calculate_scale_offset
 * (amct_pytorch/quantize_op/utils.py:75-108) -> convert_dtype(x / scale)
 * (amct_pytorch/utils/quant_util.py:57-73), and, when `smooth` is given, the
 * `x * scale_factor` pass of NpuQuantizationLinear.forward
 * (amct_pytorch/deploy_op/npu_quantization_linear.py:96-97).
 * rule = AMCT_RULE_EXPERIMENTAL follows ActivationQuantizer.get_scale_zero
 * (amct_pytorch/experimental/quantization/DeepSeekV3.2/cores/quantization/node.py:181-204).
 * x [rows, k] (ld_x), smooth [k] in x's dtype or NULL, q int8 [rows, k] (ld_q),
 * scale fp32 [rows]. */
int amct_quant_dynamic_pertoken(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x,
                                const void* smooth, int rule, int8_t* q, int64_t ld_q, float* scale,
                                int* status, void* stream);

/* Row-wise quantizer over a [rows, k] matrix; each row is read once.
 * compute=1 derives scale/offset per row (AMCT_STRATEGY_CHANNEL) or per group of
 * `group` elements (AMCT_STRATEGY_GROUP, a ragged last group is zero padded) and
 * writes them; compute=0 reads them (also AMCT_STRATEGY_TENSOR: one value).
 * Replaces get_weight_min_max_by_granularity + calculate_scale_offset
 * (amct_pytorch/quantize_op/utils.py:75-136), quant_weight / convert_dtype
 * (amct_pytorch/utils/quant_util.py:57-93), NpuQuantizationLinear.quant_wts
 * (amct_pytorch/deploy_op/npu_quantization_linear.py:72-87), quant_dequant_weight
 * (amct_pytorch/utils/quant_util.py:162-188, AMCT_OUT_FAKE) and do_quant ->
 * convert_precision -> do_dequant (amct_pytorch/algorithm/awq.py:129-170,
 * AMCT_OUT_FAKE_AWQ).  pre/pre_op fold apply_smooth_weight (MUL) or
 * apply_awq_quantize_weight (DIV) (amct_pytorch/utils/quant_util.py:96-159) into
 * the load.  AMCT_OUT_PACK4 writes two INT4 codes per byte (code + 8, even k in
 * the low nibble), standing in for torch_npu.npu_convert_weight_to_int4pack
 * (amct_pytorch/deploy_op/weight_npu_quant_module.py:54-57).
 * scale fp32 / offset int32: [1] | [rows] | [rows, ceil(k/group)]; offset may be
 * NULL when symmetric.  out: int8 | int32 | uint8 [rows, k/2] | x's dtype. */
int amct_quant_rows(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x,
                    const void* pre, int pre_op, int compute, int strategy, int group, int bits,
                    int symmetric, float* scale, int* offset, int out_mode, void* out, int64_t ld_out,
                    int* status, void* stream);

/* min and max of a [rows, k] matrix over the whole tensor (AMCT_AXIS_TENSOR, one
 * value) or per column over all rows (AMCT_AXIS_COLUMN, k values), in x's dtype.
 * merge=1 folds the result into the values already in out_min/out_max (running
 * observers).  Replaces torch.max/min (amct_pytorch/quantize_op/minmax_module.py:96-98,
 * :107-110) and amax/amin over tokens
 * (amct_pytorch/quantize_op/smooth_quant_module.py:79-91).
 * workspace: at least amct_minmax_workspace_bytes(k) bytes of device memory. */
int64_t amct_minmax_workspace_bytes(int64_t k);
int amct_minmax(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int axis, int merge,
                void* out_min, void* out_max, void* workspace, int* status, void* stream);

/* amct_minmax for callers that cannot give it a workspace and must not see a
 * device allocation -- a server whose memory budget is fixed at start-up, a plugin
 * host that passes inputs and outputs only.  Same arguments and results as
 * amct_minmax minus `workspace`: the partials live in an 8 MiB array built into
 * the library (held by every GPU that loads it, until the process exits).  It has
 * no counterpart in the reference; it exists for embedding, not for parity.
 *   - limit: AMCT_AXIS_COLUMN needs k <= amct_minmax_noalloc_max_k() (16384);
 *     larger k returns AMCT_ERR_TOO_LARGE and launches nothing.  AMCT_AXIS_TENSOR
 *     has no size limit.
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine.  The
 *     first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before any stream capture.
 *   - all calls share the one array, which keeps whatever the last call left in
 *     it (nothing needs clearing: each call overwrites what it reads).  Two calls
 *     that can overlap on the GPU -- different streams, no ordering -- race on it:
 *     serialize them. */
int64_t amct_minmax_noalloc_max_k(void);
int amct_minmax_noalloc(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int axis, int merge,
                        void* out_min, void* out_max, int* status, void* stream);

/* min and max of every row of a [rows, k] matrix, in x's dtype; `pre`/pre_op
 * apply an element-wise factor [k] first (rounded to x's dtype), merge=1 folds
 * into existing values.  Replaces torch.amax/amin over all axes but the token
 * axis (amct_pytorch/quantize_op/minmax_module.py:99-105) and the per-token
 * statistics of the smoothed stash
 * (amct_pytorch/quantize_op/smooth_quant_module.py:155-168). */
int amct_minmax_rows(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, const void* pre,
                     int pre_op, int merge, void* out_min, void* out_max, int* status, void* stream);

/* scale/offset from n (max, min) pairs given in `dtype`.
 * Replaces calculate_scale_offset (amct_pytorch/quantize_op/utils.py:75-108). */
int amct_scale_offset(const void* vmax, const void* vmin, int dtype, int64_t n, int bits, int symmetric,
                      float* scale, int* offset, int* status, void* stream);

/* Static activation quantization q = sat_int8(rne(x * scale + offset)), scale
 * and offset in x's dtype: one element (per-tensor) or one per token, i.e. per
 * index of the second-to-last axis (x is [outer, tokens, k] contiguous).
 * Stands in for torch_npu.npu_quantize(x, scales, zero_points, torch.int8, axis,
 * div_mode=False) as called at amct_pytorch/deploy_op/npu_quantization_linear.py:98-99;
 * `smooth` folds the multiply at :96-97. */
int amct_quantize_static(const void* x, int dtype, int64_t outer, int64_t tokens, int64_t k,
                         const void* scale, const void* offset, int per_token, const void* smooth,
                         int8_t* q, void* stream);

/* rowsum[n] = sum_k wq[n, k] over INT8 codes stored K-major ([n_rows, k], ld).
 * The integer statement of the fp32 matmul that builds offset_bias
 * (amct_pytorch/deploy_op/npu_quantization_linear.py:56-59). */
int amct_rowsum_i8(const int8_t* wq, int64_t n_rows, int64_t k, int64_t ld, int32_t* out, void* stream);

/* Out-of-place transpose of an INT8 matrix [rows, cols] -> [cols, rows]
 * (the `torch.transpose(...)` the reference applies to the weight codes,
 * amct_pytorch/deploy_op/npu_quantization_linear.py:54). */
int amct_transpose_i8(const int8_t* in, int64_t rows, int64_t cols, int8_t* out, void* stream);

/* ---- tensor-core GEMMs (tcgen05, TMEM accumulators, TMA-fed) -------------- */
enum { AMCT_BIAS_NONE = 0, AMCT_BIAS_I32 = 1, AMCT_BIAS_F32 = 2, AMCT_BIAS_F16 = 3, AMCT_BIAS_BF16 = 4 };
enum { AMCT_GEMM_OUT_F32 = 0, AMCT_GEMM_OUT_F16 = 1, AMCT_GEMM_OUT_BF16 = 2, AMCT_GEMM_OUT_I32 = 3 };

/* W8A8 quantized matmul: acc_i32[m, n] = sum_k a[m, k] * b[n, k], then
 *   bias int32 (per-tensor mode): out = float(acc + bias[n]) * deq_scale[n]
 *   otherwise  (per-token mode) : out = float(acc) * deq_scale[n] (* pertoken_scale[m]) (+ bias[n])
 * each step a separately rounded fp32 operation; AMCT_GEMM_OUT_I32 stores the
 * raw accumulators.  Stands in for torch_npu.npu_quant_matmul(x1, x2, scale=,
 * pertoken_scale=, bias=, output_dtype=) as called at
 * amct_pytorch/deploy_op/npu_quantization_linear.py:100-102.  a [m, k] and
 * b [n, k] are INT8, K contiguous (b is the reference's [K, N] weight buffer
 * stored transposed); both base pointers and both leading dimensions must be
 * multiples of 16 bytes.  bit 1 of *status is set if a device-side wait timed out. */
int amct_gemm_w8a8(const int8_t* a, const int8_t* b, int64_t m, int64_t n, int64_t k, int64_t ld_a, int64_t ld_b,
                   const float* deq_scale, const float* pertoken_scale, const void* bias, int bias_kind,
                   void* out, int out_kind, int64_t ld_out, int* status, void* stream);

/* Which kernel takes m > 128: chosen by the size of b (AUTO), or pinned to the one-CTA / the CTA-pair kernel
 * (tests and comparisons).  Process-wide; returns AMCT_ERR_ARG for another value. */
enum { AMCT_GEMM_VARIANT_AUTO = 0, AMCT_GEMM_VARIANT_SINGLE = 1, AMCT_GEMM_VARIANT_PAIR = 2 };
int amct_gemm_set_variant(int variant);

/* amct_gemm_w8a8 in per-token mode with a SwiGLU epilogue, for a fused gate/up projection
 * whose weight rows are interleaved in blocks of 128: rows [256 j, 256 j + 128) are gate
 * channels [128 j, 128 j + 128) and the next 128 rows the matching up channels (n % 256 == 0).
 * gate and up are dequantized and rounded to bf16 exactly as amct_gemm_w8a8 would store
 * them; out[m, c] = bf16(bf16(silu(gate[m, c])) * up[m, c]), bf16 [m, n/2].  Saves writing
 * and re-reading the [m, n] intermediate of the Llama MLP; the reference has no such
 * fusion (its deploy forward ends at npu_quant_matmul,
 * amct_pytorch/deploy_op/npu_quantization_linear.py:100-102). */
int amct_gemm_w8a8_swiglu(const int8_t* a, const int8_t* b, int64_t m, int64_t n, int64_t k, int64_t ld_a,
                          int64_t ld_b, const float* deq_scale, const float* pertoken_scale, const void* bias,
                          int bias_kind, void* out, int64_t ld_out, int* status, void* stream);

/* 16-bit float GEMM out[m, n] = sum_k a[m, k] * b[n, k] (+ bias[n]), fp32
 * accumulation; dtype AMCT_DTYPE_F16 or AMCT_DTYPE_BF16 for both operands.  The
 * tensor-core stage behind npu_weight_quant_batchmatmul
 * (amct_pytorch/deploy_op/weight_npu_quant_module.py:116-117) once the weight
 * has been dequantized, and behind the HiFloat8 Linear. */
int amct_gemm_f16(const void* a, const void* b, int dtype, int64_t m, int64_t n, int64_t k, int64_t ld_a,
                  int64_t ld_b, const void* bias, int bias_kind, void* out, int out_kind, int64_t ld_out,
                  int* status, void* stream);

/* Dequantize weight codes for the weight-only Linear:
 *   out[n, k] = (q[n, k] + offset[g(k), n]) * scale[g(k), n]   (fp32 steps, rounded to dtype)
 * codes: INT8 [n_rows, k] (bits = 8) or two nibbles per byte [n_rows, k/2] (bits = 4,
 * code + 8, even k in the low nibble), K contiguous.  scale / offset (may be NULL)
 * are in `dtype` (F16 or BF16), laid out [k/group, n_rows], or [1, n_rows] when
 * group == 0 -- the scale_w / offset_w buffers (offset already negated) of
 * amct_pytorch/deploy_op/weight_npu_quant_module.py:59-64.  First stage of
 * torch_npu.npu_weight_quant_batchmatmul (call site :116-117). */
int amct_dequant_weight(const void* codes, int bits, int64_t n_rows, int64_t k, int64_t ld_codes,
                        const void* scale, const void* offset, int group, int dtype, void* out,
                        int64_t ld_out, void* stream);

/* The weight-only quantized Linear in one kernel:
 *   out[m, n] = sum_k x[m, k] * w[n, k] + bias[n],  w[n, k] = (code[n, k] + offset[g(k), n]) * scale[g(k), n]
 * with w rounded to `dtype` exactly as amct_dequant_weight rounds it, dequantized in shared memory
 * ahead of the tcgen05 MMA (the 16-bit weight is never written to HBM).  Replaces
 * torch_npu.npu_weight_quant_batchmatmul (amct_pytorch/deploy_op/weight_npu_quant_module.py:116-117).
 * x [m, k] in `dtype` (F16 / BF16), codes / scale / offset / group as for amct_dequant_weight;
 * bias_kind: AMCT_BIAS_NONE / F32 / F16 / BF16; out_kind: AMCT_GEMM_OUT_F32 / F16 / BF16.
 * k % 64 == 0, group % 64 == 0 (or 0), k % group == 0; other shapes: AMCT_ERR_UNSUPPORTED (use
 * amct_dequant_weight + amct_gemm_f16).  *status bit 1: a bounded wait expired. */
int amct_gemm_w4a16(const void* x, int dtype, const void* codes, int bits, int64_t m, int64_t n, int64_t k,
                    int64_t ld_x, int64_t ld_codes, const void* scale, const void* offset, int group,
                    const void* bias, int bias_kind, void* out, int out_kind, int64_t ld_out, int* status,
                    void* stream);

/* Same kernel with a table instead of the integer rule: one code byte per weight, w[n, k] = lut[code[n, k]],
 * lut = 256 values in `dtype`.  Used for HiFloat8 weights (lut = the exact decode of every code; no counterpart
 * in the reference).  codes [n, k] uint8, K contiguous; k % 64 == 0. */
int amct_gemm_lut8(const void* x, int dtype, const void* codes, const void* lut, int64_t m, int64_t n, int64_t k,
                   int64_t ld_x, int64_t ld_codes, const void* bias, int bias_kind, void* out, int out_kind,
                   int64_t ld_out, int* status, void* stream);

/* ---- MX formats (no counterpart in the reference: amct_pytorch/utils/vars.py:19-20
 * admits int8 / int4 only; the rule is the public OCP Microscaling v1.0 conversion) ---- */

/* MXFP8-E4M3 (elem_bits = 8) or MXFP4-E2M1 (elem_bits = 4) quantization of x [rows, k]
 * (k % 32 == 0) with one E8M0 scale per 32 elements of K.  payload: uint8 [rows, k]
 * (E4M3 bit patterns) or [rows, k/2] (two E2M1 codes per byte, even k in the low
 * nibble).  scales_rowmajor: uint8 [rows, k/32] or NULL.  scales_tiled: NULL or a buffer
 * of amct_mx_tiled_scale_bytes(rows, k, scale_tile_rows) bytes in the tiling the
 * block-scaled GEMM consumes.  scale_tile_rows is the GEMM tile height of the operand:
 * AMCT_MX_TILE_ROWS_A (128) for A, AMCT_MX_TILE_ROWS_B (224) for B.  With
 *   t = r / tile_rows, q = r % tile_rows, atom = t * ceil(tile_rows/128) + q/128:
 *   offset(r, kb) = (atom * ceil(k/128) + kb/4) * 512 + (q%32)*16 + ((q%128)/32)*4 + kb%4 */
enum { AMCT_MX_TILE_ROWS_A = 128, AMCT_MX_TILE_ROWS_B = 224 };
int64_t amct_mx_tiled_scale_bytes(int64_t rows, int64_t k, int scale_tile_rows);
int amct_mx_quant(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int elem_bits, void* payload,
                  void* scales_rowmajor, void* scales_tiled, int scale_tile_rows, void* stream);

/* Block-scaled MX GEMM: out[m, n] = sum over 32-element K blocks of
 *   2^(sfa[m,blk]-127) * 2^(sfb[n,blk]-127) * dot(a[m, blk], b[n, blk])      (+ bias[n])
 * a [m, k] and b [n, k]: E4M3 bytes (elem_bits = 8, k % 128 == 0) or packed E2M1 nibbles
 * (elem_bits = 4, k % 256 == 0), K contiguous, leading dimensions in BYTES (multiples of
 * 16); sfa_tiled / sfb_tiled: the tiled scale buffers written by amct_mx_quant with
 * scale_tile_rows = AMCT_MX_TILE_ROWS_A resp. AMCT_MX_TILE_ROWS_B.  fp32
 * accumulation on the tensor cores (tcgen05 kind::mxf8f6f4 / kind::mxf4 block_scale).
 * bias_kind: AMCT_BIAS_NONE / F32 / F16 / BF16; out_kind: AMCT_GEMM_OUT_F32 / F16 / BF16. */
int amct_gemm_mx(const void* a, const void* sfa_tiled, const void* b, const void* sfb_tiled, int elem_bits,
                 int64_t m, int64_t n, int64_t k, int64_t ld_a_bytes, int64_t ld_b_bytes, const void* bias,
                 int bias_kind, void* out, int out_kind, int64_t ld_out, int* status, void* stream);

/* ---- HiFloat8 (no counterpart in the reference; format and rounding as documented in
 * amct_b200/csrc/hif8.cu and oracle/hif8.py) ---- */

/* x [n] contiguous -> HiF8 codes uint8 [n] (codes != NULL, fake == NULL), or the
 * fake-quantized values decode(encode(x)) in x's dtype (fake != NULL, codes == NULL). */
int amct_hif8_encode(const void* x, int dtype, int64_t n, void* codes, void* fake, void* stream);

/* HiF8 codes uint8 [n] -> values in `dtype` (exact in fp16, bf16 and fp32). */
int amct_hif8_decode(const void* codes, int64_t n, int dtype, void* out, void* stream);

/* ---- Offline checkpoint formats
 * (amct_pytorch/experimental/quantization/DeepSeekV3.2/deploy.py, "deploy.py" below) ---- */

/* E4M3 weight [rows, cols] (uint8 bit patterns, ld_w) times one fp32 scale per block x block tile ->
 * out [rows, cols] in out_dtype (ld_out).  scale is [ceil(rows / block), ceil(cols / block)] with row stride
 * ld_scale; ragged edges use the last tile's scale.  The product is formed in fp32 and rounded once.
 * Replaces weight_dequant (deploy.py:48-90; block = 128, out_dtype = the default dtype, bf16 in its main). */
int amct_ckpt_block_dequant(const void* w_fp8, int64_t rows, int64_t cols, int64_t ld_w, const float* scale,
                            int64_t ld_scale, int block, void* out, int out_dtype, int64_t ld_out, void* stream);

/* Symmetric per-row (per output channel) quantization of w [rows, k] (ld) carried out in w's own dtype T:
 * scale = T(T(max|w| [* clip_factor]) / qmax), code = clamp(round(T(w / scale)), -qmax, qmax), qmax = 2^(bits-1) - 1.
 * bits = 8: codes int8 [rows, k] (ld_codes), scale fp32 [rows], bias unused (may be NULL).
 * bits = 4: rows must be even; codes int8 [rows / 2, k], byte [j, c] = (code[2j, c] & 15) | (code[2j+1, c] << 4)
 *           (pack_4bit, deploy.py:109-125); scale uint64 [rows], low word = the fp32 bit pattern
 *           (scale_fp32_to_u64, deploy.py:93-106); bias fp32 [rows] = T(sum_c T(T(scale * code) * 8))
 *           (int4_assistance_bias, deploy.py:149-157; the sum is exact, hence order independent, for bf16 with
 *           k < 8192 and fp16 with k < 1024, and an fp32 sum in this kernel's own order otherwise).
 * use_clip != 0 applies clip_factor (a host value, sigmoid of the stored clip parameter).  An all-zero row gives
 * scale 0 and codes 0.  Replaces int_weight_quant (deploy.py:128-146). */
int amct_ckpt_rowquant(const void* w, int dtype, int64_t rows, int64_t k, int64_t ld, int bits, int use_clip,
                       float clip_factor, int8_t* codes, int64_t ld_codes, void* scale, float* bias, void* stream);

/* amct_ckpt_block_dequant followed by amct_ckpt_rowquant in ONE pass, for the weights the export both dequantizes
 * and re-quantizes (deploy.py:437-463): each E4M3 element is scaled, rounded to `dtype` (the value weight_dequant
 * would have stored) and quantized from registers, so the 16-bit copy of the weight never goes to memory --
 * 1 byte read and 1 (INT8) or 0.5 (INT4) written per element instead of 1 + 2 and 2 + 1.  Results are bit-identical
 * to the two calls.  w_fp8 [rows, k] (ld_w), block_scale [ceil(rows / block), ceil(k / block)] (ld_scale); the other
 * arguments as amct_ckpt_rowquant. */
int amct_ckpt_dequant_rowquant(const void* w_fp8, int64_t rows, int64_t k, int64_t ld_w, const float* block_scale,
                               int64_t ld_scale, int block, int dtype, int bits, int use_clip, float clip_factor,
                               int8_t* codes, int64_t ld_codes, void* scale, float* bias, void* stream);

/* pack_4bit alone (deploy.py:109-125): codes int8 [rows, k] (ld), rows even -> out int8 [rows / 2, k] (ld_out). */
int amct_ckpt_pack4_rows(const int8_t* codes, int64_t rows, int64_t k, int64_t ld, int8_t* out, int64_t ld_out,
                         void* stream);

/* int4_assistance_bias alone (deploy.py:149-157): codes int8 [rows, k] (ld), scale [rows, groups] contiguous in
 * `dtype` with k % groups == 0 (each scale covers k / groups consecutive codes) -> bias fp32 [rows]. */
int amct_ckpt_int4_bias(const int8_t* codes, int64_t rows, int64_t k, int64_t ld, const void* scale, int dtype,
                        int64_t groups, float* bias, void* stream);

/* Sylvester Hadamard matrix out [n, n] in `dtype`, n a power of two <= 32768.  norm != 0: every doubling divides
 * by fp32 sqrt(2) and rounds to dtype, as the reference does on a tensor of its default dtype, so the magnitude is
 * that chain of log2(n) rounded divisions.  Replaces get_had_pow2 (deploy.py:32-45). */
int amct_hadamard_pow2(int n, int norm, int dtype, void* out, void* stream);

/* ---- KV-cache / indexer activation path
 * (amct_pytorch/experimental/quantization/DeepSeekV3.2/cores, "cores" below) ---- */

/* Per row of x [rows, k] (ld_x), in this order:
 *   rotate != 0: r = dtype(x @ (H / sqrt(k))) in fp32, H the k x k Sylvester Hadamard matrix, k a power of two in
 *                32 .. 512 (rotate_activation, cores/models/deepseek_v3_2/indexer.py:140-151); else r = x;
 *   y = out_dtype(r) (the `.half()` of cores/models/deepseek_v3_2/quant_dsa.py:78-79 when out_dtype differs);
 *   bits == 16: out = y.  Otherwise out = the fake quantization of y, any k (ActivationQuantizer.fake_quant,
 *   cores/quantization/node.py:140-215 and :39-66), per token and dynamic unless the mode is static:
 *     bounds hi = max(row max, 0), lo = min(row min, 0);
 *     AMCT_DSA_DYNAMIC, symmetric: scale = hi / qmax (the negative side does not widen it; 1 when hi == 0), codes in
 *       [-(qmax + 1), qmax], qmax = 2^(bits-1) - 1; asymmetric: a row of zeros uses [-1, 1], scale = (hi - lo) / qmax,
 *       zero = round(-lo / scale), codes in [0, qmax], qmax = 2^bits - 1; every step rounded to out_dtype;
 *     AMCT_DSA_LEARNED_CLIP (lac=True): symmetric bound = max(|lo|, hi) * a; asymmetric hi *= a, lo *= b; a, b = the
 *       sigmoid of clip_factor_a_max / clip_factor_a_min; every step in fp32 (the fp32 parameter promotes);
 *     AMCT_DSA_CLIP_RATIO (clip_ratio): hi *= a, lo *= a, rounded to out_dtype, then as AMCT_DSA_DYNAMIC;
 *     AMCT_DSA_STATIC / AMCT_DSA_STATIC_F32 (per_tensor=True): scale = a, zero = b for every element; steps
 *       rounded to out_dtype / kept in fp32 -- torch's promotion of the activation with the module's scale tensor
 *       (a 0-dim scale taken from observed 16-bit data keeps 16-bit steps; a one-element fp32 buffer promotes).
 *   a and b are host values.
 * out [rows, k] in out_dtype (ld_out).  One warp per row (up to four rows at a time when rotating); one pass over HBM. */
int amct_dsa_rotate_fakequant(const void* x, int dtype, int64_t rows, int64_t k, int64_t ld_x, int rotate, int out_dtype,
                              int bits, int symmetric, int mode, float a, float b, void* out, int64_t ld_out,
                              void* stream);

/* GPTQ: the column-by-column update of one block of b <= 128 (permuted) weight columns, the inner loop of
 * amct_pytorch/quantize_op/gptq_module.py:137-151, in one launch.  w [n, ldw] fp32 holds the block's columns and is
 * updated in place: for i = 0 .. b-1: q = quant_dequant(w[:, i]) (amct_pytorch/utils/quant_util.py:162-188, fp32);
 * e = (w[:, i] - q) / hinv[i, i]; w[:, i:b] -= e (x) hinv[i, i:b]; err[:, i] = e.  hinv [b, ldh]: the block's corner of
 * the upper Cholesky factor of the inverse Hessian.  scale fp32 / offset int32 (NULL: symmetric): [n, factors_ld]
 * when row_factors, else [1, factors_ld]; block column i uses column col_group[i] of them (the group of its
 * original index).  The trailing update w[:, i2:] -= err @ hinv[i1:i2, i2:] stays with the caller (one GEMM). */
int amct_gptq_block(float* w, int64_t n, int64_t ldw, int b, const float* hinv, int64_t ldh, const float* scale,
                    const int* offset, int64_t factors_ld, int row_factors, const int* col_group, int bits,
                    float* err, int64_t lde, void* stream);

/* ---- Glue of the sharded deploy workload (no counterpart in the reference) ---- */

/* h = x + residual (rounded to dtype; residual may be NULL: h = x); n = round(h * rstd * gamma) with
 * rstd = 1 / sqrt(mean(h^2) + eps) in fp32; then the dynamic per-token symmetric INT8 rule of
 * amct_quant_dynamic_pertoken (AMCT_RULE_RELEASED) applied to n: q int8 [rows, k], scale fp32 [rows].
 * residual_out (NULL or [rows, k]) receives h, norm_out (NULL or [rows, k]) receives n.
 * fp16 / bf16 only, k % 8 == 0, k <= 16384, 16-byte aligned rows; other shapes: AMCT_ERR_UNSUPPORTED.
 * One pass: replaces a torch add, a torch rms_norm and the activation-quant kernel of
 * NpuQuantizationLinear.forward (amct_pytorch/deploy_op/npu_quantization_linear.py:95-99). */
int amct_addnorm_quant_pertoken(const void* x, const void* residual, int dtype, int64_t rows, int64_t k,
                                int64_t ld_x, int64_t ld_res, const void* gamma, float eps,
                                void* residual_out, int64_t ld_res_out, void* norm_out, int64_t ld_norm,
                                int8_t* q, int64_t ld_q, float* scale, int* status, void* stream);

/* Rotary embedding (rotate-half) in place on the first `heads` heads of each row of x [tokens, ld]:
 * head h occupies columns [h * head_dim, (h + 1) * head_dim).  cos_table / sin_table [seq, head_dim / 2]
 * in x's dtype; token t uses table row t % seq.  fp16 / bf16, head_dim % 16 == 0.  Each product and sum
 * is rounded to dtype, like the same expression in torch ops. */
int amct_rope_inplace(void* x, int dtype, int64_t tokens, int64_t ld, int heads, int head_dim,
                      const void* cos_table, const void* sin_table, int64_t seq, void* stream);

/* Tensor-core peak of the device, measured (no counterpart in the reference): `ctas` CTAs (one per SM) each issue
 * `steps` K blocks of four tcgen05.mma (M128 x N256, or N224 for the block-scaled kinds, x 32 bytes of K) back to
 * back on operands resident in shared memory: no loads, no stores.  kind: 0 INT8, 1 bf16, 2 MXFP8 (E4M3, E8M0 block
 * scales), 3 MXFP4.  The caller times the launch; one launch performs
 * ctas * steps * amct_mma_peak_ops_per_cta_step(kind) operations.  Bit 1 of *status: a bounded wait expired. */
int amct_mma_peak(int kind, int steps, int ctas, int* status, void* stream);
int64_t amct_mma_peak_ops_per_cta_step(int kind);

/* amct_gemm_w8a8 (per-token mode, no bias, fp16 / bf16 output) for a K-sharded ("row-parallel") Linear under tensor
 * parallelism, whose [m, n] result is one rank's PARTIAL sum: instead of one output matrix, output row r is
 * written to row (slot * rows_per_rank + r % rows_per_rank) of out_ptrs[r / rows_per_rank], the staging buffer
 * [world * rows_per_rank, ld_out] of the rank that owns token rows [j rows_per_rank, (j + 1) rows_per_rank).
 * out_ptrs is a host array of `world` device pointers (this process's peer mappings of every rank's buffer, its
 * own included); slot = this rank.  The epilogue stores whole 128-byte row segments with plain st.global, so
 * the reduce-scatter's transfer runs tile by tile inside the GEMM; the caller orders it against the readers with
 * amct_peer_barrier.  n % 64 == 0; m <= world * rows_per_rank.  The sharded form of
 * NpuQuantizationLinear.forward (amct_pytorch/deploy_op/npu_quantization_linear.py:89-103); the reference has no
 * multi-device path. */
int amct_gemm_w8a8_scatter(const int8_t* a, const int8_t* b, int64_t m, int64_t n, int64_t k, int64_t ld_a,
                           int64_t ld_b, const float* deq_scale, const float* pertoken_scale, void* const* out_ptrs,
                           int world, int slot, int64_t rows_per_rank, int out_kind, int64_t ld_out, int* status,
                           void* stream);

/* amct_addnorm_quant_pertoken for the token-sharded residual stream of that workload.  Input: `parts` holds
 * n_parts partial sums of this rank's `rows` rows, part j at parts + j * part_stride elements (what
 * amct_gemm_w8a8_scatter staged); x = their fp32 sum in that order rounded once to dtype, then as
 * amct_addnorm_quant_pertoken (residual add, RMSNorm, per-token INT8 rule).  Output: codes and scale of row r go
 * to row (row0 + r) of EVERY rank's buffers q_all[d] [*, ld_q] / scale_all[d] (host arrays of `world` device
 * pointers, peer mappings), i.e. the all-gather of the codes happens in this kernel's stores. */
int amct_addnorm_quant_pertoken_tp(const void* parts, int n_parts, int64_t part_stride, const void* residual,
                                   int dtype, int64_t rows, int64_t k, int64_t ld_x, int64_t ld_res,
                                   const void* gamma, float eps, void* residual_out, int64_t ld_res_out,
                                   int8_t* const* q_all, float* const* scale_all, int world, int64_t row0,
                                   int64_t ld_q, int* status, void* stream);

/* Barrier number `seq` between the `world` ranks of one node, in stream order, for collectives made of plain
 * device-to-device copies: flag_arrays[r] is rank r's array of `world` zero-initialised 32-bit words in memory every
 * rank has mapped (host array of device pointers, r = 0 .. world-1; world <= 16).  Callers count seq 1, 2, 3 ... the
 * same on every rank.  One 32-thread block; a peer that has not arrived within two seconds sets bit 1 of *status and
 * the kernel returns; with that bit already set the barrier still signals its peers but does not wait.  No counterpart in the reference (it
 * has no multi-device path); serves the tensor-parallel workload around NpuQuantizationLinear. */
int amct_peer_barrier(void* const* flag_arrays, int world, int rank, uint32_t seq, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AMCT_B200_H_ */
