"""CPU statement of the four external ops the deploy modules call.

TEST INFRASTRUCTURE.  PARITY UNPINNED: ``torch_npu`` (unversioned dependency,
requirements.txt:2) is not part of the reference tree and the reference's
tests mock these ops without rounding, clamping or per-token / group factors
(tests/amct_pytorch/mock_torch_npu.py:33-87).  What is written here follows
(i) the documented formula ``clip(round(x/scale + offset), -128, 127)``
(docs/量化概念.md:31-34), (ii) how the call sites build the operands
(amct_pytorch/deploy_op/npu_quantization_linear.py:36-68,98-130,
amct_pytorch/deploy_op/weight_npu_quant_module.py:53-73,116-117) and
(iii) ``torch.round`` (half to even) as used by every in-tree quantizer.
The fp32 operation order below is the contract of the CUDA epilogues.
"""
import torch


def _along(v, ndim, axis):
    shape = [1] * ndim
    shape[axis] = -1
    return v.float().reshape(shape)


def npu_quantize(x, scales, zero_points, dtype=torch.int8, axis=-1, div_mode=False):
    """q = sat_int8(rne(x*scale + zero_point)); ``scales`` is the reciprocal
    scale already rounded to x's dtype (npu_quantization_linear.py:42-45).
    axis=-1 with one element is per-tensor, axis=-2 is per-token."""
    assert dtype == torch.int8 and not div_mode
    s = scales.float() if scales.numel() == 1 else _along(scales, x.dim(), axis)
    y = x.float() * s
    if zero_points is not None:
        z = zero_points.float() if zero_points.numel() == 1 else _along(zero_points, x.dim(), axis)
        y = y + z
    return y.round().clamp(-128, 127).to(torch.int8)


def int32_matmul(q, wq_kn, fast=False):
    """Exact INT8 x INT8 -> INT32 accumulation.  fast=True uses torch's CPU int8
    GEMM (same exact result, all host threads) -- the CPU-baseline timing path."""
    q2 = q.reshape(-1, q.shape[-1])
    if fast:
        return torch._int_mm(q2, wq_kn)
    return (q2.to(torch.int64) @ wq_kn.to(torch.int64)).to(torch.int32)


def npu_quant_matmul(q, wq_kn, scale, pertoken_scale=None, bias=None, output_dtype=torch.bfloat16, fast=False):
    """INT32 GEMM, then: (+ int32 bias) * scale[n] (* pertoken[m]) (+ float
    bias), in that order, each step a separately rounded fp32 operation.
    int32 bias = per-tensor mode (npu_quantization_linear.py:117-120), float
    bias = per-token mode (:121-122)."""
    lead = q.shape[:-1]
    acc = int32_matmul(q, wq_kn, fast)
    if bias is not None and bias.dtype == torch.int32:
        acc = acc + bias
    y = acc.float() * scale.float().reshape(1, -1)
    if pertoken_scale is not None:
        y = y * pertoken_scale.float().reshape(-1, 1)
    if bias is not None and bias.dtype != torch.int32:
        y = y + bias.float().reshape(1, -1)
    return y.to(output_dtype).reshape(*lead, -1)


def dequant_weight(wq_kn, antiquant_scale, antiquant_offset, group_size, dtype):
    """(q + aoff[g(k), n]) * ascale[g(k), n], rounded to ``dtype`` (the MMA
    operand dtype).  aoff is the NEGATED offset
    (weight_npu_quant_module.py:62-64)."""
    k = wq_kn.shape[0]

    def rows(v):
        v = v.float()
        return v.repeat_interleave(group_size, 0)[:k] if group_size else v.reshape(1, -1)

    w = wq_kn.float()
    if antiquant_offset is not None:
        w = w + rows(antiquant_offset)
    return (w * rows(antiquant_scale)).to(dtype)


def npu_weight_quant_batchmatmul(x, wq_kn, antiquant_scale, antiquant_offset=None,
                                 bias=None, antiquant_group_size=0):
    """x @ dequant(w) + bias with fp32 accumulation; output in x's dtype."""
    w = dequant_weight(wq_kn, antiquant_scale, antiquant_offset, antiquant_group_size, x.dtype)
    y = x.reshape(-1, x.shape[-1]).float() @ w.float()
    if bias is not None:
        y = y + bias.float().reshape(1, -1)
    return y.to(x.dtype).reshape(*x.shape[:-1], -1)


def npu_convert_weight_to_int4pack(w_kn_int32):
    """[K, N] int32 codes in [-8, 7] -> int32 [K, N / 8]: eight two's-complement nibbles per word along N, column
    8 j + i in bits [4 i, 4 i + 4) of word j -- the form the device op hands back to
    amct_pytorch/deploy_op/weight_npu_quant_module.py:53-57 and a deployed checkpoint stores."""
    k, n = w_kn_int32.shape
    nib = (w_kn_int32.to(torch.int64) & 0xF).reshape(k, n // 8, 8)
    word = sum(nib[..., i] << (4 * i) for i in range(8))
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


def pack_int4_along_k(w_kn_int32):
    """[K, N] int32 codes in [-8, 7] -> uint8 [K/2, N], the payload this build's kernels read: u = q + 8, row 2j in the
    low nibble and row 2j+1 in the high nibble of byte [j, n] (low nibble =
    first element, as the in-tree ``pack_4bit`` does, amct_pytorch/experimental/
    quantization/DeepSeekV3.2/deploy.py:109-125).  Pairing along K and the bias
    of 8 are this build's choices: the GEMM streams K-contiguous bytes, and
    zero-points then live in [0, 15].  The result is a transposed view of a
    contiguous [N, K/2] buffer."""
    u = (w_kn_int32 + 8).to(torch.uint8)
    packed_nk = (u[0::2, :] | (u[1::2, :] << 4)).t().contiguous()
    return packed_nk.t()


def unpack_int4(packed_k2n):
    """Inverse of the pack: uint8 [K/2, N] -> int32 [K, N]."""
    lo = (packed_k2n & 0xF).to(torch.int32) - 8
    hi = (packed_k2n >> 4).to(torch.int32) - 8
    return torch.stack((lo, hi), dim=1).reshape(-1, packed_k2n.shape[1])
