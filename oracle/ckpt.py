"""Offline checkpoint formats of the reference's DeepSeek-V3.2 export script, restated on CPU.

TEST INFRASTRUCTURE: the CUDA kernels of ``amct_b200/csrc/ckpt_formats.cu`` are compared against these
functions.  The reference file is ``amct_pytorch/experimental/quantization/DeepSeekV3.2/deploy.py`` (cited
as ``deploy.py`` below).

The reference runs these steps on tensors of the checkpoint's dtype (bfloat16 in its ``main``), so every
intermediate is rounded to that dtype.  The restatement makes that explicit: every step is one correctly
rounded fp32 operation followed by a round trip through the tensor dtype ``T`` (written ``rt``), which is what
torch's CPU kernels do for 16-bit floats.  The CUDA kernels follow the same recipe step by step.

PINNED against the imported reference through ``tests/golden/ckpt_golden.npz`` (made by
``tests/golden/make_ckpt_golden.py``); the one step that is order dependent, the fp32 row sum of the INT4
bias for float32 inputs, is compared with a tolerance there.
"""
import math

import numpy as np
import torch


def rt(x, dtype):
    """fp32 tensor -> the value a tensor of ``dtype`` holds, back in fp32."""
    return x.to(dtype).to(torch.float32)


# deploy.py:48-90
def weight_dequant(weight_fp8, scale, block_size=128, out_dtype=torch.bfloat16):
    """E4M3 weight [M, N] times one fp32 scale per block_size x block_size tile -> ``out_dtype``.

    ``scale`` is [ceil(M / b), ceil(N / b)]; ragged edges use the last tile's scale (deploy.py:78-83).
    The product is formed in fp32 and rounded once (deploy.py:75, :86-88).
    """
    m, n = weight_fp8.shape
    if tuple(scale.shape) != ((m + block_size - 1) // block_size, (n + block_size - 1) // block_size):
        raise AssertionError('scale shape does not match the weight')
    rows = torch.arange(m) // block_size
    cols = torch.arange(n) // block_size
    s = scale.to(torch.float32)[rows][:, cols]
    return (weight_fp8.to(torch.float32) * s).to(out_dtype)


# deploy.py:93-106
def scale_fp32_to_u64(scale):
    """[k, n] scales -> [k, n] uint64 whose low 32 bits are the fp32 bit pattern (high word zero)."""
    bits = scale.to(torch.float32).contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return bits.view(torch.uint64)


# deploy.py:109-125
def pack_4bit(codes):
    """int8 [N, K] holding 4-bit values -> int8 [N / 2, K]: rows 2j (low nibble) and 2j + 1 (high nibble)."""
    assert codes.dtype == torch.int8 and codes.shape[0] % 2 == 0
    lo = codes[0::2].to(torch.int32) & 0xF
    hi = (codes[1::2].to(torch.int32) & 0xF) << 4
    return (lo | hi).to(torch.uint8).view(torch.int8).contiguous()


# deploy.py:149-157
def int4_assistance_bias(codes, scale_t, dtype):
    """sum_k(scale * q * 8) per row with every product rounded to ``dtype``; fp32 result."""
    term = rt(rt(scale_t * codes.to(torch.float32), dtype) * 8.0, dtype)
    if dtype == torch.float32:
        return term.sum(dim=1)
    return rt(term.sum(dim=1, dtype=torch.float32), dtype)


# deploy.py:128-146
def int_weight_quant(weight, bits=8, weight_clip_factor=None):
    """Symmetric per-row quantization in the weight's own dtype.

    Returns (codes, scale, bias): INT8 -> int8 [N, K], fp32 [N, 1], None;
    INT4 -> packed int8 [N / 2, K], uint64 [N, 1], fp32 [N] (deploy.py:139-144).
    """
    assert weight.dim() == 2
    dtype = weight.dtype
    qmax = float(2 ** (bits - 1) - 1)
    w = weight.to(torch.float32)
    absmax = w.abs().amax(dim=1, keepdim=True)
    if weight_clip_factor is not None:
        # a 0-dim fp32 factor does not promote the 16-bit tensor; the product is rounded to T (deploy.py:132-133)
        absmax = rt(absmax * weight_clip_factor.to(torch.float32).reshape(()), dtype)
    scale = rt(absmax / qmax, dtype)                                       # deploy.py:134
    level = torch.round(rt(w / scale, dtype)).clamp(-qmax, qmax)           # deploy.py:136-137
    codes = level.to(torch.int8)
    if bits == 4:
        return pack_4bit(codes), scale_fp32_to_u64(scale), int4_assistance_bias(codes, scale, dtype)
    return codes, scale, None


# deploy.py:32-45
def get_had_pow2(n, norm=True, dtype=torch.bfloat16):
    """Sylvester Hadamard matrix; with ``norm`` each doubling divides by sqrt(2) IN ``dtype`` (the reference
    builds it from ``torch.ones(1, 1)`` of the default dtype, bfloat16 in its ``main``), so the magnitude is
    log2(n) successively rounded divisions and not 1 / sqrt(n)."""
    if n <= 0 or n & (n - 1):
        raise ValueError(f'n must be a positive power of 2, got{n}')
    mag = torch.ones((), dtype=torch.float32)
    if norm:
        for _ in range(n.bit_length() - 1):
            mag = rt(mag / np.float32(math.sqrt(2)), dtype)
    i = torch.arange(n)
    parity = torch.zeros(n, n, dtype=torch.int64)
    both = i[:, None] & i[None, :]
    for b in range(n.bit_length()):
        parity ^= (both >> b) & 1
    return (mag * (1 - 2 * parity).to(torch.float32)).to(dtype)
