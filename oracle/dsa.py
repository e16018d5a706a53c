"""KV-cache / indexer activation path of the reference's DeepSeek-V3.2 tree, restated on CPU.

TEST INFRASTRUCTURE: the CUDA kernel of ``amct_b200/csrc/kv_quant.cu`` is compared against these functions.
Reference files, relative to amct_pytorch/experimental/quantization/DeepSeekV3.2/cores:
``quantization/node.py`` (ActivationQuantizer, "node.py" below) and ``models/deepseek_v3_2/indexer.py``
(rotate_activation, "indexer.py" below); call sites in ``models/deepseek_v3_2/quant_dsa.py:75-82, 116-125, 195-199``.

The fake quantization is restated as single correctly rounded fp32 operations, each followed by a rounding to
the dtype torch carries the value in (``rt``).  Which dtype that is follows torch's promotion rules and is part of
the contract: without learned clipping everything stays in the activation dtype; with it the clip parameter, an
fp32 tensor of one element, promotes the bounds -- and every step after them -- to fp32, and only the final
result is cast back (node.py:154-159).

PINNED against the imported reference through ``tests/golden/dsa_golden.npz``
(``tests/golden/make_dsa_golden.py``): the fake quantization bit for bit; the rotation, an fp32 matrix product
whose summation order is the BLAS library's, to one unit in the last place of the activation dtype.
"""
import numpy as np
import torch


def rt(x, dtype):
    return x.to(dtype).to(torch.float32)


# node.py:181-215 (bounds and scale), :39-66 (quantize / dequantize), :140-159 (fake_quant)
def activation_fake_quant(x, bits=8, sym=True, lac=False, clip_max_raw=None, clip_min_raw=None, clip_ratio=None):
    """Per-token (last axis) dynamic fake quantization of ActivationQuantizer with per_tensor=False.

    Bounds: hi = max(row max, 0), lo = min(row min, 0) (node.py:186-188).
    sym, no clipping: scale = hi / qmax -- the negative side does NOT widen the bound -- and 1 where hi == 0.
    sym, clipping: bound = max(|lo|, hi) * sigmoid(clip_max_raw).
    asym (clipping): hi *= sigmoid(clip_max_raw), lo *= sigmoid(clip_min_raw); a row of zeros uses [-1, 1];
    scale = (hi - lo) / qmax, zero = round(-lo / scale).
    Codes are clamped to [-(qmax + 1), qmax] (sym) or [0, qmax] (asym).
    clip_ratio (a plain number, only without learned clipping): both bounds times the ratio, rounded to the
    activation dtype (node.py:198-200).
    """
    if bits == 16:
        return x
    dtype = x.dtype
    comp = torch.float32 if lac else dtype          # the fp32 clip parameter promotes everything after it
    shape = x.shape
    xf = x.reshape(-1, shape[-1]).to(torch.float32)
    hi = xf.amax(1, keepdim=True).clamp(min=0)
    lo = xf.amin(1, keepdim=True).clamp(max=0)
    if clip_ratio is not None and not lac:
        hi, lo = rt(hi * clip_ratio, dtype), rt(lo * clip_ratio, dtype)
    if sym:
        qmax = float(2 ** (bits - 1) - 1)
        if lac:
            bound = torch.maximum(lo.abs(), hi) * torch.sigmoid(torch.tensor(clip_max_raw, dtype=torch.float32))
        else:
            bound = hi
        scale = rt(bound / qmax, comp)
        scale[bound == 0] = 1.0
        # round_ste computes (round(t) - t) + t (node.py:23-27): exact, except that a zero comes out as +0
        level = (torch.round(rt(xf / scale, comp)) + 0.0).clamp(-(qmax + 1), qmax)
        return rt(scale * level, comp).to(dtype).reshape(shape)
    qmax = float(2 ** bits - 1)
    if lac:
        hi = hi * torch.sigmoid(torch.tensor(clip_max_raw, dtype=torch.float32))
        lo = lo * torch.sigmoid(torch.tensor(clip_min_raw, dtype=torch.float32))
    flat = (hi == 0) & (lo == 0)
    hi = torch.where(flat, torch.ones_like(hi), hi)
    lo = torch.where(flat, -torch.ones_like(lo), lo)
    scale = rt(rt(hi - lo, comp) / qmax, comp)
    zero = torch.round(rt(-lo / scale, comp))
    level = rt(torch.round(rt(xf / scale, comp)) + zero, comp).clamp(0, qmax)
    return rt(scale * rt(level - zero, comp), comp).to(dtype).reshape(shape)


# node.py:161-179 (per-tensor bounds -> scale / zero), :117-128 (observation)
def observe(chunks):
    """Running bounds as the observe mode keeps them: fp32 one-element buffers of zeros, REPLACED by the chunk's own
    0-dim max / min (in the chunk's dtype) whenever that exceeds them."""
    hi, lo = torch.zeros(1), torch.zeros(1)
    for x in chunks:
        if x.max() > hi:
            hi = x.max()
        if x.min() < lo:
            lo = x.min()
    return hi, lo


def per_tensor_scale_zero(hi, lo, bits=8, sym=True, lac=False, clip_max_raw=None, clip_min_raw=None):
    """(scale, zero) tensors with the dtypes and shapes torch gives them: they decide, by promotion against the
    activation, whether the quantization runs in the activation dtype or in fp32."""
    if lac:
        hi = hi * torch.sigmoid(torch.full((1,), clip_max_raw))
        lo = lo * torch.sigmoid(torch.full((1,), clip_min_raw))
    if sym:
        bound = torch.maximum(lo.abs(), hi)
        scale = bound / torch.tensor(2 ** (bits - 1) - 1)
        return scale, torch.zeros_like(scale)
    scale = (hi - lo) / torch.tensor(2 ** bits - 1)
    return scale, torch.round(-lo / scale)


# node.py:140-159 with a given scale and zero point, :39-66
def static_fake_quant(x, scale, zero, bits=8, sym=True):
    """Fake quantization with one given scale / zero point; the arithmetic dtype is torch's promotion of the
    activation with the scale tensor (a 0-dim scale of a 16-bit dtype keeps 16-bit steps, a one-element fp32
    buffer promotes to fp32)."""
    dtype = x.dtype
    comp = torch.result_type(x, scale)
    xf = x.to(torch.float32)
    s, z = float(scale), float(zero)
    if sym:
        qmax = float(2 ** (bits - 1) - 1)
        level = (torch.round(rt(xf / s, comp)) + 0.0).clamp(-(qmax + 1), qmax)
        return rt(s * level, comp).to(dtype)
    qmax = float(2 ** bits - 1)
    level = rt(torch.round(rt(xf / s, comp)) + z, comp).clamp(0, qmax)
    return rt(s * rt(level - z, comp), comp).to(dtype)


# indexer.py:140-151
def rotate_activation(x):
    """x @ (H / sqrt(d)) over the last axis in fp32, H the Sylvester Hadamard matrix, result in x's dtype.
    The entries of the matrix are +-fl32(1 / fl32(sqrt(d))) as the reference builds them."""
    d = x.shape[-1]
    if d <= 0 or d & (d - 1):
        raise ValueError('the rotated axis must be a power of two')
    i = torch.arange(d)
    both = i[:, None] & i[None, :]
    parity = torch.zeros(d, d, dtype=torch.int64)
    for b in range(d.bit_length()):
        parity ^= (both >> b) & 1
    entry = np.float32(1.0) / np.float32(d ** 0.5)
    h = (1 - 2 * parity).to(torch.float32) * float(entry)
    return (x.to(torch.float32) @ h).to(x.dtype)
