"""Integer quantization arithmetic of the reference, restated on CPU torch.

TEST INFRASTRUCTURE: the CUDA kernels are compared against these functions.
Every function names the reference lines it follows (paths are relative to the
reference project root).  Operation ORDER and intermediate dtypes are part of
the contract, because integer codes must come out bit-identical:

* max/min are taken in the input dtype, then cast to fp32;
* every division is a true IEEE fp32 division (never a reciprocal multiply);
* rounding is round-half-to-even (``torch.round``);
* ``x / scale + offset`` is two separately rounded fp32 operations.

PINNED against the imported reference through ``tests/golden/*.npz``.
"""
import math

import torch

FLT_EPSILON = 1.192092896e-7  # amct_pytorch/quantize_op/utils.py:23


def _bits(quant_type):
    return int(quant_type.replace('int', ''))


# --------------------------------------------------------------------------
# K0  scale / offset from (max, min)      amct_pytorch/quantize_op/utils.py:75-108
# --------------------------------------------------------------------------
def scale_offset(data_max, data_min, symmetric, quant_type):
    """(max, min) per unit -> (scale fp32, offset int32 | None).

    Symmetric: divisor is 2^(b-1)-1, plus one when the largest-magnitude value
    is negative (quantize_op/utils.py:87-91, :158-176).  Asymmetric: the range
    is widened to contain zero, offset = round(-2^(b-1) - min/scale)
    (:93-103).  A scale below FLT_EPSILON becomes 1 (and the offset -2^(b-1))
    (:26-51).  Non-finite scale raises (:54-72).
    """
    bits = _bits(quant_type)
    hi = data_max.to(torch.float32)
    lo = data_min.to(torch.float32)
    if symmetric:
        neg_dominates = hi.abs() < lo.abs()
        divisor = neg_dominates + (2 ** (bits - 1) - 1)
        bound = torch.where(hi.abs() > lo.abs(), hi.abs(), lo.abs())
        scale = bound / divisor
        offset = None
        scale = torch.where(scale < FLT_EPSILON, torch.tensor(1.0), scale)
    else:
        hi = hi.clamp(min=0)
        lo = lo.clamp(max=0)
        span = 2 ** bits - 1
        half = math.ceil(span / 2)
        scale = (hi - lo) / span
        offset = torch.where(hi != lo, -half - lo / scale,
                             torch.tensor(float(-half)))
        tiny = scale < FLT_EPSILON
        offset = torch.where(tiny, torch.tensor(-(2.0 ** (bits - 1))), offset)
        scale = torch.where(tiny, torch.tensor(1.0), scale)
    if not (torch.isfinite(scale).all() and torch.isfinite(1 / scale).all()):
        raise RuntimeError("Param scale has invalid value inf, nan or zeros!")
    if offset is not None and not torch.isfinite(offset).all():
        raise RuntimeError("Param offset has invalid value inf or nan!")
    scale = scale.to(torch.float32)
    if offset is not None:
        offset = offset.round().to(torch.int32)
    return scale, offset


# --------------------------------------------------------------------------
# K3  min / max by granularity     amct_pytorch/quantize_op/utils.py:111-136
#                                  amct_pytorch/utils/quant_util.py:23-53
# --------------------------------------------------------------------------
def to_groups(t, group_size):
    """[N, K] -> [N, ceil(K/g), g]; the zero padding of the tail takes part in
    the min/max (utils/quant_util.py:34-35)."""
    pad = (-t.shape[-1]) % group_size
    t = torch.nn.functional.pad(t, (0, pad))
    return t.reshape(t.shape[0], t.shape[1] // group_size, group_size)


def weight_min_max(weight, strategy, group_size=None):
    if strategy == 'channel':
        return weight.amin(dim=1, keepdim=True), weight.amax(dim=1, keepdim=True)
    if strategy == 'tensor':
        return weight.min().reshape(1, 1), weight.max().reshape(1, 1)
    g = to_groups(weight, group_size)
    return g.amin(dim=-1, keepdim=True), g.amax(dim=-1, keepdim=True)


def weight_scale_offset(weight, quant_type, symmetric, strategy, group_size=None):
    """MinMaxQuant.calculate_weights_scale_factor_and_quantize
    (amct_pytorch/quantize_op/minmax_module.py:67-76)."""
    lo, hi = weight_min_max(weight, strategy, group_size)
    return scale_offset(hi, lo, symmetric, quant_type)


def column_min_max(x):
    """Per-input-channel observer over all tokens
    (amct_pytorch/quantize_op/smooth_quant_module.py:79-80)."""
    flat = x.reshape(-1, x.shape[-1])
    return flat.amin(dim=0, keepdim=True), flat.amax(dim=0, keepdim=True)


# --------------------------------------------------------------------------
# K4 / K5  integer codes            amct_pytorch/utils/quant_util.py:57-93
# --------------------------------------------------------------------------
def to_codes(t, quant_type):
    """round -> clamp -> container dtype (int8 for int8, int32 for int4)
    (utils/quant_util.py:57-73)."""
    if quant_type == 'int8':
        return t.round().clamp(-128, 127).to(torch.int8)
    if quant_type == 'int4':
        return t.round().clamp(-8, 7).to(torch.int32)
    raise ValueError('Not supported quant_dtype {}'.format(quant_type))


def weight_codes(weight, quant_type, scale, offset=None, group_size=None):
    """utils/quant_util.py:76-93.  Returns codes in the (grouped, padded) shape
    the reference returns; ``crop_groups`` restores [N, K]."""
    t = to_groups(weight, group_size) if group_size else weight
    t = t / scale
    if offset is not None:
        t = t + offset
    return to_codes(t, quant_type)


def crop_groups(t, shape):
    if tuple(t.shape) == tuple(shape):
        return t
    return t.reshape(t.shape[0], -1)[:shape[0], :shape[1]]


def w8a8_weight_codes(weight, scale_w_flat, quant_type='int8'):
    """NpuQuantizationLinear.quant_wts
    (amct_pytorch/deploy_op/npu_quantization_linear.py:72-87)."""
    s = scale_w_flat.reshape(-1, 1) if scale_w_flat.shape[0] > 1 else scale_w_flat
    return to_codes(weight / s, quant_type)


# --------------------------------------------------------------------------
# K1  dynamic per-token activation quantization
# --------------------------------------------------------------------------
def dynamic_per_token(x, rule='released', smooth_recip=None):
    """Row-wise symmetric INT8: returns (codes int8 [M,K], scale fp32 [M]).

    rule='released': amax/amin per row (amct_pytorch/quantize_op/
    minmax_module.py:99-105) -> ``scale_offset`` -> round(x / scale)
    (utils/quant_util.py:57-73,90).  Divisor 127, or 128 when the
    largest-magnitude element of the row is negative.
    rule='experimental': ActivationQuantizer.get_scale_zero + sym_quant
    (amct_pytorch/experimental/quantization/DeepSeekV3.2/cores/quantization/
    node.py:181-204, :39-43) as constructed with sym=True, lac=False: the bound
    is max(row max, 0) -- the negative side does not widen it -- the divisor is
    always 127, a zero bound gives scale 1, and both divisions happen in the
    INPUT dtype.
    smooth_recip: optional [1,K] factor multiplied in first, in the input
    dtype (deploy_op/npu_quantization_linear.py:96-97).
    """
    if smooth_recip is not None:
        x = x * smooth_recip
    x2 = x.reshape(-1, x.shape[-1])
    hi = x2.amax(dim=1, keepdim=True)
    lo = x2.amin(dim=1, keepdim=True)
    if rule == 'released':
        scale, _ = scale_offset(hi, lo, True, 'int8')
        q = to_codes(x2 / scale, 'int8')
        return q.reshape(x.shape), scale.reshape(-1)
    bound = torch.maximum(hi, torch.zeros_like(hi))
    scale = bound / torch.tensor(127)
    scale[bound == 0] = 1
    q = torch.clamp(torch.round(x2 / scale), -128, 127)
    return q.to(torch.int8).reshape(x.shape), scale.reshape(-1).float()


def addnorm_dynamic_per_token(x, gamma, eps, residual=None):
    """Decoder-layer glue in front of a dynamic W8A8 Linear: h = x + residual (a torch add in
    the tensor dtype), n = RMSNorm(h) * gamma evaluated in fp32 and rounded once to the tensor
    dtype, then ``dynamic_per_token(n)``.  Returns (h, n, codes, scale).  The reference has no
    fused form; the quantizer is the one of deploy_op/npu_quantization_linear.py's input path
    with per-token dynamic scales, applied to the rounded n."""
    h = x if residual is None else x + residual
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(dim=-1, keepdim=True) + eps)
    n = ((hf * rstd) * gamma.float()).to(x.dtype)
    q, scale = dynamic_per_token(n)
    return h, n, q, scale


# --------------------------------------------------------------------------
# K7  fake quantization
# --------------------------------------------------------------------------
def fake_quant(weight, quant_type, scale, offset=None, group_size=None):
    """quant_dequant_weight (amct_pytorch/utils/quant_util.py:162-188): all
    intermediate values stay fp32, one rounding to the input dtype at the end."""
    bits = _bits(quant_type)
    shape = weight.shape
    t = to_groups(weight, group_size) if group_size else weight
    t = t / scale
    if offset is not None:
        t = t + offset
    t = torch.clamp(torch.round(t), -2 ** (bits - 1), 2 ** (bits - 1) - 1)
    if offset is not None:
        t = t - offset
    t = t * scale
    return t.reshape(shape[0], -1)[:, :shape[1]].to(weight.dtype)


def fake_quant_awq(weight, quant_type, scale, offset=None, group_size=None):
    """AWQ grid-search variant: do_quant -> convert_precision -> do_dequant
    (amct_pytorch/algorithm/awq.py:129-170, utils/data_utils.py:49-66).  The
    scaled value is rounded to the INPUT dtype before the integer rounding,
    and the offset subtraction happens in that dtype too."""
    bits = _bits(quant_type)
    shape = weight.shape
    t = to_groups(weight, group_size) if group_size else weight
    t = t / scale
    if offset is not None:
        t = t + offset
    t = crop_groups(t, shape).to(weight.dtype)
    t = torch.clamp(torch.round(t), -2 ** (bits - 1), 2 ** (bits - 1) - 1)
    t = to_groups(t, group_size) if group_size else t
    if offset is not None:
        t = t - offset
    t = t * scale
    return crop_groups(t, shape).to(weight.dtype)


# --------------------------------------------------------------------------
# K6  SmoothQuant factor and fold
# --------------------------------------------------------------------------
def smooth_factor(act_absmax, weight, strength):
    """SmoothQuant.calculate_smooth
    (amct_pytorch/quantize_op/smooth_quant_module.py:113-133), computed in the
    dtype of its inputs.  Non-finite or below-eps factors become 1."""
    w_absmax = weight.abs().amax(dim=0, keepdim=True)
    s = (act_absmax ** strength) / (w_absmax ** (1 - strength))
    bad = (s < torch.finfo(act_absmax.dtype).eps) | ~torch.isfinite(s)
    return torch.where(bad, torch.tensor(1.0, dtype=s.dtype), s)


def fold_smooth_into_weight(weight, factor):
    """apply_smooth_weight (amct_pytorch/utils/quant_util.py:96-111): product
    rounded to the weight dtype."""
    return weight * factor.to(weight.dtype)


# --------------------------------------------------------------------------
# K8  deploy constants of the W8A8 module
#     amct_pytorch/deploy_op/npu_quantization_linear.py:27-70, :105-130
# --------------------------------------------------------------------------
def w8a8_deploy_buffers(weight, bias, scale_w, scale_d, offset_d, smooth=None):
    """Returns the dict of buffers NpuQuantizationLinear registers."""
    out_dtype = weight.dtype
    per_token = scale_d.dim() > 1
    off = offset_d if offset_d is not None else torch.tensor([0])
    off = off.repeat(scale_d.shape)
    buf = {
        'act_scale': (1 / scale_d).reshape(-1).to(out_dtype),
        'act_offset': off.reshape(-1).to(out_dtype),
    }
    w = weight
    if smooth is not None:
        w = fold_smooth_into_weight(w, smooth)
        buf['scale_factor'] = 1 / smooth
    sw = scale_w.reshape(-1)
    wq = w8a8_weight_codes(w, sw).transpose(1, 0)          # [K, N]
    buf['quantized_weight'] = wq
    offset_bias = None
    if offset_d is not None:
        row = offset_d.float().repeat(1, weight.shape[-1])
        offset_bias = -1 * (row.float() @ wq.float()).round().to(torch.int32).reshape(-1)
    if per_token:
        buf['deq_scale'] = sw
        buf['pertoken_scale'] = scale_d.reshape(-1).to(torch.float32)
    else:
        buf['deq_scale'] = scale_d * sw
    if bias is not None:
        if per_token:
            b = bias
        else:
            b = (bias.data / (scale_d * sw)).round().to(torch.int32)
        if offset_bias is not None:
            b = b + offset_bias
    else:
        b = offset_bias
    buf['bias'] = b
    return buf


def w4a16_deploy_buffers(weight, bias, quant_type, scale_w, offset_w, group_size, awq_scale=None):
    """NpuWeightQuantizedLinear.__init__ minus the external int4 pack
    (amct_pytorch/deploy_op/weight_npu_quant_module.py:29-100)."""
    w = weight
    buf = {}
    if awq_scale is not None:
        w = w / awq_scale
        buf['scale_factor'] = awq_scale
    q = weight_codes(w, quant_type, scale_w, offset_w, group_size)
    if group_size is not None:
        sw = scale_w.reshape(scale_w.shape[0], scale_w.shape[1])
        ow = None if offset_w is None else offset_w.reshape(sw.shape)
        q = crop_groups(q, weight.shape)
        gs = group_size
    else:
        sw = scale_w.reshape(-1, 1)
        sw = sw.repeat(weight.shape[0], 1) if sw.shape[0] == 1 else sw
        ow = offset_w
        if ow is not None:
            ow = ow.reshape(-1, 1)
            ow = ow.repeat(weight.shape[0], 1) if ow.shape[0] == 1 else ow
        gs = 0
    buf['quantized_weight'] = q.transpose(-1, -2).contiguous()      # [K, N]
    buf['scale_w'] = sw.to(weight.dtype).transpose(-1, -2).contiguous()
    buf['offset_w'] = None if ow is None else (ow * -1).to(weight.dtype).transpose(-1, -2).contiguous()
    b = bias
    if b is not None and weight.dtype == torch.bfloat16:
        b = b.to(torch.float32)
    buf['bias'] = b
    buf['group_size'] = gs
    return buf
