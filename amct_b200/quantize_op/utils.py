"""Scale/offset and weight statistics, computed by the CUDA kernels.

Function names and return shapes follow amct_pytorch/quantize_op/utils.py:75-136;
the arithmetic runs in amct_quant_rows / amct_minmax* / amct_scale_offset.
"""
import torch

from ..backend import ops

FLT_EPSILON = 1.192092896e-7


def calculate_scale_offset(data_max, data_min, symmetric, data_type):
    """(max, min) -> (scale fp32, offset int32 | None), same shape as data_max."""
    return ops.scale_offset(data_max, data_min, symmetric, data_type)


def _grouped_rows(weight, group_size):
    """[N, K] -> contiguous [N * G, g] with the ragged tail zero padded
    (amct_pytorch/utils/quant_util.py:23-53)."""
    n, k = weight.shape
    pad = (-k) % group_size
    if pad:
        weight = torch.nn.functional.pad(weight, (0, pad))
    return weight.reshape(n * ((k + pad) // group_size), group_size), (k + pad) // group_size


def get_weight_min_max_by_granularity(weight_data, quant_config):
    cfg = quant_config.get('weights_cfg')
    strategy = cfg.get('strategy')
    n = weight_data.shape[0]
    if strategy == 'channel':
        mn, mx = ops.minmax_rows(weight_data)
        return mn.reshape(n, 1), mx.reshape(n, 1)
    if strategy == 'tensor':
        mn, mx = ops.minmax(weight_data, 'tensor')
        return mn.reshape(1, 1), mx.reshape(1, 1)
    rows, groups = _grouped_rows(weight_data, cfg.get('group_size'))
    mn, mx = ops.minmax_rows(rows)
    return mn.reshape(n, groups, 1), mx.reshape(n, groups, 1)


def weight_scale_offset(weight, wts_type, symmetric, strategy, group_size=None, pre=None, pre_op='none'):
    """Fused min/max + scale rule over a weight, one read of the weight.  `pre`
    is an optional [1, K] factor applied first in the weight dtype (SmoothQuant
    multiply / AWQ divide).  Shapes: [N,1] | [1,1] | [N, ceil(K/g), 1]."""
    n, k = weight.shape
    if strategy == 'tensor':
        w = weight
        if pre is not None:
            w = weight * pre.to(weight.dtype) if pre_op == 'mul' else weight / pre.to(weight.dtype)
        mn, mx = ops.minmax(w, 'tensor')
        scale, offset = ops.scale_offset(mx, mn, symmetric, wts_type)
        return scale.reshape(1, 1), None if offset is None else offset.reshape(1, 1)
    scale, offset, _ = ops.quant_rows(weight, wts_type, symmetric, strategy, group_size, out='none',
                                      pre=pre, pre_op=pre_op if pre is not None else 'none')
    shape = (n, 1) if strategy == 'channel' else (n, -1, 1)
    return scale.reshape(shape), None if offset is None else offset.reshape(shape)


# ---------------------------------------------------------------------------------------------
# The smaller pieces of the scale rule under the reference's names (amct_pytorch/quantize_op/utils.py:26-72,
# :139-176).  calculate_scale_offset above evaluates the whole rule in one kernel; these act on factor-sized tensors
# (one value per channel or group) and exist for callers that use them one by one.
# ---------------------------------------------------------------------------------------------
def get_int_quant_scope(data_type, symmetric, abs_max_is_negative=False):
    """Divisor of the scale rule: 2^b - 1 (asymmetric) or 2^(b-1) - 1, plus one when the largest magnitude is
    negative (utils.py:158-176)."""
    quant_bits = int(data_type.replace('int', ''))
    if not symmetric:
        return pow(2, quant_bits) - 1
    return abs_max_is_negative + pow(2, quant_bits - 1) - 1


def check_scale_offset(scale, offset):
    """Raises the reference's errors for a non-finite or zero scale and a non-finite offset (utils.py:54-72)."""
    if not (torch.all(torch.isfinite(scale)) and torch.all(torch.isfinite(1 / scale))):
        raise RuntimeError("Param scale has invalid value inf, nan or zeros!")
    if offset is not None and not torch.all(torch.isfinite(offset)):
        raise RuntimeError("Param offset has invalid value inf or nan!")


def process_scale(scale, offset, symmetric, numbit=8):
    """A scale below FLT_EPSILON becomes 1 (and its offset -2^(b-1)); then check_scale_offset (utils.py:26-51)."""
    tiny = scale < FLT_EPSILON
    if not symmetric:
        offset = torch.where(tiny, torch.tensor(-pow(2.0, numbit - 1), device=offset.device), offset)
    scale = torch.where(tiny, torch.tensor(1.0, device=scale.device), scale)
    check_scale_offset(scale, offset)
    return scale, offset


def convert_to_dst_shape(input_tensor, dst_shape):
    """[N, G, g] (padded) -> [N, K]: flattens the groups and drops the padded tail (utils.py:139-155)."""
    if input_tensor.shape == dst_shape:
        return input_tensor
    flat = input_tensor.reshape(input_tensor.shape[0], input_tensor.shape[1] * input_tensor.shape[2])
    return flat[:dst_shape[0], :dst_shape[1]]
