"""AWQ scale search (host control flow of amct_pytorch/algorithm/awq.py:52-118); the
fake quantization inside the loop is one launch of the row kernel per candidate
(AMCT_OUT_FAKE_AWQ = do_quant -> convert_precision -> do_dequant, awq.py:129-170)."""
import torch

from ..backend import ops

GRIDS_NUM = 'grids_num'


def fake_quantize_scaled(weight, scale_awq, quant_config):
    """((W * s) fake-quantized with fresh min-max factors) / s, as process_weights_for_layers
    (awq.py:30-49) leaves it in layer.weight.  Channel and group granularity: ONE kernel launch does the multiply by
    s (rounded to the weight dtype like the reference's tensor op), the min-max factors and the AWQ fake quantization
    from a single read of W; the tensor granularity needs the tensor-wide bounds first."""
    cfg = quant_config.get('weights_cfg')
    qt, sym, strat, gs = cfg.get('quant_type'), cfg.get('symmetric'), cfg.get('strategy'), cfg.get('group_size')
    if strat == 'tensor':
        scaled = weight.mul(scale_awq)
        mn, mx = ops.minmax(scaled, 'tensor')
        s, o = ops.scale_offset(mx, mn, sym, qt)
        _, _, fq = ops.quant_rows(scaled, qt, sym, strat, gs, scale=s, offset=o, out='fake_awq', check=False)
    else:
        _, _, fq = ops.quant_rows(weight, qt, sym, strat, gs, out='fake_awq', pre=scale_awq, pre_op='mul', check=False)
    return fq / scale_awq


def _per_unit(weight, granularity, group_size):
    """weight viewed so that the quant factors broadcast over it: [N, K/g, g] for groups, as it is otherwise."""
    if granularity != 'group':
        return weight
    n, k = weight.shape
    pad = (-k) % group_size
    if pad:
        weight = torch.nn.functional.pad(weight, (0, pad))
    return weight.reshape(n, -1, group_size)


def do_quant(weight, scale_w, offset_w, weight_granularity, group_size=None):
    """weight / scale_w (+ offset_w) in the weight's dtype, not yet rounded to integers: the first of the three steps the
    reference composes its AWQ fake quantization from (awq.py:129-149).  The search loop here uses the fused kernel
    mode instead (AMCT_OUT_FAKE_AWQ: this step, convert_precision and do_dequant in one pass); the step is offered
    under its own name for callers that used it directly.  Device tensors in, device tensor out."""
    shape, dtype = weight.shape, weight.dtype
    t = _per_unit(weight, weight_granularity, group_size) / scale_w
    if offset_w is not None:
        t = t + offset_w
    return t.reshape(shape[0], -1)[:, :shape[1]].to(dtype)


def do_dequant(weight, scale, offset, weight_granularity, group_size=None):
    """(weight - offset) * scale, the last of the three steps (awq.py:152-170)."""
    shape = weight.shape
    t = _per_unit(weight, weight_granularity, group_size)
    if offset is not None:
        t = t - offset
    return (t * scale).reshape(shape[0], -1)[:, :shape[1]].to(weight.dtype)


def calculate_scale_offset_by_granularity(weight, quant_config):
    """(scale, offset) of a weight by the configured granularity, one read of the weight (awq.py:121-126)."""
    from ..quantize_op.utils import weight_scale_offset
    cfg = quant_config.get('weights_cfg')
    return weight_scale_offset(weight, cfg.get('quant_type'), cfg.get('symmetric'), cfg.get('strategy'), cfg.get('group_size'))


def process_weights_for_layers(layers, scale_awq, quant_config):
    """Leaves ((W * s) fake-quantized) / s in every layer's weight (awq.py:30-49).  The reference's three passes per
    layer -- do_quant, convert_precision, do_dequant (awq.py:129-170) -- are one kernel mode here and are not offered
    one by one."""
    for layer in layers:
        layer.weight.data = fake_quantize_scaled(layer.weight.data, scale_awq, quant_config)


def apply_scale(scale_awq, ori_module, input_data):
    """W *= s and x /= s in place, as the reference does with tensor ops (awq.py:108-118)."""
    scale = scale_awq.to(ori_module.weight.device)
    ori_module.weight.data.mul_(scale)
    input_data.div_(scale)


@torch.no_grad()
def search_scale(inputs, layer, quant_config):
    """Grid search over s = mean|x|^(i/grids) (normalised), minimising the 4th-power output error of
    the fake-quantized layer; returns the best [1, cin] scale."""
    if not torch.isfinite(inputs).all():
        raise RuntimeError("Run AWQ error! Invalid value(nan or inf) in activation!")
    if not torch.isfinite(layer.weight.data).all():
        raise RuntimeError("Run AWQ error! Invalid value(nan or inf) in weight!")
    grids = quant_config.get('algorithm').get('awq').get(GRIDS_NUM)
    ori_out = layer(inputs)
    ori_weight = layer.weight.data.clone()
    mean = inputs.abs().contiguous().view(-1, inputs.shape[-1]).mean(0)
    # the whole search stays on the device: candidate scale, fused scale + fake-quant kernel, the layer's GEMM, the
    # 4th-power loss, and the running best kept with torch.where -- the host reads one number, after the last candidate
    best = torch.ones((1, inputs.shape[-1]), dtype=inputs.dtype, device=inputs.device)
    best_loss = torch.full((), float('inf'), device=inputs.device)
    for grid in range(grids):
        s = mean.pow(grid / grids).clamp(min=1e-4).to(torch.float64).view(1, -1)
        s = s / (s.max() * s.min()).sqrt()
        s = torch.clamp(s.to(inputs.dtype), 1e-4, torch.finfo(inputs.dtype).max)
        layer.weight.data = fake_quantize_scaled(ori_weight, s, quant_config)
        loss = (ori_out - layer(inputs)).float().pow(4).mean()
        better = ~torch.isnan(loss) & (loss < best_loss)
        best_loss = torch.where(better, loss, best_loss)
        best = torch.where(better, s, best)
        layer.weight.data = ori_weight
    if bool(torch.isinf(best_loss)):
        raise RuntimeError("Run AWQ error! Got invalid loss.")
    return best
