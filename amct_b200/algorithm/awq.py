"""AWQ scale search (host control flow of amct_pytorch/algorithm/awq.py:52-118); the
fake quantization inside the loop is one launch of the row kernel per candidate
(AMCT_OUT_FAKE_AWQ = do_quant -> convert_precision -> do_dequant, awq.py:129-170)."""
import torch

from ..backend import ops

GRIDS_NUM = 'grids_num'


def fake_quantize_scaled(weight, scale_awq, quant_config):
    """((W * s) fake-quantized with fresh min-max factors) / s, as process_weights_for_layers
    (awq.py:30-49) leaves it in layer.weight."""
    cfg = quant_config.get('weights_cfg')
    qt, sym, strat, gs = cfg.get('quant_type'), cfg.get('symmetric'), cfg.get('strategy'), cfg.get('group_size')
    scaled = weight.mul(scale_awq)
    if strat == 'tensor':
        mn, mx = ops.minmax(scaled, 'tensor')
        s, o = ops.scale_offset(mx, mn, sym, qt)
        _, _, fq = ops.quant_rows(scaled, qt, sym, strat, gs, scale=s, offset=o, out='fake_awq')
    else:
        s, o, _ = ops.quant_rows(scaled, qt, sym, strat, gs, out='none')
        _, _, fq = ops.quant_rows(scaled, qt, sym, strat, gs, scale=s, offset=o, out='fake_awq')
    return fq / scale_awq


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
    best, best_loss = None, torch.tensor(float('inf'), device=inputs.device)
    for grid in range(grids):
        s = mean.pow(grid / grids).clamp(min=1e-4).to(torch.float64).view(1, -1)
        s = s / (s.max() * s.min()).sqrt()
        s = torch.clamp(s.to(inputs.dtype), 1e-4, torch.finfo(inputs.dtype).max)
        layer.weight.data = fake_quantize_scaled(ori_weight, s, quant_config)
        loss = (ori_out - layer(inputs)).float().pow(4).mean()
        if not torch.isnan(loss) and loss < best_loss:
            best_loss, best = loss, s
        layer.weight.data = ori_weight
    if best is None or torch.isinf(best_loss):
        raise RuntimeError("Run AWQ error! Got invalid loss.")
    return best
