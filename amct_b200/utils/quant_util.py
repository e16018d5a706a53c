"""Weight quantization helpers with the names and results of amct_pytorch/utils/quant_util.py ("quant_util.py"
below), on the CUDA row quantizer.

Rounding, clamping and the fake-quantization round trip run in ``amct_quant_rows`` (``amct_b200/csrc/quant_rows.cu``
and the kernels it dispatches to); what stays in torch here is what the reference also does as a plain tensor op and
what is layout only: zero padding and group reshape, and the broadcast multiply / divide by a SmoothQuant or AWQ
factor (the quantizers of this package fold that factor into their load instead of calling these two functions).
CPU tensors raise, as everywhere in this package.
"""
import torch

from ..backend import ops
from ..deploy_op.weight_npu_quant_module import check_scale_offset_shape  # noqa: F401  (quant_util.py:114-140)
from .vars import INT4, INT8


def pad_zero_by_group(tensor, group_size):
    """Zero-pads the last axis up to a multiple of ``group_size`` (quant_util.py:23-36)."""
    pad = (group_size - (tensor.shape[-1] % group_size)) % group_size
    return torch.nn.functional.pad(tensor, (0, pad), 'constant', 0)


def convert_to_per_group_shape(input_tensor, group_size):
    """[N, K] -> [N, ceil(K / g), g], the tail zero padded (quant_util.py:39-53)."""
    padded = pad_zero_by_group(input_tensor, group_size)
    return padded.reshape(padded.shape[0], padded.shape[1] // group_size, group_size)


def _strategy(rows, scale, group_size):
    if group_size:
        return 'group'
    return 'tensor' if scale.numel() == 1 else 'channel'


def _as_rows(tensor):
    """Any rank -> [rows, last]; the quantizer works on two dimensions."""
    return tensor.reshape(-1, tensor.shape[-1]) if tensor.dim() != 2 else tensor


@torch.no_grad()
def convert_dtype(ori_tensor, quant_dtype):
    """round -> clamp -> int8 (INT8) or int32 (INT4) (quant_util.py:56-73): the row quantizer with a scale of one."""
    if quant_dtype not in (INT8, INT4):
        raise ValueError('Not supported quant_dtype {}'.format(quant_dtype))
    rows = _as_rows(ori_tensor)
    if rows.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        rows = rows.to(torch.float32)
    one = torch.ones(1, dtype=torch.float32, device=rows.device)
    _, _, codes = ops.quant_rows(rows, quant_dtype, True, 'tensor', scale=one, out='i8' if quant_dtype == INT8 else 'i32',
                                 check=False)
    return codes.reshape(ori_tensor.shape)


def quant_weight(tensor, wts_type, scale, offset=None, group_size=None):
    """clamp(round(w / scale [+ offset])) as integer codes (quant_util.py:76-93).  With ``group_size`` the result has
    the grouped shape [N, ceil(K / g), g] like the reference's, the padded tail quantized along with the rest."""
    if wts_type not in (INT8, INT4):
        raise ValueError('Not supported quant_dtype {}'.format(wts_type))
    work = pad_zero_by_group(tensor, group_size) if group_size else tensor
    _, _, codes = ops.quant_rows(work, wts_type, offset is None, _strategy(work.shape[0], scale, group_size), group_size,
                                 scale=scale, offset=offset, out='i8' if wts_type == INT8 else 'i32', check=False)
    if group_size:
        return codes.reshape(work.shape[0], work.shape[1] // group_size, group_size)
    return codes


def apply_smooth_weight(smooth_factor, ori_weight):
    """weight * smooth_factor ([1, cin]) in the weight's dtype (quant_util.py:96-111)."""
    smooth_factor = smooth_factor.to(device=ori_weight.device, dtype=ori_weight.dtype)
    if list(smooth_factor.shape) != [1, ori_weight.shape[1]]:
        raise RuntimeError("smooth_factor shape should be {} current shape is {}"
                           .format([1, ori_weight.shape[1]], list(smooth_factor.shape)))
    return ori_weight * smooth_factor


def apply_awq_quantize_weight(weight_tensor, awq_scale, group_size):
    """weight / awq_scale ([1, cin]) (quant_util.py:143-159)."""
    cin = weight_tensor.shape[1]
    if list(awq_scale.shape) != [1, cin]:
        raise RuntimeError("AWQ params scale.shape should be [1, {}] current shape is {}".format(
            cin, list(awq_scale.shape)))
    return weight_tensor / awq_scale


def quant_dequant_weight(tensor, quant_params=None, scale=None, offset=None):
    """Quantize and dequantize in one pass: all steps in fp32, one rounding to the weight dtype at the end, the padded
    tail of a ragged last group dropped (quant_util.py:162-188)."""
    cfg = quant_params.get('weights_cfg')
    wts_dtype, group_size = cfg.get('quant_type'), cfg.get('group_size')
    _, _, fake = ops.quant_rows(tensor, wts_dtype, offset is None, _strategy(tensor.shape[0], scale, group_size),
                                group_size, scale=scale, offset=offset, out='fake', check=False)
    return fake
