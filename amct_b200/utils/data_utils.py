"""Input checks shared by the quant modules (amct_pytorch/utils/data_utils.py:26-46)."""


def check_linear_input_dim(input_tensor):
    if not 2 <= input_tensor.dim() <= 6:
        raise RuntimeError("Linear quant only support dim from 2 to 6")


def check_data_type(tensor_dtype, data_types):
    if tensor_dtype not in data_types:
        raise RuntimeError('Not support tensor dtype {}, support dtypes {}.'.format(tensor_dtype, data_types))


def convert_precision(ori_tensor, quant_dtype):
    """clamp(round(x)) to the integer range of ``quant_dtype``, kept in x's dtype (amct_pytorch/utils/data_utils.py:49-66):
    one launch of the row quantizer's fake-quant mode with a scale of one."""
    import torch
    from ..backend import ops
    if ori_tensor.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(
            "dtype {} not support now, only support float32/float16/bfloat16.".format(ori_tensor.dtype))
    rows = ori_tensor.reshape(-1, ori_tensor.shape[-1])
    one = torch.ones(1, dtype=torch.float32, device=rows.device)
    _, _, out = ops.quant_rows(rows, quant_dtype, True, 'tensor', scale=one, out='fake', check=False)
    return out.reshape(ori_tensor.shape)
