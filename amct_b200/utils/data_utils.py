"""Input checks shared by the quant modules (amct_pytorch/utils/data_utils.py:26-46)."""


def check_linear_input_dim(input_tensor):
    if not 2 <= input_tensor.dim() <= 6:
        raise RuntimeError("Linear quant only support dim from 2 to 6")


def check_data_type(tensor_dtype, data_types):
    if tensor_dtype not in data_types:
        raise RuntimeError('Not support tensor dtype {}, support dtypes {}.'.format(tensor_dtype, data_types))
