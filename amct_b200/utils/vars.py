"""Constants of the quantization schema (same names and meaning as
amct_pytorch/utils/vars.py:19-47)."""
import torch

SUPPORT_WEIGHT_QUANT_DTYPE = ['int8', 'int4', 'hifloat8']          # 'hifloat8' is additive
SUPPORT_INPUT_QUANT_DTYPE = ['int8', 'hifloat8']
SUPPORT_QUANT_STRATEGY_WEIGHT = ['tensor', 'channel', 'group']
SUPPORT_QUANT_STRATEGY_INPUT = ['tensor', 'token']

INT8, INT4 = 'int8', 'int4'
INT8_MIN, INT8_MAX = -128, 127
INT4_MIN, INT4_MAX = -8, 7

SUPPORTED_QUANT_DTYPE_COMB = ['int8 int8', 'NOT_QUANTIZE int8', 'NOT_QUANTIZE int4']

ALGORITHM_SUPPORTED_QUANT_TYPE_COMB = {
    'int8 int8': ['minmax', 'smoothquant'],
    'NOT_QUANTIZE int8': ['minmax', 'awq', 'gptq'],
    'NOT_QUANTIZE int4': ['minmax', 'awq', 'gptq'],
}

_HALF = [torch.bfloat16, torch.float16]
ALLOWED_WEIGHT_DTYPES = {
    'NOT_QUANTIZE int4': [torch.float32] + _HALF,
    'NOT_QUANTIZE int8': list(_HALF),
    'int8 int8': list(_HALF),
}
