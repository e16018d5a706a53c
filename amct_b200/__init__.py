"""amct_b200: the quantization hot path of AMCT on NVIDIA B200 (sm_100a).

Same public surface as ``amct_pytorch`` (amct_pytorch/__init__.py:18-25):
``quantize``, ``convert``, ``algorithm_register`` and the preset configs.  The
arithmetic runs in hand-written CUDA kernels behind a C ABI
(include/amct_b200.h); tensors must live on a CUDA device.
"""
from .quantize import quantize, convert, algorithm_register
from .config import (INT4_AWQ_WEIGHT_QUANT_CFG, INT4_GPTQ_WEIGHT_QUANT_CFG, INT8_SMOOTHQUANT_CFG,
                     INT8_MINMAX_WEIGHT_QUANT_CFG)

__all__ = ['quantize', 'convert', 'algorithm_register', 'INT4_AWQ_WEIGHT_QUANT_CFG', 'INT4_GPTQ_WEIGHT_QUANT_CFG',
           'INT8_SMOOTHQUANT_CFG', 'INT8_MINMAX_WEIGHT_QUANT_CFG']
