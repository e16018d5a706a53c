from .npu_quantization_linear import NpuQuantizationLinear
from .weight_npu_quant_module import NpuWeightQuantizedLinear

__all__ = ['NpuQuantizationLinear', 'NpuWeightQuantizedLinear']
