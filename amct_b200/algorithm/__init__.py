"""Built-in algorithms (amct_pytorch/algorithm/__init__.py:32-38)."""
from .register_algo import Algorithm
from ..quantize_op.minmax_module import MinMaxQuant
from ..quantize_op.smooth_quant_module import SmoothQuant
from ..deploy_op.npu_quantization_linear import NpuQuantizationLinear
from ..deploy_op.weight_npu_quant_module import NpuWeightQuantizedLinear
from ..config.schema import BUILT_IN_ALGORITHM

__all__ = ['AlgorithmRegistry', 'BUILT_IN_ALGORITHM']

AlgorithmRegistry = Algorithm()
AlgorithmRegistry.register('smoothquant', 'Linear', SmoothQuant, NpuQuantizationLinear)
AlgorithmRegistry.register('minmax', 'Linear', MinMaxQuant, [NpuWeightQuantizedLinear, NpuQuantizationLinear])
