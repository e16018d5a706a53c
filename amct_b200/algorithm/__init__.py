"""Built-in algorithms (amct_pytorch/algorithm/__init__.py:32-38)."""
from .register_algo import Algorithm
from ..quantize_op.minmax_module import MinMaxQuant
from ..quantize_op.smooth_quant_module import SmoothQuant
from ..deploy_op.npu_quantization_linear import NpuQuantizationLinear
from ..deploy_op.weight_npu_quant_module import NpuWeightQuantizedLinear
from ..quantize_op.hif8_module import HiFloat8Quant
from ..quantize_op.linear_awq_module import LinearAWQuant
from ..quantize_op.gptq_module import GPTQuant
from ..deploy_op.hif8_linear import HiFloat8Linear
from ..config.schema import BUILT_IN_ALGORITHM

__all__ = ['AlgorithmRegistry', 'BUILT_IN_ALGORITHM']

AlgorithmRegistry = Algorithm()
AlgorithmRegistry.register('gptq', 'Linear', GPTQuant, NpuWeightQuantizedLinear)
AlgorithmRegistry.register('awq', 'Linear', LinearAWQuant, NpuWeightQuantizedLinear)
AlgorithmRegistry.register('smoothquant', 'Linear', SmoothQuant, NpuQuantizationLinear)
AlgorithmRegistry.register('minmax', 'Linear', MinMaxQuant, [NpuWeightQuantizedLinear, NpuQuantizationLinear])
# additive: HiFloat8 weight + activation quantization (not a built-in of the reference; it goes through the
# custom-algorithm path of the config parser, so no dtype-combination rules apply)
AlgorithmRegistry.register('hifloat8', 'Linear', HiFloat8Quant, HiFloat8Linear)
