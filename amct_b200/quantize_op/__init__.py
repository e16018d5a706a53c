from .base_quant_module import BaseQuantizeModule
from .minmax_module import MinMaxQuant
from .smooth_quant_module import SmoothQuant
from .linear_awq_module import LinearAWQuant
from .gptq_module import GPTQuant

__all__ = ['BaseQuantizeModule', 'MinMaxQuant', 'SmoothQuant', 'LinearAWQuant', 'GPTQuant']
