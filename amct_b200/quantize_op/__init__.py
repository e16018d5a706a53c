from .base_quant_module import BaseQuantizeModule
from .minmax_module import MinMaxQuant
from .smooth_quant_module import SmoothQuant

__all__ = ['BaseQuantizeModule', 'MinMaxQuant', 'SmoothQuant']
