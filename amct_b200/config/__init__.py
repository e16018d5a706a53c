from .presets import (INT4_AWQ_WEIGHT_QUANT_CFG, INT4_GPTQ_WEIGHT_QUANT_CFG, INT8_SMOOTHQUANT_CFG,
                      INT8_MINMAX_WEIGHT_QUANT_CFG)
from .schema import parse_config, set_default_config, get_alg_name_from_config, QuantConfig

__all__ = ['INT4_AWQ_WEIGHT_QUANT_CFG', 'INT4_GPTQ_WEIGHT_QUANT_CFG', 'INT8_SMOOTHQUANT_CFG',
           'INT8_MINMAX_WEIGHT_QUANT_CFG', 'parse_config', 'set_default_config', 'get_alg_name_from_config',
           'QuantConfig']
