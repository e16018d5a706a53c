"""Ready-made configuration dicts (values of amct_pytorch/config/config.py:19-76)."""


def _weights(quant_type):
    return {'type': quant_type, 'symmetric': True, 'strategy': 'channel'}


INT4_AWQ_WEIGHT_QUANT_CFG = {
    'batch_num': 1,
    'quant_cfg': {'weights': _weights('int4')},
    'algorithm': {'awq': {'grids_num': 20}},
    'skip_layers': {'lm_head'},
}

INT4_GPTQ_WEIGHT_QUANT_CFG = {
    'batch_num': 1,
    'quant_cfg': {'weights': _weights('int4')},
    'algorithm': {'gptq'},
    'skip_layers': {'lm_head'},
}

INT8_SMOOTHQUANT_CFG = {
    'batch_num': 1,
    'quant_cfg': {'weights': _weights('int8'),
                  'inputs': {'type': 'int8', 'symmetric': True, 'strategy': 'tensor'}},
    'algorithm': {'smoothquant': {'smooth_strength': 0.5}},
    'skip_layers': {'lm_head'},
}

INT8_MINMAX_WEIGHT_QUANT_CFG = {
    'batch_num': 1,
    'quant_cfg': {'weights': _weights('int8')},
    'algorithm': {'minmax'},
}
