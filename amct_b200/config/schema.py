"""Validation of the user configuration dict and its expansion to one detail
dict per quantizable layer.

Schema, rules and error texts follow amct_pytorch/config/fields.py:23-258 and
amct_pytorch/config/parser.py:26-146; the detail dict
{'batch_num', 'weights_cfg', 'inputs_cfg', 'algorithm'} is what every quant_op
constructor receives (parser.py:137-138).
"""
import torch

from ..utils.log import LOGGER
from ..utils import vars as V
from .presets import INT8_MINMAX_WEIGHT_QUANT_CFG

BUILT_IN_ALGORITHM = ['minmax', 'awq', 'gptq', 'smoothquant']


def get_alg_name_from_config(alg):
    """'minmax' | {'minmax'} | {'awq': {...}} -> (name, attrs)  (config/utils.py:18-25)."""
    if isinstance(alg, dict):
        name = next(iter(alg))
        return name, alg[name]
    if isinstance(alg, set):
        return next(iter(alg)), None
    if isinstance(alg, str):
        return alg, None
    raise ValueError('invalid algo name, pls check config')


class _Field:
    """A validated slice of the configuration; ``get_value()`` is its normalised dict."""
    value = None

    def get_value(self):
        return self.value


class BatchNumField(_Field):
    def __init__(self, batch_num):
        if not isinstance(batch_num, int) or batch_num <= 0:
            raise ValueError(f'Batch num only support positive int, but got {batch_num}')
        self.batch_num = batch_num
        self.value = {'batch_num': batch_num}


class WeightsCfgField(_Field):
    def __init__(self, config):
        self.quant_type = config.get('type')
        self.symmetric = config.get('symmetric')
        self.strategy = config.get('strategy')
        self.group_size = config.get('group_size', None)
        self._check()
        self.value = {'quant_type': self.quant_type, 'symmetric': self.symmetric, 'strategy': self.strategy}
        if self.group_size is not None:
            self.value['group_size'] = self.group_size

    def _check(self):
        if self.quant_type not in V.SUPPORT_WEIGHT_QUANT_DTYPE:
            raise ValueError(f'Weights quant_dtype only support {V.SUPPORT_WEIGHT_QUANT_DTYPE}, '
                             f'but got {self.quant_type}')
        if self.symmetric not in [True, False]:
            raise ValueError(f'Weights symmetric only support bool [True, False], but got {self.symmetric}')
        if self.strategy not in V.SUPPORT_QUANT_STRATEGY_WEIGHT:
            raise ValueError(f'Weights strategy only support{V.SUPPORT_QUANT_STRATEGY_WEIGHT}, but got {self.strategy}')
        grouped = self.strategy == 'group'
        if self.group_size is not None and not grouped:
            raise ValueError(f'Weights group_size only support strategy group, but got {self.strategy}')
        if self.group_size is None and grouped:
            raise ValueError('Weights group_size is necessary, when weights strategy is group')
        if self.group_size is not None and (not isinstance(self.group_size, int) or self.group_size <= 0):
            raise ValueError(f'group_size only support positive int, but got {self.group_size}')


class InputsCfgField(_Field):
    def __init__(self, config):
        self.quant_input = config.get('enable_quant', True)
        if not self.quant_input:
            self.value = {'enable_quant': False}
            return
        self.quant_type = config.get('type')
        self.symmetric = config.get('symmetric')
        self.strategy = config.get('strategy')
        if self.quant_type not in V.SUPPORT_INPUT_QUANT_DTYPE:
            raise ValueError(f'Inputs quant_dtype only support {V.SUPPORT_INPUT_QUANT_DTYPE}, but got {self.quant_type}')
        if self.symmetric not in [True, False]:
            raise ValueError(f'Inputs symmetric only support bool [True, False], but got {self.symmetric}')
        if self.strategy not in V.SUPPORT_QUANT_STRATEGY_INPUT:
            raise ValueError(f'Inputs strategy only support{V.SUPPORT_QUANT_STRATEGY_INPUT}, but got {self.strategy}')
        if self.strategy == 'token' and self.symmetric is False:
            raise ValueError('Inputs strategy token do not support asymmetric quantization')
        self.value = {'quant_type': self.quant_type, 'symmetric': self.symmetric, 'strategy': self.strategy}
        # additive key (not in the reference schema): per-token scales computed at run time
        if config.get('dynamic', False):
            if self.strategy != 'token':
                raise ValueError('Inputs dynamic quantization only support strategy token')
            self.value['dynamic'] = True


class QuantCfgField(_Field):
    def __init__(self, config):
        self.weights_cfg = WeightsCfgField(config.get('weights', {}))
        self.inputs_cfg = InputsCfgField(config.get('inputs', {'enable_quant': False}))
        self.value = {'weights_cfg': self.weights_cfg.get_value(), 'inputs_cfg': self.inputs_cfg.get_value()}


def _awq_value(attrs):
    if attrs is None or attrs.get('grids_num') is None:
        raise ValueError('Awq grids_num is necessary param, pls check and set')
    grids = attrs.get('grids_num')
    if not isinstance(grids, int) or grids <= 0:
        raise ValueError(f'Awq grids_num only support positive int, but got {grids}')
    return {'awq': {'grids_num': grids}}


def _smoothquant_value(attrs):
    if attrs is None or attrs.get('smooth_strength') is None:
        raise ValueError('Smoothquant smooth_strength is necessary param, pls check and set')
    strength = attrs.get('smooth_strength')
    if not isinstance(strength, float) or strength <= 0 or strength >= 1:
        raise ValueError(f'Smoothquant smooth_strength only support float (0, 1), but got {strength}')
    return {'smoothquant': {'smooth_strength': strength}}


_ALG_VALUE = {
    'awq': _awq_value,
    'smoothquant': _smoothquant_value,
    'gptq': lambda attrs: {'gptq'},
    'minmax': lambda attrs: {'minmax'},
}


class AlgorithmField(_Field):
    def __init__(self, alg_cfg, registry):
        if not isinstance(alg_cfg, str) and len(alg_cfg) != 1:
            raise ValueError(f'Algorithm only support 1 str, but got {alg_cfg}')
        name, attrs = get_alg_name_from_config(alg_cfg)
        if registry.algo.get(name) is None:
            raise ValueError(f'Not support algorithm {name}, pls regiter it first')
        self.name = name
        build = _ALG_VALUE.get(name)
        self.value = {'algorithm': build(attrs) if build else {name: attrs}}


class SkipLayersField(_Field):
    def __init__(self, layers):
        for layer in layers:
            if not isinstance(layer, str):
                raise ValueError('Skip layers must be str')
        self.skip_layers = layers
        self.value = {'skip_layers': layers}


class QuantConfig:
    def __init__(self, config, registry):
        self.batch_num = BatchNumField(config.get('batch_num', 1))
        self.quant_cfg = QuantCfgField(config.get('quant_cfg', {}))
        self.algorithm = AlgorithmField(config.get('algorithm', {}), registry)
        self.skip_layers = SkipLayersField(config.get('skip_layers', []))


# ---------------------------------------------------------------------------
def set_default_config():
    LOGGER.logd('Using INT8_MINMAX_WEIGHT_QUANT_CFG as default config')
    return INT8_MINMAX_WEIGHT_QUANT_CFG


def check_skip_layer(layer_name, skip_layers):
    """Substring match against every entry (config/parser.py:32-49)."""
    hit = bool(skip_layers) and any(s in layer_name for s in skip_layers)
    if hit:
        LOGGER.logd('The {} quantifiable module is skipped'.format(layer_name))
    return hit


def check_config(comb, quant_config, algo):
    """Global combination rules (config/parser.py:52-74)."""
    if comb not in V.SUPPORTED_QUANT_DTYPE_COMB:
        raise ValueError(f'Do not support combination {comb} of act and weight quant dtype.')
    if algo not in V.ALGORITHM_SUPPORTED_QUANT_TYPE_COMB[comb]:
        raise ValueError(f'Algorithm {algo} do not support act and weight quant dtype {comb}')
    weights = quant_config.quant_cfg.weights_cfg
    if comb == 'int8 int8' and weights.strategy == 'group':
        raise ValueError(f'act_dtype and wts dtype {comb} do not support weight quant strategy group')
    gs = weights.group_size
    if gs is not None and (gs < 32 or gs % 32 != 0):
        raise ValueError(f'act_type and wts_type {comb} only support group_size larger than 32 and '
                         f'integer multiple of 32, current is {gs}')


def check_quant_op_constraint(mod, layer_name, comb, quant_config):
    """Per-layer shape rules of the weight-only deploy op (config/parser.py:77-102)."""
    if comb not in ('NOT_QUANTIZE int4', 'NOT_QUANTIZE int8'):
        return True
    cout, cin = mod.weight.shape[0], mod.weight.shape[1]
    if comb == 'NOT_QUANTIZE int4' and (cout % 8 != 0 or cin % 8 != 0):
        LOGGER.logd('layer:{} cannot be quantized, act_dtype and wts dtype {} has shape requirement'
                    ' cin and cout length should be integer multiple of 8'.format(layer_name, comb))
        return False
    gs = quant_config.quant_cfg.weights_cfg.group_size
    if gs is not None and gs >= cin:
        LOGGER.logd(f'group size should less than cout, current group_size is {gs}, '
                    f'cout is {cin}, skip quantization of current layer {layer_name}')
        return False
    return True


# fp32 Linears may take the W8A8 path here (additive to the reference's allow-list,
# amct_pytorch/utils/vars.py:43-47, which silently leaves them unquantized).
EXTRA_ALLOWED_WEIGHT_DTYPES = {'int8 int8': [torch.float32], 'NOT_QUANTIZE int8': [torch.float32]}


def get_supported_layers(model, quant_config, registry, extra_dtypes=False):
    algo = quant_config.algorithm.name
    src_op = registry.algo.get(algo)[0]
    built_in = algo in BUILT_IN_ALGORITHM
    comb = None
    if built_in:
        inputs = quant_config.quant_cfg.inputs_cfg
        act = inputs.quant_type if inputs.quant_input else 'NOT_QUANTIZE'
        comb = act + ' ' + quant_config.quant_cfg.weights_cfg.quant_type
        check_config(comb, quant_config, algo)
        allowed = list(V.ALLOWED_WEIGHT_DTYPES.get(comb))
        if extra_dtypes:
            allowed += EXTRA_ALLOWED_WEIGHT_DTYPES.get(comb, [])
    else:
        LOGGER.logd("Customized Algorithm {} is used fot quant".format(algo))

    detail = {}
    for name, mod in model.named_modules():
        if type(mod) is not src_op and type(mod).__name__ != src_op:
            continue
        if check_skip_layer(name, quant_config.skip_layers.skip_layers):
            LOGGER.logd('layer:{} is skipped'.format(name))
            continue
        if built_in:
            if mod.weight.dtype not in allowed:
                LOGGER.logd('layer:{} cannot be quantized, act_dtype and wts dtype {} only support ori dtype {} '
                            'but got {}'.format(name, comb, allowed, mod.weight.dtype))
                continue
            if not check_quant_op_constraint(mod, name, comb, quant_config):
                continue
        detail[name] = {**quant_config.batch_num.get_value(), **quant_config.quant_cfg.get_value(),
                        **quant_config.algorithm.get_value()}
    return detail


def parse_config(model, config, registry):
    """User dict -> {layer name: detail dict} (config/parser.py:142-146).
    The key 'allow_fp32' (not in the reference schema) opts fp32 Linears into W8A8."""
    quant_config = QuantConfig(config, registry)
    return get_supported_layers(model, quant_config, registry, extra_dtypes=bool(config.get('allow_fp32', False)))
