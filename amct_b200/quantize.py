"""Public entry points: quantize(), convert(), algorithm_register()
(signatures and behaviour of amct_pytorch/quantize.py:28-73)."""
from torch import nn

from .algorithm import AlgorithmRegistry
from .config import set_default_config, parse_config
from .optimizer import ModelOptimizer, ReplaceNpuQuantModulePass, InsertQuantizeModulePass
from .quantize_op.base_quant_module import BaseQuantizeModule
from .utils.check_params import check_params


@check_params(model=nn.Module, config=(dict, type(None)))
def quantize(model, config=None):
    """Replace every quantizable layer of `model`, in place, by its calibration module."""
    if config is None:
        config = set_default_config()
    layer_config = parse_config(model, config, AlgorithmRegistry)
    optimizer = ModelOptimizer()
    optimizer.add_pass(InsertQuantizeModulePass(layer_config))
    optimizer.do_optimizer(model)


@check_params(model=nn.Module)
def convert(model):
    """Replace every calibration module of `model`, in place, by its deploy module."""
    optimizer = ModelOptimizer()
    optimizer.add_pass(ReplaceNpuQuantModulePass())
    optimizer.do_optimizer(model)


@check_params(name=str, src_op=str, quant_op=BaseQuantizeModule, deploy_op=(nn.Module, type(None)))
def algorithm_register(name, src_op, quant_op, deploy_op=None):
    """Register a user algorithm: name -> (source op type name, calibration module class, deploy module class)."""
    AlgorithmRegistry.register(name, src_op, quant_op, deploy_op=deploy_op)
