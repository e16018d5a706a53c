"""Module-replacement passes behind quantize() and convert()
(amct_pytorch/optimizer/*.py)."""
from ..utils.log import LOGGER
from ..utils.model_util import ModuleHelper
from ..config.schema import get_alg_name_from_config


class BaseModuleFusionPass:
    """A pass matches modules by (module, name) and rewrites each match."""

    def match_pattern(self, module, name):
        return False

    def do_pass(self, model, object_module, object_name):
        pass

    def run(self, model):
        helper = ModuleHelper(model)
        matched = {n: m for n, m in helper.named_module_dict.items() if self.match_pattern(m, n)}
        for name, module in matched.items():
            self.do_pass(model, module, name)


class InsertQuantizeModulePass(BaseModuleFusionPass):
    """Wraps every configured layer in its algorithm's calibration module
    (amct_pytorch/optimizer/insert_quantize_op_pass.py:26-77)."""

    def __init__(self, quant_config):
        self.config = quant_config
        self.quant_layers = list(quant_config.keys())
        self.quantize_op = None

    def match_pattern(self, module, name):
        from ..algorithm import AlgorithmRegistry
        if name not in self.quant_layers:
            return False
        alg_name, _ = get_alg_name_from_config(self.config[name].get('algorithm'))
        entry = AlgorithmRegistry.algo.get(alg_name)
        return bool(entry) and type(module).__name__ == entry[0]

    def do_pass(self, model, object_module, object_name):
        from ..algorithm import AlgorithmRegistry
        layer_config = self.config.get(object_name)
        alg_name, _ = get_alg_name_from_config(layer_config.get('algorithm'))
        quant_op = AlgorithmRegistry.algo.get(alg_name)[1]
        ModuleHelper.replace_module_by_name(model, object_name, quant_op(object_module, object_name, layer_config))
        LOGGER.logd("Insert quantize op module to '{}' success!".format(object_name), 'InsertQuantizeModulePass')


class ReplaceNpuQuantModulePass(BaseModuleFusionPass):
    """Swaps every calibration module for its deploy module
    (amct_pytorch/optimizer/replace_npu_quant_pass.py:27-75)."""

    def match_pattern(self, module, name):
        from ..algorithm import AlgorithmRegistry
        return isinstance(module, tuple(AlgorithmRegistry.quant_op))

    def do_pass(self, model, object_module, object_name):
        from ..algorithm import AlgorithmRegistry
        from ..quantize_op import MinMaxQuant
        from ..deploy_op import NpuQuantizationLinear, NpuWeightQuantizedLinear
        deploy = AlgorithmRegistry.quant_to_deploy[type(object_module)]
        if not deploy:
            raise RuntimeError(f"The deploy_op for {type(object_module).__name__} is None! "
                               "pls invoke algorithm_register to register deploy_op!")
        if isinstance(object_module, MinMaxQuant):
            deploy = NpuQuantizationLinear if object_module.scale_d is not None else NpuWeightQuantizedLinear
        ModuleHelper.replace_module_by_name(model, object_name, deploy(object_module))
        LOGGER.logd("Replace npu module to '{}' success!".format(object_name), 'ReplaceNpuQuantPass')


class ModelOptimizer:
    """Runs passes in the order they were added (amct_pytorch/optimizer/model_optimizer.py:21-58)."""

    def __init__(self):
        self._passes = []

    def add_pass(self, model_pass):
        self._passes.append(model_pass)

    def clear_pass(self):
        self._passes.clear()

    def do_optimizer(self, model):
        for model_pass in self._passes:
            LOGGER.logi('Do {}'.format(type(model_pass)), 'Optimizer')
            model_pass.run(model)
