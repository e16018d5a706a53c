from ..utils.log import LOGGER


class Algorithm:
    """Plugin registry: algorithm name -> (source op name, quant module class), and
    quant module class -> deploy module class(es)
    (amct_pytorch/algorithm/register_algo.py:22-35)."""

    def __init__(self):
        self.algo = {}
        self.quant_to_deploy = {}
        self.quant_op = []

    def register(self, name, src_op, quant_op, deploy_op):
        if self.algo.get(name) is not None:
            raise ValueError(f'{name} is already registered')
        self.algo[name] = (src_op, quant_op)
        self.quant_op.append(quant_op)
        self.quant_to_deploy[quant_op] = deploy_op
        LOGGER.logd(f'register algorithm {name} success.')
