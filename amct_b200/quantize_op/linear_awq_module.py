import copy

import torch
import torch.nn.functional as F

from .base_quant_module import BaseQuantizeModule
from .utils import weight_scale_offset
from ..algorithm.awq import search_scale
from ..utils.data_utils import check_linear_input_dim
from ..utils.log import LOGGER


class LinearAWQuant(BaseQuantizeModule):
    """AWQ calibration of one Linear (contract of
    amct_pytorch/quantize_op/linear_awq_module.py:30-81): the first forward searches the
    per-input-channel scale, folds it into the wrapped Linear's weight, and derives the weight
    quantization factors; ``scale`` holds 1 / awq_scale for the deploy module."""

    def __init__(self, ori_module, layer_name, quant_config):
        super().__init__(ori_module, layer_name, quant_config)
        self.weight = copy.deepcopy(ori_module.weight)
        self.bias = ori_module.bias
        self.layer_name = layer_name
        self.quant_config = quant_config
        cfg = quant_config.get('weights_cfg')
        self.wts_symmetric = cfg.get('symmetric')
        self.wts_type = cfg.get('quant_type')
        self.ori_module = ori_module
        if cfg.get('group_size') is not None:
            self.group_size = cfg.get('group_size')
        self.calc_done = False

    @torch.no_grad()
    def forward(self, inputs):
        data = inputs.clone()
        check_linear_input_dim(data)
        data = data.to(self.weight.device)
        output = F.linear(data, self.weight, self.bias)
        if self.calc_done:
            return output
        scale_awq = search_scale(data, self.ori_module, self.quant_config)
        self.ori_module.weight.data.mul_(scale_awq.to(self.ori_module.weight.device))
        self.scale = 1 / scale_awq.detach()
        cfg = self.quant_config.get('weights_cfg')
        self.scale_w, self.offset_w = weight_scale_offset(self.ori_module.weight.data, self.wts_type, self.wts_symmetric,
                                                          cfg.get('strategy'), cfg.get('group_size'))
        self.calc_done = True
        LOGGER.logd("Calculate awq quant params of layer '{}' success!".format(self.layer_name), 'LinearAWQuant')
        return output
