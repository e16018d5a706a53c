import torch

from .base_quant_module import BaseQuantizeModule
from .utils import calculate_scale_offset, weight_scale_offset
from ..backend import ops
from ..utils.data_utils import check_linear_input_dim
from ..utils.log import LOGGER


class MinMaxQuant(BaseQuantizeModule):
    """Min-max calibration of one Linear.

    Same constructor, attributes and forward contract as
    amct_pytorch/quantize_op/minmax_module.py:28-117.  Weight factors come from
    one fused pass of the row kernel; activation observers are the device
    min/max kernels with a running merge, so calibration keeps no copy of the
    inputs.  With inputs_cfg {'strategy': 'token', 'dynamic': True} (not in the
    reference schema) no activation statistics are collected: the deploy module
    quantizes each token row at run time.
    """

    def __init__(self, ori_module, layer_name, quant_config):
        super().__init__(ori_module, layer_name, quant_config)
        self.weight = ori_module.weight
        self.bias = ori_module.bias
        self.layer_name = layer_name
        self.cur_batch = 0
        self.weight_compress_only = True
        self.ori_module = ori_module
        self.dynamic_act = False

        self.batch_num = quant_config.get('batch_num')
        inputs_cfg = quant_config.get('inputs_cfg')
        if inputs_cfg.get('enable_quant') in (None, True):
            self.weight_compress_only = False
            self.act_type = inputs_cfg.get('quant_type')
            self.act_symmetric = inputs_cfg.get('symmetric')
            self.act_granularity = inputs_cfg.get('strategy')
            self.dynamic_act = bool(inputs_cfg.get('dynamic', False))
            self.data_max = None
            self.data_min = None

        weights_cfg = quant_config.get('weights_cfg')
        self.wts_type = weights_cfg.get('quant_type')
        self.wts_symmetric = weights_cfg.get('symmetric')
        self.group_size = weights_cfg.get('group_size', None)
        self.weight_granularity = weights_cfg.get('strategy')

        self.scale_w, self.offset_w = self.calculate_weights_scale_factor_and_quantize(self.weight.data, quant_config)
        if self.dynamic_act:
            # placeholder that routes convert() to the W8A8 deploy module (its rank marks per-token)
            self.scale_d = torch.ones((1, 1), dtype=torch.float32, device=self.weight.device)

    def calculate_weights_scale_factor_and_quantize(self, weight_data, quant_config):
        return weight_scale_offset(weight_data, self.wts_type, self.wts_symmetric, self.weight_granularity,
                                   self.group_size)

    @torch.no_grad()
    def forward(self, inputs):
        check_linear_input_dim(inputs)
        fp_out = self.ori_module(inputs)
        if self.weight_compress_only or self.dynamic_act:
            return fp_out

        self.cur_batch += 1
        if self.cur_batch > self.batch_num:
            return fp_out
        if self.act_granularity == 'tensor':
            if self.data_max is None:
                self.data_min, self.data_max = ops.minmax(inputs, 'tensor')
            else:
                ops.minmax(inputs, 'tensor', running=(self.data_min, self.data_max))
        elif self.act_granularity == 'token':
            # one (min, max) per index of axis -2, reduced over every other axis
            tokens, k = inputs.shape[-2], inputs.shape[-1]
            x3 = inputs.reshape(-1, tokens, k)
            shape = [1] * inputs.dim()
            shape[-2] = tokens
            for b in range(x3.shape[0]):
                if self.data_max is None:
                    mn, mx = ops.minmax_rows(x3[b])
                    self.data_min, self.data_max = mn.reshape(shape), mx.reshape(shape)
                else:
                    ops.minmax_rows(x3[b], running=(self.data_min.view(-1), self.data_max.view(-1)))

        if self.cur_batch == self.batch_num:
            self.scale_d, self.offset_d = calculate_scale_offset(self.data_max, self.data_min, self.act_symmetric,
                                                                 self.act_type)
            LOGGER.logd("Calculate minmax quant params of layer '{}' success!".format(self.layer_name), 'MinMaxQuant')
        return fp_out
