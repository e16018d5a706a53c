import torch
import torch.nn.functional as F

from .base_quant_module import BaseQuantizeModule
from .utils import calculate_scale_offset, weight_scale_offset
from ..backend import ops
from ..utils.data_utils import check_linear_input_dim
from ..utils.log import LOGGER


class SmoothQuant(BaseQuantizeModule):
    """SmoothQuant calibration of one Linear
    (contract of amct_pytorch/quantize_op/smooth_quant_module.py:26-178).

    Per-channel activation extrema are a running device reduction; the per-token
    variant keeps the calibration batches in HBM (the reference moves them to
    host memory) and takes the per-token statistics of x / smooth with the
    division folded into the row reduction.
    """

    def __init__(self, ori_module, layer_name, quant_config):
        super().__init__(ori_module, layer_name, quant_config)
        self.weight = ori_module.weight
        self.bias = ori_module.bias
        self.layer_name = layer_name
        self.quant_config = quant_config
        self.group_size = quant_config.get('group_size')
        self.batch_num = quant_config.get('batch_num')
        inputs_cfg, weights_cfg = quant_config.get('inputs_cfg'), quant_config.get('weights_cfg')
        self.act_granularity = inputs_cfg.get('strategy')
        self.wts_granularity = weights_cfg.get('strategy')
        self.act_symmetric = inputs_cfg.get('symmetric')
        self.wts_symmetric = weights_cfg.get('symmetric')
        self.act_type = inputs_cfg.get('quant_type')
        self.wts_type = weights_cfg.get('quant_type')
        self.cur_batch = 0
        self.device = ori_module.weight.device
        self.data_max = None
        self.data_min = None
        self.batch_input = []

    @torch.no_grad()
    def forward(self, inputs):
        check_linear_input_dim(inputs)
        inputs = inputs.to(self.weight.device)
        output = F.linear(inputs, self.weight, self.bias)

        self.cur_batch += 1
        if self.cur_batch > self.batch_num:
            return output
        if self.data_max is None:
            self.data_min, self.data_max = ops.minmax(inputs, 'column')
        else:
            ops.minmax(inputs, 'column', running=(self.data_min.view(-1), self.data_max.view(-1)))
        if self.act_granularity == 'token':
            self.batch_input.append(inputs.detach())

        if self.cur_batch == self.batch_num:
            act_max = torch.max(self.data_max.abs(), self.data_min.abs())
            smooth_factor = self.calculate_smooth(act_max)
            self.scale_w, self.offset_w = weight_scale_offset(self.weight.data, self.wts_type, self.wts_symmetric,
                                                              self.wts_granularity, pre=smooth_factor, pre_op='mul')
            if self.act_granularity == 'tensor':
                self.scale_d, self.offset_d = self._calculate_per_tensor_params(smooth_factor)
            else:
                self.scale_d, self.offset_d = self._calculate_per_token_params(smooth_factor)
            self.scale = smooth_factor
            self.batch_input = []
            LOGGER.logd("Calculate smooth quant params of layer '{}' success!".format(self.layer_name), 'SmoothQuant')
        return output

    def calculate_smooth(self, act_max):
        """act^a / w^(1-a) per input channel, in the weight dtype; non-finite or
        below-eps entries become 1 (smooth_quant_module.py:113-133)."""
        w_min, w_max = ops.minmax(self.weight.data, 'column')
        wts_max = torch.max(w_max.abs(), w_min.abs())
        strength = self.quant_config.get('algorithm').get('smoothquant').get('smooth_strength')
        smooth = (act_max ** strength) / (wts_max ** (1 - strength))
        bad = (smooth < torch.finfo(act_max.dtype).eps) | ~torch.isfinite(smooth)
        if bad.any().item():
            smooth = torch.where(bad, torch.ones((), dtype=smooth.dtype, device=smooth.device), smooth)
            LOGGER.logd("The smooth factor is calculated as abnormal and set to 1")
        return smooth

    def _calculate_per_token_params(self, smooth_factor):
        first = self.batch_input[0]
        tokens, k = first.shape[-2], first.shape[-1]
        shape = [1] * first.dim()
        shape[-2] = tokens
        running = None
        for batch in self.batch_input:
            x3 = batch.reshape(-1, tokens, k)
            for b in range(x3.shape[0]):
                if running is None:
                    running = ops.minmax_rows(x3[b], pre=smooth_factor, pre_op='div')
                else:
                    ops.minmax_rows(x3[b], pre=smooth_factor, pre_op='div', running=running)
        return calculate_scale_offset(running[1].reshape(shape), running[0].reshape(shape), self.act_symmetric,
                                      self.act_type)

    def _calculate_per_tensor_params(self, smooth_factor):
        max_val = (self.data_max / smooth_factor).max().reshape(-1)
        min_val = (self.data_min / smooth_factor).min().reshape(-1)
        return calculate_scale_offset(max_val, min_val, self.act_symmetric, self.act_type)
