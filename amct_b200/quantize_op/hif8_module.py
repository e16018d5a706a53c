import torch
import torch.nn.functional as F

from .base_quant_module import BaseQuantizeModule
from ..backend import ops
from ..utils.data_utils import check_linear_input_dim
from ..utils.log import LOGGER


class HiFloat8Quant(BaseQuantizeModule):
    """Calibration module of the 'hifloat8' algorithm: SmoothQuant-style per-channel smoothing
    (same factor rule as amct_pytorch/quantize_op/smooth_quant_module.py:113-133) ahead of
    HiFloat8 weight + activation quantization.  HiFloat8 needs no scale: the only calibrated
    quantity is the smoothing factor ``scale`` [1, K].  Algorithm attribute
    ``smooth_strength`` (float in (0, 1)) may be omitted to disable smoothing.
    The reference has no HiFloat8 path; this module plugs in through algorithm_register().
    """

    def __init__(self, ori_module, layer_name, quant_config):
        super().__init__(ori_module, layer_name, quant_config)
        self.ori_module = ori_module
        self.weight = ori_module.weight
        self.bias = ori_module.bias
        self.layer_name = layer_name
        self.batch_num = quant_config.get('batch_num')
        attrs = (quant_config.get('algorithm') or {}).get('hifloat8') or {}
        self.smooth_strength = attrs.get('smooth_strength')
        self.act_type = self.wts_type = 'hifloat8'
        self.cur_batch = 0
        self.data_max = None
        self.data_min = None

    @torch.no_grad()
    def forward(self, inputs):
        check_linear_input_dim(inputs)
        output = F.linear(inputs, self.weight, self.bias)
        self.cur_batch += 1
        if self.smooth_strength is None or self.cur_batch > self.batch_num:
            return output
        if self.data_max is None:
            self.data_min, self.data_max = ops.minmax(inputs, 'column')
        else:
            ops.minmax(inputs, 'column', running=(self.data_min.view(-1), self.data_max.view(-1)))
        if self.cur_batch == self.batch_num:
            act_max = torch.max(self.data_max.abs(), self.data_min.abs())
            w_min, w_max = ops.minmax(self.weight.data, 'column')
            wts_max = torch.max(w_max.abs(), w_min.abs())
            s = (act_max ** self.smooth_strength) / (wts_max ** (1 - self.smooth_strength))
            bad = (s < torch.finfo(act_max.dtype).eps) | ~torch.isfinite(s)
            self.scale = torch.where(bad, torch.ones((), dtype=s.dtype, device=s.device), s)
            LOGGER.logd("Calculate hifloat8 smooth factor of layer '{}' success!".format(self.layer_name), 'HiFloat8Quant')
        return output
