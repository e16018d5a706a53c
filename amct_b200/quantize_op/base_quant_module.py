import torch.nn as nn


class BaseQuantizeModule(nn.Module):
    """Base class of calibration modules; the attributes every deploy module reads
    (amct_pytorch/quantize_op/base_quant_module.py:21-35)."""

    def __init__(self, ori_module, layer_name, quant_config):
        super().__init__()
        self.act_type = None
        self.wts_type = None
        self.scale_w = None
        self.scale_d = None
        self.offset_w = None
        self.offset_d = None
        self.group_size = None
        self.scale = None
        self.clip_max = None

    def forward(self, inputs):
        pass
