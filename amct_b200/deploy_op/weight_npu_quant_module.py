import math

import torch
from torch import nn

from ..backend import ops


def check_scale_offset_shape(weight, scale_w, offset_w=None, group_size=None):
    """Shape rules of the quant factors (amct_pytorch/utils/quant_util.py:114-140)."""
    if group_size is None:
        if scale_w.shape[0] in (1, weight.shape[0]):
            return
        raise RuntimeError("scale.shape should be equal to 1 or cout. current is {}, "
                           "pls check quant factors from quantize model".format(scale_w.shape[0]))
    want = [weight.shape[0], math.ceil(weight.shape[1] / group_size), 1]
    if list(scale_w.shape) != want:
        raise RuntimeError(
            "scale.shape should be [{}] current shape is {}, please check quant factors from quantize model.".format(
                tuple(want), list(scale_w.shape)))
    if offset_w is not None and scale_w.shape != offset_w.shape:
        raise RuntimeError("offset_w.shape should be equal to scale_w.shape,"
                           " pls check quant factors from quantize model")


class NpuWeightQuantizedLinear(nn.Module):
    """Weight-only (INT8 / INT4) quantized Linear for deployment.

    Constructor argument and buffers follow
    amct_pytorch/deploy_op/weight_npu_quant_module.py:24-121:
      quantized_weight  [K, N] int8, or packed INT4 uint8 [K/2, N] (two codes per byte
                        along K, code + 8, even k in the low nibble) -- both are
                        transposed views of K-contiguous storage
      scale_w           [K/group, N] (or [1, N]) in the weight dtype
      offset_w          same shape, the NEGATED offset, or None
      bias              [N], fp32 when the weight is bf16
      scale_factor      [1, K] AWQ factor or None;  group_size (0 = per channel)
    forward() dequantizes the codes with the rounded scale_w / offset_w buffers and
    multiplies on the tensor cores with fp32 accumulation.
    """

    def __init__(self, quant_module):
        super().__init__()
        wts_type = quant_module.wts_type
        device = quant_module.weight.device
        self.group_size = quant_module.group_size
        self.wts_bits = ops.bits_of(wts_type)
        weight = quant_module.weight.data
        n, k = weight.shape

        awq = getattr(quant_module, 'scale', None)
        if awq is not None:
            awq = awq.to(device=device)
            if list(awq.shape) != [1, k]:
                raise RuntimeError("AWQ params scale.shape should be [1, {}] current shape is {}".format(
                    k, list(awq.shape)))
            self.register_buffer('scale_factor', awq)
        else:
            self.scale_factor = None

        scale_w = quant_module.scale_w.to(device)
        offset_w = quant_module.offset_w
        if offset_w is not None:
            offset_w = offset_w.to(device)
        check_scale_offset_shape(weight, scale_w, offset_w, self.group_size)
        if self.group_size is not None and k % self.group_size != 0:
            raise RuntimeError("cin {} should be an integer multiple of group_size {}".format(k, self.group_size))

        if self.group_size is not None:
            strategy = 'group'
            scale_nk = scale_w.reshape(n, -1)
            offset_nk = None if offset_w is None else offset_w.reshape(n, -1)
        else:
            strategy = 'channel' if scale_w.numel() == n else 'tensor'
            scale_nk = scale_w.reshape(-1, 1)
            offset_nk = None if offset_w is None else offset_w.reshape(-1, 1)
        out = 'pack4' if wts_type == 'int4' else 'i8'
        _, _, codes = ops.quant_rows(weight, wts_type, offset_w is None, strategy, self.group_size,
                                     scale=scale_nk, offset=offset_nk, out=out,
                                     pre=awq, pre_op='div' if awq is not None else 'none')
        self.register_buffer('quantized_weight', codes.t())

        if self.group_size is None:
            # per-tensor factors are repeated to one per output channel (the op is per-channel)
            if scale_nk.shape[0] == 1:
                scale_nk = scale_nk.repeat(n, 1)
                offset_nk = None if offset_nk is None else offset_nk.repeat(n, 1)
            self.group_size = 0
        self.register_buffer('scale_w', scale_nk.to(weight.dtype).t().contiguous())
        if offset_nk is not None:
            self.register_buffer('offset_w', (offset_nk * -1).to(self.scale_w.dtype).t().contiguous())
        else:
            self.offset_w = None

        if quant_module.bias is not None:
            bias = quant_module.bias.to(device=device)
            if weight.dtype == torch.bfloat16:
                bias = bias.to(torch.float32)
            self.register_buffer('bias', bias)
        else:
            self.bias = None

    @torch.no_grad()
    def forward(self, inputs):
        from ..torch_npu_shim import npu_weight_quant_batchmatmul
        ori_shape = inputs.shape
        inputs = inputs.to(self.quantized_weight.device).reshape(-1, inputs.shape[-1])
        if self.scale_factor is not None:
            inputs = torch.mul(inputs, self.scale_factor)
        output = npu_weight_quant_batchmatmul(inputs, self.quantized_weight, self.scale_w,
                                              antiquant_offset=self.offset_w, bias=self.bias,
                                              antiquant_group_size=self.group_size)
        return output.reshape(*ori_shape[:-1], -1)
