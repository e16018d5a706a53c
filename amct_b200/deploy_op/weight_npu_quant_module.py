import math

import torch
from torch import nn

from ..backend import ops
from ..utils import int4pack


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
      quantized_weight  INT8: [K, N] int8 (a transposed view of K-contiguous storage).
                        INT4: int32 [K, N / 8], the int4pack form the reference stores (the result of
                        torch_npu.npu_convert_weight_to_int4pack on the [K, N] codes; int32 [K, N] unpacked when N is
                        not a multiple of 8), so state dicts go both ways; what the kernels read is the additional,
                        non-persistent buffer ``weight_payload`` uint8 [N, K / 2] (two codes per byte along K, code
                        + 8, even k in the low nibble), rebuilt from quantized_weight whenever a state dict is loaded
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
        _, _, codes = ops.quant_rows(weight, wts_type, offset_w is None, strategy, self.group_size,
                                     scale=scale_nk, offset=offset_nk, out='i8',
                                     pre=awq, pre_op='div' if awq is not None else 'none')
        if self.wts_bits == 4:
            codes_kn = codes.t()
            self.register_buffer('quantized_weight',
                                 int4pack.to_int4pack(codes_kn) if n % 8 == 0 else codes_kn.to(torch.int32).contiguous())
            self.register_buffer('weight_payload', int4pack.to_payload(codes), persistent=False)
        else:
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

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """Accepts every form of ``quantized_weight`` a checkpoint can hold (see int4pack.codes_from_buffer) and derives
        what the kernels read from it once, here, not on the forward path."""
        key = prefix + 'quantized_weight'
        n = self.scale_w.shape[-1]
        if self.wts_bits == 4 and key in state_dict:
            codes_kn = int4pack.codes_from_buffer(state_dict[key], n)
            state_dict = dict(state_dict)
            state_dict[key] = int4pack.to_int4pack(codes_kn) if n % 8 == 0 else codes_kn.to(torch.int32).contiguous()
            if tuple(self.quantized_weight.shape) != tuple(state_dict[key].shape):
                self.quantized_weight = torch.empty_like(state_dict[key], device=self.quantized_weight.device)
            self.weight_payload = int4pack.to_payload(codes_kn.t().contiguous()).to(self.quantized_weight.device)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        if self.wts_bits == 8 and self.quantized_weight.stride(0) != 1:
            # a checkpoint stores [K, N] row-major; the MMA wants K contiguous: transpose once, keep the shape
            self.quantized_weight = self.quantized_weight.t().contiguous().t()

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        if self.wts_bits == 8 and self.quantized_weight.stride(0) != 1:
            self.quantized_weight = self.quantized_weight.t().contiguous().t()     # .to() / .cuda() copies lose the view's strides
        return out

    @torch.no_grad()
    def forward(self, inputs):
        from ..torch_npu_shim import weight_quant_matmul
        ori_shape = inputs.shape
        inputs = inputs.to(self.quantized_weight.device).reshape(-1, inputs.shape[-1])
        if self.scale_factor is not None:
            inputs = torch.mul(inputs, self.scale_factor)
        codes_nk = self.weight_payload if self.wts_bits == 4 else self.quantized_weight.t()
        output = weight_quant_matmul(inputs, codes_nk, self.wts_bits, self.scale_w, self.offset_w, self.bias, self.group_size)
        return output.reshape(*ori_shape[:-1], -1)
