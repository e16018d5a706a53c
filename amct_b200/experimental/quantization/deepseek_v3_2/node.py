"""Activation quantizer of the reference's DeepSeek-V3.2 tree on the CUDA kernel.

Drop-in for ``ActivationQuantizer`` of amct_pytorch/experimental/quantization/DeepSeekV3.2/cores/quantization/node.py
("node.py" below): dynamic per-token fake quantization -- symmetric without learned clipping, symmetric or
asymmetric with it, as its attention module builds them (cores/models/deepseek_v3_2/quant_dsa.py:46-49, :113-124),
or with a ``clip_ratio`` -- and per-tensor quantization with the scale taken from observed bounds or loaded
(``deploy`` / ``load_deploy``).  Same constructor arguments, parameter and buffer names (``clip_factor_a_max``,
``clip_factor_a_min``, ``maxval``, ``minval``, ``scale``, ``zero``), observe mode and bits=16 pass-through.  The
quantization itself is ``amct_dsa_rotate_fakequant`` (``amct_b200/csrc/kv_quant.cu``); it is an inference-time path:
the kernel has no backward, so the learned clip factors are read, not trained, here.  What stays on the host is the
per-tensor scale and zero point: a handful of operations on one-element tensors, written with torch so that their
dtypes -- which decide, by promotion, whether the kernel rounds every step to the activation dtype or works in
fp32 -- come out as in the reference.
"""
import torch

from ....backend import ops as _ops


def get_qmin_qmax(bits, sym):
    """(q_max, q_min) as node.py:30-36."""
    if sym:
        q_max = torch.tensor(2 ** (bits - 1) - 1)
        return q_max, -q_max - 1
    return torch.tensor(2 ** bits - 1), 0


class ActivationQuantizer(torch.nn.Module):
    """Per-token (last axis) dynamic activation fake quantizer (node.py:85-215)."""

    def __init__(self, bits, sym=False, lac=False, groupsize=-1, clip_ratio=None, per_tensor=False, head_num=-1):
        super().__init__()
        if groupsize > 0:
            raise NotImplementedError('Not support per-group quantization for activation yet.')       # node.py:98-99
        self.bits, self.sym, self.lac, self.groupsize = bits, sym, lac, groupsize
        self.q_max, self.q_min = get_qmin_qmax(bits, sym)
        self._clip_ratio = clip_ratio
        if lac:
            self.sigmoid = torch.nn.Sigmoid()
            self.clip_factor_a_max = torch.nn.Parameter(torch.ones((1,)) * 4.0, requires_grad=True)
            self.clip_factor_a_min = torch.nn.Parameter(torch.ones((1,)) * 4.0, requires_grad=True)
        self.enable = True
        self.register_buffer('maxval', torch.zeros(1))
        self.register_buffer('minval', torch.zeros(1))
        self.register_buffer('scale', torch.ones(1))
        self.register_buffer('zero', torch.zeros(1))
        self.is_observe = False
        self.is_deploy = False
        self.is_per_tensor = per_tensor
        self.cnt = 0
        self._deployed = None           # (key, kernel arguments) read from the deployed scale / zero

    def forward(self, x):
        if self.bits == 16:
            return x
        if self.is_observe:                                                    # node.py:121-128
            hi, lo = x.max(), x.min()
            if hi > self.maxval.to(x.device):
                self.maxval.data = hi
            if lo < self.minval.to(x.device):
                self.minval.data = lo
            return x
        return self.fake_quant(x)

    def _bounds_device(self):
        """The device the per-tensor arithmetic runs on: where the observed bounds live.  Observe mode replaces a
        bound by a 0-dim tensor on the activation's device, so a module that was built on the host and fed device
        activations holds bounds (and clip parameters) on different devices; a bound that was never exceeded is
        still the constructor's host tensor."""
        for t in (self.maxval, self.minval):
            if t.device.type != 'cpu':
                return t.device
        return self.maxval.device

    def get_scale_zero_pertensor(self):
        """(scale, zero) from the observed bounds (node.py:161-179), every operand moved to one device first (the
        dynamic rule does the same with its clip parameters, node.py:192-196); dtypes, and with them torch's
        promotion, are left as they are."""
        dev = self._bounds_device()
        q_max = self.q_max.to(dev)
        hi, lo = self.maxval.to(dev).clone(), self.minval.to(dev).clone()
        if self.lac:
            hi = hi * self.sigmoid(self.clip_factor_a_max.to(dev))
            lo = lo * self.sigmoid(self.clip_factor_a_min.to(dev))
        elif self._clip_ratio is not None:
            hi, lo = hi * self._clip_ratio, lo * self._clip_ratio
        if self.sym:
            scale = torch.maximum(lo.abs(), hi) / q_max
            return scale, torch.zeros_like(scale)
        scale = (hi - lo) / q_max
        return scale, torch.round(-lo / scale)

    def deploy(self):
        scale, zero = self.get_scale_zero_pertensor()
        self.scale.data, self.zero.data = scale, zero
        self._deployed = None

    def load_deploy(self, scale, zero):
        self.scale.data, self.zero.data = scale, zero
        self.is_deploy = True
        self._deployed = None

    def _sigmoids(self):
        if not self.lac:
            return None, None
        if self.clip_factor_a_max.dtype != torch.float32:
            raise NotImplementedError('the kernel follows torch promotion for fp32 clip parameters only')
        with torch.no_grad():
            return (float(torch.sigmoid(self.clip_factor_a_max.float())),
                    float(torch.sigmoid(self.clip_factor_a_min.float())))

    @staticmethod
    def promoted_dtype(x_dtype, scale):
        """dtype of ``x / scale`` for an activation of ``x_dtype`` (one or more dimensions) under torch's promotion
        rules, evaluated without touching a device."""
        probe = torch.empty(1, dtype=x_dtype, device='meta')
        return torch.result_type(probe, torch.empty(scale.shape, dtype=scale.dtype, device='meta'))

    def _static_arguments(self, x_dtype):
        """Kernel arguments of the per-tensor modes.  Scale and zero point reach the kernel as host floats, and
        reading them waits for the device: once deployed (``load_deploy``) the pair is read once and kept until the
        buffers are replaced or written in place (``load_state_dict``); before that it is derived from the observed
        bounds on every call, as the reference does."""
        key = (x_dtype,) + tuple((t.data_ptr(), t._version, t.device) for t in (self.scale, self.zero))
        if self.is_deploy and self._deployed is not None and self._deployed[0] == key:
            return self._deployed[1]
        with torch.no_grad():
            scale, zero = (self.scale.data, self.zero.data) if self.is_deploy else self.get_scale_zero_pertensor()
        if scale.numel() != 1:
            raise NotImplementedError('per-tensor quantization takes a one-element scale')
        promoted = self.promoted_dtype(x_dtype, scale)
        if promoted not in (x_dtype, torch.float32):
            raise NotImplementedError(f'arithmetic in {promoted} is not built')
        args = {'static': (float(scale), float(zero)),
                'static_fp32': promoted == torch.float32 and x_dtype != torch.float32}
        if self.is_deploy:
            self._deployed = (key, args)
        return args

    def kernel_arguments(self, x_dtype):
        """Keyword arguments of ``ops.dsa_rotate_fakequant`` for an activation of ``x_dtype``."""
        if self.is_per_tensor:
            return self._static_arguments(x_dtype)
        if self.lac:
            sig_max, sig_min = self._sigmoids()
            return {'clip_max_sigmoid': sig_max, 'clip_min_sigmoid': sig_min}
        if self._clip_ratio is not None:
            return {'clip_ratio': float(self._clip_ratio)}
        return {}

    def fake_quant(self, x):
        if self.sym:
            self.cnt += 1
        return _ops.dsa_rotate_fakequant(x, rotate=False, bits=self.bits, symmetric=self.sym,
                                         **self.kernel_arguments(x.dtype))
