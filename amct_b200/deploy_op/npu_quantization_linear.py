import torch

from ..backend import ops


class NpuQuantizationLinear(torch.nn.Module):
    """W8A8 quantized Linear for deployment.

    Constructor argument, buffer names, shapes and dtypes follow
    amct_pytorch/deploy_op/npu_quantization_linear.py:22-130:
      act_scale / act_offset  [1] or [tokens], output dtype (reciprocal activation scale, offset)
      scale_factor            [1, K] reciprocal SmoothQuant factor (only with SmoothQuant)
      quantized_weight        [K, N] int8
      deq_scale               [N] fp32;  pertoken_scale [tokens] fp32 (per-token mode)
      bias                    [N] int32 (per-tensor mode, offset_bias folded in) or float (per-token)
    quantized_weight is a transposed VIEW of a contiguous [N, K] buffer: the MMA
    wants both operands K-contiguous, and a view keeps the reference's shape
    without a second copy of the weight.

    forward() is two kernels: activation quantization (SmoothQuant multiply
    folded into the load) and the tcgen05 INT8 GEMM with the dequant epilogue.
    With a quant module marked ``dynamic_act`` the activation scale is computed
    per token row at run time, so the token count of the input is free.
    """

    def __init__(self, quant_module):
        super().__init__()
        self.output_dtype = quant_module.weight.dtype
        device = quant_module.weight.device
        self.offset_bias = None
        self.act_type = quant_module.act_type
        self.dynamic_act = bool(getattr(quant_module, 'dynamic_act', False))
        self.dynamic_rule = 'released'
        # opt-in (not in the reference): 'swiglu' fuses silu(gate) * up into the GEMM epilogue of a fused
        # gate/up projection whose weight rows are interleaved in blocks of 128 (see interleave_gate_up)
        self.fused_act = None
        self.act_granularity = 'PER_TENSOR'
        self.quantize_axis = -1

        scale_d = quant_module.scale_d.to(device=device)
        offset_d = quant_module.offset_d
        if scale_d.dim() > 1:
            self.act_granularity = 'PER_TOKEN'
            self.quantize_axis = -2
        if not self.dynamic_act:
            off = offset_d if offset_d is not None else torch.zeros(1, dtype=torch.int32, device=device)
            off = off.to(device).repeat(scale_d.shape)
            self.register_buffer('act_scale', (1 / scale_d).reshape(-1).to(self.output_dtype))
            self.register_buffer('act_offset', off.reshape(-1).to(self.output_dtype))

        weight = quant_module.weight.data
        smooth = quant_module.scale
        if smooth is not None:
            smooth = smooth.to(device=device, dtype=weight.dtype)
            if list(smooth.shape) != [1, weight.shape[1]]:
                raise RuntimeError("smooth_factor shape should be {} current shape is {}".format(
                    [1, weight.shape[1]], list(smooth.shape)))
            self.register_buffer('scale_factor', (1 / quant_module.scale).to(device=device))
        scale_w = quant_module.scale_w.reshape(-1).to(device=device)
        codes_nk = self.quant_wts(weight, scale_w, quant_module.wts_type, smooth)
        self.register_buffer('quantized_weight', codes_nk.t())

        if offset_d is not None:
            # -round(offset_d * sum_k Wq[k, n]): integer row sums instead of the fp32 matmul
            self.offset_bias = -(offset_d.reshape(-1)[0].to(device=device, dtype=torch.int32) * ops.rowsum_i8(codes_nk))

        if self.act_granularity == 'PER_TENSOR':
            self.register_buffer('deq_scale', scale_d * scale_w)
            self.pertoken_scale = None
        else:
            self.register_buffer('deq_scale', scale_w)
            if self.dynamic_act:
                self.pertoken_scale = None
            else:
                self.register_buffer('pertoken_scale', quant_module.scale_d.reshape(-1).to(torch.float32).to(device))
        self._init_bias(quant_module, scale_d, scale_w)

    @staticmethod
    def quant_wts(weight, scale_w_tensor, wts_type, smooth=None):
        """round(weight / scale) codes as a contiguous int8 [N, K] tensor; `smooth`
        ([1, K]) is multiplied in first, rounded to the weight dtype."""
        strategy = 'channel' if scale_w_tensor.shape[0] > 1 else 'tensor'
        _, _, codes = ops.quant_rows(weight, wts_type, True, strategy, scale=scale_w_tensor, out='i8',
                                     pre=smooth, pre_op='mul' if smooth is not None else 'none')
        return codes

    def _init_bias(self, module, scale_d, scale_w):
        bias = module.bias
        if bias is not None:
            if self.act_granularity == 'PER_TENSOR':
                bias = (bias.data / (scale_d * scale_w)).round().to(torch.int32)
            else:
                bias = bias.data
            self.register_buffer('bias', bias)
            if self.offset_bias is not None:
                self.bias = self.bias + self.offset_bias
        else:
            self.bias = self.offset_bias

    @torch.no_grad()
    def forward(self, x, out=None):
        """`out` (optional, not in the reference): a preallocated [rows, N] tensor the GEMM writes into, e.g. a
        peer-mapped buffer the other ranks read the partial result from."""
        smooth = getattr(self, 'scale_factor', None)
        k = x.shape[-1]
        wq_nk = self.quantized_weight.t()
        if self.dynamic_act:
            q, pertoken = ops.quant_dynamic_per_token(x, smooth=smooth, rule=self.dynamic_rule)
        else:
            q = ops.quantize_static(x, self.act_scale, self.act_offset, axis=self.quantize_axis, smooth=smooth)
            pertoken = self.pertoken_scale
            if pertoken is not None and x.dim() > 2:
                pertoken = pertoken.repeat(x.numel() // (x.shape[-2] * k))
        return self._gemm(q, pertoken, out)

    def _deq_scales(self, n):
        """deq_scale with one value per output channel.  For one scale for the whole weight (strategy 'tensor') the
        buffer keeps the reference's one element and the expanded copy is kept until the buffer is replaced or
        written (no device read on the forward path)."""
        deq = self.deq_scale
        if deq.numel() == n:
            return deq
        key = (deq.data_ptr(), deq._version, deq.device)
        cached = getattr(self, '_deq_per_channel', None)
        if cached is None or cached[0] != key:
            cached = (key, deq.reshape(-1)[:1].to(torch.float32).expand(n).contiguous())
            self._deq_per_channel = cached
        return cached[1]

    def _gemm(self, q, pertoken, out=None):
        k = q.shape[-1]
        wq_nk = self.quantized_weight.t()
        deq = self._deq_scales(wq_nk.shape[0])
        if self.fused_act == 'swiglu':
            res = ops.gemm_w8a8_swiglu(q.reshape(-1, k), wq_nk, deq, pertoken, self.bias, out=out)
            return res.reshape(*q.shape[:-1], -1)
        res = ops.gemm_w8a8(q.reshape(-1, k), wq_nk, deq, pertoken, self.bias, out_dtype=self.output_dtype, out=out)
        return res.reshape(*q.shape[:-1], -1)

    @torch.no_grad()
    def forward_scatter(self, x, out_ptrs, slot, rows_per_rank, ld_out):
        """forward() of a K-sharded (row-parallel) Linear under tensor parallelism; not in the reference.  The result is
        this rank's partial sum, and instead of returning it the GEMM writes output row r into row
        (slot * rows_per_rank + r % rows_per_rank) of the staging buffer of rank r // rows_per_rank (out_ptrs: the
        device addresses of every rank's buffer as mapped into this process).  Dynamic per-token scales, no bias."""
        if not self.dynamic_act or self.bias is not None or self.fused_act is not None:
            raise RuntimeError('forward_scatter needs dynamic per-token activation scales, no bias and no fused activation')
        k = x.shape[-1]
        q, pertoken = ops.quant_dynamic_per_token(x, smooth=getattr(self, 'scale_factor', None), rule=self.dynamic_rule)
        wq_nk = self.quantized_weight.t()
        ops.gemm_w8a8_scatter(q.reshape(-1, k), wq_nk, self._deq_scales(wq_nk.shape[0]), pertoken, out_ptrs, slot,
                              rows_per_rank, ld_out, out_dtype=self.output_dtype)

    @torch.no_grad()
    def forward_quantized(self, q, pertoken_scale):
        """The GEMM half of forward() for an input some producer kernel has already quantized with
        the dynamic per-token rule (q int8 [..., K], pertoken_scale fp32 [rows]); not in the
        reference.  Only for modules with dynamic activation scales and no SmoothQuant factor."""
        if not self.dynamic_act or getattr(self, 'scale_factor', None) is not None:
            raise RuntimeError('forward_quantized needs dynamic per-token activation scales and no smooth factor')
        return self._gemm(q, pertoken_scale)


def interleave_gate_up(w_gate, w_up, block=128):
    """Rows of a fused gate/up weight in the order the SwiGLU epilogue expects: 128 gate rows,
    then the 128 matching up rows, and so on.  [I, K] + [I, K] -> [2 I, K] (I % 128 == 0)."""
    i, k = w_gate.shape
    assert w_up.shape == w_gate.shape and i % block == 0
    return torch.stack((w_gate.reshape(i // block, block, k), w_up.reshape(i // block, block, k)), dim=1).reshape(2 * i, k)
