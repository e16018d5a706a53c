import torch

from ..backend import ops


class HiFloat8Linear(torch.nn.Module):
    """Linear with HiFloat8 weights and activations.

    Buffers: ``quantized_weight`` uint8 HiF8 codes [K, N] (a transposed view of the
    K-contiguous [N, K] storage), ``scale_factor`` [1, K] reciprocal smoothing factor (only
    when the calibration produced one), ``bias``.  forward(): activations are multiplied by
    scale_factor, rounded to HiFloat8 and back in one pass; the weight codes are decoded
    (exactly) to the activation dtype -- in shared memory, ahead of the MMA, inside the GEMM
    kernel -- and the product runs on the tensor cores with fp32 accumulation.  B200 has no HiFloat8 MMA, so the 16-bit MMA on exactly decoded operands
    is the arithmetic definition of this layer.
    """

    def __init__(self, quant_module):
        super().__init__()
        weight = quant_module.weight.data
        self.output_dtype = weight.dtype
        smooth = quant_module.scale
        if smooth is not None:
            smooth = smooth.to(device=weight.device, dtype=weight.dtype)
            weight = weight * smooth
            self.register_buffer('scale_factor', 1 / smooth)
        else:
            self.scale_factor = None
        self.register_buffer('quantized_weight', ops.hif8_encode(weight).t())
        if quant_module.bias is not None:
            self.register_buffer('bias', quant_module.bias.data.to(torch.float32))
        else:
            self.bias = None
        self._decoded = None
        self.cache_decoded_weight = False

    @torch.no_grad()
    def forward(self, x):
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if self.scale_factor is not None:
            x2 = x2 * self.scale_factor
        xq = ops.hif8_fake_quant(x2)
        w = self._decoded
        n_out = self.quantized_weight.shape[1]
        if w is None and x.dtype in (torch.float16, torch.bfloat16) and x2.shape[0] <= 128 and n_out >= 3 * k:
            # one kernel: the weight codes are decoded in shared memory ahead of the MMA.  It gives every 128 output
            # channels to one CTA and walks K serially, so it only beats decode + GEMM for a few tokens and a wide,
            # shallow weight (14336 x 4096, 128 tokens: 70 us against 81; 4096 x 4096: 66 against 36; 4096 x 14336:
            # 193 against 95)
            out = ops.gemm_hif8_weight(xq, self.quantized_weight.t(), bias=self.bias, out_dtype=x.dtype)
            if out is not None:
                return out.reshape(*x.shape[:-1], -1)
        if w is None:
            w = ops.hif8_decode(self.quantized_weight.t(), dtype=x.dtype)
            if self.cache_decoded_weight:
                self._decoded = w
        out = ops.gemm_f16(xq, w, bias=self.bias, out_dtype=x.dtype)
        return out.reshape(*x.shape[:-1], -1)
