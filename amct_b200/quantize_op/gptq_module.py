import math

import torch
import torch.nn.functional as F

from .base_quant_module import BaseQuantizeModule
from .utils import weight_scale_offset
from ..backend import ops
from ..utils.data_utils import check_linear_input_dim
from ..utils.log import LOGGER


class GPTQuant(BaseQuantizeModule):
    """GPTQ calibration of one Linear (contract of amct_pytorch/quantize_op/gptq_module.py:29-186).

    The Hessian X^T X accumulates on the device over ``batch_num`` batches; then columns are
    quantized in order of decreasing Hessian diagonal, each column's error being pushed into
    the columns not yet quantized (blocks of 128).  The per-column fake quantization is the
    row kernel (quant_dequant_weight, amct_pytorch/utils/quant_util.py:162-188) on the
    transposed block; the Cholesky factorisations are torch.linalg.
    """

    def __init__(self, ori_module, layer_name, quant_config):
        super().__init__(ori_module, layer_name, quant_config)
        self.weight = ori_module.weight
        if not torch.isfinite(self.weight.data).all():
            raise ValueError("{}'s weight has invalid value, inf or nan.".format(layer_name))
        self.bias = ori_module.bias
        self.layer_name = layer_name
        self.quant_config = quant_config
        self.cur_batch = 0
        self.nsamples = 0
        self.perc_damp = 0.01
        self.block_size = 128
        self.hessian = None

    @torch.no_grad()
    def forward(self, inputs):
        check_linear_input_dim(inputs)
        inputs = inputs.to(self.weight.device)
        if self.cur_batch < self.quant_config.get('batch_num'):
            self.update_hessian(inputs)
            self.cur_batch += 1
        if self.cur_batch == self.quant_config.get('batch_num'):
            self.cur_batch += 1
            self.weight.data, self.scale_w, self.offset_w = self.get_opt_weight_and_quant_factor()
            LOGGER.logd("Calculate gptq quant params of layer '{}' success!".format(self.layer_name), 'GPTQuant')
        return F.linear(inputs, self.weight, self.bias)

    def update_hessian(self, input_data):
        if input_data.dim() == 2:
            input_data = input_data.unsqueeze(0)
        batch = input_data.shape[0]
        x = input_data.reshape(-1, input_data.shape[-1]).t()
        if self.hessian is None:
            k = self.weight.shape[1]
            self.hessian = torch.zeros((k, k), dtype=torch.float32, device=x.device)
        self.hessian *= self.nsamples / (self.nsamples + batch)
        self.nsamples += batch
        x = math.sqrt(2 / self.nsamples) * x.float()
        self.hessian += x.matmul(x.t())
        if not torch.isfinite(self.hessian).all():
            raise RuntimeError("{}'s hessian matrix has invalid value, inf or nan.".format(self.layer_name))

    def _fake_quant_column(self, w, scale, offset):
        """w [N] with one (scale, offset) per row -> quantize-dequantize, fp32."""
        _, _, fq = ops.quant_rows(w.reshape(-1, 1).contiguous(), self.wts_type, offset is None, 'channel',
                                  scale=scale.reshape(-1), offset=None if offset is None else offset.reshape(-1), out='fake')
        return fq.reshape(-1)

    def get_opt_weight_and_quant_factor(self):
        cfg = self.quant_config.get('weights_cfg')
        self.group_size = cfg.get('group_size')
        self.wts_type = cfg.get('quant_type')
        columns = self.weight.shape[1]
        n = self.weight.shape[0]
        weight = self.weight.clone().float()
        hessian = self.hessian
        dead = torch.diag(hessian) == 0
        hessian[dead, dead] = 1
        weight[:, dead] = 0
        perm = torch.argsort(torch.diag(hessian), descending=True)
        invperm = torch.argsort(perm)

        scale_w, offset_w = weight_scale_offset(weight, self.wts_type, cfg.get('symmetric'), cfg.get('strategy'),
                                                self.group_size)
        w_sorted = weight[:, perm]
        h = hessian[perm][:, perm]
        diag = torch.arange(columns, device=weight.device)
        h[diag, diag] += self.perc_damp * torch.mean(torch.diag(h))
        h = torch.linalg.cholesky(h)
        h = torch.cholesky_inverse(h)
        h_inv = torch.linalg.cholesky(h, upper=True)
        del h
        self.hessian = None

        def factors(col):
            """(scale, offset) [N] for the original column index `col`."""
            if self.group_size:
                g = int(col) // self.group_size
                return scale_w[:, g].reshape(-1), None if offset_w is None else offset_w[:, g].reshape(-1)
            s = scale_w.reshape(-1)
            o = None if offset_w is None else offset_w.reshape(-1)
            return (s.expand(n) if s.numel() == 1 else s), (None if o is None else (o.expand(n) if o.numel() == 1 else o))

        perm_host = perm.tolist()
        for i1 in range(0, columns, self.block_size):
            i2 = min(i1 + self.block_size, columns)
            block = w_sorted[:, i1:i2]
            err_block = torch.zeros_like(block)
            h_block = h_inv[i1:i2, i1:i2]
            for i in range(i2 - i1):
                w = block[:, i]
                s, o = factors(perm_host[i1 + i])
                err = (w - self._fake_quant_column(w, s.contiguous(), None if o is None else o.contiguous())) / h_block[i, i]
                block[:, i:] -= err.unsqueeze(1).matmul(h_block[i, i:].unsqueeze(0))
                err_block[:, i] = err
            w_sorted[:, i2:] -= err_block.matmul(h_inv[i1:i2, i2:])
        return w_sorted[:, invperm].to(self.weight.dtype), scale_w, offset_w
