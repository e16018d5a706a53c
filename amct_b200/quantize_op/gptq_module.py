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
    the columns not yet quantized (blocks of 128).  The column loop of a block -- fake quantization
    (quant_dequant_weight, amct_pytorch/utils/quant_util.py:162-188), error, rank-1 update -- is one kernel
    (amct_gptq_block); the trailing update of a block is one GEMM; the Cholesky factorisations are torch.linalg.
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
        w_sorted = weight[:, perm].contiguous()             # row-major: the block kernel walks rows
        h = hessian[perm][:, perm]
        diag = torch.arange(columns, device=weight.device)
        h[diag, diag] += self.perc_damp * torch.mean(torch.diag(h))
        h = torch.linalg.cholesky(h)
        h = torch.cholesky_inverse(h)
        h_inv = torch.linalg.cholesky(h, upper=True).contiguous()       # (the upper factor comes back as a transposed view)
        del h
        self.hessian = None

        # quant factors as [N or 1, G] tables; a block column takes the entry of its original column's group
        groups = scale_w.shape[1] if self.group_size else 1
        scale_tab = scale_w.reshape(-1, groups) if self.group_size else scale_w.reshape(-1, 1)
        offset_tab = None if offset_w is None else (offset_w.reshape(-1, groups) if self.group_size else offset_w.reshape(-1, 1))
        col_groups = (perm // self.group_size if self.group_size else torch.zeros_like(perm)).to(torch.int32)
        bits = ops.bits_of(self.wts_type)
        for i1 in range(0, columns, self.block_size):
            i2 = min(i1 + self.block_size, columns)
            # the whole column loop of the block is one kernel (one warp per weight row); the trailing update is one GEMM
            err_block = ops.gptq_block(w_sorted[:, i1:i2], h_inv[i1:i2, i1:i2], scale_tab, offset_tab, col_groups[i1:i2], bits)
            w_sorted[:, i2:] -= err_block.matmul(h_inv[i1:i2, i2:])
        return w_sorted[:, invperm].to(self.weight.dtype), scale_w, offset_w
