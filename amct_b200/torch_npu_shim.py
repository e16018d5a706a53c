"""The four backend ops of the deploy path with ``torch_npu``'s call signatures,
running on the CUDA kernels of this package.

``install()`` registers this module as ``sys.modules['torch_npu']`` so that code
written against the reference (``import torch_npu; torch_npu.npu_quantize(...)``,
amct_pytorch/deploy_op/npu_quantization_linear.py:95-102,
amct_pytorch/deploy_op/weight_npu_quant_module.py:55-57,108-117) runs unchanged.
"""
import sys

import torch

from .backend import ops


def npu_quantize(input, scales, zero_points=None, dtype=torch.int8, axis=-1, div_mode=False):
    if dtype != torch.int8 or div_mode:
        raise NotImplementedError('npu_quantize: only dtype=torch.int8, div_mode=False')
    return ops.quantize_static(input, scales, zero_points, axis=axis)


def _as_nk(w_kn):
    """[K, N] weight -> K-contiguous [N, K] tensor (free when it already is a transposed view)."""
    if w_kn.stride(0) == 1:
        return w_kn.t()
    return ops.transpose_i8(w_kn) if w_kn.dtype == torch.int8 else w_kn.t().contiguous()


def npu_quant_matmul(x1, x2, scale, offset=None, bias=None, pertoken_scale=None, output_dtype=torch.bfloat16, **_):
    if offset is not None:
        raise NotImplementedError('npu_quant_matmul: offset is not used by the deploy modules')
    k = x1.shape[-1]
    out = ops.gemm_w8a8(x1.reshape(-1, k), _as_nk(x2), scale, pertoken_scale, bias, out_dtype=output_dtype)
    return out.reshape(*x1.shape[:-1], -1)


FUSED_MAX_TOKENS = 128


def weight_quant_matmul(x, codes_nk, bits, antiquant_scale, antiquant_offset, bias, group_size):
    """x [..., K] (fp16 / bf16) times the dequantized weight, codes in the kernels' own form: int8 [N, K], or the INT4
    payload uint8 [N, K / 2]."""
    k = x.shape[-1]
    # up to FUSED_MAX_TOKENS rows: one kernel that streams the packed weight once (a weight-streaming kernel for up to
    # 16 rows, codes dequantized in shared memory ahead of the MMA beyond that).  More rows, or shapes those kernels do
    # not take: dequantize to HBM once and run the 16-bit GEMM, whose larger tiles win once the work is tensor-bound
    # (config 2's shape, one kernel against dequant + GEMM: 23 / 60 us at 16 rows, 45 / 62 at 128, 70 / 65 at 256,
    # 147 / 114 at 1024).
    x2 = x.reshape(-1, k)
    out = None
    if x2.shape[0] <= FUSED_MAX_TOKENS:
        out = ops.gemm_w4a16(x2, codes_nk, bits, antiquant_scale, antiquant_offset, group_size, bias=bias, out_dtype=x.dtype)
    if out is None:
        w = ops.dequant_weight(codes_nk, bits, antiquant_scale.to(x.dtype), antiquant_offset, group_size)
        out = ops.gemm_f16(x2, w, bias=bias, out_dtype=x.dtype)
    return out.reshape(*x.shape[:-1], -1)


_PAYLOADS = {}


def npu_weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset=None, quant_scale=None,
                                 quant_offset=None, bias=None, antiquant_group_size=0, **_):
    """torch_npu's call: weight is int8 [K, N], or INT4 as int32 [K, N / 8] (the result of
    npu_convert_weight_to_int4pack) -- converted to the kernels' K-major payload on first sight and kept while the
    tensor lives; the deploy module holds that payload itself and does not come through here."""
    n = antiquant_scale.shape[-1]
    if weight.dtype == torch.int8:
        return weight_quant_matmul(x, _as_nk(weight), 8, antiquant_scale, antiquant_offset, bias, antiquant_group_size)
    key = (weight.data_ptr(), weight._version, tuple(weight.shape), weight.dtype)
    payload = _PAYLOADS.get(key)
    if payload is None:
        from .utils import int4pack
        _PAYLOADS.clear()                              # one weight at a time: a cache, not a store
        payload = int4pack.to_payload(int4pack.codes_from_buffer(weight, n).t().contiguous())
        _PAYLOADS[key] = payload
    return weight_quant_matmul(x, payload, 4, antiquant_scale, antiquant_offset, bias, antiquant_group_size)


def npu_convert_weight_to_int4pack(weight, inner_k_tiles=0):
    """int32 codes [K, N] in [-8, 7] -> int32 [K, N / 8], eight nibbles per word along N."""
    from .utils import int4pack
    return int4pack.to_int4pack(weight)


class _Npu:
    @staticmethod
    def is_available():
        return False

    @staticmethod
    def empty_cache():
        torch.cuda.empty_cache()


npu = _Npu()


def install():
    sys.modules['torch_npu'] = sys.modules[__name__]
    if not hasattr(torch.Tensor, 'npu'):
        torch.Tensor.npu = lambda self, *a, **k: self
