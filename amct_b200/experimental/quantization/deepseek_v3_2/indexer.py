"""Hadamard rotation of the lightning indexer's activations on the CUDA kernel.

``rotate_activation`` / ``hadamard_transform_fix`` stand in for the functions of the same names in
amct_pytorch/experimental/quantization/DeepSeekV3.2/cores/models/deepseek_v3_2/indexer.py:140-151: the last axis (a
power of two, 32 .. 512; the indexer's head_dim is 128) is multiplied by H / sqrt(d) in fp32 and the result is
returned in the input dtype.  The reference multiplies by the dense matrix; the kernel runs the equivalent fast
transform inside a warp, so results agree to the last place of the 16-bit dtype, not bit for bit.
``rotate_half_fake_quant`` is the indexer's whole sequence for q and k -- rotate, ``.half()``, per-token symmetric
fake quantization (cores/models/deepseek_v3_2/quant_dsa.py:75-82) -- in one pass over the data.
"""
import torch

from ....backend import ops as _ops


def hadamard_transform_fix(x):
    return _ops.dsa_rotate_fakequant(x, rotate=True, bits=16)


def rotate_activation(x):
    return hadamard_transform_fix(x)


def rotate_half_fake_quant(x, quantizer):
    """quantizer(rotate_activation(x).half()) for a symmetric or asymmetric ``ActivationQuantizer`` of this package."""
    return _ops.dsa_rotate_fakequant(x, rotate=True, out_dtype=torch.float16, bits=quantizer.bits,
                                     symmetric=quantizer.sym, **quantizer.kernel_arguments(torch.float16))
