"""Generate golden vectors for the KV-cache / indexer activation path by running the REFERENCE on CPU.

    AMCT_REFERENCE=/path/to/amct python tests/golden/make_dsa_golden.py

Imports, from amct_pytorch/experimental/quantization/DeepSeekV3.2, ``cores.quantization.node.ActivationQuantizer``
(per-token dynamic fake quantization as the attention module constructs it: symmetric without learned clipping,
symmetric and asymmetric with it) and ``cores.models.deepseek_v3_2.indexer.rotate_activation`` (the 128-wide
Hadamard rotation), runs them on seeded inputs and writes ``tests/golden/dsa_golden.npz`` (16-bit floats as raw bit
patterns, the key suffix carries the dtype).  The tests need neither the reference nor scipy / loguru.
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get('AMCT_REFERENCE') or sys.exit('set AMCT_REFERENCE to a checkout of the reference (read only)')
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REF, 'amct_pytorch', 'experimental', 'quantization', 'DeepSeekV3.2'))
from cores.quantization.node import ActivationQuantizer  # noqa: E402
from cores.models.deepseek_v3_2.indexer import rotate_activation  # noqa: E402

store = {}
TAG = {torch.bfloat16: 'bf16', torch.float16: 'fp16'}


def put(name, t):
    t = t.detach().cpu().contiguous()
    if t.dtype in TAG:
        store[f'{name}|{TAG[t.dtype]}'] = t.view(torch.int16).numpy()
    else:
        store[name] = t.numpy()


def activations(gen, rows, k, dtype):
    x = torch.randn(rows, k, generator=gen) * torch.exp(torch.randn(rows, 1, generator=gen))
    x[1] = x[1].abs()                    # all positive: the lower bound stays 0
    x[2] = -x[2].abs()                   # all negative: the symmetric rule without clipping sees a zero bound
    x[3] = 0                             # all zero
    x[4, ::7] *= 30                      # outliers
    return x.to(dtype)


def main():
    gen = torch.Generator().manual_seed(31)
    for dname, dt in {'fp16': torch.float16, 'bf16': torch.bfloat16, 'fp32': torch.float32}.items():
        for k in (128, 512, 200):
            x = activations(gen, 12, k, dt)
            put(f'fq.{dname}.{k}.x', x)
            with torch.no_grad():
                # afq1 / afq2 / afq_rot_q / afq_rot_k of the attention module: symmetric, no learned clipping
                aq = ActivationQuantizer(bits=8, sym=True, lac=False, groupsize=-1, per_tensor=False)
                put(f'fq.{dname}.{k}.sym', aq(x))
                # k_cache_quantizer: learned clipping, symmetric or asymmetric
                for sym in (True, False):
                    aq = ActivationQuantizer(bits=8, sym=sym, lac=True, groupsize=-1, per_tensor=False)
                    aq.clip_factor_a_max.data.fill_(1.7)
                    aq.clip_factor_a_min.data.fill_(0.9)
                    put(f"fq.{dname}.{k}.lac.{'sym' if sym else 'asym'}", aq(x))
    store['fq.clip_max_raw'] = np.float32([1.7])
    store['fq.clip_min_raw'] = np.float32([0.9])
    for dname, dt in {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp32': torch.float32}.items():
        for d in (128, 64):
            x = activations(gen, 40, d, dt)
            put(f'rot.{dname}.{d}.x', x)
            put(f'rot.{dname}.{d}.out', rotate_activation(x))
    # the indexer's sequence: rotate in bf16, cast to half, fake-quantize (quant_dsa.py:75-82)
    x = activations(gen, 40, 128, torch.bfloat16)
    put('chain.x', x)
    with torch.no_grad():
        aq = ActivationQuantizer(bits=8, sym=True, lac=False, groupsize=-1, per_tensor=False)
        r = rotate_activation(x)
        put('chain.rotated', r)
        put('chain.out', aq(r.half()))
    # clip_ratio (a plain number: the bounds stay in the activation dtype) and per-tensor static scales taken from an
    # observation pass (fp32 buffers of one element: they promote the arithmetic to fp32)
    for dname, dt in {'fp16': torch.float16, 'bf16': torch.bfloat16, 'fp32': torch.float32}.items():
        x = activations(gen, 12, 256, dt)
        put(f'ext.{dname}.x', x)
        with torch.no_grad():
            for sym in (True, False):
                tag = 'sym' if sym else 'asym'
                aq = ActivationQuantizer(bits=8, sym=sym, lac=False, groupsize=-1, clip_ratio=0.9, per_tensor=False)
                put(f'ext.{dname}.ratio.{tag}', aq(x))
                for lac in (False, True):
                    aq = ActivationQuantizer(bits=8, sym=sym, lac=lac, groupsize=-1, per_tensor=True)
                    if lac:
                        aq.clip_factor_a_max.data.fill_(1.7)
                        aq.clip_factor_a_min.data.fill_(0.9)
                    aq.is_observe = True
                    aq(x[:6])
                    aq(x[6:])
                    aq.is_observe = False
                    put(f"ext.{dname}.tensor.{tag}.{'lac' if lac else 'plain'}", aq(x))
                    if dname == 'fp16' and lac:
                        aq.deploy()
                        put(f'ext.deploy.{tag}.scale', aq.scale.data.float().reshape(-1))
                        put(f'ext.deploy.{tag}.zero', aq.zero.data.float().reshape(-1))
    np.savez_compressed(os.path.join(HERE, 'dsa_golden.npz'), **store)
    print(len(store), 'arrays')


if __name__ == '__main__':
    main()
