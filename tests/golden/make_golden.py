"""Generate golden vectors by running the REFERENCE implementation on CPU.

Run where the reference checkout is available (it is not needed to run the
tests):

    AMCT_REFERENCE=/path/to/amct python tests/golden/make_golden.py

Writes ``tests/golden/intq_golden.npz``.  Inputs are seeded; both inputs and the
reference's outputs are stored, so the tests need neither the reference nor a
particular RNG implementation.  bf16/fp16 tensors are stored as raw 16-bit
patterns; the key suffix carries the dtype (``name|bf16``).

``torch_npu`` does not exist here; the one call that construction of a deploy
module makes (int4 pack) is stubbed with the identity, exactly as the
reference's own tests do (tests/amct_pytorch/mock_torch_npu.py:86-90).
"""
import os
import sys
import types
import itertools

import numpy as np
import torch

REF = os.environ.get('AMCT_REFERENCE') or sys.exit('set AMCT_REFERENCE to a checkout of the reference (read only)')
HERE = os.path.dirname(os.path.abspath(__file__))

DT = {'fp32': torch.float32, 'bf16': torch.bfloat16, 'fp16': torch.float16}
store = {}


def put(name, t):
    if t is None:
        return
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        store[name + '|bf16'] = t.view(torch.int16).numpy()
    elif t.dtype == torch.float16:
        store[name + '|fp16'] = t.view(torch.int16).numpy()
    else:
        store[name] = t.numpy()


def main():
    os.chdir('/tmp')                       # the reference logger writes ./amct_log
    sys.path.insert(0, REF)
    stub = types.ModuleType('torch_npu')
    stub.npu_convert_weight_to_int4pack = lambda w, inner_k_tiles=0: w
    sys.modules['torch_npu'] = stub
    torch.Tensor.npu = lambda self: self

    from amct_pytorch.quantize_op.utils import calculate_scale_offset, get_weight_min_max_by_granularity
    from amct_pytorch.utils.quant_util import convert_dtype, quant_weight, quant_dequant_weight
    from amct_pytorch.utils.data_utils import convert_precision
    from amct_pytorch.algorithm.awq import do_quant, do_dequant
    from amct_pytorch.deploy_op.npu_quantization_linear import NpuQuantizationLinear
    from amct_pytorch.deploy_op.weight_npu_quant_module import NpuWeightQuantizedLinear
    import amct_pytorch as amct

    g = torch.Generator().manual_seed(1234)

    # ---- K0: scale/offset from hand-picked and random (max, min) pairs
    hi = torch.cat([torch.tensor([1.0, 0.5, 0.0, 2.0, -1.0, 3e-8, 0.0, 5.0, 1.0]),
                    torch.randn(23, generator=g).abs() * 3])
    lo = torch.cat([torch.tensor([-0.5, -1.0, 0.0, 1.0, -2.0, -3e-8, -4.0, 5.0, -1.0]),
                    -torch.randn(23, generator=g).abs() * 3])
    put('k0/max', hi)
    put('k0/min', lo)
    for sym, qt in itertools.product((True, False), ('int8', 'int4')):
        s, o = calculate_scale_offset(hi.reshape(-1, 1), lo.reshape(-1, 1), sym, qt)
        put(f'k0/{qt}/{int(sym)}/scale', s)
        put(f'k0/{qt}/{int(sym)}/offset', o)

    # ---- K3/K4/K5/K7: weights through every granularity
    n, k = 24, 72                                     # 72 % 32 != 0 -> zero-padded tail group
    for dname, dt in DT.items():
        w = (torch.randn(n, k, generator=g) * 0.05).to(dt)
        w[3] = 0                                       # an all-zero channel
        w[5] = w[5].abs()                              # an all-positive channel
        w[7] = -w[7].abs()                             # negative-dominant
        put(f'w/{dname}/weight', w)
        for qt, sym, strat in itertools.product(('int8', 'int4'), (True, False), ('tensor', 'channel', 'group')):
            gs = 32 if strat == 'group' else None
            cfg = {'weights_cfg': {'quant_type': qt, 'symmetric': sym, 'strategy': strat}}
            if gs:
                cfg['weights_cfg']['group_size'] = gs
            wmin, wmax = get_weight_min_max_by_granularity(w, cfg)
            s, o = calculate_scale_offset(wmax, wmin, sym, qt)
            tag = f'w/{dname}/{qt}/{int(sym)}/{strat}'
            put(tag + '/scale', s)
            put(tag + '/offset', o)
            put(tag + '/codes', quant_weight(w, qt, s, o, gs))
            put(tag + '/fake', quant_dequant_weight(w, cfg, s, o))
            t = do_quant(w, s, o, strat, gs)
            t = convert_precision(t, qt)
            put(tag + '/fake_awq', do_dequant(t, s, o, strat, gs))

    # ---- K1: dynamic per-token, released rule = observer + scale rule + code rule
    for dname, dt in DT.items():
        x = torch.randn(19, 200, generator=g)
        x[:, 7] *= 20
        x[4] = 0
        x[6, 11] = -x[6].abs().max() * 1.5             # negative-dominant row -> divisor 128
        x = x.to(dt)
        put(f'k1/{dname}/x', x)
        hi_r = torch.amax(x, dim=(1,), keepdim=True)
        lo_r = torch.amin(x, dim=(1,), keepdim=True)
        s, _ = calculate_scale_offset(hi_r, lo_r, True, 'int8')
        put(f'k1/{dname}/scale', s.reshape(-1))
        put(f'k1/{dname}/codes', convert_dtype(x / s, 'int8'))

    # experimental dynamic rule (needs only torch from that tree's node.py)
    sys.path.insert(0, os.path.join(REF, 'amct_pytorch/experimental/quantization/DeepSeekV3.2'))
    try:
        from cores.quantization.node import ActivationQuantizer, sym_quant
        for dname, dt in DT.items():
            x = torch.from_numpy(store[f'k1/{dname}/x' + ('' if dname == 'fp32' else '|' + dname)].copy())
            x = x.view(dt) if dname != 'fp32' else x
            aq = ActivationQuantizer(bits=8, sym=True, lac=False, groupsize=-1, clip_ratio=None)
            s, _ = aq.get_scale_zero(x)
            q, _ = sym_quant(x, s, aq.q_max)
            put(f'k1x/{dname}/scale', s[:, 0].float())
            put(f'k1x/{dname}/codes', q.to(torch.int8))
    except Exception as exc:                           # optional dependency of that tree missing
        print('experimental rule skipped:', exc)

    # ---- deploy modules through the public API (bf16 model, seeded)
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1 = torch.nn.Linear(64, 64)
            self.fc2 = torch.nn.Linear(64, 32, bias=False)

        def forward(self, x):
            return self.fc2(self.fc1(x))

    def run(tag, cfg, calib):
        torch.manual_seed(7)
        net = Net().to(torch.bfloat16)
        put(f'{tag}/fc1.weight', net.fc1.weight)
        put(f'{tag}/fc1.bias', net.fc1.bias)
        put(f'{tag}/fc2.weight', net.fc2.weight)
        amct.quantize(net, cfg)
        for c in calib:
            net(c)
        for name in ('fc1', 'fc2'):
            m = getattr(net, name)
            for attr in ('scale_w', 'offset_w', 'scale_d', 'offset_d', 'scale'):
                put(f'{tag}/{name}.q.{attr}', getattr(m, attr, None))
        amct.convert(net)
        for name in ('fc1', 'fc2'):
            m = getattr(net, name)
            for attr in ('act_scale', 'act_offset', 'scale_factor', 'quantized_weight', 'deq_scale',
                         'pertoken_scale', 'bias', 'scale_w', 'offset_w'):
                v = getattr(m, attr, None)
                if isinstance(v, torch.Tensor):
                    put(f'{tag}/{name}.d.{attr}', v)

    calib = [torch.randn(16, 64, generator=g).to(torch.bfloat16) * 2 for _ in range(2)]
    calib[0][:, 5] *= 12
    put('deploy/calib0', calib[0])
    put('deploy/calib1', calib[1])
    w8 = {'type': 'int8', 'symmetric': True, 'strategy': 'channel'}
    run('deploy/sq_tensor', {'batch_num': 2, 'quant_cfg': {'weights': w8,
        'inputs': {'type': 'int8', 'symmetric': True, 'strategy': 'tensor'}},
        'algorithm': {'smoothquant': {'smooth_strength': 0.5}}}, calib)
    run('deploy/sq_tensor_asym', {'batch_num': 2, 'quant_cfg': {'weights': w8,
        'inputs': {'type': 'int8', 'symmetric': False, 'strategy': 'tensor'}},
        'algorithm': {'smoothquant': {'smooth_strength': 0.4}}}, calib)
    run('deploy/sq_token', {'batch_num': 2, 'quant_cfg': {'weights': w8,
        'inputs': {'type': 'int8', 'symmetric': True, 'strategy': 'token'}},
        'algorithm': {'smoothquant': {'smooth_strength': 0.5}}}, calib)
    run('deploy/mm_tensor_asym', {'batch_num': 2, 'quant_cfg': {'weights': w8,
        'inputs': {'type': 'int8', 'symmetric': False, 'strategy': 'tensor'}},
        'algorithm': {'minmax'}}, calib)
    run('deploy/mm_token', {'batch_num': 2, 'quant_cfg': {'weights': w8,
        'inputs': {'type': 'int8', 'symmetric': True, 'strategy': 'token'}},
        'algorithm': {'minmax'}}, calib)
    run('deploy/w4_group_asym', {'batch_num': 1, 'quant_cfg': {'weights':
        {'type': 'int4', 'symmetric': False, 'strategy': 'group', 'group_size': 32}},
        'algorithm': {'minmax'}}, calib[:1])
    run('deploy/w8_channel', {'batch_num': 1, 'quant_cfg': {'weights':
        {'type': 'int8', 'symmetric': True, 'strategy': 'channel'}},
        'algorithm': {'minmax'}}, calib[:1])
    run('deploy/w8_tensor_asym', {'batch_num': 1, 'quant_cfg': {'weights':
        {'type': 'int8', 'symmetric': False, 'strategy': 'tensor'}},
        'algorithm': {'minmax'}}, calib[:1])

    out = os.path.join(HERE, 'intq_golden.npz')
    np.savez_compressed(out, **store)
    print('wrote', out, len(store), 'arrays', os.path.getsize(out), 'bytes')


if __name__ == '__main__':
    main()
