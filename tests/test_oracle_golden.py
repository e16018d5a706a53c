"""The CPU oracle against vectors produced by the reference implementation.

This pins oracle/intq.py: every function there must reproduce, bit for bit,
what the reference computed for the stored inputs."""
import itertools

import pytest
import torch

from golden_io import Golden, bits_equal
from oracle import intq

G = Golden()
DTYPES = ('fp32', 'bf16', 'fp16')
WCASES = list(itertools.product(DTYPES, ('int8', 'int4'), (True, False), ('tensor', 'channel', 'group')))


@pytest.mark.parametrize('qt,sym', list(itertools.product(("int8", "int4"), (True, False))))
def test_scale_offset_rule(qt, sym):
    hi, lo = G.get('k0/max').reshape(-1, 1), G.get('k0/min').reshape(-1, 1)
    s, o = intq.scale_offset(hi, lo, sym, qt)
    assert bits_equal(s, G.get(f'k0/{qt}/{int(sym)}/scale'))
    assert bits_equal(o, G.get(f'k0/{qt}/{int(sym)}/offset'))


@pytest.mark.parametrize('dname,qt,sym,strat', WCASES)
def test_weight_paths(dname, qt, sym, strat):
    w = G.get(f'w/{dname}/weight')
    gs = 32 if strat == 'group' else None
    tag = f'w/{dname}/{qt}/{int(sym)}/{strat}'
    s, o = intq.weight_scale_offset(w, qt, sym, strat, gs)
    assert bits_equal(s, G.get(tag + '/scale'))
    assert bits_equal(o, G.get(tag + '/offset'))
    assert bits_equal(intq.weight_codes(w, qt, s, o, gs), G.get(tag + '/codes'))
    assert bits_equal(intq.fake_quant(w, qt, s, o, gs), G.get(tag + '/fake'))
    assert bits_equal(intq.fake_quant_awq(w, qt, s, o, gs), G.get(tag + '/fake_awq'))


@pytest.mark.parametrize('dname', DTYPES)
def test_dynamic_per_token_released(dname):
    x = G.get(f'k1/{dname}/x')
    q, s = intq.dynamic_per_token(x, 'released')
    assert bits_equal(s, G.get(f'k1/{dname}/scale'))
    assert bits_equal(q, G.get(f'k1/{dname}/codes'))


@pytest.mark.parametrize('dname', DTYPES)
def test_dynamic_per_token_experimental(dname):
    if not G.has(f'k1x/{dname}/codes'):
        pytest.skip('fixture lacks the experimental rule')
    x = G.get(f'k1/{dname}/x')
    q, s = intq.dynamic_per_token(x, 'experimental')
    assert bits_equal(s, G.get(f'k1x/{dname}/scale'))
    assert bits_equal(q, G.get(f'k1x/{dname}/codes'))


W8A8 = ('sq_tensor', 'sq_tensor_asym', 'sq_token', 'mm_tensor_asym', 'mm_token')


@pytest.mark.parametrize('case', W8A8)
def test_w8a8_deploy_buffers(case):
    tag = f'deploy/{case}'
    w, b = G.get(f'{tag}/fc1.weight'), G.get(f'{tag}/fc1.bias')
    q = lambda a: G.get(f'{tag}/fc1.q.{a}')
    buf = intq.w8a8_deploy_buffers(w, b, q('scale_w'), q('scale_d'), q('offset_d'), q('scale'))
    for name in ('act_scale', 'act_offset', 'scale_factor', 'quantized_weight', 'deq_scale',
                 'pertoken_scale', 'bias'):
        assert bits_equal(buf.get(name), G.get(f'{tag}/fc1.d.{name}')), name


@pytest.mark.parametrize('case', ('sq_tensor', 'sq_tensor_asym', 'sq_token'))
def test_smooth_factor(case):
    tag = f'deploy/{case}'
    w = G.get(f'{tag}/fc1.weight')
    c0, c1 = G.get('deploy/calib0'), G.get('deploy/calib1')
    lo0, hi0 = intq.column_min_max(c0)
    lo1, hi1 = intq.column_min_max(c1)
    hi, lo = torch.maximum(hi0, hi1), torch.minimum(lo0, lo1)
    act = torch.max(hi.abs(), lo.abs())
    strength = 0.4 if case == 'sq_tensor_asym' else 0.5
    f = intq.smooth_factor(act, w, strength)
    assert bits_equal(f, G.get(f'{tag}/fc1.q.scale'))
    s, o = intq.weight_scale_offset(intq.fold_smooth_into_weight(w, f), 'int8', True, 'channel')
    assert bits_equal(s, G.get(f'{tag}/fc1.q.scale_w'))


@pytest.mark.parametrize('case,qt,gs', (('w4_group_asym', 'int4', 32), ('w8_channel', 'int8', None),
                                        ('w8_tensor_asym', 'int8', None)))
def test_weight_only_deploy_buffers(case, qt, gs):
    tag = f'deploy/{case}'
    for layer in ('fc1', 'fc2'):
        w, b = G.get(f'{tag}/{layer}.weight'), G.get(f'{tag}/{layer}.bias')
        q = lambda a: G.get(f'{tag}/{layer}.q.{a}')
        buf = intq.w4a16_deploy_buffers(w, b, qt, q('scale_w'), q('offset_w'), gs)
        for name in ('quantized_weight', 'scale_w', 'offset_w', 'bias'):
            assert bits_equal(buf.get(name), G.get(f'{tag}/{layer}.d.{name}')), (layer, name)
