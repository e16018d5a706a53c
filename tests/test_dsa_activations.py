"""KV-cache / indexer activation path on the CPU: the oracle against the reference's outputs
(tests/golden/dsa_golden.npz) and the host side of the drop-in modules (names, refusals)."""
import os

import pytest
import torch

from golden_io import Golden, bits_equal
from oracle import dsa as O

GOLD = Golden(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'dsa_golden.npz'))
CLIP_MAX, CLIP_MIN = float(GOLD.get('fq.clip_max_raw')), float(GOLD.get('fq.clip_min_raw'))


@pytest.mark.parametrize('dtype', ['fp16', 'bf16', 'fp32'])
@pytest.mark.parametrize('k', [128, 512, 200])
def test_oracle_fake_quant(dtype, k):
    x = GOLD.get(f'fq.{dtype}.{k}.x')
    assert bits_equal(O.activation_fake_quant(x), GOLD.get(f'fq.{dtype}.{k}.sym'))
    assert bits_equal(O.activation_fake_quant(x, 8, True, True, CLIP_MAX, CLIP_MIN), GOLD.get(f'fq.{dtype}.{k}.lac.sym'))
    assert bits_equal(O.activation_fake_quant(x, 8, False, True, CLIP_MAX, CLIP_MIN), GOLD.get(f'fq.{dtype}.{k}.lac.asym'))
    assert O.activation_fake_quant(x, bits=16) is x


@pytest.mark.parametrize('dtype', ['bf16', 'fp16', 'fp32'])
@pytest.mark.parametrize('d', [128, 64])
def test_oracle_rotation(dtype, d):
    """Bit-equal here because the oracle's matmul and the reference's ran on the same BLAS; one unit in the last place
    is what the contract promises."""
    x = GOLD.get(f'rot.{dtype}.{d}.x')
    got, want = O.rotate_activation(x), GOLD.get(f'rot.{dtype}.{d}.out')
    assert got.dtype == want.dtype
    ulp = torch.finfo(x.dtype).eps * want.float().abs().clamp_min(float(torch.finfo(x.dtype).tiny))
    assert bool(((got.float() - want.float()).abs() <= ulp).all())


@pytest.mark.parametrize('dtype', ['fp16', 'bf16', 'fp32'])
def test_oracle_clip_ratio_and_per_tensor(dtype):
    x = GOLD.get(f'ext.{dtype}.x')
    for sym in (True, False):
        tag = 'sym' if sym else 'asym'
        assert bits_equal(O.activation_fake_quant(x, 8, sym, False, clip_ratio=0.9), GOLD.get(f'ext.{dtype}.ratio.{tag}'))
        hi, lo = O.observe([x[:6], x[6:]])
        for lac in (False, True):
            scale, zero = O.per_tensor_scale_zero(hi, lo, 8, sym, lac, CLIP_MAX, CLIP_MIN)
            want = GOLD.get(f"ext.{dtype}.tensor.{tag}.{'lac' if lac else 'plain'}")
            assert bits_equal(O.static_fake_quant(x, scale, zero, 8, sym), want)


def test_oracle_indexer_chain():
    r = O.rotate_activation(GOLD.get('chain.x'))
    assert bits_equal(O.activation_fake_quant(GOLD.get('chain.rotated').half()), GOLD.get('chain.out'))
    assert bits_equal(r, GOLD.get('chain.rotated'))


def test_rotation_is_orthonormal_and_rejects_other_widths():
    x = torch.randn(5, 256, generator=torch.Generator().manual_seed(1))
    y = O.rotate_activation(O.rotate_activation(x))
    assert torch.allclose(x, y, atol=1e-5)
    with pytest.raises(ValueError):
        O.rotate_activation(torch.zeros(2, 48))


def test_module_mirror_names_and_refusals():
    from amct_b200.experimental.quantization.deepseek_v3_2.node import ActivationQuantizer, get_qmin_qmax
    q = ActivationQuantizer(bits=8, sym=True, lac=True, groupsize=-1, per_tensor=False)
    assert sorted(q.state_dict()) == ['clip_factor_a_max', 'clip_factor_a_min', 'maxval', 'minval', 'scale', 'zero']
    assert float(q.clip_factor_a_max.detach()) == 4.0 and int(q.q_max) == 127 and int(q.q_min) == -128
    assert [int(v) for v in get_qmin_qmax(8, False)] == [255, 0]
    x = torch.randn(3, 8)
    assert ActivationQuantizer(bits=16)(x) is x                                # pass-through needs no kernel
    obs = ActivationQuantizer(bits=8, sym=True)
    obs.is_observe = True
    assert obs(x) is x and float(obs.maxval) == float(x.max()) and float(obs.minval) == float(x.min())
    with pytest.raises(NotImplementedError):
        ActivationQuantizer(bits=8, sym=True, groupsize=64)
    # per-tensor: the host side (bounds -> scale / zero, and which arithmetic dtype torch would use)
    x16 = GOLD.get('ext.fp16.x')
    for sym in (True, False):
        tag = 'sym' if sym else 'asym'
        pt = ActivationQuantizer(bits=8, sym=sym, lac=True, per_tensor=True)
        pt.clip_factor_a_max.data.fill_(CLIP_MAX)
        pt.clip_factor_a_min.data.fill_(CLIP_MIN)
        pt.is_observe = True
        pt(x16[:6])
        pt(x16[6:])
        pt.is_observe = False
        assert pt.maxval.dtype == torch.float16 and pt.maxval.dim() == 0          # replaced by the chunk's own max
        args = pt.kernel_arguments(torch.float16)
        assert args['static_fp32'] is True                                        # the fp32 clip parameter promotes
        assert args['static'][0] == float(GOLD.get(f'ext.deploy.{tag}.scale')) and args['static'][1] == float(GOLD.get(f'ext.deploy.{tag}.zero'))
        pt.deploy()
        assert bits_equal(pt.scale.data.float().reshape(-1), GOLD.get(f'ext.deploy.{tag}.scale'))
        plain = ActivationQuantizer(bits=8, sym=sym, lac=False, per_tensor=True)
        plain.is_observe = True
        plain(x16)
        plain.is_observe = False
        assert plain.kernel_arguments(torch.float16)['static_fp32'] is False      # 0-dim fp16 bounds: fp16 steps
    assert ActivationQuantizer(bits=8, sym=True, clip_ratio=0.9).kernel_arguments(torch.bfloat16) == {'clip_ratio': 0.9}
    from amct_b200.backend.lib import BackendError
    with pytest.raises(BackendError):                                          # no CPU fallback
        ActivationQuantizer(bits=8, sym=True)(x)


@pytest.mark.parametrize('lac', [False, True])
@pytest.mark.parametrize('sym', [True, False])
def test_per_tensor_bounds_on_another_device_than_the_module(sym, lac):
    """A module built on the host whose observed bounds were replaced by 0-dim tensors on the activation's device
    (what observe mode leaves) must derive scale and zero on that device: a one-element host parameter cannot be
    mixed with a 0-dim device tensor.  The meta device stands in for the accelerator, so this runs without one; an
    unexceeded bound stays the constructor's host tensor, which is the other half of the case."""
    from amct_b200.experimental.quantization.deepseek_v3_2.node import ActivationQuantizer
    q = ActivationQuantizer(bits=8, sym=sym, lac=lac, per_tensor=True)
    q._buffers['maxval'] = torch.empty((), dtype=torch.float16, device='meta')   # `.data =` refuses a meta tensor
    scale, zero = q.get_scale_zero_pertensor()                                  # minval still on the host
    assert scale.device.type == 'meta' and zero.device.type == 'meta'
    q._buffers['minval'] = torch.empty((), dtype=torch.float16, device='meta')
    scale, zero = q.get_scale_zero_pertensor()
    assert scale.device.type == 'meta' and scale.numel() == 1
    assert scale.dtype == (torch.float32 if lac else torch.float16)
    assert q.promoted_dtype(torch.float16, scale) == scale.dtype
    assert q.promoted_dtype(torch.bfloat16, torch.ones(1)) == torch.float32      # a loaded fp32 buffer promotes
    assert q.promoted_dtype(torch.bfloat16, torch.ones((), dtype=torch.float32)) == torch.bfloat16


def test_deployed_scale_is_read_once_and_reread_when_replaced():
    from amct_b200.experimental.quantization.deepseek_v3_2.node import ActivationQuantizer
    q = ActivationQuantizer(bits=8, sym=False, per_tensor=True)
    q.load_deploy(torch.tensor([0.5]), torch.tensor([3.0]))
    first = q.kernel_arguments(torch.float16)
    assert first['static'] == (0.5, 3.0) and q.kernel_arguments(torch.float16) is first
    assert q.kernel_arguments(torch.bfloat16)['static'] == (0.5, 3.0)
    q.load_deploy(torch.tensor([0.25]), torch.tensor([1.0]))
    assert q.kernel_arguments(torch.float16)['static'] == (0.25, 1.0)
    q.load_state_dict({**q.state_dict(), 'scale': torch.tensor([2.0])})          # an in-place write is seen too
    assert q.kernel_arguments(torch.float16)['static'] == (2.0, 1.0)
