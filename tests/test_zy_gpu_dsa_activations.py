"""GPU parity of amct_dsa_rotate_fakequant (amct_b200/csrc/kv_quant.cu) against the reference's own outputs
(tests/golden/dsa_golden.npz) and, at other shapes, oracle/dsa.py.

The fake quantization is compared bit for bit.  The rotation is an fp32 sum of k terms taken in another order than
the reference's matrix product: its result may differ by one unit in the last place of the activation dtype
(relative 2^-7 for bf16, 2^-10 for fp16, 2^-23 x a few for fp32), and the fused chain is therefore checked as
fake_quant(the kernel's own rotation), bit for bit, plus the rotation tolerance."""
import os

import pytest
import torch

from golden_io import Golden, bits_equal
from oracle import dsa as O

pytestmark = pytest.mark.gpu
GOLD = Golden(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'dsa_golden.npz'))
CLIP_MAX, CLIP_MIN = float(GOLD.get('fq.clip_max_raw')), float(GOLD.get('fq.clip_min_raw'))
SIG_MAX = float(torch.sigmoid(torch.tensor(CLIP_MAX)))
SIG_MIN = float(torch.sigmoid(torch.tensor(CLIP_MIN)))


def ops():
    from amct_b200.backend import ops as o
    return o


def close_rotation(got, want):
    """Within one unit in the last place of the dtype, measured against the row's largest magnitude for values that
    cancel to (almost) nothing."""
    assert got.dtype == want.dtype and got.shape == want.shape
    g, w = got.cpu().float(), want.cpu().float()
    eps = torch.finfo(want.dtype).eps * (4 if want.dtype == torch.float32 else 1)
    floor = w.abs().amax(-1, keepdim=True) * 2e-6 + torch.finfo(want.dtype).tiny * torch.finfo(want.dtype).eps    # + one step of a subnormal
    return bool(((g - w).abs() <= eps * w.abs() + floor).all())


@pytest.mark.parametrize('dtype', ['fp16', 'bf16', 'fp32'])
@pytest.mark.parametrize('k', [128, 512, 200])
def test_fake_quant_golden(dtype, k):
    x = GOLD.get(f'fq.{dtype}.{k}.x').cuda()
    assert bits_equal(ops().dsa_rotate_fakequant(x), GOLD.get(f'fq.{dtype}.{k}.sym'))
    got = ops().dsa_rotate_fakequant(x, symmetric=True, clip_max_sigmoid=SIG_MAX, clip_min_sigmoid=SIG_MIN)
    assert bits_equal(got, GOLD.get(f'fq.{dtype}.{k}.lac.sym'))
    got = ops().dsa_rotate_fakequant(x, symmetric=False, clip_max_sigmoid=SIG_MAX, clip_min_sigmoid=SIG_MIN)
    assert bits_equal(got, GOLD.get(f'fq.{dtype}.{k}.lac.asym'))


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize('shape', [(3, 70, 1536), (1000, 128), (5, 16384), (7, 33), (2, 4, 9, 512), (6, 8)])
def test_fake_quant_oracle(dtype, shape):
    gen = torch.Generator().manual_seed(41)
    x = (torch.randn(*shape, generator=gen) * torch.exp(torch.randn(*shape[:-1], 1, generator=gen))).to(dtype)
    flat = x.view(-1, shape[-1])
    flat[0] = 0
    flat[1] = -flat[1].abs()
    xd = x.cuda()
    assert bits_equal(ops().dsa_rotate_fakequant(xd), O.activation_fake_quant(x))
    assert bits_equal(ops().dsa_rotate_fakequant(xd, bits=4), O.activation_fake_quant(x, bits=4))
    got = ops().dsa_rotate_fakequant(xd, symmetric=True, clip_max_sigmoid=SIG_MAX)
    assert bits_equal(got, O.activation_fake_quant(x, 8, True, True, CLIP_MAX, CLIP_MIN))
    got = ops().dsa_rotate_fakequant(xd, symmetric=False, clip_max_sigmoid=SIG_MAX, clip_min_sigmoid=SIG_MIN)
    assert bits_equal(got, O.activation_fake_quant(x, 8, False, True, CLIP_MAX, CLIP_MIN))


def test_fake_quant_scale_underflow_keeps_nan():
    """fp16 rows so small that hi / 127 rounds to zero in fp16: x / 0 is +-inf (clamped) or, for a zero element, NaN,
    which torch.clamp keeps and the kernel must keep too."""
    gen = torch.Generator().manual_seed(45)
    x = (torch.randn(6, 64, generator=gen) * 1e-6).half()
    x[:, 5] = 0
    got = ops().dsa_rotate_fakequant(x.cuda()).cpu()
    want = O.activation_fake_quant(x)
    assert bool(torch.isnan(want).any())
    assert bool((torch.isnan(got) == torch.isnan(want)).all())
    keep = ~torch.isnan(want)
    assert bits_equal(torch.where(keep, got, torch.zeros_like(got)), torch.where(keep, want, torch.zeros_like(want)))


def test_fake_quant_nan_input_makes_the_row_nan():
    """torch.amax / amin carry a NaN of the row into its bounds, so scale and every output of that row are NaN; the
    other rows are untouched.  Plain and rotated path, symmetric and asymmetric."""
    gen = torch.Generator().manual_seed(46)
    for dtype in (torch.bfloat16, torch.float16):
        x = torch.randn(9, 128, generator=gen).to(dtype)
        x[2, 17] = float('nan')
        x[5, 127] = float('nan')
        for kwargs, ref in (({}, ()), ({'bits': 4}, (4,)),
                            ({'symmetric': False, 'clip_max_sigmoid': SIG_MAX, 'clip_min_sigmoid': SIG_MIN}, (8, False, True, CLIP_MAX, CLIP_MIN))):
            got = ops().dsa_rotate_fakequant(x.cuda(), **kwargs).cpu()
            want = O.activation_fake_quant(x, *ref)
            assert bool(torch.isnan(want[2]).all()) and bool(torch.isnan(want[5]).all())
            assert bool((torch.isnan(got) == torch.isnan(want)).all())
            keep = ~torch.isnan(want)
            assert bits_equal(torch.where(keep, got, torch.zeros_like(got)), torch.where(keep, want, torch.zeros_like(want)))
        rot = ops().dsa_rotate_fakequant(x.cuda(), rotate=True, out_dtype=torch.float16).cpu()
        assert bool(torch.isnan(rot[2]).all()) and bool(torch.isnan(rot[5]).all())
        assert not bool(torch.isnan(rot[[0, 1, 3, 4, 6, 7, 8]]).any())


def test_fake_quant_strided_and_cast():
    gen = torch.Generator().manual_seed(42)
    big = torch.randn(9, 300, generator=gen).to(torch.bfloat16)
    got = ops().dsa_rotate_fakequant(big.cuda()[:, 3:259])                     # unaligned start, row stride 300
    assert bits_equal(got, O.activation_fake_quant(big[:, 3:259].contiguous()))
    x = (torch.randn(6, 128, generator=gen) * 3).to(torch.bfloat16)
    got = ops().dsa_rotate_fakequant(x.cuda(), out_dtype=torch.float16)        # .half() then quantize
    assert bits_equal(got, O.activation_fake_quant(x.half()))


@pytest.mark.parametrize('dtype', ['bf16', 'fp16', 'fp32'])
@pytest.mark.parametrize('d', [128, 64])
def test_rotation_golden(dtype, d):
    x = GOLD.get(f'rot.{dtype}.{d}.x')
    got = ops().dsa_rotate_fakequant(x.cuda(), rotate=True, bits=16)
    assert close_rotation(got, GOLD.get(f'rot.{dtype}.{d}.out'))


@pytest.mark.parametrize('d', [32, 64, 128, 256, 512])
def test_rotation_widths_and_round_trip(d, rows=257):
    gen = torch.Generator().manual_seed(43)
    x = torch.randn(rows, d, generator=gen)
    got = ops().dsa_rotate_fakequant(x.cuda(), rotate=True, bits=16)
    assert close_rotation(got, O.rotate_activation(x))
    back = ops().dsa_rotate_fakequant(got, rotate=True, bits=16)               # H / sqrt(d) is its own inverse
    assert torch.allclose(back.cpu(), x, atol=1e-5)
    basis = torch.eye(d)                                                       # row i of H / sqrt(d), signs exact
    rows = ops().dsa_rotate_fakequant(basis.cuda(), rotate=True, bits=16).cpu()
    assert bool((torch.sign(rows) == torch.sign(O.rotate_activation(basis))).all())


def test_rotation_unaligned_rows():
    """Rows that do not start on a multiple of a lane's run take the element-wise loads and stores."""
    gen = torch.Generator().manual_seed(44)
    for dtype, start in ((torch.float32, 3), (torch.bfloat16, 2), (torch.bfloat16, 1), (torch.float16, 4)):
        big = torch.randn(11, 200, generator=gen).to(dtype)
        view = big[:, start:start + 128]
        got = ops().dsa_rotate_fakequant(big.cuda()[:, start:start + 128], rotate=True, bits=16)
        assert close_rotation(got, O.rotate_activation(view.contiguous()))
        fused = ops().dsa_rotate_fakequant(big.cuda()[:, start:start + 128], rotate=True, out_dtype=torch.float16, bits=8)
        assert bits_equal(fused, O.activation_fake_quant(got.cpu().half()))


def test_indexer_chain():
    """rotate -> .half() -> symmetric fake quantization, one launch, against the same steps launched one by one and
    against the reference's result for the chain."""
    x = GOLD.get('chain.x').cuda()
    rotated = ops().dsa_rotate_fakequant(x, rotate=True, bits=16)
    assert close_rotation(rotated, GOLD.get('chain.rotated'))
    fused = ops().dsa_rotate_fakequant(x, rotate=True, out_dtype=torch.float16, bits=8)
    assert bits_equal(fused, O.activation_fake_quant(rotated.cpu().half()))
    # where the kernel's rotation equals the reference's bit for bit over a whole row, so does the chain's output
    same_rows = (rotated.cpu().view(torch.int16) == GOLD.get('chain.rotated').view(torch.int16)).all(dim=1)
    assert int(same_rows.sum()) > 0
    assert bits_equal(fused.cpu()[same_rows], GOLD.get('chain.out')[same_rows])
    from amct_b200.experimental.quantization.deepseek_v3_2.indexer import rotate_activation, rotate_half_fake_quant
    from amct_b200.experimental.quantization.deepseek_v3_2.node import ActivationQuantizer
    assert bits_equal(rotate_activation(x), rotated)
    quantizer = ActivationQuantizer(bits=8, sym=True, lac=False, groupsize=-1, per_tensor=False)
    assert bits_equal(rotate_half_fake_quant(x, quantizer), fused)
    assert bits_equal(quantizer(rotated.half()), fused)


def test_module_with_learned_clipping():
    from amct_b200.experimental.quantization.deepseek_v3_2.node import ActivationQuantizer
    x = GOLD.get('fq.bf16.512.x').cuda()
    for sym in (True, False):
        q = ActivationQuantizer(bits=8, sym=sym, lac=True, groupsize=-1, per_tensor=False)
        q.clip_factor_a_max.data.fill_(CLIP_MAX)
        q.clip_factor_a_min.data.fill_(CLIP_MIN)
        assert bits_equal(q(x.unsqueeze(1)).squeeze(1), GOLD.get(f"fq.bf16.512.lac.{'sym' if sym else 'asym'}"))
        assert bits_equal(q.cuda()(x.unsqueeze(1)).squeeze(1), GOLD.get(f"fq.bf16.512.lac.{'sym' if sym else 'asym'}"))


@pytest.mark.parametrize('on_device', [True, False])
@pytest.mark.parametrize('dtype', ['fp16', 'bf16', 'fp32'])
def test_clip_ratio_and_per_tensor_modules(dtype, on_device):
    """ActivationQuantizer with a clip_ratio, and per-tensor with observed bounds (with and without learned clipping:
    fp32 and activation-dtype arithmetic), through the module, against the reference's outputs.  The module is
    moved to the activations' device as a model would be, or left on the host (its bounds and clip parameters
    then live on different devices)."""
    from amct_b200.experimental.quantization.deepseek_v3_2.node import ActivationQuantizer

    def place(module):
        return module.cuda() if on_device else module

    x = GOLD.get(f'ext.{dtype}.x').cuda()
    for sym in (True, False):
        tag = 'sym' if sym else 'asym'
        q = place(ActivationQuantizer(bits=8, sym=sym, lac=False, groupsize=-1, clip_ratio=0.9, per_tensor=False))
        assert bits_equal(q(x), GOLD.get(f'ext.{dtype}.ratio.{tag}'))
        for lac in (False, True):
            q = ActivationQuantizer(bits=8, sym=sym, lac=lac, groupsize=-1, per_tensor=True)
            if lac:
                q.clip_factor_a_max.data.fill_(CLIP_MAX)
                q.clip_factor_a_min.data.fill_(CLIP_MIN)
            q = place(q)
            q.is_observe = True
            q(x[:6])
            q(x[6:])
            q.is_observe = False
            assert bits_equal(q(x), GOLD.get(f"ext.{dtype}.tensor.{tag}.{'lac' if lac else 'plain'}"))
            scale, zero = q.get_scale_zero_pertensor()
            q.load_deploy(scale, zero)
            assert bits_equal(q(x), GOLD.get(f"ext.{dtype}.tensor.{tag}.{'lac' if lac else 'plain'}"))
            assert bits_equal(q(x), GOLD.get(f"ext.{dtype}.tensor.{tag}.{'lac' if lac else 'plain'}"))   # kept pair


def test_argument_errors():
    from amct_b200.backend.lib import BackendError
    x = torch.zeros(4, 48, device='cuda')
    with pytest.raises(BackendError):
        ops().dsa_rotate_fakequant(x, rotate=True, bits=16)                    # not a power of two
    with pytest.raises(BackendError):
        ops().dsa_rotate_fakequant(torch.zeros(4, 1024, device='cuda'), rotate=True, bits=16)   # wider than one warp holds
    with pytest.raises(BackendError):
        ops().dsa_rotate_fakequant(x, bits=9)
    with pytest.raises(ValueError):
        ops().dsa_rotate_fakequant(x, symmetric=False, clip_max_sigmoid=0.5)
    with pytest.raises(ValueError):
        ops().dsa_rotate_fakequant(x, clip_ratio=0.9, static=(1.0, 0.0))
