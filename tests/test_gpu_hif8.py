"""GPU parity of the HiFloat8 kernels and the HiFloat8 Linear against oracle/hif8.py (the
reference has no HiFloat8 code: parity is against the builder's CPU restatement only)."""
import numpy as np
import pytest
import torch

from oracle import hif8

pytestmark = pytest.mark.gpu


def ops():
    from amct_b200.backend import ops as o
    return o


def probe_values():
    """All representable values, all midpoints between neighbours, neighbours of both, specials,
    range edges, and a log-uniform random sample."""
    t = hif8.DECODE_TABLE
    fin = np.unique(np.abs(t[np.isfinite(t)]))
    mids = ((fin[1:] + fin[:-1]) / 2).astype(np.float32)
    base = np.concatenate([fin, mids])
    around = np.concatenate([base, np.nextafter(base, np.float32(0)), np.nextafter(base, np.float32(np.inf))])
    rng = np.random.default_rng(0)
    rand = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 13, 20000))).astype(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 2 ** -23, 2 ** -23 * 0.999, 2 ** -24, 1e-30, 1e-45, 32768, 33000,
                        49151.9, 49152, 65504, 1e9, 3e38], dtype=np.float32)
    v = np.concatenate([around, -around, rand, special, -special]).astype(np.float32)
    return v[:-3] if len(v) % 8 == 0 else v                            # keep a ragged tail


def test_decode_all_codes():
    codes = torch.arange(256, dtype=torch.uint8)
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        got = ops().hif8_decode(codes.cuda(), dtype).cpu().float().numpy()
        want = hif8.DECODE_TABLE
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got[ok], want[ok])              # exact in every float dtype


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
def test_encode_matches_oracle(dtype):
    x = torch.from_numpy(probe_values()).to(dtype)
    want = hif8.encode(x.float().numpy())
    got = ops().hif8_encode(x.cuda()).cpu().numpy()
    assert np.array_equal(got, want)
    fake = ops().hif8_fake_quant(x.cuda()).cpu().float().numpy()
    ref = hif8.decode(want)
    assert np.array_equal(np.isnan(fake), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.array_equal(fake[ok], torch.from_numpy(ref).to(dtype).float().numpy()[ok])


def test_encode_is_monotonic_and_idempotent():
    x = torch.linspace(-40000, 40000, 1 << 16)
    c = ops().hif8_encode(x.cuda())
    v = ops().hif8_decode(c, torch.float32)
    assert (v[1:] >= v[:-1]).all()
    assert torch.equal(ops().hif8_encode(v), c)


def test_hifloat8_linear_through_the_public_api():
    import amct_b200 as amct
    torch.manual_seed(3)
    net = torch.nn.Sequential(torch.nn.Linear(256, 136)).to(torch.bfloat16).cuda()
    w, b = net[0].weight.data.cpu().clone(), net[0].bias.data.cpu().clone()
    cfg = {'batch_num': 2, 'quant_cfg': {'weights': {'type': 'hifloat8', 'symmetric': True, 'strategy': 'channel'},
                                         'inputs': {'type': 'hifloat8', 'symmetric': True, 'strategy': 'tensor'}},
           'algorithm': {'hifloat8': {'smooth_strength': 0.5}}}
    amct.quantize(net, cfg)
    calib = [(torch.randn(64, 256) * 2).to(torch.bfloat16), (torch.randn(64, 256) * 2).to(torch.bfloat16)]
    calib[0][:, 3] *= 15
    for c in calib:
        net(c.cuda())
    smooth = net[0].scale.cpu()
    amct.convert(net)
    assert type(net[0]).__name__ == 'HiFloat8Linear' and net[0].quantized_weight.shape == (256, 136)
    # smoothing factor as the SmoothQuant rule gives it on the CPU
    both = torch.cat(calib)
    act = torch.max(both.amax(0, keepdim=True).abs(), both.amin(0, keepdim=True).abs())
    want_s = (act ** 0.5) / (w.abs().amax(0, keepdim=True) ** 0.5)
    assert torch.equal(smooth.view(torch.int16), want_s.view(torch.int16))
    # weight codes and forward
    wq = hif8.encode((w * smooth).float().numpy())
    assert np.array_equal(net[0].quantized_weight.t().cpu().numpy(), wq)
    x = (torch.randn(40, 256) * 3).to(torch.bfloat16)
    got = net(x.cuda()).cpu().float()
    xq = hif8.decode(hif8.encode((x * (1 / smooth)).float().numpy()))
    want = torch.from_numpy(xq).double() @ torch.from_numpy(hif8.decode(wq)).double().t() + b.double()
    err = ((got.double() - want).abs().max() / want.abs().max()).item()
    assert err < 1e-2, err
