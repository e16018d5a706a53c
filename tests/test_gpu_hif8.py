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


def test_encode_every_bfloat16_pattern():
    """All 65536 bfloat16 patterns (the bf16 kernels index their tables with the pattern's top 13 bits): codes and
    fake-quantized values against the oracle, NaNs of every payload and sign included; a ragged tail as well."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    for x in (bits.view(torch.bfloat16), bits.view(torch.bfloat16)[3:-2].clone()):
        want = hif8.encode(x.float().numpy())
        got = ops().hif8_encode(x.cuda()).cpu().numpy()
        assert np.array_equal(got, want)
        fake = ops().hif8_fake_quant(x.cuda()).cpu()
        ref = torch.from_numpy(hif8.decode(want)).to(torch.bfloat16)
        assert np.array_equal(torch.isnan(fake).numpy(), torch.isnan(ref).numpy())
        ok = ~torch.isnan(ref)
        assert torch.equal(fake.view(torch.int16)[ok], ref.view(torch.int16)[ok])       # bit for bit, the sign of zero included


def test_decode_long_and_ragged():
    """Decoding 16 codes per thread: every code, many times over, lengths that are and are not multiples of 16."""
    codes = torch.randint(0, 256, (100003,), dtype=torch.uint8, generator=torch.Generator().manual_seed(2))
    want = hif8.DECODE_TABLE
    for n in (100003, 99984, 16, 15):
        for dtype in (torch.bfloat16, torch.float16, torch.float32):
            got = ops().hif8_decode(codes[:n].clone().cuda(), dtype).cpu().float().numpy()
            ref = want[codes[:n].numpy()]
            assert np.array_equal(np.isnan(got), np.isnan(ref)) and np.array_equal(got[~np.isnan(ref)], ref[~np.isnan(ref)])


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


def test_llama_layer_smoothquant_hifloat8_workload():
    """The SmoothQuant (a = 0.5) + HiFloat8 decoder-layer workload at a toy size: calibration through quantize(), seven
    HiFloat8Linear modules after convert(), smoothing factors by the reference's rule from the calibration inputs, and
    every Linear's output against the oracle's HiFloat8 round trip of its actual input and an fp64 product."""
    from amct_b200.workloads import llama_hif8
    from amct_b200.workloads.llama_tp import LlamaShape
    shape = LlamaShape(hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, intermediate=512, n_layers=1, vocab=1000)
    # the float layer first, to record what calibration will see
    ref_layer = llama_hif8.LlamaLayer(shape, 'cuda', seed=3)
    seen = {name: [] for name in llama_hif8.LINEARS}
    hooks = [getattr(ref_layer, name).register_forward_pre_hook(lambda m, a, name=name: seen[name].append(a[0].reshape(-1, a[0].shape[-1]).cpu()))
             for name in llama_hif8.LINEARS]
    work = llama_hif8.build(shape, 'cuda', seed=3, calib_sequences=8, calib_seq=32, calib_batch=4)
    float_work = llama_hif8.HiF8LayerWorkload(ref_layer, work.embed, 0, 32)
    ids_gen = torch.Generator().manual_seed(3)
    for _ in range(2):
        float_work(torch.randint(0, 1000, (4, 32), generator=ids_gen).cuda())
    for h in hooks:
        h.remove()
    # evaluation inputs of every deployed Linear
    inputs, outputs = {}, {}
    for name in llama_hif8.LINEARS:
        mod = getattr(work.layer, name)
        assert type(mod).__name__ == 'HiFloat8Linear'
        def record(m, a, out, name=name):
            inputs[name], outputs[name] = a[0].cpu(), out.cpu()            # (returns None: the output stays as it is)
        mod.register_forward_hook(record)
    ids = torch.randint(0, 1000, (2, 32), generator=torch.Generator().manual_seed(9)).cuda()
    y = work(ids)
    assert y.shape == (2, 32, 256) and torch.isfinite(y.float()).all()
    for name in llama_hif8.LINEARS:
        mod, w = getattr(work.layer, name), getattr(ref_layer, name).weight.data.cpu()
        # smoothing factor: s = amax_x^0.5 / amax_w^0.5 per input channel (bf16 torch ops, as the reference computes it)
        act = torch.cat(seen[name]).abs().amax(0, keepdim=True)
        s = (act ** 0.5) / (w.abs().amax(0, keepdim=True) ** 0.5)
        assert torch.equal((1 / s).view(torch.int16), mod.scale_factor.cpu().view(torch.int16)), name
        # weight codes: HiFloat8 of the smoothed weight
        wq = hif8.encode((w * s).float().numpy())
        assert np.array_equal(mod.quantized_weight.t().cpu().numpy(), wq), name
        x = inputs[name].reshape(-1, w.shape[1])
        xq = hif8.decode(hif8.encode((x * mod.scale_factor.cpu()).float().numpy()))
        want = torch.from_numpy(xq).double() @ torch.from_numpy(hif8.decode(wq)).double().t()
        got = outputs[name].reshape(-1, w.shape[0]).double()
        assert float((got - want).abs().max() / want.abs().max()) < 1e-2, name          # bf16 output rounding
