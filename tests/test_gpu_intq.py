"""GPU parity of the integer quantization kernels, called through the C ABI.

Bit-exact against (a) the golden vectors produced by the reference and (b) the
CPU oracle on seeded inputs, including ragged / unaligned / large-K shapes."""
import itertools

import pytest
import torch

from golden_io import Golden, bits_equal
from oracle import intq, npu_ops

pytestmark = pytest.mark.gpu
G = Golden()
DT = {'fp32': torch.float32, 'bf16': torch.bfloat16, 'fp16': torch.float16}
WCASES = list(itertools.product(DT, ('int8', 'int4'), (True, False), ('tensor', 'channel', 'group')))


def ops():
    from amct_b200.backend import ops as o
    return o


def dev(t):
    return None if t is None else t.cuda()


@pytest.mark.parametrize('qt,sym', list(itertools.product(('int8', 'int4'), (True, False))))
def test_scale_offset_golden(qt, sym):
    s, o = ops().scale_offset(dev(G.get('k0/max')).reshape(-1, 1), dev(G.get('k0/min')).reshape(-1, 1), sym, qt)
    assert bits_equal(s, G.get(f'k0/{qt}/{int(sym)}/scale'))
    assert bits_equal(o, G.get(f'k0/{qt}/{int(sym)}/offset'))


@pytest.mark.parametrize('dname,qt,sym,strat', WCASES)
def test_weight_paths_golden(dname, qt, sym, strat):
    from amct_b200.quantize_op.utils import weight_scale_offset, get_weight_min_max_by_granularity
    w = dev(G.get(f'w/{dname}/weight'))
    gs = 32 if strat == 'group' else None
    tag = f'w/{dname}/{qt}/{int(sym)}/{strat}'
    s, o = weight_scale_offset(w, qt, sym, strat, gs)
    assert bits_equal(s, G.get(tag + '/scale'))
    assert bits_equal(o, G.get(tag + '/offset'))
    # unfused observer + rule gives the same factors
    cfgd = {'weights_cfg': {'strategy': strat, 'group_size': gs}}
    mn, mx = get_weight_min_max_by_granularity(w, cfgd)
    s2, o2 = ops().scale_offset(mx, mn, sym, qt)
    assert bits_equal(s2, s) and bits_equal(o2, o)

    gold = intq.crop_groups(G.get(tag + '/codes'), w.shape)
    _, _, codes = ops().quant_rows(w, qt, sym, strat, gs, scale=s, offset=o, out='i8' if qt == 'int8' else 'i32')
    assert bits_equal(codes, gold.contiguous())
    # fused: factors and codes from one read of the weight
    if strat != 'tensor':
        s3, o3, codes3 = ops().quant_rows(w, qt, sym, strat, gs, out='i8' if qt == 'int8' else 'i32')
        assert bits_equal(s3.reshape(s.shape), s) and bits_equal(codes3, gold.contiguous())
    _, _, fake = ops().quant_rows(w, qt, sym, strat, gs, scale=s, offset=o, out='fake')
    assert bits_equal(fake, G.get(tag + '/fake'))
    _, _, fake_awq = ops().quant_rows(w, qt, sym, strat, gs, scale=s, offset=o, out='fake_awq')
    assert bits_equal(fake_awq, G.get(tag + '/fake_awq'))
    if qt == 'int4':
        _, _, packed = ops().quant_rows(w, qt, sym, strat, gs, scale=s, offset=o, out='pack4')
        want = npu_ops.pack_int4_along_k(gold.t().contiguous()).t()
        assert bits_equal(packed, want.contiguous())


@pytest.mark.parametrize('dname', list(DT))
@pytest.mark.parametrize('rule', ['released', 'experimental'])
def test_dynamic_per_token_golden(dname, rule):
    x = dev(G.get(f'k1/{dname}/x'))
    q, s = ops().quant_dynamic_per_token(x, rule=rule, check=True)
    pre = 'k1' if rule == 'released' else 'k1x'
    assert bits_equal(s, G.get(f'{pre}/{dname}/scale'))
    assert bits_equal(q, G.get(f'{pre}/{dname}/codes'))


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('rows,k', [(1, 8), (3, 67), (5, 1000), (7, 4096), (4, 8192), (3, 28672), (2, 40000), (0, 64)])
@pytest.mark.parametrize('smooth', [False, True])
def test_dynamic_per_token_oracle(dtype, rows, k, smooth):
    g = torch.Generator().manual_seed(rows * 131 + k)
    x = torch.randn(rows, k, generator=g)
    if rows:
        x[:, :: max(1, k // 41)] *= 20
        x[0, 0] = -x[0].abs().max() * 2
    x = x.to(dtype)
    f = (torch.rand(1, k, generator=g) + 0.5).to(dtype) if smooth else None
    q_ref, s_ref = intq.dynamic_per_token(x, 'released', f)
    q, s = ops().quant_dynamic_per_token(x.cuda(), smooth=dev(f))
    assert bits_equal(s, s_ref)
    assert bits_equal(q, q_ref)


def test_dynamic_per_token_strided_rows_and_3d():
    g = torch.Generator().manual_seed(5)
    big = torch.randn(6, 512, generator=g).to(torch.bfloat16)
    view = big[:, 128:384]                                     # ld 512, k 256, 16-byte aligned
    q, s = ops().quant_dynamic_per_token(view.cuda())
    q_ref, s_ref = intq.dynamic_per_token(view.contiguous())
    assert bits_equal(q, q_ref) and bits_equal(s, s_ref)
    x3 = torch.randn(2, 3, 136, generator=g)
    q, s = ops().quant_dynamic_per_token(x3.cuda())
    q_ref, s_ref = intq.dynamic_per_token(x3)
    assert bits_equal(q, q_ref) and bits_equal(s, s_ref)


def test_nonfinite_input_raises_like_reference():
    x = torch.randn(4, 64)
    x[2, 3] = float('nan')
    with pytest.raises(RuntimeError, match='invalid value inf, nan or zeros'):
        ops().quant_dynamic_per_token(x.cuda(), check=True)
    w = torch.randn(8, 64)
    w[1, 1] = float('inf')
    with pytest.raises(RuntimeError, match='invalid value inf, nan or zeros'):
        ops().quant_rows(w.cuda(), 'int8', True, 'channel')


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('rows,k', [(1, 1), (9, 67), (300, 256), (2049, 136), (64, 4096)])
def test_minmax_observers(dtype, rows, k):
    g = torch.Generator().manual_seed(rows + k)
    x = torch.randn(rows, k, generator=g).to(dtype)
    xc = x.cuda()
    mn, mx = ops().minmax(xc, 'tensor')
    assert bits_equal(mn, x.min().reshape(1)) and bits_equal(mx, x.max().reshape(1))
    mn, mx = ops().minmax(xc, 'column')
    assert bits_equal(mn, x.amin(0, keepdim=True)) and bits_equal(mx, x.amax(0, keepdim=True))
    mn, mx = ops().minmax_rows(xc)
    assert bits_equal(mn, x.amin(1)) and bits_equal(mx, x.amax(1))
    # running merge with a second batch
    y = (torch.randn(rows, k, generator=g) * 2).to(dtype)
    run = ops().minmax(xc, 'column')
    ops().minmax(y.cuda(), 'column', running=(run[0].view(-1), run[1].view(-1)))
    both = torch.cat((x, y))
    assert bits_equal(run[0], both.amin(0, keepdim=True)) and bits_equal(run[1], both.amax(0, keepdim=True))
    f = (torch.rand(1, k, generator=g) + 0.5).to(dtype)
    mn, mx = ops().minmax_rows(xc, pre=f.cuda(), pre_op='div')
    assert bits_equal(mn, (x / f).amin(1)) and bits_equal(mx, (x / f).amax(1))


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('rows,k', [(9, 67), (300, 256), (2049, 136)])
def test_minmax_observers_propagate_nan(dtype, rows, k):
    """torch.amax / amin / max / min return NaN where an operand is NaN (so the scale rule then raises); the running
    merge is torch.where(batch > running, batch, running): a NaN batch value is dropped, a NaN running value stays."""
    g = torch.Generator().manual_seed(7 * rows + k)
    x = torch.randn(rows, k, generator=g).to(dtype)
    x[rows // 2, k // 3] = float('nan')
    x[rows - 1, k - 1] = float('nan')
    xc = x.cuda()

    def same(a, b):                                     # NaN payloads are not part of the contract
        a, b = a.cpu().float().reshape(-1), b.float().reshape(-1)
        return bool((torch.isnan(a) == torch.isnan(b)).all()) and bits_equal(torch.nan_to_num(a), torch.nan_to_num(b))

    mn, mx = ops().minmax(xc, 'tensor')
    assert torch.isnan(mn).all() and torch.isnan(mx).all()
    mn, mx = ops().minmax(xc, 'column')
    assert same(mn, x.amin(0)) and same(mx, x.amax(0)) and int(torch.isnan(mn).sum()) == 2
    mn, mx = ops().minmax_rows(xc)
    assert same(mn, x.amin(1)) and same(mx, x.amax(1)) and int(torch.isnan(mx).sum()) == 2
    # an unaligned view takes the scalar kernels
    if k > 8:
        v = x[:, 1:k - 2]
        mn, mx = ops().minmax(xc[:, 1:k - 2], 'column')
        assert same(mn, v.amin(0)) and same(mx, v.amax(0))
        mn, mx = ops().minmax(xc[:, 1:k - 2], 'tensor')
        assert torch.isnan(mn).all() and torch.isnan(mx).all()
    with pytest.raises(RuntimeError, match='invalid value inf, nan or zeros'):
        lo, hi = ops().minmax(xc, 'tensor')
        ops().scale_offset(hi, lo, True, 'int8')
    # merge: clean running values + NaN batch -> the NaN is dropped; NaN running values stay
    clean = torch.randn(rows, k, generator=g).to(dtype)
    run = ops().minmax(clean.cuda(), 'column')
    run = (run[0].view(-1), run[1].view(-1))
    ops().minmax(xc, 'column', running=run)
    bmax, bmin = x.amax(0), x.amin(0)
    want_max = torch.where(bmax > clean.amax(0), bmax, clean.amax(0))
    want_min = torch.where(bmin < clean.amin(0), bmin, clean.amin(0))
    assert same(run[0], want_min) and same(run[1], want_max)
    run = ops().minmax(xc, 'column')
    run = (run[0].view(-1), run[1].view(-1))
    ops().minmax(clean.cuda(), 'column', running=run)
    assert int(torch.isnan(run[0]).sum()) == 2 and int(torch.isnan(run[1]).sum()) == 2


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('shape', [(5, 64), (2, 7, 72), (3, 33), (1, 4, 16, 40)])
@pytest.mark.parametrize('per_token,offset,smooth', [(False, False, False), (False, True, True), (True, False, False),
                                                     (True, True, True)])
def test_quantize_static_oracle(dtype, shape, per_token, offset, smooth):
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    n = shape[-2] if per_token else 1
    s = (torch.rand(n, generator=g) * 40 + 5).to(dtype)
    z = torch.randint(-20, 20, (n,), generator=g).to(dtype) if offset else None
    f = (torch.rand(1, shape[-1], generator=g) + 0.5).to(dtype) if smooth else None
    axis = -2 if per_token else -1
    want = npu_ops.npu_quantize(x * f if smooth else x, s, z, torch.int8, axis)
    got = ops().quantize_static(x.cuda(), s.cuda(), dev(z), axis=axis, smooth=dev(f))
    assert bits_equal(got, want)


def test_rowsum_and_transpose():
    g = torch.Generator().manual_seed(3)
    for n, k in ((1, 1), (17, 67), (64, 4096), (33, 272)):
        w = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
        assert bits_equal(ops().rowsum_i8(w.cuda()), w.to(torch.int32).sum(1).to(torch.int32))
        assert bits_equal(ops().transpose_i8(w.cuda()), w.t().contiguous())


@pytest.mark.parametrize('bits,group,offset', [(8, 0, False), (8, 0, True), (4, 32, True), (4, 128, False), (8, 64, True)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_dequant_weight_oracle(bits, group, offset, dtype):
    g = torch.Generator().manual_seed(bits + group)
    n, k = 40, 256
    lo, hi = (-8, 8) if bits == 4 else (-128, 128)
    q_kn = torch.randint(lo, hi, (k, n), generator=g, dtype=torch.int32)
    ng = k // group if group else 1
    s = (torch.rand(ng, n, generator=g) * 0.01 + 0.001).to(dtype)
    o = torch.randint(-8, 8, (ng, n), generator=g).to(dtype) if offset else None
    want = npu_ops.dequant_weight(q_kn, s, o, group, dtype).t().contiguous()
    if bits == 4:
        codes = npu_ops.pack_int4_along_k(q_kn).t().contiguous()
    else:
        codes = q_kn.to(torch.int8).t().contiguous()
    got = ops().dequant_weight(codes.cuda(), bits, s.cuda(), dev(o), group)
    assert bits_equal(got, want)


def test_config1_shape_properties():
    """Full size of the W8A8 single-Linear configuration: properties that hold at
    any size -- full use of the code range and |x - q*scale| <= scale/2 away from the clamp."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2048, 4096, generator=g)
    idx = torch.randperm(4096, generator=g)[:41]
    x[:, idx] *= 20
    xc = x.cuda()
    q, s = ops().quant_dynamic_per_token(xc, check=True)
    deq = q.float() * s[:, None]
    # half a step everywhere except at the positive clamp (a negative-dominant row divides by 128)
    ok = (deq - xc).abs().le(s[:, None] * 0.5 * (1 + 1e-5)) | (q == 127)
    assert ok.all()
    assert (q.int().abs().amax(1) >= 127).all()                    # every row uses its full range
    # a stripe of rows against the oracle
    q_ref, s_ref = intq.dynamic_per_token(x[1000:1032])
    assert bits_equal(q[1000:1032], q_ref) and bits_equal(s[1000:1032], s_ref)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('rows,k', [(64, 1024), (200, 4096), (333, 8192), (70, 28672), (129, 16384), (4096, 512)])
@pytest.mark.parametrize('smooth', [False, True])
def test_dynamic_per_token_streaming_kernel(dtype, rows, k, smooth):
    """Shapes the shared-memory-staged kernel takes (many rows, aligned K): bit-exact codes and
    scales, with outliers, a zero row, a negative-dominant row and a strided input."""
    g = torch.Generator().manual_seed(rows + k)
    x = torch.randn(rows, k, generator=g)
    x[:, :: max(1, k // 41)] *= 20
    x[1] = 0
    x[2, 5] = -x[2].abs().max() * 2
    x = x.to(dtype)
    f = (torch.rand(1, k, generator=g) + 0.5).to(dtype) if smooth else None
    q_ref, s_ref = intq.dynamic_per_token(x, 'released', f)
    q, s = ops().quant_dynamic_per_token(x.cuda(), smooth=dev(f), check=True)
    assert bits_equal(s, s_ref)
    assert bits_equal(q, q_ref)


def test_dynamic_per_token_rounding_ties():
    """Quotients that sit exactly on, and one ulp around, rounding ties: the reciprocal-multiply
    fast path must hand these to the IEEE division."""
    rows, k = 128, 2048
    g = torch.Generator().manual_seed(9)
    for scale_target in (1.0, 0.37, 3.0e-3, 17.25):
        n = torch.randint(-127, 127, (rows, k), generator=g).float() + 0.5
        x = n * scale_target
        ulp = torch.randint(-2, 3, (rows, k), generator=g, dtype=torch.int32)
        x = (x.view(torch.int32) + ulp).view(torch.float32)          # a few ulps around each tie
        x[:, 0] = 127 * scale_target                                  # pins the row scale
        q_ref, s_ref = intq.dynamic_per_token(x)
        q, s = ops().quant_dynamic_per_token(x.cuda())
        assert bits_equal(s, s_ref) and bits_equal(q, q_ref)


def test_dynamic_per_token_streaming_nonfinite():
    x = torch.randn(256, 1024)
    x[100, 77] = float('nan')
    with pytest.raises(RuntimeError, match='invalid value inf, nan or zeros'):
        ops().quant_dynamic_per_token(x.cuda(), check=True)
    x[100, 77] = float('inf')
    with pytest.raises(RuntimeError, match='invalid value inf, nan or zeros'):
        ops().quant_dynamic_per_token(x.to(torch.bfloat16).cuda(), check=True)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('smooth', [False, True])
def test_channel_int8_weight_quant_streaming_path(dtype, smooth):
    """Per-channel symmetric INT8 weight codes on a shape large enough for the streaming kernel."""
    g = torch.Generator().manual_seed(17)
    w = (torch.randn(320, 4096, generator=g) * 0.02).to(dtype)
    w[5] = 0
    w[9] = -w[9].abs()
    f = (torch.rand(1, 4096, generator=g) + 0.5).to(dtype) if smooth else None
    ws = intq.fold_smooth_into_weight(w, f) if smooth else w
    s_ref, _ = intq.weight_scale_offset(ws, 'int8', True, 'channel')
    q_ref = intq.weight_codes(ws, 'int8', s_ref)
    s, o, q = ops().quant_rows(w.cuda(), 'int8', True, 'channel', out='i8', pre=dev(f), pre_op='mul' if smooth else 'none')
    assert o is None and bits_equal(s.reshape(-1, 1), s_ref) and bits_equal(q, q_ref)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('qt,sym', [('int4', False), ('int4', True), ('int8', False)])
@pytest.mark.parametrize('rows,k,gs', [(37, 1024, 128), (300, 4096, 32), (64, 2048, 256), (5, 512, 64), (16, 96, 48)])
def test_group_weight_quant_oracle(dtype, qt, sym, rows, k, gs):
    """Group-wise weight quantization (warp-shuffle kernel where the group fits a warp, row kernel
    otherwise) against the oracle: factors, codes, packed nibbles and both fake-quant variants,
    with and without an AWQ-style pre-division."""
    g = torch.Generator().manual_seed(rows + k + gs)
    w = (torch.randn(rows, k, generator=g) * 0.05).to(dtype)
    w[0, :gs] = 0                                            # an all-zero group: scale becomes 1
    w[1 % rows, gs:2 * gs] = w[1 % rows, gs:2 * gs].abs() * -1       # a negative-only group
    pre = (torch.rand(k, generator=g) + 0.5).to(dtype)
    for pre_t, pre_op in ((None, 'none'), (pre, 'div')):
        wp = w if pre_t is None else w / pre_t
        s, o = intq.weight_scale_offset(wp, qt, sym, 'group', gs)
        kw = dict(pre=None if pre_t is None else pre_t.cuda(), pre_op=pre_op)
        s2, o2, codes = ops().quant_rows(w.cuda(), qt, sym, 'group', gs, out='i32', **kw)
        assert bits_equal(s2.reshape(s.shape), s)
        if not sym:
            assert bits_equal(o2.reshape(o.shape), o.to(torch.int32))
        want = intq.crop_groups(intq.weight_codes(wp, qt, s, o, gs), w.shape).to(torch.int32)
        assert bits_equal(codes, want.contiguous())
        # given factors (the deploy path), int8 codes
        _, _, c8 = ops().quant_rows(w.cuda(), qt, sym, 'group', gs, scale=s.cuda(), offset=dev(o), out='i8', **kw)
        assert bits_equal(c8, want.to(torch.int8).contiguous())
        if qt == 'int4':
            _, _, packed = ops().quant_rows(w.cuda(), qt, sym, 'group', gs, scale=s.cuda(), offset=dev(o), out='pack4', **kw)
            nib = (want + 8).to(torch.uint8)
            assert bits_equal(packed, (nib[:, 0::2] | (nib[:, 1::2] << 4)).contiguous())
        _, _, fake = ops().quant_rows(w.cuda(), qt, sym, 'group', gs, scale=s.cuda(), offset=dev(o), out='fake', **kw)
        assert bits_equal(fake, intq.fake_quant(wp, qt, s, o, gs))
        _, _, fake_awq = ops().quant_rows(w.cuda(), qt, sym, 'group', gs, scale=s.cuda(), offset=dev(o), out='fake_awq', **kw)
        assert bits_equal(fake_awq, intq.fake_quant_awq(wp, qt, s, o, gs))
        # factors and fake quantization from one read of the weight (what the AWQ search launches per candidate)
        for mode, want_fake in (('fake', intq.fake_quant(wp, qt, s, o, gs)), ('fake_awq', intq.fake_quant_awq(wp, qt, s, o, gs))):
            s4, o4, fake4 = ops().quant_rows(w.cuda(), qt, sym, 'group', gs, out=mode, **kw)
            assert bits_equal(s4.reshape(s.shape), s) and bits_equal(fake4, want_fake), mode


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_group_weight_quant_rounding_ties(dtype):
    """Weights that are exact multiples of half a quantization step: every quotient is an integer or
    a tie, where a reciprocal-multiply shortcut and the IEEE division may disagree."""
    g = torch.Generator().manual_seed(9)
    rows, k, gs = 64, 1024, 128
    steps = torch.randint(-15, 16, (rows, k), generator=g).float() * 0.5          # multiples of 0.5 in [-7.5, 7.5]
    scale = torch.tensor([0.0078125, 0.013671875, 0.1, 0.3]).repeat(rows * k // gs // 4 + 1)[:rows * k // gs].reshape(rows, k // gs, 1)
    w = (steps.reshape(rows, k // gs, gs) * scale).reshape(rows, k).to(dtype)
    for off in (None, torch.randint(-3, 4, (rows, k // gs, 1), generator=g).to(torch.int32)):
        want = intq.crop_groups(intq.weight_codes(w, 'int4', scale, off, gs), w.shape).to(torch.int32)
        _, _, codes = ops().quant_rows(w.cuda(), 'int4', off is None, 'group', gs, scale=scale.cuda(), offset=dev(off), out='i32')
        assert bits_equal(codes, want.contiguous())
        _, _, fake_awq = ops().quant_rows(w.cuda(), 'int4', off is None, 'group', gs, scale=scale.cuda(), offset=dev(off), out='fake_awq')
        assert bits_equal(fake_awq, intq.fake_quant_awq(w, 'int4', scale, off, gs))
