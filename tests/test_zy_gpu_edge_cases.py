"""Corner cases of the integer quantizers that the CPU emulation of the kernel source turned up (see
tests/test_kernel_source_emulation.py); on the GPU they run after the long-standing parity tests."""
import pytest
import torch

from golden_io import bits_equal
from oracle import intq

pytestmark = pytest.mark.gpu


def ops():
    from amct_b200.backend import ops as o
    return o


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('strategy,group,k', [('channel', None, 200), ('group', 64, 256), ('group', 48, 96)])
def test_fake_quant_keeps_the_sign_of_a_zero_input(dtype, strategy, group, k):
    """-0.0 / scale is -0.0 in the reference's torch division; both fake-quant variants show it."""
    gen = torch.Generator().manual_seed(51)
    w = (torch.randn(4, k, generator=gen) * 0.05).to(dtype)
    w[:, ::3] = -0.0
    w[1] = -0.0                                            # a whole row of negative zeros: scale becomes 1
    for qt, sym in (('int4', True), ('int4', False), ('int8', True)):
        scale, offset = intq.weight_scale_offset(w, qt, sym, strategy, group)
        dev_off = None if offset is None else offset.cuda()
        fake = ops().quant_rows(w.cuda(), qt, sym, strategy, group, scale=scale.cuda(), offset=dev_off, out='fake')[2]
        assert bits_equal(fake, intq.fake_quant(w, qt, scale, offset, group))
        fake = ops().quant_rows(w.cuda(), qt, sym, strategy, group, scale=scale.cuda(), offset=dev_off, out='fake_awq')[2]
        assert bits_equal(fake, intq.fake_quant_awq(w, qt, scale, offset, group))


def test_experimental_rule_with_a_scale_that_underflows():
    """fp16 rows around 1e-7: max / 127 rounds to zero in fp16, x / 0 is +-inf (clamped) or NaN for a zero element,
    which the reference's int8 cast turns into code 0."""
    gen = torch.Generator().manual_seed(52)
    x = (torch.randn(5, 64, generator=gen) * 1e-7).half()
    x[:, 7] = 0
    want_q, want_s = intq.dynamic_per_token(x, 'experimental')
    got_q, got_s = ops().quant_dynamic_per_token(x.cuda(), rule='experimental')
    assert bool((want_s == 0).any())
    assert bits_equal(got_s, want_s) and bits_equal(got_q, want_q)


@pytest.mark.parametrize('dynamic', [True, False])
def test_w8a8_linear_with_one_scale_for_the_whole_weight(dynamic):
    """weights.strategy = 'tensor' (the reference's test_int8_int8_tensor_sym_minmax_success configuration): the
    deq_scale buffer keeps one element as in the reference; the GEMM gets it per output channel."""
    import amct_b200 as amct
    from oracle import npu_ops
    torch.manual_seed(5)
    net = torch.nn.Sequential(torch.nn.Linear(256, 192)).to(torch.bfloat16).cuda()
    w, b = net[0].weight.data.cpu().clone(), net[0].bias.data.cpu().clone()
    inputs = {'type': 'int8', 'symmetric': True, 'strategy': 'token', 'dynamic': True} if dynamic else \
        {'type': 'int8', 'symmetric': True, 'strategy': 'tensor'}
    amct.quantize(net, {'batch_num': 1, 'quant_cfg': {'weights': {'type': 'int8', 'symmetric': True, 'strategy': 'tensor'},
                                                       'inputs': inputs}, 'algorithm': {'minmax'}})
    x = (torch.randn(64, 256) * 2).to(torch.bfloat16)
    net(x.cuda())                                          # calibration batch
    amct.convert(net)
    assert net[0].deq_scale.numel() == 1
    got = net(x.cuda()).cpu()
    sw, _ = intq.weight_scale_offset(w, 'int8', True, 'tensor')
    wq = intq.w8a8_weight_codes(w, sw.reshape(-1))
    if dynamic:
        q, s = intq.dynamic_per_token(x)
        want = npu_ops.npu_quant_matmul(q, wq.t(), sw.reshape(-1).expand(192), s, b, torch.bfloat16)
        assert bits_equal(got, want)
    else:
        # static per-tensor activations: codes from the calibrated scale; compare against the float Linear loosely
        ref = torch.nn.functional.linear(x.float(), w.float(), b.float())
        assert float((got.float() - ref).abs().max()) < 0.05 * float(ref.abs().max())


def _check_empty(cases):
    failures = []
    for name, fn, shape, dtype in cases:
        try:
            out = fn()
            out.cpu()                                                 # any launch error surfaces here
            if tuple(out.shape) != shape or out.dtype != dtype:
                failures.append((name, tuple(out.shape), out.dtype))
        except Exception as exc:                                      # noqa: BLE001 -- collected, reported together
            failures.append((name, repr(exc)[:120]))
    assert not failures, failures


def test_zero_rows_are_a_no_op_in_the_quantizers():
    """An empty batch (zero token rows) goes through every activation-side quantizer without a launch error and comes
    back with zero rows of the right width and dtype."""
    o = ops()
    k = 128
    x = torch.empty(0, k, dtype=torch.bfloat16).cuda()
    one, zero = torch.ones(1).cuda(), torch.zeros(1).cuda()
    gamma = torch.ones(k, dtype=torch.bfloat16).cuda()
    _check_empty([
        ('quant_dynamic_per_token', lambda: o.quant_dynamic_per_token(x)[0], (0, k), torch.int8),
        ('quantize_static', lambda: o.quantize_static(x, one, zero), (0, k), torch.int8),
        ('addnorm_quant_per_token', lambda: o.addnorm_quant_per_token(x, gamma, 1e-5)[0], (0, k), torch.int8),
        ('hif8_encode', lambda: o.hif8_encode(x), (0, k), torch.uint8),
        ('hif8_fake_quant', lambda: o.hif8_fake_quant(x), (0, k), torch.bfloat16),
        ('dsa_rotate_fakequant', lambda: o.dsa_rotate_fakequant(x), (0, k), torch.bfloat16),
        ('dsa_rotate_fakequant rotate', lambda: o.dsa_rotate_fakequant(x, rotate=True, out_dtype=torch.float16), (0, k), torch.float16),
    ])


def test_zero_rows_through_the_gemms():
    o = ops()
    k, n = 128, 256
    w = torch.randint(-128, 128, (n, k), dtype=torch.int8).cuda()
    q = torch.empty(0, k, dtype=torch.int8).cuda()
    x = torch.empty(0, k, dtype=torch.bfloat16).cuda()
    wf = torch.randn(n, k).to(torch.bfloat16).cuda()
    _check_empty([
        ('gemm_w8a8', lambda: o.gemm_w8a8(q, w, torch.ones(n).cuda(), torch.empty(0).cuda(), None), (0, n), torch.bfloat16),
        ('gemm_f16', lambda: o.gemm_f16(x, wf), (0, n), torch.bfloat16),
    ])
