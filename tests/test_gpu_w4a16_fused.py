"""The weight-only quantized Linear as one kernel (codes dequantized in shared memory ahead of the
tensor-core MMA), through the C ABI, against the CPU oracle and against the two-kernel route
(dequantize to HBM, then the 16-bit GEMM) on the same device."""
import pytest
import torch

from oracle import npu_ops

pytestmark = pytest.mark.gpu
TOL_16 = 1e-2          # max error relative to the largest reference magnitude, 16-bit outputs


def ops():
    from amct_b200.backend import ops as o
    return o


def make_case(g, m, n, k, group, bits, dtype, asym):
    x = torch.randn(m, k, generator=g).to(dtype)
    ng = k // group if group else 1
    lo, hi = (-8, 8) if bits == 4 else (-128, 128)
    q_kn = torch.randint(lo, hi, (k, n), generator=g, dtype=torch.int32)
    scale = (torch.rand(ng, n, generator=g) * 0.02 + 0.005).to(dtype)
    aoff = torch.randint(-7, 8, (ng, n), generator=g).to(dtype) if asym else None
    bias = torch.randn(n, generator=g).float()
    return x, q_kn, scale, aoff, bias


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('bits,group,asym', [(4, 128, True), (4, 64, False), (4, 0, True), (8, 128, True), (8, 0, False)])
@pytest.mark.parametrize('m,n,k', [(1, 256, 256), (16, 136, 512), (33, 384, 1024), (128, 264, 256), (300, 520, 1280)])
def test_fused_w4a16_matches_oracle_and_two_kernel_route(dtype, bits, group, asym, m, n, k):
    g = torch.Generator().manual_seed(m * 3 + n + k + bits)
    x, q_kn, scale, aoff, bias = make_case(g, m, n, k, group, bits, dtype, asym)
    wq = npu_ops.pack_int4_along_k(q_kn) if bits == 4 else q_kn.to(torch.int8)
    want = npu_ops.npu_weight_quant_batchmatmul(x, q_kn, scale, aoff, bias, group)     # the oracle takes unpacked codes [K, N]
    codes_nk = wq.t().contiguous().cuda() if bits == 8 else wq.t().cuda()
    assert codes_nk.is_contiguous()
    st = torch.zeros(1, dtype=torch.int32, device='cuda')
    got = ops().gemm_w4a16(x.cuda(), codes_nk, bits, scale.cuda(), None if aoff is None else aoff.cuda(), group,
                           bias=bias.cuda(), out_dtype=dtype, status=st)
    assert got is not None, 'shape should be taken by the fused kernel'
    ops().raise_if_timed_out(st)
    ref_mag = want.float().abs().max()
    err = ((got.cpu().float() - want.float()).abs().max() / ref_mag).item()
    assert err < TOL_16, err
    # the two-kernel route feeds the MMA the same operand bits: fp32 outputs agree to accumulation order
    w = ops().dequant_weight(codes_nk, bits, scale.cuda(), None if aoff is None else aoff.cuda(), group)
    two = ops().gemm_f16(x.cuda(), w, bias=bias.cuda(), out_dtype=torch.float32)
    one = ops().gemm_w4a16(x.cuda(), codes_nk, bits, scale.cuda(), None if aoff is None else aoff.cuda(), group,
                           bias=bias.cuda(), out_dtype=torch.float32)
    assert float((one - two).abs().max() / two.abs().max()) < 1e-5


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('group,asym', [(128, True), (32, True), (64, False), (0, True)])
@pytest.mark.parametrize('m,n,k', [(1, 16, 128), (5, 130, 384), (8, 1000, 1024), (9, 256, 2048), (16, 408, 1152), (3, 129, 8192)])
def test_streaming_kernel_for_up_to_16_tokens(dtype, group, asym, m, n, k):
    """INT4 weights and at most 16 tokens take the weight-streaming kernel (the K steps of a 16-row tile dealt to four
    warps, their partial sums added in warp order): every step count (K / 128 = 1, 3, 8, 16, 9, 64), ragged and odd N,
    one or two token groups, all group sizes; against the oracle, against the two-kernel route, and bit-identical from run to run."""
    if group and k % group:
        pytest.skip('K is not a multiple of the group')
    g = torch.Generator().manual_seed(m * 5 + n + k + group)
    x, q_kn, scale, aoff, bias = make_case(g, m, n, k, group, 4, dtype, asym)
    wq = npu_ops.pack_int4_along_k(q_kn)
    want = npu_ops.npu_weight_quant_batchmatmul(x, q_kn, scale, aoff, bias, group)
    codes_nk = wq.t().cuda()
    args = (x.cuda(), codes_nk, 4, scale.cuda(), None if aoff is None else aoff.cuda(), group)
    got = ops().gemm_w4a16(*args, bias=bias.cuda(), out_dtype=dtype)
    assert got is not None
    err = ((got.cpu().float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert err < TOL_16, err
    one = ops().gemm_w4a16(*args, bias=bias.cuda(), out_dtype=torch.float32)
    again = ops().gemm_w4a16(*args, bias=bias.cuda(), out_dtype=torch.float32)
    assert torch.equal(one, again)
    w = ops().dequant_weight(codes_nk, 4, scale.cuda(), None if aoff is None else aoff.cuda(), group)
    two = ops().gemm_f16(x.cuda(), w, bias=bias.cuda(), out_dtype=torch.float32)
    assert float((one - two).abs().max() / two.abs().max()) < 3e-5           # fp32 sums of up to 8192 terms in two different orders
    # the fp64 product with the oracle's dequantized weight: the kernel's weights are those values bit for bit
    w_ref = npu_ops.dequant_weight(q_kn, scale, aoff, group, dtype)
    exact = x.double() @ w_ref.double() + bias.double()
    assert float((one.cpu().double() - exact).abs().max() / exact.abs().max()) < 3e-5


def test_fused_w4a16_declines_what_it_cannot_do():
    g = torch.Generator().manual_seed(1)
    x, q_kn, scale, aoff, bias = make_case(g, 4, 64, 96, 32, 4, torch.bfloat16, True)      # K % 64 != 0
    wq = npu_ops.pack_int4_along_k(q_kn)
    assert ops().gemm_w4a16(x.cuda(), wq.t().cuda(), 4, scale.cuda(), aoff.cuda(), 32) is None
    # the shim then takes the two-kernel route and still matches the oracle
    from amct_b200 import torch_npu_shim
    got = torch_npu_shim.npu_weight_quant_batchmatmul(x.cuda(), wq.cuda(), scale.cuda(), antiquant_offset=aoff.cuda(),
                                                      bias=bias.cuda(), antiquant_group_size=32)
    want = npu_ops.npu_weight_quant_batchmatmul(x, q_kn, scale, aoff, bias, 32)
    assert float((got.cpu().float() - want.float()).abs().max() / want.float().abs().max()) < TOL_16


def test_fused_w4a16_config2_shape_checksum():
    """N = 11008, K = 4096, group 128 (the W4A16 benchmark shape), 16 tokens: a column checksum against
    an fp64 product with the oracle's dequantized weight."""
    g = torch.Generator().manual_seed(2)
    m, n, k, group = 16, 11008, 4096, 128
    x, q_kn, scale, aoff, _ = make_case(g, m, n, k, group, 4, torch.bfloat16, True)
    wq = npu_ops.pack_int4_along_k(q_kn)
    got = ops().gemm_w4a16(x.cuda(), wq.t().cuda(), 4, scale.cuda(), aoff.cuda(), group, out_dtype=torch.float32)
    w = npu_ops.dequant_weight(q_kn, scale, aoff, group, torch.bfloat16)            # [K, N]
    want = x.double() @ w.double()
    err = (got.cpu().double() - want).abs().max() / want.abs().max()
    assert float(err) < 1e-5


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('m,n,k', [(3, 128, 128), (70, 200, 320), (256, 384, 1024)])
def test_fused_hif8_weight_gemm(dtype, m, n, k):
    """HiFloat8 weight codes decoded in shared memory ahead of the MMA against decode-then-GEMM."""
    from oracle import hif8
    g = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, k, generator=g).to(dtype)
    w = (torch.randn(n, k, generator=g) * 0.05).to(dtype)
    codes = ops().hif8_encode(w.cuda())
    assert torch.equal(codes.cpu(), torch.from_numpy(hif8.encode(w.float().numpy())))
    bias = torch.randn(n, generator=g).float()
    got = ops().gemm_hif8_weight(x.cuda(), codes, bias=bias.cuda(), out_dtype=torch.float32)
    assert got is not None
    wd = torch.from_numpy(hif8.decode(codes.cpu().numpy()))                   # float32, exactly representable in 16 bits
    want = x.double() @ wd.double().t() + bias.double()
    assert float((got.cpu().double() - want).abs().max() / want.abs().max()) < 1e-5
    two = ops().gemm_f16(x.cuda(), ops().hif8_decode(codes, dtype=dtype), bias=bias.cuda(), out_dtype=torch.float32)
    assert float((got - two).abs().max() / two.abs().max()) < 1e-5
