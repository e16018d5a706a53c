"""GPU parity of the MX (MXFP8-E4M3 / MXFP4-E2M1, E8M0 block scales) kernels through the
C ABI against the CPU restatement of the public MX rule (oracle/mx.py; the reference has no
MX code, so this parity is against the builder's oracle only).  Payloads and scale bytes
must be bit-exact; the block-scaled GEMM is compared within a floating-point tolerance."""
import numpy as np
import pytest
import torch

from oracle import mx

pytestmark = pytest.mark.gpu
GEMM_TOL = 2e-3          # max |got - ref| / max |ref| for the fp32-accumulating tensor-core GEMM


def ops():
    from amct_b200.backend import ops as o
    return o


def tiled_to_rowmajor(tiled, rows, k, tile_rows=128):
    """Undo the scale tiling documented in include/amct_b200.h."""
    kb = k // 32
    kb4 = (kb + 3) // 4
    t = tiled.cpu().numpy()
    r = np.arange(rows)[:, None]
    c = np.arange(kb)[None, :]
    q = r % tile_rows
    atom = (r // tile_rows) * ((tile_rows + 127) // 128) + q // 128
    off = (atom * kb4 + c // 4) * 512 + (q % 32) * 16 + ((q % 128) // 32) * 4 + c % 4
    return torch.from_numpy(t[off])


def padding_is_zero(tiled, rows, k, tile_rows=128):
    """Every byte of the tiled layout that no (row, K block) maps to is zero (the GEMM copies whole atoms)."""
    kb = k // 32
    kb4 = (kb + 3) // 4
    t = tiled.cpu().numpy().copy()
    r = np.arange(rows)[:, None]
    c = np.arange(kb)[None, :]
    q = r % tile_rows
    atom = (r // tile_rows) * ((tile_rows + 127) // 128) + q // 128
    t[(atom * kb4 + c // 4) * 512 + (q % 32) * 16 + ((q % 128) // 32) * 4 + c % 4] = 0
    return not t.any()


def dirty_allocator(nbytes):
    """Leaves a freed block full of 0xAB behind, so that the next torch.empty of that size does not start out zero."""
    junk = torch.full((nbytes,), 0xAB, dtype=torch.uint8).cuda()
    del junk


def make_input(rows, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, k, generator=g) * torch.exp(torch.randn(rows, 1, generator=g) * 3)
    if rows > 3 and k >= 64:
        x[1, :32] = 0                                  # an all-zero block
        x[2, 32:64] *= 1e-30                           # tiny block
        x[3, :32] = x[3, :32].abs() + 300              # values that saturate after scaling
    return x.to(dtype)


@pytest.mark.parametrize('fmt', ['fp8', 'fp4'])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('rows,k', [(1, 32), (5, 96), (130, 256), (257, 1024), (64, 8192)])
def test_mx_quant_matches_oracle(fmt, dtype, rows, k):
    x = make_input(rows, k, dtype, rows * 7 + k)
    want_p, want_s = mx.quantize(x, fmt)
    dirty_allocator(((rows + 127) // 128) * ((k // 32 + 3) // 4) * 512)
    got_p, got_s, got_t = ops().mx_quant(x.cuda(), fmt)
    assert torch.equal(got_s.cpu(), want_s)
    assert torch.equal(got_p.cpu(), want_p)
    assert torch.equal(tiled_to_rowmajor(got_t, rows, k), want_s) and padding_is_zero(got_t, rows, k)
    dirty_allocator(((rows + 223) // 224) * 2 * ((k // 32 + 3) // 4) * 512)
    _, _, got_tb = ops().mx_quant(x.cuda(), fmt, operand='b')
    assert torch.equal(tiled_to_rowmajor(got_tb, rows, k, 224), want_s) and padding_is_zero(got_tb, rows, k, 224)


@pytest.mark.parametrize('fmt', ['fp8', 'fp4'])
def test_mx_quant_nonfinite_blocks(fmt):
    x = make_input(8, 128, torch.float32, 3)
    x[0, 5] = float('nan')
    x[4, 40] = float('inf')
    x[5, 100] = float('-inf')
    want_p, want_s = mx.quantize(x, fmt)
    got_p, got_s, _ = ops().mx_quant(x.cuda(), fmt)
    assert torch.equal(got_s.cpu(), want_s) and int(want_s[0, 0]) == 0xFF
    assert torch.equal(got_p.cpu(), want_p)


def test_mx_roundtrip_properties_full_width():
    """Size-independent properties on a K = 8192 stripe: dequantized values are within half a
    quantization step of the input unless saturated, and re-quantizing them is the identity."""
    x = (torch.randn(512, 8192) * 2).to(torch.bfloat16)
    for fmt in ('fp8', 'fp4'):
        p, s, _ = ops().mx_quant(x.cuda(), fmt)
        deq = mx.dequantize(p.cpu(), s.cpu(), fmt)
        p2, s2, _ = ops().mx_quant(deq.cuda(), fmt)
        assert torch.equal(p2.cpu(), p.cpu()) and torch.equal(s2.cpu(), s.cpu())
        rel = ((deq - x.float()).abs().max() / x.float().abs().max()).item()
        assert rel < (0.13 if fmt == 'fp8' else 0.5)


@pytest.mark.parametrize('fmt', ['fp8', 'fp4'])
@pytest.mark.parametrize('m,n,k', [(128, 224, 256), (7, 40, 512), (300, 520, 1024), (129, 449, 768), (256, 1000, 2048)])
def test_mx_gemm_matches_oracle(fmt, m, n, k):
    if fmt == 'fp4' and k % 256:
        pytest.skip('fp4 needs K % 256 == 0')
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * torch.exp(torch.randn(m, 1, generator=g))).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g) * 0.015).to(torch.bfloat16)
    bias = torch.randn(n, generator=g)
    ap, asr, at = ops().mx_quant(a.cuda(), fmt)
    bp, bsr, bt = ops().mx_quant(b.cuda(), fmt, operand='b')
    want = mx.gemm(ap.cpu(), asr.cpu(), bp.cpu(), bsr.cpu(), fmt) + bias
    st = torch.zeros(1, dtype=torch.int32, device='cuda')
    got = ops().gemm_mx(ap, at, bp, bt, fmt, bias=bias.cuda(), out_dtype=torch.float32, status=st)
    ops().raise_if_timed_out(st)
    err = ((got.cpu() - want).abs().max() / want.abs().max()).item()
    assert err < GEMM_TOL, err
    got16 = ops().gemm_mx(ap, at, bp, bt, fmt, bias=bias.cuda(), out_dtype=torch.bfloat16, status=st)
    err16 = ((got16.cpu().float() - want).abs().max() / want.abs().max()).item()
    assert err16 < 1e-2, err16


@pytest.mark.parametrize('fmt', ['fp8', 'fp4'])
def test_mx_gemm_exact_on_small_integers(fmt):
    """With values that MX represents exactly and sums that fp32 holds exactly, the block-scaled
    GEMM must reproduce the integer matrix product bit for bit -- checks operand order, scale
    addressing (including tiles that start in the middle of a scale atom) and K slicing."""
    g = torch.Generator().manual_seed(1)
    m, n, k = 200, 700, 512
    a = torch.randint(-2, 3, (m, k), generator=g).float() * (2.0 ** torch.randint(-3, 4, (m, 1), generator=g))
    b = torch.randint(-2, 3, (n, k), generator=g).float() * (2.0 ** torch.randint(-3, 4, (n, 1), generator=g))
    ap, asr, at = ops().mx_quant(a.cuda(), fmt)
    bp, bsr, bt = ops().mx_quant(b.cuda(), fmt, operand='b')
    assert torch.equal(mx.dequantize(ap.cpu(), asr.cpu(), fmt), a)
    st = torch.zeros(1, dtype=torch.int32, device='cuda')
    got = ops().gemm_mx(ap, at, bp, bt, fmt, out_dtype=torch.float32, status=st)
    ops().raise_if_timed_out(st)
    assert torch.equal(got.cpu(), a @ b.t())
