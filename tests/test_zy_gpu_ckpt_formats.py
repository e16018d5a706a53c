"""GPU parity of the offline checkpoint kernels (amct_b200/csrc/ckpt_formats.cu) against the reference's own
outputs (tests/golden/ckpt_golden.*) and, at other shapes, against oracle/ckpt.py; then the whole export through
``deploy.main`` on the tiny two-shard checkpoint, compared file by file with what the reference wrote.

Integer codes, packed nibbles, scale words, bf16 / fp16 values and the 16-bit INT4 bias are compared bit for bit;
the INT4 bias of an fp32 weight is an fp32 sum in a different order from torch's and is held to 1e-6 of the
largest value the sum of magnitudes can take (k * 56 * scale)."""
import ctypes

import pytest
import torch

from ckpt_fixture import QUANT_CASES, compare_export, golden, write_checkpoint
from golden_io import bits_equal
from oracle import ckpt as O

pytestmark = pytest.mark.gpu
GOLD, META = golden()


def ops():
    from amct_b200.backend import ops as o
    return o


def deploy():
    from amct_b200.experimental.quantization.deepseek_v3_2 import deploy as d
    return d


def fp8_weight(gen, m, n):
    raw = torch.randint(0, 256, (m, n), generator=gen, dtype=torch.int32)
    count = min(256, raw.numel())
    raw.view(-1)[:count] = torch.arange(256, dtype=torch.int32)[-count:]   # every bit pattern, NaN included
    return raw.to(torch.uint8).view(torch.float8_e4m3fn)


def same_or_both_nan(got, want):
    got, want = got.cpu(), want.cpu()
    if got.dtype != want.dtype or got.shape != want.shape:
        return False
    g, w = got.float(), want.float()
    nan = torch.isnan(w)
    return bool((torch.isnan(g) == nan).all()) and bits_equal(torch.where(nan, torch.zeros_like(g), g).to(got.dtype),
                                                              torch.where(nan, torch.zeros_like(w), w).to(want.dtype))


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize('tag', ['ragged', 'even'])
def test_block_dequant_golden(tag):
    got = ops().ckpt_block_dequant(GOLD.get(f'dequant.{tag}.w').cuda(), GOLD.get(f'dequant.{tag}.scale').cuda())
    assert bits_equal(got, GOLD.get(f'dequant.{tag}.out'))


@pytest.mark.parametrize('shape', [(256, 7168), (130, 96), (1, 16), (257, 2064), (5, 3)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
def test_block_dequant_oracle(shape, dtype):
    gen = torch.Generator().manual_seed(21)
    m, n = shape
    w = fp8_weight(gen, m, n)
    s = torch.rand((m + 127) // 128, (n + 127) // 128, generator=gen) * 0.02 + 1e-4
    got = ops().ckpt_block_dequant(w.cuda(), s.cuda(), out_dtype=dtype)
    assert same_or_both_nan(got, O.weight_dequant(w, s, 128, dtype))


def test_block_dequant_other_block_and_errors():
    gen = torch.Generator().manual_seed(22)
    w = fp8_weight(gen, 96, 160)
    w.view(torch.uint8)[(w.view(torch.uint8) & 0x7F) == 0x7F] = 0x31
    s = torch.rand(3, 5, generator=gen) + 0.5
    got = ops().ckpt_block_dequant(w.cuda(), s.cuda(), block_size=32)
    assert bits_equal(got, O.weight_dequant(w, s, 32))
    with pytest.raises(AssertionError):
        ops().ckpt_block_dequant(w.cuda(), s[:2].cuda(), block_size=32)


# ---------------------------------------------------------------------------------------------
def words_to_scale(scale_words):
    return (scale_words.cpu().view(torch.int64) & 0xFFFFFFFF).to(torch.int32).view(torch.float32)


def check_quant(got, want, dtype):
    codes, scale, bias = got
    w_codes, w_scale, w_bias = want
    assert bits_equal(codes, w_codes)
    assert bits_equal(scale, w_scale)
    if w_bias is None:
        assert bias is None
    elif dtype == torch.float32:
        # an fp32 sum of k signed terms of at most 56 * scale each, added in another order than torch's
        k = w_codes.shape[1]
        bound = 1e-6 * k * 56.0 * words_to_scale(w_scale).reshape(-1)
        assert bool(((bias.cpu() - w_bias).abs() <= bound).all())
    else:
        assert bits_equal(bias, w_bias)


@pytest.mark.parametrize('dtype', ['bf16', 'fp16', 'fp32'])
@pytest.mark.parametrize('bits', [8, 4])
@pytest.mark.parametrize('clip', ['noclip', 'clip'])
def test_rowquant_golden(dtype, bits, clip):
    w = GOLD.get(f'quant.{dtype}.w')
    factor = float(GOLD.get('clip')) if clip == 'clip' else None
    key = f'quant.{dtype}.int{bits}.{clip}'
    want = (GOLD.get(key + '.q'), GOLD.get(key + '.scale'), GOLD.get(key + '.bias'))
    check_quant(ops().ckpt_rowquant(w.cuda(), bits, factor), want, w.dtype)


@pytest.mark.parametrize('shape', [(64, 7168), (6, 515), (2, 8), (130, 96), (4, 20000)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('bits', [8, 4])
def test_rowquant_oracle(shape, dtype, bits):
    gen = torch.Generator().manual_seed(23)
    n, k = shape
    if bits == 4 and dtype != torch.float32 and k > (8000 if dtype == torch.bfloat16 else 1000):
        pytest.skip('the 16-bit INT4 bias is order independent only below this row length')
    w = torch.randn(n, k, generator=gen) * 0.05
    w[0] *= 40.0
    w[n - 1, k // 2] = 3.0
    w = w.to(dtype)
    clip = torch.sigmoid(torch.tensor(0.7))
    for factor in (None, clip):
        got = ops().ckpt_rowquant(w.cuda(), bits, None if factor is None else float(factor))
        check_quant(got, O.int_weight_quant(w, bits, factor), dtype)


def test_rowquant_strided_rows_zero_row_and_nan():
    gen = torch.Generator().manual_seed(24)
    big = (torch.randn(8, 300, generator=gen) * 0.1).to(torch.bfloat16)
    view = big[:, 4:260]                                   # row stride 300, start not 16-byte aligned
    got = ops().ckpt_rowquant(big.cuda()[:, 4:260], 8)
    check_quant(got, O.int_weight_quant(view.contiguous(), 8), torch.bfloat16)
    w = (torch.randn(4, 128, generator=gen) * 0.1).to(torch.bfloat16)
    w[1] = 0
    w[2, 7] = float('nan')
    codes, scale, _ = ops().ckpt_rowquant(w.cuda(), 8)
    assert int(codes[1].abs().sum()) == 0 and float(scale[1]) == 0.0       # 0 / 0 -> code 0
    assert int(codes[2].abs().sum()) == 0 and bool(torch.isnan(scale[2]))  # torch.max propagates NaN
    want = O.int_weight_quant(w[[0, 3]], 8)
    assert bits_equal(codes[[0, 3]], want[0]) and bits_equal(scale[[0, 3]], want[1])


@pytest.mark.parametrize('shape', [(128, 7168), (130, 96), (6, 200), (258, 2064)])
@pytest.mark.parametrize('bits', [8, 4])
def test_fused_dequant_rowquant(shape, bits):
    """One pass over the FP8 weight gives exactly what dequantize-then-quantize gives (the reference's two steps), for
    bf16 and fp16 intermediates, with and without a clip factor, on the vector and the element-wise path."""
    gen = torch.Generator().manual_seed(27)
    m, n = shape
    w = fp8_weight(gen, m, n)
    w.view(torch.uint8)[(w.view(torch.uint8) & 0x7F) == 0x7F] = 0x2C                # a checkpoint holds no NaN
    s = torch.rand((m + 127) // 128, (n + 127) // 128, generator=gen) * 0.02 + 1e-4
    clip = torch.sigmoid(torch.tensor(1.1))
    for dtype in (torch.bfloat16, torch.float16):
        if bits == 4 and n > (8000 if dtype == torch.bfloat16 else 1000):
            continue                                                               # bias order dependent beyond this
        for factor in (None, clip):
            got = ops().ckpt_dequant_rowquant(w.cuda(), s.cuda(), bits, None if factor is None else float(factor), dtype=dtype)
            check_quant(got, O.int_weight_quant(O.weight_dequant(w, s, 128, dtype), bits, factor), dtype)
    two_steps = ops().ckpt_rowquant(ops().ckpt_block_dequant(w.cuda(), s.cuda()), bits)
    fused = ops().ckpt_dequant_rowquant(w.cuda(), s.cuda(), bits)
    for a, b in zip(fused, two_steps):
        assert bits_equal(a, b)


def test_rowquant_argument_errors():
    w = torch.zeros(3, 16, dtype=torch.bfloat16, device='cuda')
    with pytest.raises(ValueError):
        ops().ckpt_rowquant(w, 4)                          # odd number of output channels
    with pytest.raises(ValueError):
        ops().ckpt_rowquant(w, 2)
    from amct_b200.backend import lib
    out = torch.zeros(3, 16, dtype=torch.int8, device='cuda')
    scale = torch.zeros(3, dtype=torch.int64, device='cuda')
    bias = torch.zeros(3, dtype=torch.float32, device='cuda')
    p = lambda t: ctypes.c_void_p(t.data_ptr())                                     # noqa: E731
    rc = lib.load().amct_ckpt_rowquant(p(w), ctypes.c_int(2), ctypes.c_int64(3), ctypes.c_int64(16), ctypes.c_int64(16),
                                       ctypes.c_int(4), ctypes.c_int(0), ctypes.c_float(1.0), p(out), ctypes.c_int64(16),
                                       p(scale), p(bias), ctypes.c_void_p(0))
    assert rc == -1


# ---------------------------------------------------------------------------------------------
def test_pack4_bias_scale_words_hadamard():
    assert bits_equal(ops().ckpt_pack4_rows(GOLD.get('pack.codes').cuda()), GOLD.get('pack.out'))
    gen = torch.Generator().manual_seed(25)
    codes = torch.randint(-8, 8, (34, 777), generator=gen, dtype=torch.int32).to(torch.int8)
    assert bits_equal(ops().ckpt_pack4_rows(codes.cuda()), O.pack_4bit(codes))
    codes = torch.randint(-7, 8, (12, 768), generator=gen, dtype=torch.int32).to(torch.int8)
    for dtype in (torch.bfloat16, torch.float16):
        scale = (torch.rand(12, 1, generator=gen) * 0.01 + 1e-4).to(dtype)
        want = O.int4_assistance_bias(codes, scale.float(), dtype)
        assert bits_equal(ops().ckpt_int4_bias(codes.cuda(), scale.cuda()), want)
        scale3 = (torch.rand(12, 3, generator=gen) * 0.01 + 1e-4).to(dtype)
        want = O.int4_assistance_bias(codes, scale3.float().repeat_interleave(256, dim=1), dtype)
        assert bits_equal(ops().ckpt_int4_bias(codes.cuda(), scale3.cuda()), want)
    s = torch.rand(9, 2, generator=gen)
    assert bits_equal(deploy().scale_fp32_to_u64(s.cuda()), O.scale_fp32_to_u64(s))
    assert bits_equal(ops().hadamard_pow2(128, True, torch.bfloat16), GOLD.get('had128'))
    assert bits_equal(ops().hadamard_pow2(8, False, torch.bfloat16), GOLD.get('had8_unnormalised'))
    for dtype in (torch.float16, torch.float32):
        assert bits_equal(ops().hadamard_pow2(64, True, dtype), O.get_had_pow2(64, True, dtype))
    h = ops().hadamard_pow2(256, True, torch.float32).double()
    assert torch.allclose(h @ h.T, torch.eye(256, dtype=torch.float64, device=h.device), atol=1e-5)
    with pytest.raises(ValueError):
        ops().hadamard_pow2(12)


def test_full_size_properties():
    """An expert-sized weight (2048 x 7168): dequant -> INT8 -> dequantized codes stay within half a step of the
    bf16 weight, and packing two INT4 rows then unpacking the nibbles returns the codes."""
    gen = torch.Generator().manual_seed(26)
    m, n = 2048, 7168
    raw = torch.randint(0, 256, (m, n), generator=gen, dtype=torch.int32)
    raw[(raw & 0x7F) == 0x7F] = 0x3A
    w8 = raw.to(torch.uint8).view(torch.float8_e4m3fn).cuda()
    s = (torch.rand(m // 128, n // 128, generator=gen) * 0.01 + 1e-3).cuda()
    bf = ops().ckpt_block_dequant(w8, s)
    codes, scale, _ = ops().ckpt_rowquant(bf, 8)
    assert int(codes.abs().max()) <= 127
    err = (codes.float() * scale - bf.float()).abs()
    # one bf16 rounding of the quotient (2^-8 relative at |q| <= 127) on top of the half step
    assert bool((err <= scale * 1.01).all())
    packed, scale_words, bias = ops().ckpt_rowquant(bf, 4)
    lo = (packed.to(torch.int32) << 28) >> 28
    hi = (packed.to(torch.int32) << 24) >> 28
    scale4 = words_to_scale(scale_words).to(bf.device)
    level = torch.round((bf.float() / scale4).to(torch.bfloat16).float()).clamp(-7, 7).to(torch.int32)
    assert bool((lo == level[0::2]).all()) and bool((hi == level[1::2]).all())
    assert bool((scale_words.view(torch.int64) >> 32 == 0).all())
    assert bits_equal(ops().ckpt_pack4_rows(level.to(torch.int8)), packed)
    assert bits_equal(ops().ckpt_int4_bias(level.to(torch.int8), scale4.to(torch.bfloat16)), bias)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize('quant_type,clip', QUANT_CASES)
def test_export_end_to_end(quant_type, clip, tmp_path):
    src, dst, par = tmp_path / 'src', tmp_path / 'dst', tmp_path / 'par'
    src.mkdir()
    mla, moe = write_checkpoint(GOLD, META, str(src), str(par))
    deploy().main(str(src), str(dst), quant_type, clip, mla, moe, device='cuda')
    compare_export(GOLD, META, quant_type, str(dst))
