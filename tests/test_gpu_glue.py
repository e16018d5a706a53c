"""GPU parity of the decoder-layer glue kernels (residual add + RMSNorm + per-token quant in one
pass; in-place rotary embedding), called through the C ABI, and of the workload that uses them.

The add and the codes / scales are bit-exact; the normalised values are within one unit in the
last place of the oracle's (the fp32 sum of squares is order dependent), and the codes are
bit-exact with the oracle quantizer applied to the kernel's own normalised values."""
import pytest
import torch
import torch.nn.functional as F

from golden_io import bits_equal
from oracle import intq

pytestmark = pytest.mark.gpu


def ops():
    from amct_b200.backend import ops as o
    return o


def ulp_distance(a, b):
    """Distance in units of the last place between two 16-bit float tensors of equal dtype."""
    ia = a.contiguous().view(torch.int16).to(torch.int32)
    ib = b.contiguous().view(torch.int16).to(torch.int32)
    ia = torch.where(ia < 0, -(ia & 0x7fff), ia)
    ib = torch.where(ib < 0, -(ib & 0x7fff), ib)
    return (ia - ib).abs()


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('rows,k', [(1, 8), (3, 1000), (64, 1024), (257, 2048), (130, 4096), (100, 8192), (17, 8200), (9, 16384)])
@pytest.mark.parametrize('with_res', [True, False])
def test_addnorm_quant_matches_oracle(dtype, rows, k, with_res):
    g = torch.Generator().manual_seed(rows * 131 + k)
    x = (torch.randn(rows, k, generator=g) * 1.7).to(dtype)
    res = (torch.randn(rows, k, generator=g) * 3.1).to(dtype) if with_res else None
    gamma = (1 + 0.1 * torch.randn(k, generator=g)).to(dtype)
    if rows > 2:
        x[1] = -x[1].abs()                       # negative-dominant row: divisor 128 and the clamp at 127
        if with_res:
            res[1] = -res[1].abs()
        x[2] = 0                                 # all-zero row without residual: scale becomes 1
    eps = 1e-5
    q, scale, h, n = ops().addnorm_quant_per_token(x.cuda(), gamma.cuda(), eps, residual=None if res is None else res.cuda(),
                                                   want_norm=True, check=True)
    ho, no, _, _ = intq.addnorm_dynamic_per_token(x, gamma, eps, res)
    if with_res:
        assert bits_equal(h, ho)
    else:
        assert h is None
    d = ulp_distance(n.cpu(), no)
    assert int(d.max()) <= 1
    assert float((d > 0).float().mean()) < 0.02
    # codes and scales: exactly the quantizer of the normalised values this kernel produced
    qo, so = intq.dynamic_per_token(n.cpu())
    assert bits_equal(scale, so)
    assert bits_equal(q, qo)
    # and the separate kernel agrees on the same input
    q2, s2 = ops().quant_dynamic_per_token(n)
    assert bits_equal(q2, q) and bits_equal(s2, scale)
    # torch's own rms_norm on the device is within one unit in the last place as well
    nt = F.rms_norm(h if with_res else x.cuda(), (k,), gamma.cuda(), eps)
    assert int(ulp_distance(n, nt).max()) <= 2


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('n_parts,rows,k,world', [(1, 5, 1024, 2), (2, 33, 2048, 2), (4, 20, 8192, 4), (8, 9, 4096, 8), (3, 7, 520, 3)])
@pytest.mark.parametrize('with_res', [True, False])
def test_addnorm_quant_tp_sums_parts_and_stores_to_every_rank(dtype, n_parts, rows, k, world, with_res):
    """The tensor-parallel form: x = fp32 sum of the staged partial sums in rank order, rounded once; after that the
    very arithmetic of addnorm_quant_per_token (so codes and scales are bit-identical to that kernel on the summed
    rows); codes and scales are stored into row0 + r of every rank's buffer (here: separate local tensors)."""
    g = torch.Generator().manual_seed(n_parts * 1000 + rows * 7 + k)
    parts = (torch.randn(n_parts, rows, k, generator=g) * 1.3).to(dtype)
    res = (torch.randn(rows, k, generator=g) * 2.0).to(dtype) if with_res else None
    gamma = (1 + 0.1 * torch.randn(k, generator=g)).to(dtype)
    acc = parts[0].float()
    for j in range(1, n_parts):
        acc = acc + parts[j].float()
    x_sum = acc.to(dtype)
    eps, row0, total = 1e-5, 3, rows + 11
    q_ref, s_ref, h_ref, _ = ops().addnorm_quant_per_token(x_sum.cuda(), gamma.cuda(), eps, residual=None if res is None else res.cuda())
    q_bufs = [torch.full((total, k), 99, dtype=torch.int8).cuda() for _ in range(world)]
    s_bufs = [torch.full((total,), -1.0, dtype=torch.float32).cuda() for _ in range(world)]
    h = ops().addnorm_quant_per_token_tp(parts.cuda(), gamma.cuda(), eps, [t.data_ptr() for t in q_bufs],
                                         [t.data_ptr() for t in s_bufs], row0, residual=None if res is None else res.cuda())
    if with_res:
        assert bits_equal(h, h_ref) and bits_equal(h, x_sum + res)
    else:
        assert h is None
    for d in range(world):
        assert bits_equal(q_bufs[d][row0:row0 + rows], q_ref) and bits_equal(s_bufs[d][row0:row0 + rows], s_ref)
        assert bool((q_bufs[d][:row0] == 99).all()) and bool((q_bufs[d][row0 + rows:] == 99).all())
        assert bool((s_bufs[d][:row0] == -1).all()) and bool((s_bufs[d][row0 + rows:] == -1).all())


def test_addnorm_quant_strided_and_batched():
    g = torch.Generator().manual_seed(5)
    big = torch.randn(4, 6, 2048 + 64, generator=g).to(torch.bfloat16).cuda()
    x = big[..., :2048]                                   # row stride larger than K
    res = torch.randn(4, 6, 2048, generator=g).to(torch.bfloat16).cuda()
    gamma = torch.ones(2048, dtype=torch.bfloat16).cuda()
    q, scale, h, n = ops().addnorm_quant_per_token(x, gamma, 1e-6, residual=res, want_norm=True)
    assert q.shape == x.shape and h.shape == x.shape and scale.shape == (24,)
    assert bits_equal(h, (x + res))
    qo, so = intq.dynamic_per_token(n.cpu())
    assert bits_equal(q, qo) and bits_equal(scale, so)


def test_addnorm_quant_flags_nan_rows():
    x = torch.randn(8, 1024).to(torch.bfloat16)
    x[3, 17] = float('nan')
    with pytest.raises(RuntimeError, match='invalid value'):
        ops().addnorm_quant_per_token(x.cuda(), torch.ones(1024, dtype=torch.bfloat16).cuda(), 1e-5, check=True)


def test_addnorm_quant_rejects_what_it_cannot_do():
    from amct_b200.backend.lib import BackendError
    x = torch.randn(4, 1024).cuda()
    with pytest.raises(BackendError):
        ops().addnorm_quant_per_token(x, torch.ones(1024).cuda(), 1e-5)               # fp32
    xb = torch.randn(4, 1028).to(torch.bfloat16).cuda()
    with pytest.raises(BackendError):
        ops().addnorm_quant_per_token(xb, torch.ones(1028).cuda(), 1e-5)              # K % 8 != 0
    xl = torch.randn(2, 16392).to(torch.bfloat16).cuda()
    with pytest.raises(BackendError):
        ops().addnorm_quant_per_token(xl, torch.ones(16392).cuda(), 1e-5)             # K too long


def rotary_torch(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('b,s,heads,kv,hd', [(2, 5, 4, 2, 128), (1, 300, 8, 1, 64), (3, 64, 64, 8, 128), (1, 1, 2, 2, 32)])
def test_rope_inplace_bit_identical_to_torch_ops(dtype, b, s, heads, kv, hd):
    g = torch.Generator().manual_seed(b * 7 + s)
    ld = (heads + 2 * kv) * hd
    qkv = torch.randn(b, s, ld, generator=g).to(dtype).cuda()
    ang = torch.arange(s, dtype=torch.float32)[:, None] * (1.0 / (10000 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd)))[None, :]
    cos, sin = ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda()
    want_qk = rotary_torch(qkv[..., :(heads + kv) * hd].reshape(b, s, heads + kv, hd), cos, sin).reshape(b, s, -1)
    want_v = qkv[..., (heads + kv) * hd:].clone()
    ops().rope_inplace(qkv, heads + kv, hd, cos, sin)
    assert bits_equal(qkv[..., :(heads + kv) * hd].contiguous(), want_qk)
    assert bits_equal(qkv[..., (heads + kv) * hd:].contiguous(), want_v)            # values untouched


def test_workload_fused_glue_matches_unfused_layers():
    """Two-layer Llama-shaped stack: fused glue kernels against the torch-op glue on the same weights."""
    from amct_b200.workloads.llama_tp import LlamaW8A8, LlamaShape
    shape = LlamaShape(hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, intermediate=2048, n_layers=2, vocab=512)
    ids = torch.randint(0, 512, (2, 48), generator=torch.Generator().manual_seed(3)).cuda()
    outs = {}
    for name, kw in {'fused': dict(fused_glue=True), 'unfused': dict(fused_glue=False)}.items():
        outs[name] = LlamaW8A8(shape, device='cuda', seed=11, **kw)(ids)
    ref = outs['unfused']
    err = (outs['fused'] - ref).abs().max() / ref.abs().max()
    assert float(err) < 2e-2            # bf16 tolerance: one-ulp differences in the norm move a few codes by one
    # decode step with an in-place KV cache goes through the same kernels
    m = LlamaW8A8(shape, device='cuda', seed=11)
    caches = [(torch.zeros(2, 2, 64, 128, dtype=torch.bfloat16, device='cuda'),
               torch.zeros(2, 2, 64, 128, dtype=torch.bfloat16, device='cuda'), 0) for _ in range(2)]
    full = m(ids)
    pre = m(ids[:, :47], kv_caches=caches)
    caches = [(k, v, 47) for k, v, _ in caches]
    step = m(ids[:, 47:], kv_caches=caches, past_len=47)
    assert pre.shape == full.shape
    assert float((step - full).abs().max() / full.abs().max()) < 3e-2
