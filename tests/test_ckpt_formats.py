"""Offline checkpoint formats on the CPU: the oracle against the reference's outputs (tests/golden/ckpt_golden.*),
and the host side of the export (which tensor gets which treatment, clip-factor files, config block, index)
against the same fixtures.  The end-to-end host test swaps the CUDA tensor steps of the export module for the
oracle's -- only here, by monkeypatching; the module itself has no CPU implementation."""
import json

import pytest
import torch

from ckpt_fixture import QUANT_CASES, compare_export, golden, write_checkpoint
from golden_io import bits_equal
from oracle import ckpt as O

GOLD, META = golden()


@pytest.mark.parametrize('tag', ['ragged', 'even'])
def test_oracle_block_dequant(tag):
    out = O.weight_dequant(GOLD.get(f'dequant.{tag}.w'), GOLD.get(f'dequant.{tag}.scale'))
    assert bits_equal(out, GOLD.get(f'dequant.{tag}.out'))


@pytest.mark.parametrize('dtype', ['bf16', 'fp16', 'fp32'])
@pytest.mark.parametrize('bits', [8, 4])
@pytest.mark.parametrize('clip', ['noclip', 'clip'])
def test_oracle_int_weight_quant(dtype, bits, clip):
    w = GOLD.get(f'quant.{dtype}.w')
    codes, scale, bias = O.int_weight_quant(w, bits, GOLD.get('clip') if clip == 'clip' else None)
    key = f'quant.{dtype}.int{bits}.{clip}'
    assert bits_equal(codes, GOLD.get(key + '.q'))
    assert bits_equal(scale, GOLD.get(key + '.scale'))
    if bits == 4:
        if dtype == 'fp32':       # an fp32 sum: the order of the additions shows in the last bits
            torch.testing.assert_close(bias, GOLD.get(key + '.bias'), rtol=1e-5, atol=0)
        else:
            assert bits_equal(bias, GOLD.get(key + '.bias'))
    else:
        assert bias is None


def test_oracle_pack_and_hadamard():
    assert bits_equal(O.pack_4bit(GOLD.get('pack.codes')), GOLD.get('pack.out'))
    assert bits_equal(O.get_had_pow2(128), GOLD.get('had128'))
    assert bits_equal(O.get_had_pow2(8, norm=False), GOLD.get('had8_unnormalised'))
    with pytest.raises(ValueError):
        O.get_had_pow2(12)


def test_oracle_zero_row_and_bias_exactness():
    w = torch.zeros(2, 64, dtype=torch.bfloat16)
    w[1, 5] = -3.0
    codes, scale, _ = O.int_weight_quant(w, 8)
    assert codes[0].abs().sum() == 0 and float(scale[0]) == 0.0 and int(codes[1, 5]) <= -126   # bf16 steps
    # the INT4 bias of a 16-bit row is exact in fp32, so any summation order gives the same bits
    gen = torch.Generator().manual_seed(3)
    w = (torch.randn(4, 4096, generator=gen) * 0.05).to(torch.bfloat16)
    _, scale_u64, bias = O.int_weight_quant(w, 4)
    scale = (scale_u64.view(torch.int64) & 0xFFFFFFFF).to(torch.int32).view(torch.float32)
    level = torch.round((w.float() / scale).to(torch.bfloat16).float()).clamp(-7, 7)
    term = ((scale * level).to(torch.bfloat16).float() * 8).to(torch.bfloat16).double()
    assert bits_equal(bias, term.flip(1).sum(1).float().to(torch.bfloat16).float())


# ---------------------------------------------------------------------------------------------
# host side of amct_b200.experimental.quantization.deepseek_v3_2.deploy
# ---------------------------------------------------------------------------------------------
from amct_b200.experimental.quantization.deepseek_v3_2 import deploy as D  # noqa: E402


def test_config_generators_match_reference():
    assert D.generate_ignore_item(5, 4, 1) == META['ignore_5_4_1']
    assert D.generate_w4a8_quant(5, 1) == META['w4a8_layers_5_1']
    for c8 in (False, True):
        for w4a8 in (False, True):
            for clip in (False, True):
                made = D.generate_quant_config(c8, ['lm_head'], w4a8=w4a8, clip=clip)
                assert made == META[f'quant_config.c8={c8}.w4a8={w4a8}.clip={clip}']
                assert json.loads(json.dumps(made)) == made


@pytest.mark.parametrize('quant_type,clip', QUANT_CASES)
def test_export_plan_names(quant_type, clip):
    """The plan alone reproduces which names each output shard holds (before the extra tensors of c8)."""
    plan = D.ExportPlan(META['e2e.config_in'], quant_type, clip)
    in_index = {n for names in META['e2e.shards'].values() for n in names}
    extras = ('hadamard_matrix', 'alpha')
    for file_name, names in META['e2e.shards'].items():
        produced = []
        for n in names:
            size = GOLD.get(f'e2e.in.{n}').element_size()
            produced += plan.output_names(n, plan.action(n, size, f'{n}_scale_inv' in in_index))
        expected = [n for n in META[f'e2e.{quant_type}.files'][file_name] if not n.endswith(extras)]
        assert sorted(produced) == expected
    assert plan.config == META[f'e2e.{quant_type}.config']


def test_export_plan_refuses_what_the_reference_cannot_finish():
    with pytest.raises(ValueError):
        D.ExportPlan(META['e2e.config_in'], 'w8a8c8', clip=False)
    with pytest.raises(ValueError):
        D.ExportPlan(META['e2e.config_in'], 'w8a8c16', clip=True)
    with pytest.raises(AssertionError):
        D.ExportPlan(META['e2e.config_in'], 'w2a8', clip=False)


def test_clip_factor_conversion(tmp_path):
    mla, moe = write_checkpoint(GOLD, META, str(tmp_path), str(tmp_path / 'par'))
    kv, act, weight = D.load_clip_params(2, 1, mla, moe)
    assert sorted(kv) == [f'model.layers.{i}.self_attn.ckv_a_alpha' for i in range(3)]
    assert float(kv['model.layers.2.self_attn.ckv_a_alpha']) == 1.0          # next-token layer: factor 1
    assert float(kv['model.layers.0.self_attn.ckv_a_alpha']) == float(torch.sigmoid(torch.tensor(2.0)))
    assert sorted(act) == [f'model.layers.{i}.mlp.down_proj.alpha' for i in range(3)]
    assert float(act['model.layers.1.mlp.down_proj.alpha']) == float(torch.sigmoid(torch.tensor(10.0)))
    assert 'model.layers.0.self_attn.q_b_proj.w_alpha' in weight and 'model.layers.1.mlp.experts.0.up_proj.w_alpha' in weight
    with pytest.raises(ValueError):
        D.load_clip_params(3, 0, mla, moe)                                    # a hidden layer without its file


@pytest.mark.parametrize('quant_type,clip', QUANT_CASES)
def test_export_host_logic_end_to_end(quant_type, clip, tmp_path, monkeypatch):
    """main() with the oracle standing in for the three CUDA steps: files, tensors, index and config as the
    reference wrote them."""
    def dequant(weight, scale, block_size=128):
        return O.weight_dequant(weight, scale, block_size, torch.get_default_dtype())

    def quant(tensor, bits=8, weight_clip_factor=None):
        factor = None if weight_clip_factor is None else torch.tensor(float(weight_clip_factor), dtype=torch.float32)
        return O.int_weight_quant(tensor, bits, factor)

    def hadamards(num_layers, dim=128, device='cpu'):
        had = O.get_had_pow2(dim, True, torch.get_default_dtype()).to(torch.bfloat16)
        return {f'model.layers.{i}.self_attn.indexer.hadamard_matrix': had.clone() for i in range(num_layers)}

    def dequant_quant(weight, scale, bits=8, weight_clip_factor=None, block_size=128):
        return quant(dequant(weight, scale, block_size), bits, weight_clip_factor)

    monkeypatch.setattr(D, 'weight_dequant', dequant)
    monkeypatch.setattr(D, 'int_weight_quant', quant)
    monkeypatch.setattr(D, 'dequant_int_weight_quant', dequant_quant)
    monkeypatch.setattr(D, 'generate_li_hadamard_matrix', hadamards)
    src, dst, par = tmp_path / 'src', tmp_path / 'dst', tmp_path / 'par'
    src.mkdir()
    mla, moe = write_checkpoint(GOLD, META, str(src), str(par))
    before = torch.get_default_dtype()
    D.main(str(src), str(dst), quant_type, clip, mla, moe, device='cpu')
    assert torch.get_default_dtype() == before
    compare_export(GOLD, META, quant_type, str(dst))
