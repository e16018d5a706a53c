"""One Llama-3-8B decoder layer whose seven Linears are HiFloat8 (weights and activations) behind SmoothQuant factors.

The workload: random-init weights (normal, std 0.02; RMSNorm weights 1) and a random embedding table; a calibration
pass over 128 random token sequences feeds every Linear's per-channel activation maximum to ``quantize()`` with the
'hifloat8' algorithm and smooth_strength 0.5 (the factor rule of
amct_pytorch/quantize_op/smooth_quant_module.py:113-133: s = amax_x^a / amax_w^(1-a), applied to the weight as in
amct_pytorch/utils/quant_util.py:96-111 and to the activations as its reciprocal); ``convert()`` then leaves seven
HiFloat8Linear deploy modules, and the evaluation pass runs batch 8 x 2048 tokens through the layer.

The layer is built from plain torch modules (q / k / v / o / gate / up / down are separate nn.Linear, as in the
architecture) so that the public quantize() / convert() entry points do all the work; attention, rotary embedding,
SiLU and the norms are torch ops (not part of the quantized-Linear path).
"""
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

import amct_b200 as amct

from .llama_tp import LLAMA3_8B, rotary_tables, apply_rotary

HIF8_SMOOTH_CFG = {
    'quant_cfg': {'weights': {'type': 'hifloat8', 'symmetric': True, 'strategy': 'channel'},
                  'inputs': {'type': 'hifloat8', 'symmetric': True, 'strategy': 'tensor'}},
    'algorithm': {'hifloat8': {'smooth_strength': 0.5}},
}

LINEARS = ('q_proj', 'k_proj', 'v_proj', 'o_proj', 'gate_proj', 'up_proj', 'down_proj')


class LlamaLayer(nn.Module):
    """Pre-norm decoder layer: x + attn(norm(x)), then x + mlp(norm(x)); grouped-query attention, SwiGLU."""

    def __init__(self, shape=LLAMA3_8B, device='cuda', seed=3, dtype=torch.bfloat16):
        super().__init__()
        self.shape = shape
        gen = torch.Generator(device=device).manual_seed(seed)
        h, d = shape.hidden, shape.head_dim

        def lin(k, n):
            m = nn.Linear(k, n, bias=False, device=device, dtype=dtype)
            m.weight.data.normal_(0, 0.02, generator=gen)
            m.weight.requires_grad_(False)
            return m

        self.q_proj, self.k_proj, self.v_proj = lin(h, shape.n_heads * d), lin(h, shape.n_kv_heads * d), lin(h, shape.n_kv_heads * d)
        self.o_proj = lin(shape.n_heads * d, h)
        self.gate_proj, self.up_proj, self.down_proj = lin(h, shape.intermediate), lin(h, shape.intermediate), lin(shape.intermediate, h)
        self.input_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device), requires_grad=False)
        self.post_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device), requires_grad=False)

    @torch.no_grad()
    def forward(self, x, cos, sin):
        shp = self.shape
        b, s, _ = x.shape
        hn = F.rms_norm(x, (shp.hidden,), self.input_norm, shp.rms_eps)
        q = apply_rotary(self.q_proj(hn).reshape(b, s, shp.n_heads, shp.head_dim), cos, sin).transpose(1, 2)
        k = apply_rotary(self.k_proj(hn).reshape(b, s, shp.n_kv_heads, shp.head_dim), cos, sin).transpose(1, 2)
        v = self.v_proj(hn).reshape(b, s, shp.n_kv_heads, shp.head_dim).transpose(1, 2)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.o_proj(attn.transpose(1, 2).reshape(b, s, -1))
        hn = F.rms_norm(x, (shp.hidden,), self.post_norm, shp.rms_eps)
        return x + self.down_proj(F.silu(self.gate_proj(hn)) * self.up_proj(hn))


@dataclass
class HiF8LayerWorkload:
    layer: LlamaLayer
    embed: torch.Tensor
    calib_tokens: int
    calib_seq: int

    def __call__(self, ids):
        """ids [B, S] -> hidden states [B, S, hidden] after the layer."""
        cos, sin = rotary_tables(self.layer.shape, torch.arange(ids.shape[1], device=ids.device), ids.device)
        return self.layer(F.embedding(ids, self.embed), cos, sin)

    def linear_flops_per_token(self):
        sh = self.layer.shape
        d = sh.head_dim
        return 2 * (sh.hidden * (sh.n_heads + 2 * sh.n_kv_heads) * d + sh.n_heads * d * sh.hidden + 3 * sh.hidden * sh.intermediate)


def build(shape=LLAMA3_8B, device='cuda', seed=3, calib_sequences=128, calib_seq=2048, calib_batch=8, vocab=None):
    """Random-init layer -> quantize() with SmoothQuant (a = 0.5) + HiFloat8 -> calibration over `calib_sequences`
    random sequences of `calib_seq` tokens, `calib_batch` at a time -> convert().  Returns the workload; its seven
    Linears are HiFloat8Linear modules."""
    vocab = vocab or shape.vocab
    layer = LlamaLayer(shape, device, seed)
    gen = torch.Generator(device=device).manual_seed(seed + 1)
    embed = torch.empty(vocab, shape.hidden, dtype=torch.bfloat16, device=device).normal_(0, 0.02, generator=gen)
    if calib_sequences % calib_batch:
        raise ValueError('calib_sequences must be a multiple of calib_batch')
    batches = calib_sequences // calib_batch
    cfg = dict(HIF8_SMOOTH_CFG, batch_num=batches)
    amct.quantize(layer, cfg)
    work = HiF8LayerWorkload(layer, embed, calib_sequences * calib_seq, calib_seq)
    ids_gen = torch.Generator().manual_seed(seed)
    for _ in range(batches):
        ids = torch.randint(0, vocab, (calib_batch, calib_seq), generator=ids_gen).to(device)
        work(ids)
    amct.convert(layer)
    for name in LINEARS:
        if type(getattr(layer, name)).__name__ != 'HiFloat8Linear':
            raise RuntimeError(f'{name} was not converted: {type(getattr(layer, name)).__name__}')
    return work
