"""Generate golden vectors for the offline checkpoint formats by running the REFERENCE on CPU.

    AMCT_REFERENCE=/path/to/amct python tests/golden/make_ckpt_golden.py

Runs the functions of amct_pytorch/experimental/quantization/DeepSeekV3.2/deploy.py (weight_dequant,
int_weight_quant with pack_4bit / scale_fp32_to_u64 / int4_assistance_bias, get_had_pow2, the
quantization_config generators) on seeded inputs, and its main() on a tiny synthetic two-shard checkpoint in a
temporary directory.  Writes ``tests/golden/ckpt_golden.npz`` (inputs and outputs; 16-bit floats and fp8 as raw bit
patterns, the key suffix carries the dtype) and ``tests/golden/ckpt_golden.json`` (generated configs, index files).
The tests need neither the reference nor safetensors' copy of these files.
"""
import io
import contextlib
import json
import os
import sys
import tempfile

import numpy as np
import torch

REF = os.environ.get('AMCT_REFERENCE') or sys.exit('set AMCT_REFERENCE to a checkout of the reference (read only)')
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REF, 'amct_pytorch', 'experimental', 'quantization', 'DeepSeekV3.2'))
import deploy  # noqa: E402  (the reference's script)
from safetensors.torch import load_file, save_file  # noqa: E402

store, meta = {}, {}
TAG = {torch.bfloat16: ('bf16', torch.int16), torch.float16: ('fp16', torch.int16),
       torch.float8_e4m3fn: ('fp8', torch.uint8), torch.uint64: ('u64', torch.int64)}


def put(name, t):
    t = t.detach().cpu().contiguous()
    if t.dtype in TAG:
        tag, view = TAG[t.dtype]
        store[f'{name}|{tag}'] = t.view(view).numpy()
    else:
        store[name] = t.numpy()


def rand(gen, *shape, std=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * std).to(dtype)


def fp8_weight(gen, m, n):
    """Random E4M3 values that include every finite byte pattern at least once when m * n >= 256."""
    raw = torch.randint(0, 256, (m, n), generator=gen, dtype=torch.int32)
    raw.view(-1)[:256] = torch.arange(256, dtype=torch.int32)
    raw[(raw & 0x7F) == 0x7F] = 0x3A                       # no NaN patterns in a checkpoint
    return raw.to(torch.uint8).view(torch.float8_e4m3fn)


def functions():
    torch.set_default_dtype(torch.bfloat16)                 # as the reference's main() does before anything else
    gen = torch.Generator().manual_seed(11)
    for tag, (m, n) in {'ragged': (200, 300), 'even': (256, 128)}.items():
        w = fp8_weight(gen, m, n)
        s = torch.rand((m + 127) // 128, (n + 127) // 128, generator=gen, dtype=torch.float32) * 0.01 + 1e-4
        put(f'dequant.{tag}.w', w)
        put(f'dequant.{tag}.scale', s)
        put(f'dequant.{tag}.out', deploy.weight_dequant(w, s))
    clip = torch.sigmoid(torch.tensor(1.2345, dtype=torch.float32))
    put('clip', clip.reshape(1))
    for dt_name, dt in {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp32': torch.float32}.items():
        w = rand(gen, 38, 512, std=0.05, dtype=dt)
        w[3] *= 37.0                                        # rows of different magnitude
        w[5, 7] = w[5].abs().max() * 1.5                    # a row whose maximum is positive and isolated
        put(f'quant.{dt_name}.w', w)
        for bits in (8, 4):
            for clip_tag, c in {'noclip': None, 'clip': clip}.items():
                q, s, b = deploy.int_weight_quant(w, bits=bits, weight_clip_factor=c)
                put(f'quant.{dt_name}.int{bits}.{clip_tag}.q', q)
                put(f'quant.{dt_name}.int{bits}.{clip_tag}.scale', s)
                if b is not None:
                    put(f'quant.{dt_name}.int{bits}.{clip_tag}.bias', b)
    codes = torch.randint(-8, 8, (10, 48), generator=gen, dtype=torch.int32).to(torch.int8)
    put('pack.codes', codes)
    put('pack.out', deploy.pack_4bit(codes))
    put('had128', deploy.get_had_pow2(128, norm=True))
    put('had8_unnormalised', deploy.get_had_pow2(8, norm=False))
    meta['ignore_5_4_1'] = deploy.generate_ignore_item(5, 4, 1)
    meta['w4a8_layers_5_1'] = deploy.generate_w4a8_quant(5, 1)
    for c8 in (False, True):
        for w4a8 in (False, True):
            for clip_flag in (False, True):
                meta[f'quant_config.c8={c8}.w4a8={w4a8}.clip={clip_flag}'] = deploy.generate_quant_config(
                    c8, ['lm_head'], w4a8=w4a8, clip=clip_flag)


def tiny_checkpoint(gen):
    """name -> tensor for two shards of a made-up three-layer model (2 hidden layers + 1 next-token layer)."""
    def fp8_pair(name, m, n):
        w = fp8_weight(gen, m, n)
        s = torch.rand((m + 127) // 128, (n + 127) // 128, generator=gen, dtype=torch.float32) * 0.02 + 1e-3
        return {name: w, name + '_scale_inv': s}
    a, b = {}, {}
    a['model.embed_tokens.weight'] = rand(gen, 32, 64)
    a.update(fp8_pair('model.layers.0.self_attn.q_a_proj.weight', 96, 256))
    a.update(fp8_pair('model.layers.0.self_attn.q_b_proj.weight', 130, 96))
    a.update(fp8_pair('model.layers.0.mlp.gate_proj.weight', 128, 256))
    a['model.layers.0.input_layernorm.weight'] = rand(gen, 256)
    pair = fp8_pair('model.layers.1.mlp.experts.0.up_proj.weight', 64, 256)
    a['model.layers.1.mlp.experts.0.up_proj.weight'] = pair['model.layers.1.mlp.experts.0.up_proj.weight']
    b['model.layers.1.mlp.experts.0.up_proj.weight_scale_inv'] = pair['model.layers.1.mlp.experts.0.up_proj.weight_scale_inv']
    b['model.layers.1.mlp.gate.weight'] = rand(gen, 8, 256)
    b['model.layers.1.self_attn.o_proj.weight'] = rand(gen, 256, 64, std=0.03)
    b.update(fp8_pair('model.layers.2.eh_proj.weight', 64, 128))
    b['model.layers.2.shared_head.orphan.weight'] = fp8_weight(gen, 16, 32)        # FP8 without a scale_inv tensor
    b['lm_head.weight'] = rand(gen, 32, 256)
    return {'model-00001-of-00002.safetensors': a, 'model-00002-of-00002.safetensors': b}


def end_to_end():
    gen = torch.Generator().manual_seed(12)
    shards = tiny_checkpoint(gen)
    config = {'architectures': ['Tiny'], 'num_hidden_layers': 2, 'num_nextn_predict_layers': 1, 'first_k_dense_replace': 1,
              'quantization_config': {'quant_method': 'fp8', 'weight_block_size': [128, 128]}}
    meta['e2e.config_in'] = config
    meta['e2e.shards'] = {fn: sorted(sd) for fn, sd in shards.items()}
    for fn, sd in shards.items():
        for name, t in sd.items():
            put(f'e2e.in.{name}', t)
    # clip parameters as the calibration step stores them: one file per hidden layer and per directory, raw
    # (pre-sigmoid) values; the next-token layer has none and falls back to factors of 1
    clip_files = {
        'mla': {0: {'self_attn.k_cache_quantizer.clip_factor_a_max': 2.0, 'self_attn.q_b_proj.clip_factor_w_max': 1.5,
                    'self_attn.k_cache_quantizer.clip_factor_a_min': -2.0},
                1: {'self_attn.k_cache_quantizer.clip_factor_a_max': 0.5, 'self_attn.o_proj.clip_factor_w_max': 3.0}},
        'moe': {0: {'mlp.gate_proj.clip_factor_w_max': 0.25, 'mlp.afq_down.clip_factor_a_max': 1.0},
                1: {'mlp.experts.0.up_proj.clip_factor_w_max': 2.5, 'mlp.afq_down.clip_factor_a_max': 4.0}},
    }
    meta['e2e.clip_files'] = {d: {str(k): v for k, v in files.items()} for d, files in clip_files.items()}
    for quant_type, clip in (('bfloat16', False), ('w8a8c16', False), ('w4a8c16', False), ('w8a8c8', True), ('w4a8c8', True)):
        with tempfile.TemporaryDirectory() as src, tempfile.TemporaryDirectory() as dst, tempfile.TemporaryDirectory() as par:
            weight_map = {}
            for fn, sd in shards.items():
                save_file(sd, os.path.join(src, fn), metadata={'format': 'pt'})
                weight_map.update({name: fn for name in sd})
            with open(os.path.join(src, 'model.safetensors.index.json'), 'w') as f:
                json.dump({'metadata': {}, 'weight_map': weight_map}, f)
            with open(os.path.join(src, 'config.json'), 'w') as f:
                json.dump(config, f)
            for d, files in clip_files.items():
                os.makedirs(os.path.join(par, d))
                for layer, params in files.items():
                    torch.save({k: torch.tensor(v, dtype=torch.float32) for k, v in params.items()},
                               os.path.join(par, d, f'quant_parameters_{layer}.pth'))
            with contextlib.redirect_stdout(io.StringIO()):
                deploy.main(src, dst, quant_type, clip, os.path.join(par, 'mla'), os.path.join(par, 'moe'))
            out_files = sorted(fn for fn in os.listdir(dst) if fn.endswith('.safetensors'))
            meta[f'e2e.{quant_type}.files'] = {}
            for fn in out_files:
                sd = load_file(os.path.join(dst, fn), device='cpu')
                meta[f'e2e.{quant_type}.files'][fn] = sorted(sd)
                for name, t in sd.items():
                    put(f'e2e.{quant_type}.out.{name}', t)
            with open(os.path.join(dst, 'model.safetensors.index.json')) as f:
                meta[f'e2e.{quant_type}.index'] = json.load(f)
            with open(os.path.join(dst, 'config.json')) as f:
                meta[f'e2e.{quant_type}.config'] = json.load(f)


if __name__ == '__main__':
    functions()
    end_to_end()
    np.savez_compressed(os.path.join(HERE, 'ckpt_golden.npz'), **store)
    with open(os.path.join(HERE, 'ckpt_golden.json'), 'w') as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print(len(store), 'arrays,', len(meta), 'json entries')
