"""The tiny two-shard FP8 checkpoint of tests/golden/ckpt_golden.*, rebuilt on disk, and the comparison of an
exported directory with what the reference wrote for it (helpers of the CPU and the GPU checkpoint tests)."""
import json
import os

import torch

from golden_io import CKPT_JSON, CKPT_PATH, Golden, bits_equal

QUANT_CASES = (('bfloat16', False), ('w8a8c16', False), ('w4a8c16', False), ('w8a8c8', True), ('w4a8c8', True))


def golden():
    with open(CKPT_JSON) as f:
        meta = json.load(f)
    return Golden(CKPT_PATH), meta


def write_checkpoint(gold, meta, src, par):
    """Writes shards, index, config under ``src`` and the clip-parameter files under ``par``/mla and ``par``/moe."""
    from safetensors.torch import save_file
    weight_map = {}
    for file_name, names in meta['e2e.shards'].items():
        save_file({n: gold.get(f'e2e.in.{n}') for n in names}, os.path.join(src, file_name), metadata={'format': 'pt'})
        weight_map.update({n: file_name for n in names})
    with open(os.path.join(src, 'model.safetensors.index.json'), 'w') as f:
        json.dump({'metadata': {}, 'weight_map': weight_map}, f)
    with open(os.path.join(src, 'config.json'), 'w') as f:
        json.dump(meta['e2e.config_in'], f)
    for directory, files in meta['e2e.clip_files'].items():
        os.makedirs(os.path.join(par, directory), exist_ok=True)
        for layer, params in files.items():
            torch.save({k: torch.tensor(v, dtype=torch.float32) for k, v in params.items()},
                       os.path.join(par, directory, f'quant_parameters_{layer}.pth'))
    return os.path.join(par, 'mla'), os.path.join(par, 'moe')


def compare_export(gold, meta, quant_type, dst):
    """Every output file, tensor (bit for bit), the index and the config against the reference's."""
    from safetensors.torch import load_file
    expected_files = meta[f'e2e.{quant_type}.files']
    written = sorted(fn for fn in os.listdir(dst) if fn.endswith('.safetensors'))
    assert written == sorted(expected_files)
    for file_name in written:
        tensors = load_file(os.path.join(dst, file_name), device='cpu')
        assert sorted(tensors) == expected_files[file_name], file_name
        for name, value in tensors.items():
            assert bits_equal(value, gold.get(f'e2e.{quant_type}.out.{name}')), f'{quant_type}: {name}'
    with open(os.path.join(dst, 'model.safetensors.index.json')) as f:
        assert json.load(f) == meta[f'e2e.{quant_type}.index']
    with open(os.path.join(dst, 'config.json')) as f:
        assert json.load(f) == meta[f'e2e.{quant_type}.config']
