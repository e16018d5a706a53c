"""Offline checkpoint export: FP8 block-scaled checkpoint -> bf16 / W8A8 / W4A8 compressed-tensors checkpoint.

Drop-in for ``amct_pytorch/experimental/quantization/DeepSeekV3.2/deploy.py`` ("deploy.py" below): the same
function names, arguments and results, the same ``main`` and command line.  The tensor work -- the 128 x 128
block dequantization of FP8 weights, the per-output-channel INT8 / INT4 quantization with nibble packing, the
uint64 scale words, the INT4 assistance bias and the Hadamard matrix -- runs as CUDA kernels
(``amct_b200/csrc/ckpt_formats.cu``) on tensors moved to the GPU shard by shard; there is no CPU implementation
of these steps here, so a machine without the kernel library fails on the first call.  What stays on the host is
what the reference's script does around the tensors: which weight gets which treatment, the clip-factor files,
the ``quantization_config`` block, the index.

Differences from the reference, all deliberate:
  * ``main`` sets torch's default dtype to bfloat16 like the reference (deploy.py:357) but only for its own
    duration; the previous default is restored on return.
  * ``--clip`` without a ``c8`` quant type, and a ``c8`` quant type without ``--clip``, both end in a NameError
    in the reference (deploy.py:414-416 defines the clip tables only for the two together, :448 and :543 use
    them regardless); here they are refused up front with a ValueError that says so.
"""
import json
import os
import re
import shutil
from argparse import ArgumentParser
from glob import glob

import torch

from ....backend import ops as _ops

QUANT_TYPES = ('bfloat16', 'w8a8c16', 'w8a8c8', 'w4a8c16', 'w4a8c8')           # deploy.py:360-361
_QUANTIZED_PLAIN = re.compile('(gate|up|down|o|q_b)_proj')                     # deploy.py:484


# ---------------------------------------------------------------------------------------------
# tensor steps (CUDA)
# ---------------------------------------------------------------------------------------------
def get_had_pow2(n, norm=True, device='cuda'):
    """n x n Hadamard matrix in the default dtype; with ``norm`` every doubling divides by sqrt(2), rounded to
    that dtype each time (deploy.py:32-45)."""
    return _ops.hadamard_pow2(n, norm=norm, dtype=torch.get_default_dtype(), device=device)


def weight_dequant(weight, scale, block_size=128):
    """FP8 weight [M, N] x scale [ceil(M / b), ceil(N / b)] -> default dtype (deploy.py:48-90)."""
    return _ops.ckpt_block_dequant(weight, scale, block_size=block_size, out_dtype=torch.get_default_dtype())


def scale_fp32_to_u64(weight_scale):
    """[k, n] scales -> uint64 [k, n], low word the fp32 bit pattern, high word zero (deploy.py:93-106).
    A re-layout of a few bytes per output channel: done with tensor views on the scale's device."""
    words = weight_scale.to(torch.float32).contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return words.view(torch.uint64)


def pack_4bit(x):
    """int8 [N, K] of INT4 values -> int8 [N / 2, K], two output channels per byte (deploy.py:109-125)."""
    return _ops.ckpt_pack4_rows(x)


def int4_assistance_bias(weight, weight_scale):
    """fp32 [N] = sum_k(scale * code * 8), products rounded to the scale's dtype (deploy.py:149-157)."""
    return _ops.ckpt_int4_bias(weight, weight_scale)


def int_weight_quant(tensor, bits=8, weight_clip_factor=None):
    """Symmetric per-row quantization in ``tensor``'s dtype (deploy.py:128-146).

    bits=8 -> (int8 [N, K], fp32 scale [N, 1], None); bits=4 -> (packed int8 [N / 2, K], uint64 scale [N, 1],
    fp32 bias [N]).  ``weight_clip_factor`` is a number or a one-element tensor.
    """
    assert tensor.dim() == 2
    if weight_clip_factor is not None:
        weight_clip_factor = float(weight_clip_factor)
    return _ops.ckpt_rowquant(tensor, bits=bits, clip_factor=weight_clip_factor)


def dequant_int_weight_quant(weight, scale, bits=8, weight_clip_factor=None, block_size=128):
    """int_weight_quant(weight_dequant(weight, scale), bits, weight_clip_factor) in one pass over the FP8 weight:
    the dequantized copy stays in registers.  Same results; no counterpart function in the reference, whose main
    runs the two steps one after the other (deploy.py:437-463)."""
    if weight_clip_factor is not None:
        weight_clip_factor = float(weight_clip_factor)
    return _ops.ckpt_dequant_rowquant(weight, scale, bits=bits, clip_factor=weight_clip_factor, block_size=block_size,
                                      dtype=torch.get_default_dtype())


def generate_li_hadamard_matrix(num_layers, dim=128, device='cuda'):
    """One bf16 Hadamard matrix per layer for the lightning indexer (deploy.py:241-247)."""
    had = get_had_pow2(dim, norm=True, device=device).to(torch.bfloat16)
    return {f'model.layers.{i}.self_attn.indexer.hadamard_matrix': had.clone() for i in range(num_layers)}


# ---------------------------------------------------------------------------------------------
# host logic: names, configs, clip factors
# ---------------------------------------------------------------------------------------------
def is_match_layer_name(weight_name, layer_names):
    return any(layer in weight_name for layer in layer_names)                  # deploy.py:160-166


_ALWAYS_IGNORED = ('self_attn.indexer.wk', 'self_attn.indexer.weights_proj', 'self_attn.kv_b_proj',
                   'self_attn.kv_a_proj_with_mqa', 'self_attn.q_a_proj')


def generate_ignore_item(num_layers, num_hidden_layers, first_k_dense_replace):
    """Layers left in bf16: the small attention projections, the MoE routers, the next-token heads, lm_head
    (deploy.py:169-186)."""
    ignore = []
    for i in range(num_layers):
        prefix = f'model.layers.{i}.'
        ignore += [prefix + leaf for leaf in _ALWAYS_IGNORED]
        if i >= first_k_dense_replace:
            ignore.append(prefix + 'mlp.gate')
        if i >= num_hidden_layers:
            ignore += [prefix + 'eh_proj', prefix + 'shared_head.head']
    return ignore + ['lm_head']


def generate_w4a8_quant(num_layers, first_k_dense_replace):
    """The routed experts of every MoE layer go to INT4 (deploy.py:189-194)."""
    return [f'model.layers.{i}.mlp.experts' for i in range(first_k_dense_replace, num_layers)]


def _tensor_scheme(num_bits, dynamic, observer, strategy):
    return {'actorder': None, 'block_structure': None, 'dynamic': dynamic, 'group_size': None, 'num_bits': num_bits,
            'observer': observer, 'observer_kwargs': {}, 'strategy': strategy, 'symmetric': True, 'type': 'int'}


def generate_quant_group(a_num_bits=8, w_num_bits=8, targets=None, activation_use_clip=False):
    """One compressed-tensors config group: dynamic per-token activations, static per-channel weights
    (deploy.py:197-210)."""
    return {'input_activations': _tensor_scheme(a_num_bits, True, 'memoryless', 'token'),
            'activation_use_clip': activation_use_clip,
            'output_activations': None,
            'targets': targets,
            'weights': _tensor_scheme(w_num_bits, False, 'minmax', 'channel')}


def generate_quant_config(c8, ignores, w4a8=False, clip=False):
    """The ``quantization_config`` block written into config.json (deploy.py:213-238)."""
    groups = {'group_0': generate_quant_group(a_num_bits=8, w_num_bits=8, targets=['Linear'])}
    if w4a8:
        groups['group_1'] = generate_quant_group(a_num_bits=8, w_num_bits=4, targets=['MoEGMM'],
                                                 activation_use_clip=clip)
    kv_cache = None
    if c8:      # the flags are strings in the reference's output as well
        kv_cache = {'num_bits': 8, 'type': 'float', 'strategy': 'group', 'group_size': 128, 'dynamic': 'true',
                    'symmetric': 'true'}
    return {'config_groups': groups, 'format': 'int-quantized', 'global_compression_ratio': 1, 'ignore': ignores,
            'kv_cache_scheme': kv_cache, 'quant_method': 'compressed-tensors', 'quantization_status': 'compressed'}


def copy_py_json(src, target):
    """Copies every .py and .json below ``src`` to the same relative place below ``target`` (deploy.py:250-257)."""
    for root, _, files in os.walk(src):
        for name in files:
            if name.endswith(('.py', '.json')):
                dst_dir = os.path.join(target, os.path.relpath(root, src))
                os.makedirs(dst_dir, exist_ok=True)
                shutil.copy2(os.path.join(root, name), os.path.join(dst_dir, name))


# stored parameter name -> exported name, in the order the reference tests them (deploy.py:309-323)
_CLIP_RENAMES = (('k_cache_quantizer.clip_factor_a_max', 'ckv_a_alpha'),
                 ('clip_factor_w_max', 'w_alpha'),
                 ('afq_down.clip_factor_a_max', 'down_proj.alpha'))


def convert_clip_factors(block_id, merge_quant_param):
    """Learned clip parameters of one layer -> exported clip factors: only the ``*_max`` parameters are kept,
    renamed, and passed through a sigmoid; the down-projection activation clip of layers 0-2 is forced to
    sigmoid(10) (deploy.py:299-333)."""
    out = {}
    with torch.no_grad():
        for key, val in merge_quant_param.items():
            if 'max' not in key:
                continue
            for stored, exported in _CLIP_RENAMES:
                if stored in key:
                    if exported == 'down_proj.alpha' and block_id <= 2:
                        print(f'{key} is set to 10.0')
                        val = torch.tensor(10.0)          # default dtype, as in the reference
                    out[key.replace(stored, exported)] = torch.sigmoid(val)
                    break
    return out


def _load_layer_params(mla_param_path, moe_param_path, layer_idx):
    name = f'quant_parameters_{layer_idx}.pth'
    params = torch.load(os.path.join(mla_param_path, name))
    params.update(torch.load(os.path.join(moe_param_path, name)))
    return params


def load_clip_params(num_hidden_layers, num_nextn_predict_layers, mla_param_path, moe_param_path):
    """Reads ``quant_parameters_<layer>.pth`` from both directories and sorts the converted factors into
    (kv-cache, activation, weight) tables keyed by full tensor name.  A next-token layer without a file takes
    the names of the last hidden layer with factors of 1 (deploy.py:260-296)."""
    kv, act, weight = {}, {}, {}
    last = num_hidden_layers - 1
    for layer_idx in range(num_hidden_layers + num_nextn_predict_layers):
        if os.path.exists(os.path.join(mla_param_path, f'quant_parameters_{layer_idx}.pth')):
            params = convert_clip_factors(layer_idx, _load_layer_params(mla_param_path, moe_param_path, layer_idx))
        elif layer_idx < num_hidden_layers:
            raise ValueError(f"{os.path.join(mla_param_path, f'quant_parameters_{layer_idx}.pth')} not found, "
                             f"please check the {mla_param_path}")
        else:
            borrowed = convert_clip_factors(layer_idx, _load_layer_params(mla_param_path, moe_param_path, last))
            params = {k.replace(f'layers.{last}', f'layers.{layer_idx}'): torch.tensor(1.0).to(v.dtype)
                      for k, v in borrowed.items()}
        for name, factor in params.items():
            full = f'model.layers.{layer_idx}.{name}'
            if full.endswith('w_alpha'):
                weight[full] = factor
            elif full.endswith('ckv_a_alpha'):
                kv[full] = factor
            elif full.endswith('alpha'):
                act[full] = factor
    return kv, act, weight


# ---------------------------------------------------------------------------------------------
# the export itself
# ---------------------------------------------------------------------------------------------
class ExportPlan:
    """What happens to each tensor of the checkpoint, decided from its name, its element size and whether a
    ``<name>_scale_inv`` tensor exists -- the branch structure of the reference's loop (deploy.py:428-508)
    without the tensors, so that it can be checked on its own."""

    SKIP, KEEP, DEQUANT, DEQUANT_QUANT, QUANT = 'skip', 'keep', 'dequant', 'dequant+quant', 'quant'

    def __init__(self, config, quant_type, clip=False):
        if quant_type not in QUANT_TYPES:
            raise AssertionError(f'Unsupported quant_type: {quant_type}')
        self.quant_type, self.clip = quant_type, bool(clip)
        self.c8 = quant_type.endswith('c8')
        self.w4a8 = quant_type.startswith('w4a8')
        self.w8a8 = quant_type.startswith('w8a8')
        if (self.c8 or self.clip) and not (self.c8 and self.clip):
            raise ValueError('clip factors are read only for a c8 quant type together with --clip, and the '
                             'reference fails (NameError) on either one alone: give both or neither')
        self.num_hidden_layers = config['num_hidden_layers']
        self.num_layers = self.num_hidden_layers + config['num_nextn_predict_layers']
        first_dense = config['first_k_dense_replace']
        self.config = {k: v for k, v in config.items() if k != 'quantization_config'}
        self.ignore, self.int4_layers = [], []
        if self.w8a8 or self.w4a8:
            self.ignore = generate_ignore_item(self.num_layers, self.num_hidden_layers, first_dense)
            self.config['quantization_config'] = generate_quant_config(self.c8, self.ignore, w4a8=self.w4a8,
                                                                       clip=self.clip)
        if self.w4a8:
            self.int4_layers = generate_w4a8_quant(self.num_layers, first_dense)

    def bits(self, name):
        return 4 if is_match_layer_name(name, self.int4_layers) else 8

    def action(self, name, element_size, has_scale_inv):
        if 'model.embed_tokens.weight' in name or name.endswith('_scale_inv'):
            return self.SKIP                                                    # deploy.py:430-433
        if element_size == 1:                                                   # an FP8 weight
            if not has_scale_inv:
                return self.KEEP                                                # deploy.py:476-480
            if (self.w8a8 or self.w4a8) and not is_match_layer_name(name, self.ignore):
                return self.DEQUANT_QUANT
            return self.DEQUANT
        # wider dtypes: the listed projections are quantized whatever the quant type (deploy.py:481-508)
        if _QUANTIZED_PLAIN.search(name) or 'wq_b' in name:
            return self.QUANT
        return self.KEEP

    def output_names(self, name, action):
        """Names written for one input tensor, in the order the reference inserts them into the index."""
        if action == self.SKIP:
            return []
        if action in (self.DEQUANT_QUANT, self.QUANT):
            names = [name, f'{name}_scale']
            if self.w4a8 and self.bits(name) == 4:
                names.append(name.replace('.weight', '.bias'))
            return names
        return [name]


def main(weight_path, output_path, quant_type, clip=False, mla_param_path=None, moe_param_path=None, device='cuda'):
    """Converts an FP8 block-scaled checkpoint to bf16, W8A8 or W4A8 shards plus index and config
    (deploy.py:336-572).  ``device`` is the GPU the tensor steps run on; shards are read and written on the host.
    """
    from safetensors.torch import load_file, save_file

    previous_default = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        os.makedirs(output_path, exist_ok=True)
        with open(os.path.join(weight_path, 'model.safetensors.index.json')) as f:
            weight_map = json.load(f)['weight_map']
        with open(os.path.join(weight_path, 'config.json')) as f:
            plan = ExportPlan(json.load(f), quant_type, clip)
        kv_clip, act_clip, weight_clip = {}, {}, {}
        if plan.c8 and plan.clip:
            kv_clip, act_clip, weight_clip = load_clip_params(
                plan.num_hidden_layers, plan.num_layers - plan.num_hidden_layers, mla_param_path, moe_param_path)

        shards = {}                     # file name -> tensors, the two most recent kept (deploy.py:515-518)

        def shard(file_name):
            if file_name not in shards:
                shards[file_name] = load_file(os.path.join(weight_path, file_name), device='cpu')
            return shards[file_name]

        def clip_factor(name):
            return weight_clip.get(name.replace('weight', 'w_alpha')) if plan.clip else None

        new_weight_map = {}
        files = sorted(glob(os.path.join(weight_path, '*.safetensors')))
        file_name = None
        for path in files:
            file_name = os.path.basename(path)
            shards[file_name] = load_file(path, device='cpu')
            out = {}
            for name, tensor in shards[file_name].items():
                scale_name = f'{name}_scale_inv'
                action = plan.action(name, tensor.element_size(), scale_name in weight_map)
                if action == plan.SKIP:
                    continue
                if action == plan.KEEP:
                    if tensor.element_size() == 1:
                        print(f'Warning: Missing scale_inv tensor for {name}, skipping conversion')
                    results = [tensor]
                else:
                    dev = tensor.to(device)
                    if action == plan.QUANT:
                        results = int_weight_quant(dev, bits=plan.bits(name), weight_clip_factor=clip_factor(name))
                    else:
                        scale_inv = shard(weight_map[scale_name])[scale_name].to(device)
                        if action == plan.DEQUANT:
                            if plan.w8a8 or plan.w4a8:
                                print(f'Ignore quantization {name}')
                            results = [weight_dequant(dev, scale_inv)]
                        else:           # dequantize and re-quantize without writing the bf16 weight
                            results = dequant_int_weight_quant(dev, scale_inv, bits=plan.bits(name),
                                                               weight_clip_factor=clip_factor(name))
                    results = [r for r in results if r is not None]
                for out_name, value in zip(plan.output_names(name, action), results):
                    out[out_name] = value.cpu().contiguous()
                    new_weight_map[out_name] = file_name
            save_file(out, os.path.join(output_path, file_name), metadata={'format': 'pt'})
            while len(shards) > 2:
                del shards[next(iter(shards))]

        if (plan.c8 or plan.clip) and files:
            # the extra tensors go into the LAST shard written (deploy.py:520-548)
            last_path = os.path.join(output_path, file_name)
            extra = load_file(last_path, device='cpu')
            additions = {}
            if plan.c8:
                additions.update({k: v.cpu() for k, v in
                                  generate_li_hadamard_matrix(plan.num_layers, dim=128, device=device).items()})
            if plan.clip:
                additions.update(act_clip)
            additions.update(kv_clip)
            extra.update(additions)
            for name in additions:
                new_weight_map[name] = file_name
            save_file(extra, last_path, metadata={'format': 'pt'})

        copy_py_json(weight_path, output_path)
        with open(os.path.join(output_path, 'model.safetensors.index.json'), 'w') as f:
            json.dump({'metadata': {}, 'weight_map': new_weight_map}, f, indent=2)
        with open(os.path.join(output_path, 'config.json'), 'w') as f:
            json.dump(plan.config, f, indent=2)
    finally:
        torch.set_default_dtype(previous_default)


if __name__ == '__main__':
    parser = ArgumentParser()
    parser.add_argument('--input_weight_path', type=str, required=True)
    parser.add_argument('--output_weight_path', type=str, required=True)
    parser.add_argument('--quant_type', type=str, default='bfloat16', choices=list(QUANT_TYPES))
    parser.add_argument('--clip', action='store_true')
    parser.add_argument('--mla_param_path', type=str, default=None)
    parser.add_argument('--moe_param_path', type=str, default=None)
    parser.add_argument('--device', type=str, default='cuda')
    args = parser.parse_args()
    main(args.input_weight_path, args.output_weight_path, args.quant_type, args.clip, args.mla_param_path,
         args.moe_param_path, device=args.device)
