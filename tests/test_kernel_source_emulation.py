"""The SOURCE of the checkpoint-format and KV-cache activation kernels, executed on the CPU.

``amct_b200/csrc/ckpt_formats.cu`` and ``kv_quant.cu`` are compiled with g++ under ``tests/emu/cuda_emu.h``, which
emulates blocks, threads, ``__syncthreads`` and warp shuffles with host threads and maps the rounding intrinsics to
the IEEE operations they name.  The same C ABI entry points are then called, through the same Python wrappers
(``amct_b200.backend.ops``, patched here to accept host pointers), by the very test functions that run on the GPU
(``tests/test_zy_gpu_*.py``): argument checks, launch geometry, vector and scalar paths, reductions and index
arithmetic are all exercised against the reference's golden vectors and the oracle without a GPU.  The build checks
every access for its type's alignment, so a 16-byte vector access on an address the launch conditions should have
ruled out stops the test, as it would fault on the GPU.

This is a check of the kernel source, not a product path: the emulation library is built into a temporary directory
by this test alone, and ``amct_b200`` can neither build nor load it.  What it cannot show is anything that depends on
the GPU itself (the hardware FP8 conversion, memory ordering, performance); the GPU tests remain the parity tests.
"""
import contextlib
import ctypes
import functools
import os
import shutil
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, 'amct_b200', 'csrc')
CUDA_INCLUDE = os.path.join(os.environ.get('CUDA_HOME', '/usr/local/cuda'), 'include')


@pytest.fixture(scope='module')
def emu_lib(tmp_path_factory):
    gxx = shutil.which('g++')
    if gxx is None or not os.path.exists(os.path.join(CUDA_INCLUDE, 'cuda_fp8.h')):
        pytest.skip('needs g++ and the CUDA headers')
    out = str(tmp_path_factory.mktemp('emu') / 'libamct_emu.so')
    # -fsanitize=alignment: a vector access the GPU would fault on ("misaligned address") aborts the test here
    cmd = [gxx, '-std=c++17', '-O1', '-w', '-ffp-contract=off', '-fsanitize=alignment', '-fno-sanitize-recover=alignment',
           '-fPIC', '-shared', '-x', 'c++',
           '-include', os.path.join(ROOT, 'tests', 'emu', 'cuda_emu.h'), '-I', CUDA_INCLUDE,
           os.path.join(CSRC, 'ckpt_formats.cu'), os.path.join(CSRC, 'kv_quant.cu'), '-o', out, '-lpthread']
    subprocess.check_call(cmd)
    return ctypes.CDLL(out)


@pytest.fixture
def on_cpu(emu_lib, monkeypatch):
    """The ops wrappers talking to the emulation library with host tensors."""
    from amct_b200.backend import lib, ops
    monkeypatch.setattr(lib, 'load', lambda: emu_lib)
    monkeypatch.setattr(ops, '_need_cuda', lambda *tensors: None)
    monkeypatch.setattr(ops, '_stream', lambda: ctypes.c_void_p(0))
    monkeypatch.setattr(ops, 'hadamard_pow2', functools.partial(ops.hadamard_pow2, device='cpu'))
    monkeypatch.setattr(torch.cuda, 'device', lambda device: contextlib.nullcontext())
    monkeypatch.setattr(torch.Tensor, 'cuda', lambda self, *args, **kwargs: self)
    return ops


# ---------------------------------------------------------------------------------------------
# checkpoint formats
# ---------------------------------------------------------------------------------------------
def test_emulated_block_dequant(on_cpu):
    import test_zy_gpu_ckpt_formats as G
    for tag in ('ragged', 'even'):
        G.test_block_dequant_golden(tag)
    for shape in [(256, 7168), (130, 96), (1, 16), (257, 2064), (5, 3)]:
        for dtype in (torch.bfloat16, torch.float16, torch.float32):
            G.test_block_dequant_oracle(shape, dtype)
    G.test_block_dequant_other_block_and_errors()


@pytest.mark.parametrize('dtype', ['bf16', 'fp16', 'fp32'])
def test_emulated_rowquant_golden(on_cpu, dtype):
    import test_zy_gpu_ckpt_formats as G
    for bits in (8, 4):
        for clip in ('noclip', 'clip'):
            G.test_rowquant_golden(dtype, bits, clip)


def test_emulated_rowquant_shapes(on_cpu):
    import test_zy_gpu_ckpt_formats as G
    for shape in [(64, 7168), (6, 515), (2, 8), (130, 96), (4, 20000)]:
        for dtype in (torch.bfloat16, torch.float16, torch.float32):
            for bits in (8, 4):
                try:
                    G.test_rowquant_oracle(shape, dtype, bits)
                except pytest.skip.Exception:
                    pass
    G.test_rowquant_strided_rows_zero_row_and_nan()
    for shape in [(128, 7168), (130, 96), (6, 200), (258, 2064)]:
        for bits in (8, 4):
            G.test_fused_dequant_rowquant(shape, bits)
    with pytest.raises(ValueError):
        on_cpu.ckpt_rowquant(torch.zeros(3, 16, dtype=torch.bfloat16), 4)


def test_emulated_pack_bias_hadamard(on_cpu):
    import test_zy_gpu_ckpt_formats as G
    G.test_pack4_bias_scale_words_hadamard()


def test_emulated_full_size_properties(on_cpu):
    import test_zy_gpu_ckpt_formats as G
    G.test_full_size_properties()


@pytest.mark.parametrize('quant_type,clip', [('bfloat16', False), ('w8a8c16', False), ('w4a8c16', False), ('w8a8c8', True), ('w4a8c8', True)])
def test_emulated_export_end_to_end(on_cpu, quant_type, clip, tmp_path):
    from ckpt_fixture import compare_export, golden, write_checkpoint
    from amct_b200.experimental.quantization.deepseek_v3_2 import deploy
    gold, meta = golden()
    src, dst, par = tmp_path / 'src', tmp_path / 'dst', tmp_path / 'par'
    src.mkdir()
    mla, moe = write_checkpoint(gold, meta, str(src), str(par))
    deploy.main(str(src), str(dst), quant_type, clip, mla, moe, device='cpu')
    compare_export(gold, meta, quant_type, str(dst))


# ---------------------------------------------------------------------------------------------
# KV-cache / indexer activations
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize('dtype', ['fp16', 'bf16', 'fp32'])
def test_emulated_fake_quant_golden(on_cpu, dtype):
    import test_zy_gpu_dsa_activations as G
    for k in (128, 512, 200):
        G.test_fake_quant_golden(dtype, k)
    G.test_clip_ratio_and_per_tensor_modules(dtype)


def test_emulated_fake_quant_shapes(on_cpu):
    import test_zy_gpu_dsa_activations as G
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        for shape in [(3, 70, 1536), (1000, 128), (5, 16384), (7, 33), (2, 4, 9, 512), (6, 8)]:
            G.test_fake_quant_oracle(dtype, shape)
    G.test_fake_quant_strided_and_cast()
    G.test_fake_quant_scale_underflow_keeps_nan()


def test_emulated_rotation_and_chain(on_cpu):
    import test_zy_gpu_dsa_activations as G
    for dtype in ('bf16', 'fp16', 'fp32'):
        for d in (128, 64):
            G.test_rotation_golden(dtype, d)
    for d in (32, 64, 128, 256, 512):
        G.test_rotation_widths_and_round_trip(d)
    G.test_rotation_unaligned_rows()
    G.test_indexer_chain()
    G.test_module_with_learned_clipping()


def test_emulated_argument_checks(on_cpu):
    from amct_b200.backend.lib import BackendError
    x = torch.zeros(4, 48)
    with pytest.raises(BackendError):
        on_cpu.dsa_rotate_fakequant(x, rotate=True, bits=16)
    with pytest.raises(BackendError):
        on_cpu.dsa_rotate_fakequant(torch.zeros(4, 1024), rotate=True, bits=16)
    with pytest.raises(BackendError):
        on_cpu.dsa_rotate_fakequant(x, bits=9)
