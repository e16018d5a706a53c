"""The reference's OWN unit tests, run against this package under the reference's module name.

Where a checkout of the reference is available -- ``$AMCT_REFERENCE``, or a directory ``reference`` next to this
repository -- its ``tests/amct_pytorch/test_config.py`` (config schema, presets, every error message of the parser)
and ``test_customized_algo.py`` (algorithm registry, custom quantize / deploy modules through ``quantize`` /
``convert``) are imported unchanged with ``amct_pytorch`` aliased to ``amct_b200`` and must pass.  Nothing is copied:
without the checkout the tests are skipped.

The reference's remaining test files (``test_minmax``, ``test_smoothquant``, ``test_awq``, ``test_gptq``,
``test_quantize``) drive calibration, ``convert`` and deploy forwards on CPU tensors through a mocked ``torch_npu``.
This package has no CPU path, so the second test gives it one for the duration of the run, out of test
infrastructure only: the quantization kernels' own source in the CPU emulation (``tests/emu``) and the oracle's
integer / 16-bit matmul in place of the tensor-core GEMMs.  Calibration observers, scale rules, weight codes, the
AWQ search and the GPTQ loop then run on the real kernel code, and the reference's assertions (module classes after
``quantize`` and ``convert``, buffer names, dtypes and shapes, error messages) must hold: all 47 pass (the INT4
``quantized_weight`` buffer is int32 as the reference's tests require: the int4pack form of the codes).
"""
import importlib
import os
import pkgutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get('AMCT_REFERENCE') or os.path.join(os.path.dirname(ROOT), 'reference')
REF_TESTS = os.path.join(REFERENCE, 'tests', 'amct_pytorch')

RUNNER = r'''
import importlib, pkgutil, sys, unittest
sys.path.insert(0, {root!r})
import amct_b200
sys.modules['amct_pytorch'] = amct_b200
for m in pkgutil.walk_packages(amct_b200.__path__, 'amct_b200.'):
    if any(part in m.name for part in ('.csrc', '.workloads', '.experimental')):
        continue
    sys.modules['amct_pytorch' + m.name[len('amct_b200'):]] = importlib.import_module(m.name)
sys.path.insert(0, {tests!r})
suite = unittest.defaultTestLoader.loadTestsFromNames({names!r})
result = unittest.TextTestRunner(verbosity=0).run(suite)
print('RAN', result.testsRun, 'FAILED', len(result.failures) + len(result.errors))
sys.exit(0 if result.wasSuccessful() else 1)
'''


@pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason='no checkout of the reference at hand')
def test_reference_config_and_registry_tests_pass_unchanged(tmp_path):
    names = ['test_config', 'test_customized_algo']
    code = RUNNER.format(root=ROOT, tests=REF_TESTS, names=names)
    done = subprocess.run([sys.executable, '-c', code], cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    ran = int(done.stdout.split('RAN')[1].split()[0])
    assert ran >= 29


EMULATED_RUNNER = r'''
import ctypes, importlib, pkgutil, sys, unittest
sys.path.insert(0, {root!r})
import torch
import amct_b200
sys.modules['amct_pytorch'] = amct_b200
for m in pkgutil.walk_packages(amct_b200.__path__, 'amct_b200.'):
    if any(part in m.name for part in ('.csrc', '.workloads', '.experimental')):
        continue
    sys.modules['amct_pytorch' + m.name[len('amct_b200'):]] = importlib.import_module(m.name)
from amct_b200.backend import lib, ops
from oracle import npu_ops
emu = ctypes.CDLL({library!r})
for name in ('amct_mx_tiled_scale_bytes', 'amct_minmax_workspace_bytes', 'amct_minmax_noalloc_max_k'):
    getattr(emu, name).restype = ctypes.c_int64
emu.amct_minmax_workspace_bytes.argtypes = [ctypes.c_int64]
lib.load = lambda: emu
ops._need_cuda = lambda *tensors: None
ops._stream = lambda: ctypes.c_void_p(0)
torch.Tensor.is_cuda = property(lambda self: True)


def int8_gemm(q, w_nk, deq_scale=None, pertoken_scale=None, bias=None, out_dtype=torch.bfloat16, out=None, status=None):
    assert deq_scale.numel() == w_nk.shape[0]
    return npu_ops.npu_quant_matmul(q, w_nk.t(), deq_scale, pertoken_scale, bias, out_dtype)


def float_gemm(a, b_nk, bias=None, out_dtype=None, out=None, status=None):
    y = a.float() @ b_nk.float().t()
    return (y if bias is None else y + bias.float()).to(out_dtype or a.dtype)


ops.gemm_w8a8, ops.gemm_f16 = int8_gemm, float_gemm
ops.gemm_w4a16 = lambda *args, **kwargs: None          # "not a shape for the fused kernel": dequantize, then gemm_f16
sys.path.insert(0, {tests!r})
suite = unittest.defaultTestLoader.loadTestsFromNames({names!r})
result = unittest.TextTestRunner(verbosity=0).run(suite)
bad = sorted(str(t).split()[0] for t, _ in result.failures + result.errors)
print('RAN', result.testsRun, 'BAD', ','.join(bad))
'''


@pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason='no checkout of the reference at hand')
def test_reference_algorithm_tests_on_emulated_kernels(tmp_path):
    import test_kernel_source_emulation as emulation
    library = emulation.full_library()[0]
    # two processes side by side -- the AWQ search is the slow one on emulated kernels -- and no more: the emulated
    # blocks are hundreds of host threads each
    files = [['test_awq'], ['test_minmax', 'test_smoothquant', 'test_gptq', 'test_quantize']]
    running = []
    for names in files:
        cwd = tmp_path / names[0]
        cwd.mkdir()
        code = EMULATED_RUNNER.format(root=ROOT, tests=REF_TESTS, names=names, library=library)
        running.append(subprocess.Popen([sys.executable, '-c', code], cwd=str(cwd), stdout=subprocess.PIPE,
                                        stderr=subprocess.PIPE, text=True))
    ran, bad, logs = 0, [], ''
    for name, proc in zip(files, running):
        out, err = proc.communicate(timeout=1800)
        line = [ln for ln in out.splitlines() if ln.startswith('RAN')]
        assert line, str(name) + out[-2000:] + err[-3000:]
        ran += int(line[-1].split()[1])
        bad += [b for b in line[-1].split('BAD')[1].strip().split(',') if b]
        logs += err[-1500:]
    assert ran >= 47
    assert bad == [], (bad, logs)
