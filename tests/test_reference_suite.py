"""The reference's OWN unit tests, run against this package under the reference's module name.

Where a checkout of the reference is available -- ``$AMCT_REFERENCE``, or a directory ``reference`` next to this
repository -- its ``tests/amct_pytorch/test_config.py`` (config schema, presets, every error message of the parser)
and ``test_customized_algo.py`` (algorithm registry, custom quantize / deploy modules through ``quantize`` /
``convert``) are imported unchanged with ``amct_pytorch`` aliased to ``amct_b200`` and must pass.  Nothing is copied:
without the checkout the test is skipped.  The reference's remaining test files drive calibration and deploy forwards
on CPU tensors through a mocked ``torch_npu``; this package has no CPU path for those, so they are not run here (the
GPU parity tests cover that ground against golden vectors generated from the reference).
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
