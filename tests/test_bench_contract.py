"""bench.py's command line and the reference arm's fall-back line, without a GPU."""
import importlib.util
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location('bench_under_test', os.path.join(ROOT, 'bench.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_defaults_are_one_gpu_and_at_least_three_warmup_steps(monkeypatch):
    bench = _bench()
    monkeypatch.setattr(sys, 'argv', ['bench.py'])
    args = bench.parse()
    assert args.gpus == 1 and args.impl == 'ours' and args.warmup >= 3 and args.steps >= 1
    assert args.layers == 80 and (args.batch, args.seq) == (32, 2048) and args.comm == 'auto'
    monkeypatch.setattr(sys, 'argv', ['bench.py', '--gpus', '8', '--steps', '20', '--warmup', '5', '--impl', 'reference'])
    args = bench.parse()
    assert (args.gpus, args.steps, args.warmup, args.impl) == (8, 20, 5, 'reference')


def test_reference_arm_says_unavailable_when_the_reference_is_not_installed(monkeypatch, capsys, tmp_path):
    bench = _bench()
    monkeypatch.setattr(bench, 'REF_DIR', str(tmp_path / 'nothing_here'))
    monkeypatch.setattr(sys, 'argv', ['bench.py', '--impl', 'reference', '--steps', '1', '--warmup', '0'])
    monkeypatch.delenv('RANK', raising=False)
    bench.run_reference(bench.parse())
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line['impl'] == 'reference' and 'unavailable' in line and 'missing' in line['unavailable']


def test_reference_arm_is_silent_on_other_ranks(monkeypatch, capsys):
    bench = _bench()
    monkeypatch.setenv('RANK', '3')
    monkeypatch.setattr(sys, 'argv', ['bench.py', '--impl', 'reference', '--gpus', '8'])
    bench.run_reference(bench.parse())
    assert capsys.readouterr().out == ''
