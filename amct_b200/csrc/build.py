"""Builds libamct_b200.so (all CUDA sources of this directory) for sm_100a.

    python -m amct_b200.csrc.build [--force] [--verbose]

The library lands in ``amct_b200/lib/`` inside the source tree.  It links the
CUDA runtime statically and resolves the one driver entry point it needs
(cuTensorMapEncodeTiled) at run time through cudaGetDriverEntryPoint, so it loads
on a machine without a GPU driver as well.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(os.path.dirname(HERE), 'lib')
LIB_PATH = os.path.join(LIB_DIR, 'libamct_b200.so')
INCLUDE = os.path.join(os.path.dirname(os.path.dirname(HERE)), 'include')

# numerics-critical files: no FMA contraction so that x*s+z rounds twice like torch
STRICT = {'quant_rows.cu', 'quant_token.cu', 'quant_static.cu', 'reduce.cu', 'mx_quant.cu', 'hif8.cu', 'norm_quant.cu',
          'rope.cu', 'quant_groups.cu', 'ckpt_formats.cu', 'kv_quant.cu'}


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith('.cu'))


def _stale():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(('.cu', '.cuh'))]
    deps.append(os.path.join(INCLUDE, 'amct_b200.h'))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, 'obj')
    os.makedirs(obj_dir, exist_ok=True)
    base = [nvcc, '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
            '-Xcompiler', '-fPIC', '-I', INCLUDE, '--expt-relaxed-constexpr']
    if verbose:
        base += ['-Xptxas', '-v']
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(obj_dir, src[:-3] + '.o')
        cmd = base + (['-fmad=false'] if src in STRICT else []) + ['-c', os.path.join(HERE, src), '-o', obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f'--- {src}\n{out}\n')
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError('nvcc failed')
    link = [nvcc, '-shared', '-o', LIB_PATH] + objs + ['-cudart', 'static']
    subprocess.check_call(link)
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
