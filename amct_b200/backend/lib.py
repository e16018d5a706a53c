"""ctypes loader of libamct_b200.so.

There is no CPU implementation behind this module: if the library cannot be
loaded, or a tensor is not on a CUDA device, the call fails with an exception.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), 'lib', 'libamct_b200.so')
HEADER = os.path.join(os.path.dirname(os.path.dirname(_HERE)), 'include', 'amct_b200.h')

OK = 0
ERRORS = {-1: 'invalid argument', -2: 'misaligned pointer or leading dimension', -3: 'CUDA error',
          -4: 'unsupported shape', -5: 'device-side wait timed out',
          -6: 'size exceeds the scratch memory built into the library'}

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
STRATEGY = {'tensor': 0, 'channel': 1, 'group': 2}
RULE = {'released': 0, 'experimental': 1}
PRE_NONE, PRE_MUL, PRE_DIV = 0, 1, 2
OUT_NONE, OUT_I8, OUT_I32, OUT_PACK4, OUT_FAKE, OUT_FAKE_AWQ = range(6)
AXIS_TENSOR, AXIS_COLUMN = 0, 1
DSA_DYNAMIC, DSA_LEARNED_CLIP, DSA_CLIP_RATIO, DSA_STATIC, DSA_STATIC_F32 = range(5)

_lib = None


class BackendError(RuntimeError):
    pass


def declared_symbols(header=HEADER):
    """Names of all entry points the public header declares."""
    text = open(header).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(amct_[a-z0-9_]+)\s*\(', text)))


def load():
    """Returns the ctypes handle; raises BackendError if the library is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise BackendError(
                f'{LIB_PATH} not found: build it with `python -m amct_b200.csrc.build` '
                '(there is no CPU fallback for the quantization kernels)')
        lib = ctypes.CDLL(LIB_PATH)
        lib.amct_minmax_workspace_bytes.restype = ctypes.c_int64
        lib.amct_minmax_workspace_bytes.argtypes = [ctypes.c_int64]
        lib.amct_minmax_noalloc_max_k.restype = ctypes.c_int64
        lib.amct_mx_tiled_scale_bytes.restype = ctypes.c_int64
        lib.amct_mma_peak_ops_per_cta_step.restype = ctypes.c_int64
        _lib = lib
    return _lib


def check(code, what):
    if code != OK:
        raise BackendError(f'{what} failed: {ERRORS.get(code, code)}')
