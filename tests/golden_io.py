"""Loader for the golden fixtures written by tests/golden/make_golden.py and tests/golden/make_ckpt_golden.py."""
import os

import numpy as np
import torch

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'intq_golden.npz')
CKPT_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'ckpt_golden.npz')
CKPT_JSON = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'ckpt_golden.json')
_TAGS = {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp8': torch.float8_e4m3fn, 'u64': torch.uint64}


class Golden:
    def __init__(self, path=_PATH):
        self._z = np.load(path)
        self._keys = {}
        for key in self._z.files:
            name, _, tag = key.partition('|')
            self._keys[name] = (key, tag)

    def has(self, name):
        return name in self._keys

    def names(self, prefix=''):
        return [n for n in self._keys if n.startswith(prefix)]

    def get(self, name):
        """Tensor, or None when the reference produced None (key absent)."""
        if name not in self._keys:
            return None
        key, tag = self._keys[name]
        t = torch.from_numpy(self._z[key].copy())
        return t.view(_TAGS[tag]) if tag else t


def bits_equal(a, b):
    """Bit-exact comparison that also compares dtype and shape."""
    if a is None or b is None:
        return a is None and b is None
    if a.dtype != b.dtype or tuple(a.shape) != tuple(b.shape):
        return False
    a = a.detach().cpu().contiguous()
    b = b.detach().cpu().contiguous()
    if a.dtype == torch.uint64:
        return bool((a.view(torch.int64) == b.view(torch.int64)).all())
    if a.dtype.is_floating_point:
        w = {2: torch.int16, 4: torch.int32, 8: torch.int64, 1: torch.uint8}[a.element_size()]
        return bool((a.view(w) == b.view(w)).all())
    return bool((a == b).all())
