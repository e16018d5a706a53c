"""The allocation-free observer entry point against the regular one.

Collected last on purpose: if it fails, a run that stops at the first failure has
already run everything else.  It must pass in a fresh process and after the rest
of the suite, so it makes no assumption about what the shared scratch array holds.

Who needs this entry point: a host that may not allocate device memory once it is
running (fixed memory budget carved at start-up) or that can only pass inputs and
outputs to the library.  The regular amct_minmax needs a caller workspace; this
one keeps its partial results in an array compiled into the library.
"""
import ctypes
from ctypes import c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(t.data_ptr())


def _call_both(L, x, axis, merge_from=None):
    """Runs amct_minmax (caller workspace) and amct_minmax_noalloc (built-in scratch) through the
    C ABI on the same input; returns ((min, max) regular, (min, max) no-alloc)."""
    rows, k = x.shape
    n = 1 if axis == 0 else k
    dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x.dtype]
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for noalloc in (False, True):
        if merge_from is None:
            mn = torch.empty(n, dtype=x.dtype, device='cuda')
            mx = torch.empty(n, dtype=x.dtype, device='cuda')
        else:
            mn, mx = merge_from[0].clone(), merge_from[1].clone()
        merge = c_int(0 if merge_from is None else 1)
        if noalloc:
            rc = L.amct_minmax_noalloc(_ptr(x), c_int(dt), c_int64(rows), c_int64(k), c_int64(x.stride(0)), c_int(axis),
                                       merge, _ptr(mn), _ptr(mx), c_void_p(0), stream)
        else:
            ws = torch.empty(L.amct_minmax_workspace_bytes(c_int64(k)), dtype=torch.uint8, device='cuda')
            rc = L.amct_minmax(_ptr(x), c_int(dt), c_int64(rows), c_int64(k), c_int64(x.stride(0)), c_int(axis),
                               merge, _ptr(mn), _ptr(mx), _ptr(ws), c_void_p(0), stream)
        assert rc == 0, rc
        outs.append((mn, mx))
    torch.cuda.synchronize()
    return outs


def _same_bits(a, b):
    w = {2: torch.int16, 4: torch.int32}[a.element_size()]
    return bool((a.view(w) == b.view(w)).all())


def test_noalloc_matches_regular_entry_point_on_consecutive_calls():
    from amct_b200.backend import lib
    L = lib.load()
    assert L.amct_minmax_noalloc_max_k() == 16384
    g = torch.Generator(device='cuda').manual_seed(123)
    COLUMN, TENSOR = 1, 0
    # two calls in a row on the column axis (the second one smaller, so it finds the first
    # call's partials still lying in the scratch), then the tensor axis, then a merge
    first = torch.randn(3000, 4096, device='cuda', generator=g).to(torch.bfloat16)
    second = (torch.randn(257, 520, device='cuda', generator=g) * 3).to(torch.bfloat16)
    third = torch.randn(1500, 1000, device='cuda', generator=g)
    prev = None
    for x, axis in ((first, COLUMN), (second, COLUMN), (third, TENSOR), (second, TENSOR), (first, COLUMN)):
        (mn_a, mx_a), (mn_b, mx_b) = _call_both(L, x, axis)
        assert _same_bits(mn_a, mn_b) and _same_bits(mx_a, mx_b)
        want_min = x.amin(0) if axis == COLUMN else x.min().reshape(1)
        want_max = x.amax(0) if axis == COLUMN else x.max().reshape(1)
        assert _same_bits(mn_b, want_min) and _same_bits(mx_b, want_max)
        prev = (mn_b, mx_b) if axis == COLUMN and x is first else prev
    # running merge into existing values
    shifted = (first.float() * 0.5 + 1).to(torch.bfloat16)
    (mn_a, mx_a), (mn_b, mx_b) = _call_both(L, shifted, COLUMN, merge_from=prev)
    assert _same_bits(mn_a, mn_b) and _same_bits(mx_a, mx_b)
    assert _same_bits(mx_b, torch.maximum(prev[1], shifted.amax(0)))


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    from amct_b200.backend import lib, ops
    L = lib.load()
    k = 16384 + 8
    x = torch.zeros(16, k, dtype=torch.bfloat16, device='cuda')
    mn = torch.full((k,), 7, dtype=torch.bfloat16, device='cuda')
    mx = mn.clone()
    rc = L.amct_minmax_noalloc(_ptr(x), c_int(2), c_int64(16), c_int64(k), c_int64(k), c_int(1), c_int(0), _ptr(mn), _ptr(mx),
                               c_void_p(0), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -6
    torch.cuda.synchronize()
    assert (mn == 7).all() and (mx == 7).all()                 # nothing was launched
    with pytest.raises(lib.BackendError, match='exceeds the scratch memory built into the library'):
        ops.minmax_noalloc(x, 'column', mn, mx)
    # the tensor-wide reduction has no such limit
    one_min, one_max = torch.empty(1, dtype=torch.bfloat16, device='cuda'), torch.empty(1, dtype=torch.bfloat16, device='cuda')
    ops.minmax_noalloc(x, 'tensor', one_min, one_max)
    assert float(one_min) == 0 and float(one_max) == 0
