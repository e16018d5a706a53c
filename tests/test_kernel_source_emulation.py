"""The SOURCE of the bandwidth-bound kernels, executed on the CPU.

Every ``.cu`` file of ``amct_b200/csrc`` that uses neither tensor cores, bulk asynchronous copies nor inline PTX --
``quant_rows.cu``, ``quant_groups.cu``, ``reduce.cu``, ``norm_quant.cu``, ``quant_static.cu``, ``mx_quant.cu``,
``hif8.cu``, ``w4a16.cu``, ``rope.cu``, ``ckpt_formats.cu``, ``kv_quant.cu``, ``gptq_block.cu`` -- is compiled with g++ under
``tests/emu/cuda_emu.h``, which emulates blocks, threads, ``__syncthreads`` and warp shuffles with host threads and maps
the rounding intrinsics to the IEEE operations they name.  The same C ABI entry points are then called, through the
same Python wrappers (``amct_b200.backend.ops``, patched here to accept host pointers), by the very test functions that
run on the GPU (``tests/test_gpu_*.py``, ``tests/test_zy_gpu_*.py``): argument checks, launch geometry, vector and
scalar paths, reductions and index arithmetic are exercised against the reference's golden vectors and the oracle
without a GPU.  The build checks every access for its type's alignment, so a 16-byte vector access on an address the
launch conditions should have ruled out stops the test, as it would fault on the GPU.

Not emulated: the GEMMs (tcgen05, TMA), the streaming per-row quantizer ``quant_token.cu`` (bulk copies and mbarriers;
its requests are answered by the general row kernel here, which computes the same function) and the peer barrier (PTX).
The few helpers that are one PTX instruction on the GPU (NaN-propagating fp32 min / max, the saturating integer packs)
state the instruction's effect in C++ for this build (``AMCT_CUDA_EMU``); the GPU tests check the instruction itself.

This is a check of the kernel source, not a product path: the emulation library is built into a temporary directory
by this test alone, and ``amct_b200`` can neither build nor load it.  What it cannot show is anything that depends on
the GPU itself (hardware conversions, memory ordering, performance); the GPU tests remain the parity tests.
"""
import contextlib
import ctypes
import functools
import inspect
import itertools
import os
import shutil
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, 'amct_b200', 'csrc')
EMU = os.path.join(ROOT, 'tests', 'emu')
CUDA_INCLUDE = os.path.join(os.environ.get('CUDA_HOME', '/usr/local/cuda'), 'include')
EMULATED = ('quant_rows.cu', 'quant_groups.cu', 'reduce.cu', 'norm_quant.cu', 'quant_static.cu', 'mx_quant.cu', 'hif8.cu',
            'w4a16.cu', 'rope.cu', 'ckpt_formats.cu', 'kv_quant.cu', 'gptq_block.cu')


def build(out, sources):
    gxx = shutil.which('g++')
    if gxx is None or not os.path.exists(os.path.join(CUDA_INCLUDE, 'cuda_fp4.h')):
        pytest.skip('needs g++ and the CUDA headers')
    # -fsanitize=alignment: a vector access the GPU would fault on ("misaligned address") aborts the test here
    cmd = [gxx, '-std=c++17', '-O1', '-w', '-ffp-contract=off', '-fsanitize=alignment', '-fno-sanitize-recover=alignment',
           '-fPIC', '-shared', '-x', 'c++', '-include', os.path.join(EMU, 'cuda_emu.h'), '-I', CUDA_INCLUDE, *sources,
           '-o', out, '-lpthread']
    subprocess.check_call(cmd)
    library = ctypes.CDLL(out)
    for name in ('amct_mx_tiled_scale_bytes', 'amct_minmax_workspace_bytes', 'amct_minmax_noalloc_max_k'):
        if hasattr(library, name):
            getattr(library, name).restype = ctypes.c_int64
    if hasattr(library, 'amct_minmax_workspace_bytes'):
        library.amct_minmax_workspace_bytes.argtypes = [ctypes.c_int64]
    return library


_FULL_LIBRARY = {}


def full_library():
    """(path, handle) of the library with all emulated files, built once per test session; the streaming kernel's entry
    declines every shape."""
    if not _FULL_LIBRARY:
        import tempfile
        out = os.path.join(tempfile.mkdtemp(prefix='amct_emu_'), 'libamct_emu.so')
        handle = build(out, [os.path.join(CSRC, f) for f in EMULATED] + [os.path.join(EMU, 'no_streaming_kernel.cpp')])
        _FULL_LIBRARY.update(path=out, handle=handle)
    return _FULL_LIBRARY['path'], _FULL_LIBRARY['handle']


@pytest.fixture(scope='module')
def emu_lib():
    return full_library()[1]


@pytest.fixture(scope='module')
def emu_rows_lib(tmp_path_factory):
    """quant_rows.cu on its own: the specialised kernels it would try first decline every shape, so each request runs
    through the general row kernels -- also the shapes that the group kernel serves in the full library."""
    out = str(tmp_path_factory.mktemp('emu_rows') / 'libamct_emu_rows.so')
    return build(out, [os.path.join(CSRC, 'quant_rows.cu'), os.path.join(EMU, 'no_streaming_kernel.cpp'),
                       os.path.join(EMU, 'no_group_kernel.cpp')])


def patch_ops(monkeypatch, library):
    """The ops wrappers talking to an emulation library with host tensors."""
    from amct_b200.backend import lib, ops
    monkeypatch.setattr(lib, 'load', lambda: library)
    monkeypatch.setattr(ops, '_need_cuda', lambda *tensors: None)
    monkeypatch.setattr(ops, '_stream', lambda: ctypes.c_void_p(0))
    monkeypatch.setattr(ops, 'hadamard_pow2', functools.partial(ops.hadamard_pow2, device='cpu'))
    monkeypatch.setattr(torch.cuda, 'device', lambda device: contextlib.nullcontext())
    monkeypatch.setattr(torch.Tensor, 'cuda', lambda self, *args, **kwargs: self)
    monkeypatch.setattr(torch.Tensor, 'is_cuda', property(lambda self: True))     # wrappers that check their outputs
    return ops


@pytest.fixture
def on_cpu(emu_lib, monkeypatch):
    return patch_ops(monkeypatch, emu_lib)


@pytest.fixture
def rows_on_cpu(emu_rows_lib, monkeypatch):
    return patch_ops(monkeypatch, emu_rows_lib)


def parametrizations(fn):
    """Keyword arguments of every combination of a test function's ``parametrize`` marks."""
    marks = [m for m in getattr(fn, 'pytestmark', []) if m.name == 'parametrize']
    names = [[n.strip() for n in m.args[0].split(',')] for m in marks]
    for combo in itertools.product(*[list(m.args[1]) for m in marks]):
        kwargs = {}
        for group, value in zip(names, combo):
            kwargs.update({group[0]: value} if len(group) == 1 else dict(zip(group, value)))
        yield kwargs


def run_gpu_tests(module, skip=()):
    """Calls every test function of a GPU test module with all its parameters; returns how many ran."""
    ran = 0
    for name, fn in inspect.getmembers(module, inspect.isfunction):
        if not name.startswith('test_') or name in skip:
            continue
        for kwargs in parametrizations(fn):
            try:
                fn(**kwargs)
                ran += 1
            except pytest.skip.Exception:
                pass
    return ran


# ---------------------------------------------------------------------------------------------
# whole GPU test modules on the emulated source
# ---------------------------------------------------------------------------------------------
def test_emulated_integer_quantizers(on_cpu):
    """tests/test_gpu_intq.py: scale rule, every weight granularity, per-token rules, observers, static quantize,
    weight dequantization, against the reference's golden vectors and the oracle.  The two tests aimed at the streaming
    kernel are left out (their shapes are large and the kernel is not emulated)."""
    import test_gpu_intq as G
    ran = run_gpu_tests(G, skip=('test_dynamic_per_token_streaming_kernel', 'test_channel_int8_weight_quant_streaming_path'))
    assert ran > 200


def test_emulated_decoder_glue(on_cpu):
    """tests/test_gpu_glue.py: add + RMSNorm + per-token quantization and the rotary embedding (the two tests that
    build the whole Llama workload need the GEMMs)."""
    import test_gpu_glue as G
    ran = run_gpu_tests(G, skip=('test_workload_fused_glue_matches_unfused_layers',
                                 'test_decode_in_place_kv_cache_matches_concatenation'))
    assert ran > 40


def test_emulated_edge_cases(on_cpu):
    """tests/test_zy_gpu_edge_cases.py through the full library (the group kernel takes the group-wise requests)."""
    import test_zy_gpu_edge_cases as G
    assert run_gpu_tests(G, skip=('test_w8a8_linear_with_one_scale_for_the_whole_weight', 'test_zero_rows_through_the_gemms')) >= 10


def test_emulated_edge_cases_general_kernels(rows_on_cpu):
    """The same through the general row kernels alone (that library holds no other entry point)."""
    import test_zy_gpu_edge_cases as G
    assert run_gpu_tests(G, skip=('test_w8a8_linear_with_one_scale_for_the_whole_weight', 'test_zero_rows_through_the_gemms',
                                  'test_zero_rows_are_a_no_op_in_the_quantizers')) >= 10


def test_emulated_hifloat8(on_cpu):
    import test_gpu_hif8 as G
    assert run_gpu_tests(G, skip=('test_hifloat8_linear_through_the_public_api', 'test_llama_layer_smoothquant_hifloat8_workload')) >= 5


def test_emulated_mx_block_quantization(on_cpu):
    import test_gpu_mx as G
    for fmt in ('fp8', 'fp4'):
        for dtype in (torch.bfloat16, torch.float16, torch.float32):
            for rows, k in [(1, 32), (5, 96), (130, 256), (33, 1024), (8, 8192)]:
                G.test_mx_quant_matches_oracle(fmt, dtype, rows, k)
        G.test_mx_quant_nonfinite_blocks(fmt)
    G.test_mx_roundtrip_properties_full_width()


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
    for on_device in (True, False):
        G.test_clip_ratio_and_per_tensor_modules(dtype, on_device)


def test_emulated_fake_quant_shapes(on_cpu):
    import test_zy_gpu_dsa_activations as G
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        for shape in [(3, 70, 1536), (1000, 128), (5, 16384), (7, 33), (2, 4, 9, 512), (6, 8)]:
            G.test_fake_quant_oracle(dtype, shape)
    G.test_fake_quant_strided_and_cast()
    G.test_fake_quant_scale_underflow_keeps_nan()
    G.test_fake_quant_nan_input_makes_the_row_nan()


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


# ---------------------------------------------------------------------------------------------
# the general row quantizer (quant_rows.cu): weight scales, codes, nibble packing, both fake-quant variants, and the
# per-token rules, with every shape forced through its two general kernels
# ---------------------------------------------------------------------------------------------
def test_emulated_row_quantizer_group_cases(rows_on_cpu):
    import test_gpu_intq as G
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for qt, sym in [('int4', False), ('int4', True), ('int8', False)]:
            for rows, k, gs in [(37, 1024, 128), (5, 512, 64), (16, 96, 48), (3, 200, 64)]:
                G.test_group_weight_quant_oracle(dtype, qt, sym, rows, k, gs)
    for dtype in (torch.bfloat16, torch.float32):
        G.test_group_weight_quant_rounding_ties(dtype)


def test_emulated_row_quantizer_extreme_magnitudes(rows_on_cpu):
    """Channel and group strategies, both rules per token, on magnitudes from 1e-30 to 1e30 (fp16: 1e-7 to 1e4): scales
    that underflow, saturate or are replaced by 1, all-zero and all-negative rows.  Where the oracle raises the
    reference's error for a non-finite scale, so must the kernel's status word."""
    from oracle import intq
    from golden_io import bits_equal
    ops = rows_on_cpu
    gen = torch.Generator().manual_seed(77)

    def attempt(fn):
        try:
            return fn(), None
        except RuntimeError as err:
            return None, err

    case = 0
    for dtype, mags in ((torch.bfloat16, (-30, -12, -3, 0, 4, 30)), (torch.float16, (-7, -5, 0, 4)), (torch.float32, (-30, -6, 0, 10, 30))):
        for mag in mags:
            for strat, gs, k in (('channel', None, 200), ('group', 64, 256), ('group', 48, 96)):
                case += 1
                rows = 3
                w = torch.randn(rows, k, generator=gen) * 10.0 ** mag * torch.exp(torch.randn(rows, 1, generator=gen))
                w = w.clamp(-torch.finfo(dtype).max, torch.finfo(dtype).max).to(dtype)        # finite inputs only
                w[0] = 0
                w[2] = -w[2].abs()
                w[1, ::5] = -0.0                                         # the fake-quant outputs keep the sign of a zero
                qt, sym = ('int8', 'int4')[case % 2], bool(case % 3)
                want, err_o = attempt(lambda: intq.weight_scale_offset(w, qt, sym, strat, gs))
                got, err_k = attempt(lambda: ops.quant_rows(w, qt, sym, strat, gs, out='i32'))
                assert (err_o is None) == (err_k is None), (dtype, mag, strat, qt, sym)
                if err_o is None:
                    scale, offset = want
                    assert bits_equal(got[0].reshape(scale.shape), scale)
                    codes = intq.weight_codes(w, qt, scale, offset, gs)
                    codes = (intq.crop_groups(codes, w.shape) if gs else codes).to(torch.int32).contiguous()
                    assert bits_equal(got[2], codes)
                    fake = ops.quant_rows(w, qt, sym, strat, gs, scale=scale, offset=offset, out='fake')[2]
                    assert bits_equal(fake, intq.fake_quant(w, qt, scale, offset, gs))
                    fake = ops.quant_rows(w, qt, sym, strat, gs, scale=scale, offset=offset, out='fake_awq')[2]
                    assert bits_equal(fake, intq.fake_quant_awq(w, qt, scale, offset, gs))
                for rule in ('released', 'experimental'):
                    want, err_o = attempt(lambda: intq.dynamic_per_token(w, rule))
                    got, err_k = attempt(lambda: ops.quant_dynamic_per_token(w, rule=rule, check=True))
                    assert (err_o is None) == (err_k is None), (dtype, mag, rule)
                    if err_o is None:
                        assert bits_equal(got[0], want[0]) and bits_equal(got[1], want[1]), (dtype, mag, rule)


def test_emulated_minmax_without_workspace(emu_lib):
    """amct_minmax_noalloc against amct_minmax on consecutive calls (column axis twice, tensor axis, a running merge) and
    its size limit, as tests/test_zz_no_alloc.py does on the GPU; the built-in scratch is an ordinary array here."""
    from ctypes import c_int, c_int64, c_void_p
    L = emu_lib
    assert L.amct_minmax_noalloc_max_k() == 16384

    def both(x, axis, merge_from=None):
        rows, k = x.shape
        n = 1 if axis == 0 else k
        dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x.dtype]
        outs = []
        for noalloc in (False, True):
            mn, mx = (torch.empty(n, dtype=x.dtype), torch.empty(n, dtype=x.dtype)) if merge_from is None else \
                (merge_from[0].clone(), merge_from[1].clone())
            head = (c_void_p(x.data_ptr()), c_int(dt), c_int64(rows), c_int64(k), c_int64(x.stride(0)), c_int(axis),
                    c_int(0 if merge_from is None else 1), c_void_p(mn.data_ptr()), c_void_p(mx.data_ptr()))
            if noalloc:
                rc = L.amct_minmax_noalloc(*head, c_void_p(0), c_void_p(0))
            else:
                ws = torch.empty(L.amct_minmax_workspace_bytes(c_int64(k)), dtype=torch.uint8)
                rc = L.amct_minmax(*head, c_void_p(ws.data_ptr()), c_void_p(0), c_void_p(0))
            assert rc == 0, rc
            outs.append((mn, mx))
        return outs

    def same(a, b):
        w = {2: torch.int16, 4: torch.int32}[a.element_size()]
        return bool((a.view(w) == b.view(w)).all())

    gen = torch.Generator().manual_seed(123)
    first = torch.randn(300, 1032, generator=gen).to(torch.bfloat16)
    second = (torch.randn(57, 520, generator=gen) * 3).to(torch.bfloat16)
    third = torch.randn(150, 100, generator=gen)
    prev = None
    for x, axis in ((first, 1), (second, 1), (third, 0), (second, 0), (first, 1)):
        (mn_a, mx_a), (mn_b, mx_b) = both(x, axis)
        assert same(mn_a, mn_b) and same(mx_a, mx_b)
        assert same(mn_b, x.amin(0) if axis == 1 else x.min().reshape(1))
        assert same(mx_b, x.amax(0) if axis == 1 else x.max().reshape(1))
        prev = (mn_b, mx_b) if axis == 1 and x is first else prev
    shifted = (first.float() * 0.5 + 1).to(torch.bfloat16)
    (mn_a, mx_a), (mn_b, mx_b) = both(shifted, 1, merge_from=prev)
    assert same(mn_a, mn_b) and same(mx_a, mx_b) and same(mx_b, torch.maximum(prev[1], shifted.amax(0)))
    k = 16384 + 8
    x = torch.zeros(4, k, dtype=torch.bfloat16)
    mn = torch.full((k,), 7, dtype=torch.bfloat16)
    mx = mn.clone()
    rc = L.amct_minmax_noalloc(c_void_p(x.data_ptr()), c_int(2), c_int64(4), c_int64(k), c_int64(k), c_int(1), c_int(0),
                               c_void_p(mn.data_ptr()), c_void_p(mx.data_ptr()), c_void_p(0), c_void_p(0))
    assert rc == -6 and bool((mn == 7).all()) and bool((mx == 7).all())


def test_emulated_quant_util_functions(on_cpu):
    """amct_b200.utils.quant_util (the reference's utils/quant_util.py by name) against the oracle's restatement of the
    same functions: integer codes in the reference's grouped shape, ragged tail included, and the fake quantization."""
    from golden_io import bits_equal
    from oracle import intq
    from amct_b200.utils import quant_util as U
    gen = torch.Generator().manual_seed(61)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        w = (torch.randn(9, 200, generator=gen) * 0.05).to(dtype)
        for qt, sym, strategy, gs in (('int8', True, 'channel', None), ('int8', False, 'tensor', None),
                                      ('int4', False, 'group', 64), ('int4', True, 'group', 32), ('int8', False, 'group', 128)):
            scale, offset = intq.weight_scale_offset(w, qt, sym, strategy, gs)
            codes = U.quant_weight(w, qt, scale, offset, gs)
            want = intq.weight_codes(w, qt, scale, offset, gs)
            assert codes.shape == want.shape and bits_equal(codes, want.to(codes.dtype))
            assert codes.dtype == (torch.int8 if qt == 'int8' else torch.int32)
            params = {'weights_cfg': {'quant_type': qt, 'group_size': gs}}
            assert bits_equal(U.quant_dequant_weight(w, params, scale, offset), intq.fake_quant(w, qt, scale, offset, gs))
        t = (torch.randn(3, 5, 16, generator=gen) * 60).to(dtype)
        assert bits_equal(U.convert_dtype(t, 'int8'), t.float().round().clamp(-128, 127).to(torch.int8))
        assert bits_equal(U.convert_dtype(t, 'int4'), t.float().round().clamp(-8, 7).to(torch.int32))


def test_emulated_awq_helpers(on_cpu):
    """convert_precision, calculate_scale_offset_by_granularity and process_weights_for_layers (the reference's AWQ
    helpers by name) against the oracle's statement of do_quant -> convert_precision -> do_dequant."""
    from golden_io import bits_equal
    from oracle import intq
    from amct_b200.algorithm import awq
    from amct_b200.utils.data_utils import convert_precision
    gen = torch.Generator().manual_seed(62)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        t = (torch.randn(4, 3, 40, generator=gen) * 6).to(dtype)
        assert bits_equal(convert_precision(t, 'int4'), t.float().round().clamp(-8, 7).to(dtype))
        w = (torch.randn(6, 256, generator=gen) * 0.05).to(dtype)
        s = (torch.rand(1, 256, generator=gen) + 0.5).to(dtype)
        cfg = {'weights_cfg': {'quant_type': 'int4', 'symmetric': False, 'strategy': 'group', 'group_size': 64}}
        scale, offset = awq.calculate_scale_offset_by_granularity(w * s, cfg)
        want_scale, want_offset = intq.weight_scale_offset(w * s, 'int4', False, 'group', 64)
        assert bits_equal(scale, want_scale) and bits_equal(offset, want_offset.to(offset.dtype))
        layer = torch.nn.Linear(256, 6, bias=False).to(dtype)
        layer.weight.data = w.clone()
        awq.process_weights_for_layers([layer], s, cfg)
        assert bits_equal(layer.weight.data, intq.fake_quant_awq(w * s, 'int4', want_scale, want_offset, 64) / s)


# ---------------------------------------------------------------------------------------------
# GPTQ block update
# ---------------------------------------------------------------------------------------------
def test_emulated_gptq_block(on_cpu):
    import test_gpu_awq_gptq as G
    for args in G.GPTQ_BLOCK_CASES:
        G.test_gptq_block_kernel_matches_column_loop(*args)
