"""Torch-tensor front end of the C-ABI kernels.

Every function takes CUDA tensors, allocates its outputs with torch (device
memory and streams are torch's), and enqueues the kernel on the current stream.
Nothing here computes on the CPU: a CPU tensor raises.
"""
import ctypes
from ctypes import c_int, c_int64, c_void_p

import torch

from . import lib as _l

_DT = {torch.float32: _l.DTYPE_F32, torch.float16: _l.DTYPE_F16, torch.bfloat16: _l.DTYPE_BF16}
# launches of this library's kernels since the counter was last reset (bench.py reads it)
COUNTERS = {'launches': 0}
# when set to a list, every GEMM launch appends (start event, end event, 2*M*N*K, stream handle)
GEMM_PROFILE = None

SCALE_ERROR = "Param scale has invalid value inf, nan or zeros!"      # amct_pytorch/quantize_op/utils.py:66-67


def _p(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise _l.BackendError('amct_b200 kernels need CUDA tensors (there is no CPU fallback)')


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise _l.BackendError(f'unsupported dtype {t.dtype}; float32/float16/bfloat16 only') from None


def _rows2d(x):
    """View as [rows, k] with unit inner stride; returns (tensor, rows, k, ld)."""
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) < k):
        x2 = x2.contiguous()
    ld = x2.stride(0) if x2.shape[0] > 1 else k
    return x2, x2.shape[0], k, ld


_STATUS_WORDS = {}


class Status:
    """Device word the kernels OR error bits into, read back by ``raise_if_set``.  One word per (device, stream) is
    allocated once and shared by all calls on that stream: it is zero between calls because every call that passes
    it to a kernel reads it back afterwards, in stream order, and clears it if a bit was set."""

    def __init__(self, device):
        device = torch.device(device)
        index = device.index if device.index is not None else (torch.cuda.current_device() if device.type == 'cuda' else -1)
        key = (device.type, index, _stream().value)
        word = _STATUS_WORDS.get(key)
        if word is None:
            word = torch.zeros(1, dtype=torch.int32, device=device)
            _STATUS_WORDS[key] = word
        self.word = word

    def ptr(self):
        return _p(self.word)

    def raise_if_set(self):
        bits = int(self.word.item())
        if bits:
            self.word.zero_()
        if bits & 1:
            raise RuntimeError(SCALE_ERROR)


def bits_of(quant_type):
    return int(quant_type.replace('int', ''))


# ---------------------------------------------------------------------------
def quant_dynamic_per_token(x, smooth=None, rule='released', check=False):
    """Per-row symmetric INT8 codes and fp32 scales of x[..., K] in one pass."""
    _need_cuda(x, smooth)
    x2, rows, k, ld = _rows2d(x)
    q = torch.empty((rows, k), dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    st = Status(x.device) if check else None
    if smooth is not None:
        smooth = smooth.reshape(-1).to(x.dtype).contiguous()
        assert smooth.numel() == k
    rc = _l.load().amct_quant_dynamic_pertoken(
        _p(x2), c_int(_dt(x2)), c_int64(rows), c_int64(k), c_int64(ld), _p(smooth), c_int(_l.RULE[rule]),
        _p(q), c_int64(k), _p(scale), st.ptr() if st else c_void_p(0), _stream())
    _l.check(rc, 'amct_quant_dynamic_pertoken')
    COUNTERS['launches'] += 1
    if st:
        st.raise_if_set()
    return q.reshape(x.shape), scale


def _unit_count(rows, k, strategy, group):
    if strategy == 'tensor':
        return 1, 1
    if strategy == 'channel':
        return rows, 1
    g = (k + group - 1) // group
    return rows * g, g


def quant_rows(w, quant_type, symmetric, strategy, group=None, scale=None, offset=None, out='none',
               pre=None, pre_op='none', check=True):
    """Row kernel front end.

    scale is None  -> derive scale/offset from `w` (strategy channel or group).
    out: 'none' | 'i8' | 'i32' | 'pack4' | 'fake' | 'fake_awq'.
    Returns (scale flat fp32, offset flat int32 | None, out tensor | None).
    """
    _need_cuda(w, scale, offset, pre)
    assert w.dim() == 2
    w2, rows, k, ld = _rows2d(w)
    bits = bits_of(quant_type)
    compute = scale is None
    nunits, _ = _unit_count(rows, k, strategy, group)
    if compute:
        scale = torch.empty(nunits, dtype=torch.float32, device=w.device)
        offset = None if symmetric else torch.empty(nunits, dtype=torch.int32, device=w.device)
    else:
        scale = scale.reshape(-1).to(torch.float32).contiguous()
        offset = None if offset is None else offset.reshape(-1).to(torch.int32).contiguous()
        assert scale.numel() == nunits, (scale.numel(), nunits)
    mode = {'none': _l.OUT_NONE, 'i8': _l.OUT_I8, 'i32': _l.OUT_I32, 'pack4': _l.OUT_PACK4,
            'fake': _l.OUT_FAKE, 'fake_awq': _l.OUT_FAKE_AWQ}[out]
    o, ld_out = None, 0
    if out == 'i8':
        o = torch.empty((rows, k), dtype=torch.int8, device=w.device)
    elif out == 'i32':
        o = torch.empty((rows, k), dtype=torch.int32, device=w.device)
    elif out == 'pack4':
        o = torch.empty((rows, (k + 1) // 2), dtype=torch.uint8, device=w.device)
    elif out in ('fake', 'fake_awq'):
        o = torch.empty((rows, k), dtype=w.dtype, device=w.device)
    if o is not None:
        ld_out = o.stride(0)
    pop = {'none': _l.PRE_NONE, 'mul': _l.PRE_MUL, 'div': _l.PRE_DIV}[pre_op]
    if pre is not None:
        pre = pre.reshape(-1).to(w.dtype).contiguous()
        assert pre.numel() == k
    st = Status(w.device) if check else None
    sym_flag = 1 if (symmetric or offset is None) else 0
    rc = _l.load().amct_quant_rows(
        _p(w2), c_int(_dt(w2)), c_int64(rows), c_int64(k), c_int64(ld), _p(pre), c_int(pop),
        c_int(1 if compute else 0), c_int(_l.STRATEGY[strategy]), c_int(group or 0), c_int(bits),
        c_int(sym_flag), _p(scale), _p(offset), c_int(mode), _p(o), c_int64(ld_out),
        st.ptr() if st else c_void_p(0), _stream())
    _l.check(rc, 'amct_quant_rows')
    COUNTERS['launches'] += 1
    if st:
        st.raise_if_set()
    return scale, offset, o


def minmax(x, axis, running=None):
    """(min, max) of x viewed as [rows, K]: axis 'tensor' -> shape [1], 'column' -> [1, K].
    running=(min, max) tensors are updated in place and returned."""
    _need_cuda(x)
    x2, rows, k, ld = _rows2d(x)
    n = 1 if axis == 'tensor' else k
    if running is None:
        mn = torch.empty(n, dtype=x.dtype, device=x.device)
        mx = torch.empty(n, dtype=x.dtype, device=x.device)
        merge = 0
    else:
        mn, mx = running
        assert mn.is_contiguous() and mx.is_contiguous() and mn.numel() == n and mn.dtype == x.dtype
        merge = 1
    L = _l.load()
    ws = torch.empty(L.amct_minmax_workspace_bytes(c_int64(k)), dtype=torch.uint8, device=x.device)
    # no status word: a NaN in the input shows in the result, and the scale rule refuses it there
    rc = L.amct_minmax(_p(x2), c_int(_dt(x2)), c_int64(rows), c_int64(k), c_int64(ld),
                       c_int(_l.AXIS_TENSOR if axis == 'tensor' else _l.AXIS_COLUMN), c_int(merge),
                       _p(mn), _p(mx), _p(ws), c_void_p(0), _stream())
    _l.check(rc, 'amct_minmax')
    COUNTERS['launches'] += 2
    if axis == 'column':
        return mn.reshape(1, k), mx.reshape(1, k)
    return mn, mx


def scale_offset(vmax, vmin, symmetric, quant_type):
    """calculate_scale_offset on device; keeps the shape of vmax."""
    _need_cuda(vmax, vmin)
    shape = vmax.shape
    a = vmax.reshape(-1).contiguous()
    b = vmin.reshape(-1).to(a.dtype).contiguous()
    n = a.numel()
    scale = torch.empty(n, dtype=torch.float32, device=a.device)
    offset = None if symmetric else torch.empty(n, dtype=torch.int32, device=a.device)
    st = Status(a.device)
    rc = _l.load().amct_scale_offset(_p(a), _p(b), c_int(_dt(a)), c_int64(n), c_int(bits_of(quant_type)),
                                     c_int(1 if symmetric else 0), _p(scale), _p(offset), st.ptr(), _stream())
    _l.check(rc, 'amct_scale_offset')
    COUNTERS['launches'] += 1
    st.raise_if_set()
    return scale.reshape(shape), None if offset is None else offset.reshape(shape)


def quantize_static(x, scales, zero_points, axis=-1, smooth=None):
    """npu_quantize(..., dtype=int8, div_mode=False): per-tensor (one scale) or per-token (axis=-2)."""
    _need_cuda(x, scales, zero_points, smooth)
    x = x.contiguous()
    k = x.shape[-1]
    per_token = scales.numel() != 1
    tokens = x.shape[-2] if x.dim() >= 2 else 1
    if per_token:
        if axis not in (-2, x.dim() - 2) or scales.numel() != tokens:
            raise _l.BackendError('per-token scales need axis=-2 and one scale per token position')
    outer = x.numel() // (tokens * k) if x.numel() else 0
    s = scales.reshape(-1).to(x.dtype).contiguous()
    z = None if zero_points is None else zero_points.reshape(-1).to(x.dtype).contiguous()
    if z is not None and z.numel() != s.numel():
        z = z.expand(s.numel()).contiguous()
    if smooth is not None:
        smooth = smooth.reshape(-1).to(x.dtype).contiguous()
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    rc = _l.load().amct_quantize_static(_p(x), c_int(_dt(x)), c_int64(outer), c_int64(tokens), c_int64(k),
                                        _p(s), _p(z), c_int(1 if per_token else 0), _p(smooth), _p(q), _stream())
    _l.check(rc, 'amct_quantize_static')
    COUNTERS['launches'] += 1
    return q


def rowsum_i8(wq_nk):
    _need_cuda(wq_nk)
    assert wq_nk.dtype == torch.int8 and wq_nk.dim() == 2 and wq_nk.stride(1) == 1
    out = torch.empty(wq_nk.shape[0], dtype=torch.int32, device=wq_nk.device)
    rc = _l.load().amct_rowsum_i8(_p(wq_nk), c_int64(wq_nk.shape[0]), c_int64(wq_nk.shape[1]),
                                  c_int64(wq_nk.stride(0)), _p(out), _stream())
    _l.check(rc, 'amct_rowsum_i8')
    COUNTERS['launches'] += 1
    return out


def transpose_i8(t):
    _need_cuda(t)
    t = t.contiguous()
    out = torch.empty((t.shape[1], t.shape[0]), dtype=t.dtype, device=t.device)
    rc = _l.load().amct_transpose_i8(_p(t), c_int64(t.shape[0]), c_int64(t.shape[1]), _p(out), _stream())
    _l.check(rc, 'amct_transpose_i8')
    COUNTERS['launches'] += 1
    return out


# ---------------------------------------------------------------------------
# tensor-core GEMMs
_OUT_KIND = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.int32: 3}
_BIAS_KIND = {torch.int32: 1, torch.float32: 2, torch.float16: 3, torch.bfloat16: 4}


def _prof_begin():
    if GEMM_PROFILE is None:
        return None
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    return e


def _prof_end(start, n_ops):
    if start is not None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        GEMM_PROFILE.append((start, e, n_ops, _stream().value))


def _kmajor(t):
    """[R, K] tensor with unit K stride and a 16-byte aligned leading dimension."""
    if t.stride(-1) != 1 or (t.stride(0) * t.element_size()) % 16 or t.data_ptr() % 16:
        t = t.contiguous()
    if (t.stride(0) * t.element_size()) % 16:
        raise _l.BackendError('K * element size must be a multiple of 16 bytes for the TMA-fed GEMM')
    return t


def raise_if_timed_out(status_word):
    if int(status_word.item()) & 2:
        raise _l.BackendError('a device-side wait in the GEMM kernel timed out')


def gemm_w8a8(q, w_nk, deq_scale=None, pertoken_scale=None, bias=None, out_dtype=torch.bfloat16, out=None,
              status=None):
    """q int8 [M, K] x w_nk int8 [N, K] (K-major) -> [M, N] with the W8A8 dequant epilogue;
    out_dtype=torch.int32 returns the raw accumulators."""
    _need_cuda(q, w_nk, deq_scale, pertoken_scale, bias)
    assert q.dtype == torch.int8 and w_nk.dtype == torch.int8 and q.dim() == 2 and w_nk.dim() == 2
    q, w_nk = _kmajor(q), _kmajor(w_nk)
    m, k = q.shape
    n = w_nk.shape[0]
    assert w_nk.shape[1] == k
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=q.device)
    if deq_scale is not None:
        deq_scale = deq_scale.reshape(-1).to(torch.float32).contiguous()
        assert deq_scale.numel() == n
    if pertoken_scale is not None:
        pertoken_scale = pertoken_scale.reshape(-1).to(torch.float32).contiguous()
        assert pertoken_scale.numel() == m
    bk = 0
    if bias is not None:
        bias = bias.reshape(-1).contiguous()
        bk = _BIAS_KIND[bias.dtype]
    prof = _prof_begin()
    rc = _l.load().amct_gemm_w8a8(
        _p(q), _p(w_nk), c_int64(m), c_int64(n), c_int64(k), c_int64(q.stride(0)), c_int64(w_nk.stride(0)),
        _p(deq_scale), _p(pertoken_scale), _p(bias), c_int(bk), _p(out), c_int(_OUT_KIND[out.dtype]),
        c_int64(out.stride(0)), _p(status) if status is not None else c_void_p(0), _stream())
    _l.check(rc, 'amct_gemm_w8a8')
    COUNTERS['launches'] += 1
    _prof_end(prof, 2 * m * n * k)
    return out


MMA_KINDS = {'i8': 0, 'bf16': 1, 'mxf8': 2, 'mxf4': 3}


def mma_peak(kind, steps=20000, ctas=None, status=None):
    """Enqueues the MMA-only kernel (tensor-core peak measurement) and returns the operations it performs."""
    L = _l.load()
    if ctas is None:
        ctas = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    code = MMA_KINDS[kind]
    rc = L.amct_mma_peak(c_int(code), c_int(steps), c_int(ctas), _p(status) if status is not None else c_void_p(0), _stream())
    _l.check(rc, 'amct_mma_peak')
    COUNTERS['launches'] += 1
    return ctas * steps * int(L.amct_mma_peak_ops_per_cta_step(c_int(code)))


def set_gemm_variant(variant):
    """Pins the kernel that takes GEMMs with more than 128 rows: 'auto' (by the size of the weight), 'single' (one-CTA
    kernel) or 'pair' (CTA-pair kernel).  Process-wide; for tests and comparisons."""
    code = {'auto': 0, 'single': 1, 'pair': 2}[variant]
    _l.check(_l.load().amct_gemm_set_variant(c_int(code)), 'amct_gemm_set_variant')


def _pointer_array(pointers):
    return (c_void_p * len(pointers))(*[int(p_) for p_ in pointers])


def gemm_w8a8_scatter(q, w_nk, deq_scale, pertoken_scale, out_ptrs, slot, rows_per_rank, ld_out, out_dtype=torch.bfloat16,
                      status=None):
    """The W8A8 GEMM of a K-sharded Linear whose result is this rank's partial sum: output row r is written to row
    (slot * rows_per_rank + r % rows_per_rank) of the staging buffer of rank r // rows_per_rank.  out_ptrs: device
    addresses of every rank's staging buffer [world * rows_per_rank, ld_out] as mapped into this process."""
    _need_cuda(q, w_nk, deq_scale, pertoken_scale)
    assert q.dtype == torch.int8 and w_nk.dtype == torch.int8 and q.dim() == 2 and w_nk.dim() == 2
    q, w_nk = _kmajor(q), _kmajor(w_nk)
    m, k = q.shape
    n = w_nk.shape[0]
    assert w_nk.shape[1] == k
    deq_scale = deq_scale.reshape(-1).to(torch.float32).contiguous()
    assert deq_scale.numel() == n
    if pertoken_scale is not None:
        pertoken_scale = pertoken_scale.reshape(-1).to(torch.float32).contiguous()
        assert pertoken_scale.numel() == m
    prof = _prof_begin()
    rc = _l.load().amct_gemm_w8a8_scatter(
        _p(q), _p(w_nk), c_int64(m), c_int64(n), c_int64(k), c_int64(q.stride(0)), c_int64(w_nk.stride(0)),
        _p(deq_scale), _p(pertoken_scale), _pointer_array(out_ptrs), c_int(len(out_ptrs)), c_int(slot),
        c_int64(rows_per_rank), c_int(_OUT_KIND[out_dtype]), c_int64(ld_out),
        _p(status) if status is not None else c_void_p(0), _stream())
    _l.check(rc, 'amct_gemm_w8a8_scatter')
    COUNTERS['launches'] += 1
    _prof_end(prof, 2 * m * n * k)


def gemm_f16(a, b_nk, bias=None, out_dtype=None, out=None, status=None):
    """a [M, K] x b_nk [N, K] in fp16 or bf16 -> [M, N], fp32 accumulation."""
    _need_cuda(a, b_nk, bias)
    assert a.dtype == b_nk.dtype and a.dtype in (torch.float16, torch.bfloat16)
    a, b_nk = _kmajor(a), _kmajor(b_nk)
    m, k = a.shape
    n = b_nk.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    bk = 0
    if bias is not None:
        bias = bias.reshape(-1).contiguous()
        bk = _BIAS_KIND[bias.dtype]
    prof = _prof_begin()
    rc = _l.load().amct_gemm_f16(
        _p(a), _p(b_nk), c_int(_dt(a)), c_int64(m), c_int64(n), c_int64(k), c_int64(a.stride(0)),
        c_int64(b_nk.stride(0)), _p(bias), c_int(bk), _p(out), c_int(_OUT_KIND[out.dtype]), c_int64(out.stride(0)),
        _p(status) if status is not None else c_void_p(0), _stream())
    _l.check(rc, 'amct_gemm_f16')
    COUNTERS['launches'] += 1
    _prof_end(prof, 2 * m * n * k)
    return out


def minmax_rows(x2d, pre=None, pre_op='none', running=None):
    """(min, max) per row of a [rows, K] view, optional element-wise pre-scale [K] in x's dtype."""
    _need_cuda(x2d, pre)
    x2, rows, k, ld = _rows2d(x2d)
    if running is None:
        mn = torch.empty(rows, dtype=x2.dtype, device=x2.device)
        mx = torch.empty(rows, dtype=x2.dtype, device=x2.device)
        merge = 0
    else:
        mn, mx = running
        merge = 1
    if pre is not None:
        pre = pre.reshape(-1).to(x2.dtype).contiguous()
        assert pre.numel() == k
    pop = {'none': _l.PRE_NONE, 'mul': _l.PRE_MUL, 'div': _l.PRE_DIV}[pre_op]
    rc = _l.load().amct_minmax_rows(_p(x2), c_int(_dt(x2)), c_int64(rows), c_int64(k), c_int64(ld), _p(pre), c_int(pop),
                                    c_int(merge), _p(mn), _p(mx), c_void_p(0), _stream())
    _l.check(rc, 'amct_minmax_rows')
    COUNTERS['launches'] += 1
    return mn, mx


def dequant_weight(codes_nk, bits, scale_gn, offset_gn, group, out=None):
    """K-major weight codes -> [N, K] weight in the dtype of scale_gn (fp16/bf16)."""
    _need_cuda(codes_nk, scale_gn, offset_gn)
    n = codes_nk.shape[0]
    k = codes_nk.shape[1] * (2 if bits == 4 else 1)
    assert codes_nk.stride(1) == 1
    scale_gn = scale_gn.contiguous()
    if offset_gn is not None:
        offset_gn = offset_gn.to(scale_gn.dtype).contiguous()
    if out is None:
        out = torch.empty((n, k), dtype=scale_gn.dtype, device=codes_nk.device)
    rc = _l.load().amct_dequant_weight(_p(codes_nk), c_int(bits), c_int64(n), c_int64(k), c_int64(codes_nk.stride(0)),
                                       _p(scale_gn), _p(offset_gn), c_int(group or 0), c_int(_dt(scale_gn)), _p(out),
                                       c_int64(out.stride(0)), _stream())
    _l.check(rc, 'amct_dequant_weight')
    COUNTERS['launches'] += 1
    return out


def gemm_w4a16(x, codes_nk, bits, scale_gn, offset_gn, group, bias=None, out_dtype=None, out=None, status=None):
    """x [M, K] (fp16 / bf16) times the group-dequantized weight, one kernel (dequant in shared
    memory ahead of the MMA).  Returns None when the shape is outside what the fused kernel takes
    (the caller then uses dequant_weight + gemm_f16)."""
    _need_cuda(x, codes_nk, scale_gn, offset_gn, bias)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise _l.BackendError('gemm_w4a16: float16 / bfloat16 activations only')
    x = _kmajor(x)
    m, k = x.shape
    n = codes_nk.shape[0]
    assert codes_nk.stride(1) == 1 and codes_nk.shape[1] * (2 if bits == 4 else 1) == k
    scale_gn = scale_gn.to(x.dtype).contiguous()
    if offset_gn is not None:
        offset_gn = offset_gn.to(x.dtype).contiguous()
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    bk = 0
    if bias is not None:
        bias = bias.reshape(-1).contiguous()
        bk = _BIAS_KIND[bias.dtype]
    prof = _prof_begin()
    rc = _l.load().amct_gemm_w4a16(
        _p(x), c_int(_dt(x)), _p(codes_nk), c_int(bits), c_int64(m), c_int64(n), c_int64(k), c_int64(x.stride(0)),
        c_int64(codes_nk.stride(0)), _p(scale_gn), _p(offset_gn), c_int(group or 0), _p(bias), c_int(bk), _p(out),
        c_int(_OUT_KIND[out.dtype]), c_int64(out.stride(0)), _p(status) if status is not None else c_void_p(0), _stream())
    if rc in (-4, -2):            # AMCT_ERR_UNSUPPORTED, AMCT_ERR_ALIGN: the caller takes the two-kernel route
        return None
    _l.check(rc, 'amct_gemm_w4a16')
    COUNTERS['launches'] += 1
    _prof_end(prof, 2 * m * n * k)
    return out


_HIF8_LUT = {}


def gemm_hif8_weight(x, codes_nk, bias=None, out_dtype=None, out=None, status=None):
    """x [M, K] (fp16 / bf16) times HiFloat8 weight codes [N, K], decoded exactly in shared memory
    ahead of the MMA.  Returns None for shapes the fused kernel does not take."""
    _need_cuda(x, codes_nk, bias)
    x = _kmajor(x)
    m, k = x.shape
    n = codes_nk.shape[0]
    assert codes_nk.dtype == torch.uint8 and codes_nk.stride(1) == 1 and codes_nk.shape[1] == k
    key = (x.device, x.dtype)
    if key not in _HIF8_LUT:
        _HIF8_LUT[key] = hif8_decode(torch.arange(256, dtype=torch.uint8, device=x.device), dtype=x.dtype)
    lut = _HIF8_LUT[key]
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    bk = 0
    if bias is not None:
        bias = bias.reshape(-1).contiguous()
        bk = _BIAS_KIND[bias.dtype]
    prof = _prof_begin()
    rc = _l.load().amct_gemm_lut8(
        _p(x), c_int(_dt(x)), _p(codes_nk), _p(lut), c_int64(m), c_int64(n), c_int64(k), c_int64(x.stride(0)),
        c_int64(codes_nk.stride(0)), _p(bias), c_int(bk), _p(out), c_int(_OUT_KIND[out.dtype]), c_int64(out.stride(0)),
        _p(status) if status is not None else c_void_p(0), _stream())
    if rc in (-4, -2):
        return None
    _l.check(rc, 'amct_gemm_lut8')
    COUNTERS['launches'] += 1
    _prof_end(prof, 2 * m * n * k)
    return out


def minmax_noalloc(x, axis, out_min, out_max, merge=False):
    """amct_minmax without a workspace and without any allocation: the caller passes the
    input and both outputs (in x's dtype; 1 element for axis 'tensor', K for 'column').
    For hosts that must not allocate device memory after start-up.  Column axis: K up to
    16384.  Calls share one built-in scratch array, so calls that could overlap on the
    GPU must be ordered by the caller."""
    _need_cuda(x, out_min, out_max)
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1:
        raise _l.BackendError('minmax_noalloc needs unit inner stride (it will not make a contiguous copy)')
    rows = x2.shape[0]
    ld = x2.stride(0) if rows > 1 else k
    n = 1 if axis == 'tensor' else k
    assert out_min.numel() == n and out_max.numel() == n and out_min.dtype == x.dtype and out_max.dtype == x.dtype
    assert out_min.is_contiguous() and out_max.is_contiguous()
    rc = _l.load().amct_minmax_noalloc(_p(x2), c_int(_dt(x2)), c_int64(rows), c_int64(k), c_int64(ld),
                                       c_int(_l.AXIS_TENSOR if axis == 'tensor' else _l.AXIS_COLUMN),
                                       c_int(1 if merge else 0), _p(out_min), _p(out_max), c_void_p(0), _stream())
    _l.check(rc, 'amct_minmax_noalloc')
    COUNTERS['launches'] += 2


# ---------------------------------------------------------------------------
# MX formats
MX_TILE_ROWS = {'a': 128, 'b': 224}


def mx_quant(x, fmt, operand='a', tiled=True, rowmajor=True):
    """x [R, K] -> (payload uint8, scales_rowmajor uint8 [R, K/32] | None, scales_tiled uint8 | None).
    fmt 'fp8' (E4M3, payload [R, K]) or 'fp4' (E2M1, payload [R, K/2]).  operand 'a' / 'b' picks the
    tiling of scales_tiled for the A resp. B side of gemm_mx."""
    _need_cuda(x)
    assert x.dim() == 2
    x2, rows, k, ld = _rows2d(x)
    bits = {'fp8': 8, 'fp4': 4}[fmt]
    payload = torch.empty((rows, k if bits == 8 else k // 2), dtype=torch.uint8, device=x.device)
    srm = torch.empty((rows, k // 32), dtype=torch.uint8, device=x.device) if rowmajor else None
    L = _l.load()
    st = None
    if tiled:
        # the kernel writes the layout's padding itself: no clearing pass over the buffer
        st = torch.empty(L.amct_mx_tiled_scale_bytes(c_int64(rows), c_int64(k), c_int(MX_TILE_ROWS[operand])),
                         dtype=torch.uint8, device=x.device)
    rc = L.amct_mx_quant(_p(x2), c_int(_dt(x2)), c_int64(rows), c_int64(k), c_int64(ld), c_int(bits), _p(payload),
                         _p(srm), _p(st), c_int(MX_TILE_ROWS[operand]), _stream())
    _l.check(rc, 'amct_mx_quant')
    COUNTERS['launches'] += 1
    return payload, srm, st


def gemm_mx(a_payload, a_scales_tiled, b_payload, b_scales_tiled, fmt, bias=None, out_dtype=torch.bfloat16, out=None,
            status=None):
    """Block-scaled GEMM of two MX tensors produced by mx_quant: [M, K] x [N, K] -> [M, N]."""
    _need_cuda(a_payload, a_scales_tiled, b_payload, b_scales_tiled, bias)
    bits = {'fp8': 8, 'fp4': 4}[fmt]
    m, n = a_payload.shape[0], b_payload.shape[0]
    k = a_payload.shape[1] * (2 if bits == 4 else 1)
    assert b_payload.shape[1] == a_payload.shape[1] and a_payload.stride(1) == 1 and b_payload.stride(1) == 1
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a_payload.device)
    bk = 0
    if bias is not None:
        bias = bias.reshape(-1).contiguous()
        bk = _BIAS_KIND[bias.dtype]
    prof = _prof_begin()
    rc = _l.load().amct_gemm_mx(_p(a_payload), _p(a_scales_tiled), _p(b_payload), _p(b_scales_tiled), c_int(bits),
                                c_int64(m), c_int64(n), c_int64(k), c_int64(a_payload.stride(0)), c_int64(b_payload.stride(0)),
                                _p(bias), c_int(bk), _p(out), c_int(_OUT_KIND[out.dtype]), c_int64(out.stride(0)),
                                _p(status) if status is not None else c_void_p(0), _stream())
    _l.check(rc, 'amct_gemm_mx')
    COUNTERS['launches'] += 1
    _prof_end(prof, 2 * m * n * k)
    return out


# ---------------------------------------------------------------------------
# HiFloat8
def hif8_encode(x):
    """x (any shape, contiguous) -> uint8 HiF8 codes of the same shape."""
    _need_cuda(x)
    x = x.contiguous()
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    rc = _l.load().amct_hif8_encode(_p(x), c_int(_dt(x)), c_int64(x.numel()), _p(codes), c_void_p(0), _stream())
    _l.check(rc, 'amct_hif8_encode')
    COUNTERS['launches'] += 1
    return codes


def hif8_fake_quant(x):
    """decode(encode(x)) in x's dtype, one pass."""
    _need_cuda(x)
    x = x.contiguous()
    out = torch.empty_like(x)
    rc = _l.load().amct_hif8_encode(_p(x), c_int(_dt(x)), c_int64(x.numel()), c_void_p(0), _p(out), _stream())
    _l.check(rc, 'amct_hif8_encode')
    COUNTERS['launches'] += 1
    return out


def hif8_decode(codes, dtype=torch.bfloat16, out=None):
    _need_cuda(codes)
    codes = codes.contiguous()
    if out is None:
        out = torch.empty(codes.shape, dtype=dtype, device=codes.device)
    rc = _l.load().amct_hif8_decode(_p(codes), c_int64(codes.numel()), c_int(_DT[out.dtype]), _p(out), _stream())
    _l.check(rc, 'amct_hif8_decode')
    COUNTERS['launches'] += 1
    return out


def gemm_w8a8_swiglu(q, w_nk, deq_scale, pertoken_scale=None, bias=None, out=None, status=None):
    """W8A8 GEMM of a gate/up projection with 128-row interleaved weights and a fused SwiGLU
    epilogue: returns bf16 [M, N/2]."""
    _need_cuda(q, w_nk, deq_scale, pertoken_scale, bias)
    q, w_nk = _kmajor(q), _kmajor(w_nk)
    m, k = q.shape
    n = w_nk.shape[0]
    if out is None:
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=q.device)
    deq_scale = deq_scale.reshape(-1).to(torch.float32).contiguous()
    if pertoken_scale is not None:
        pertoken_scale = pertoken_scale.reshape(-1).to(torch.float32).contiguous()
    bk = 0
    if bias is not None:
        bias = bias.reshape(-1).contiguous()
        bk = _BIAS_KIND[bias.dtype]
    prof = _prof_begin()
    rc = _l.load().amct_gemm_w8a8_swiglu(
        _p(q), _p(w_nk), c_int64(m), c_int64(n), c_int64(k), c_int64(q.stride(0)), c_int64(w_nk.stride(0)),
        _p(deq_scale), _p(pertoken_scale), _p(bias), c_int(bk), _p(out), c_int64(out.stride(0)),
        _p(status) if status is not None else c_void_p(0), _stream())
    _l.check(rc, 'amct_gemm_w8a8_swiglu')
    COUNTERS['launches'] += 1
    _prof_end(prof, 2 * m * n * k)
    return out


def addnorm_quant_per_token(x, gamma, eps, residual=None, want_norm=False, check=False, out_q=None, out_scale=None):
    """(x [+ residual]) -> RMSNorm -> dynamic per-token INT8 codes, one kernel.

    Returns (q int8 like x, scale fp32 [rows], h, n): h = x + residual in x's dtype (None without
    residual), n = the normalised values the codes were taken from (only with want_norm).
    out_q (int8 [rows, K] contiguous) / out_scale (fp32 [rows]) receive the codes and scales in
    place, e.g. a rank's slice of an all-gather buffer."""
    _need_cuda(x, gamma, residual)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise _l.BackendError('addnorm_quant_per_token: float16 / bfloat16 only')
    x2, rows, k, ld = _rows2d(x)
    r2, ld_r = None, 0
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError('residual must match x in shape and dtype')
        r2, _, _, ld_r = _rows2d(residual)
    gamma = gamma.reshape(-1).to(x.dtype).contiguous()
    if gamma.numel() != k:
        raise ValueError('gamma must have K elements')
    q = out_q if out_q is not None else torch.empty((rows, k), dtype=torch.int8, device=x.device)
    scale = out_scale if out_scale is not None else torch.empty(rows, dtype=torch.float32, device=x.device)
    if q.dtype != torch.int8 or q.numel() != rows * k or not q.is_contiguous() or not q.is_cuda:
        raise ValueError('out_q must be a contiguous CUDA int8 tensor of rows * K elements')
    if scale.dtype != torch.float32 or scale.numel() != rows or not scale.is_contiguous() or not scale.is_cuda:
        raise ValueError('out_scale must be a contiguous CUDA float32 tensor of `rows` elements')
    h = torch.empty((rows, k), dtype=x.dtype, device=x.device) if residual is not None else None
    n = torch.empty((rows, k), dtype=x.dtype, device=x.device) if want_norm else None
    st = Status(x.device) if check else None
    rc = _l.load().amct_addnorm_quant_pertoken(
        _p(x2), _p(r2), c_int(_dt(x2)), c_int64(rows), c_int64(k), c_int64(ld), c_int64(ld_r), _p(gamma),
        ctypes.c_float(eps), _p(h), c_int64(k), _p(n), c_int64(k), _p(q), c_int64(k), _p(scale),
        st.ptr() if st else c_void_p(0), _stream())
    _l.check(rc, 'amct_addnorm_quant_pertoken')
    COUNTERS['launches'] += 1
    if st:
        st.raise_if_set()
    return (q.reshape(x.shape), scale, h.reshape(x.shape) if h is not None else None,
            n.reshape(x.shape) if n is not None else None)


def addnorm_quant_per_token_tp(parts, gamma, eps, q_ptrs, scale_ptrs, row0, residual=None):
    """The tensor-parallel form of addnorm_quant_per_token.  parts [n_parts, rows, K]: partial sums of this rank's rows
    (n_parts = 1: the rows themselves); x = their fp32 sum in order, rounded once.  The codes / scale of row r are
    written to row row0 + r of every rank's code buffer [*, K] / scale buffer (q_ptrs / scale_ptrs: device addresses
    of all ranks' buffers as mapped into this process).  Returns h = x + residual (x itself without residual when
    n_parts > 1, None when the input already was the residual stream)."""
    _need_cuda(parts, gamma, residual)
    if parts.dtype not in (torch.float16, torch.bfloat16):
        raise _l.BackendError('addnorm_quant_per_token_tp: float16 / bfloat16 only')
    if parts.dim() != 3 or not parts.is_contiguous():
        raise ValueError('parts must be a contiguous [n_parts, rows, K] tensor')
    n_parts, rows, k = parts.shape
    r2 = None
    if residual is not None:
        if tuple(residual.shape) != (rows, k) or residual.dtype != parts.dtype or not residual.is_contiguous():
            raise ValueError('residual must be a contiguous [rows, K] tensor of the same dtype')
        r2 = residual
    gamma = gamma.reshape(-1).to(parts.dtype).contiguous()
    if gamma.numel() != k:
        raise ValueError('gamma must have K elements')
    h = torch.empty((rows, k), dtype=parts.dtype, device=parts.device) if residual is not None else None
    rc = _l.load().amct_addnorm_quant_pertoken_tp(
        _p(parts), c_int(n_parts), c_int64(rows * k), _p(r2), c_int(_dt(parts)), c_int64(rows), c_int64(k), c_int64(k),
        c_int64(k), _p(gamma), ctypes.c_float(eps), _p(h), c_int64(k), _pointer_array(q_ptrs), _pointer_array(scale_ptrs),
        c_int(len(q_ptrs)), c_int64(row0), c_int64(k), c_void_p(0), _stream())
    _l.check(rc, 'amct_addnorm_quant_pertoken_tp')
    COUNTERS['launches'] += 1
    return h


def gptq_block(w_block, hinv_block, scale, offset, col_group, bits):
    """One block of GPTQ's column loop in one launch.  w_block [N, b] fp32 (a column slice of the permuted weight, updated
    in place), hinv_block [b, b] fp32, scale fp32 / offset int32 [N or 1, G], col_group int32 [b].  Returns err [N, b]."""
    _need_cuda(w_block, hinv_block, scale, offset, col_group)
    n, b = w_block.shape
    assert w_block.dtype == torch.float32 and w_block.stride(1) == 1 and hinv_block.dtype == torch.float32 and hinv_block.stride(1) == 1
    scale = scale.reshape(scale.shape[0], -1).to(torch.float32).contiguous()
    if offset is not None:
        offset = offset.reshape(offset.shape[0], -1).to(torch.int32).contiguous()
    col_group = col_group.to(torch.int32).contiguous()
    err = torch.empty((n, b), dtype=torch.float32, device=w_block.device)
    rc = _l.load().amct_gptq_block(_p(w_block), c_int64(n), c_int64(w_block.stride(0)), c_int(b), _p(hinv_block),
                                   c_int64(hinv_block.stride(0)), _p(scale), _p(offset), c_int64(scale.shape[1]),
                                   c_int(1 if scale.shape[0] > 1 else 0), _p(col_group), c_int(bits), _p(err), c_int64(b), _stream())
    _l.check(rc, 'amct_gptq_block')
    COUNTERS['launches'] += 1
    return err


def rope_inplace(x, heads, head_dim, cos, sin):
    """Rotate-half rotary embedding in place on the first `heads` heads of x[..., ld]; cos / sin
    [seq, head_dim / 2] in x's dtype, row t of the flattened x uses table row t % seq."""
    _need_cuda(x, cos, sin)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise _l.BackendError('rope_inplace: float16 / bfloat16 only')
    ld = x.shape[-1]
    if not x.is_contiguous():
        raise ValueError('rope_inplace needs a contiguous tensor (it works in place)')
    cos = cos.to(x.dtype).contiguous()
    sin = sin.to(x.dtype).contiguous()
    if cos.shape != sin.shape or cos.shape[-1] != head_dim // 2:
        raise ValueError('cos / sin must be [seq, head_dim / 2]')
    tokens = x.numel() // ld
    rc = _l.load().amct_rope_inplace(_p(x), c_int(_dt(x)), c_int64(tokens), c_int64(ld), c_int(heads), c_int(head_dim),
                                     _p(cos), _p(sin), c_int64(cos.shape[0]), _stream())
    _l.check(rc, 'amct_rope_inplace')
    COUNTERS['launches'] += 1
    return x


def peer_barrier(flag_ptrs, rank, seq, status=None):
    """Barrier number `seq` between the ranks whose flag arrays (device addresses, one per rank, every one mapped
    into this process) are `flag_ptrs`, enqueued on the current stream; a wait that runs out sets bit 1 of `status`."""
    import ctypes
    arr = (ctypes.c_void_p * len(flag_ptrs))(*[int(p_) for p_ in flag_ptrs])
    rc = _l.load().amct_peer_barrier(arr, c_int(len(flag_ptrs)), c_int(rank), ctypes.c_uint32(seq & 0xFFFFFFFF), _p(status), _stream())
    _l.check(rc, 'amct_peer_barrier')
    COUNTERS['launches'] += 1


# ---------------------------------------------------------------------------
# offline checkpoint formats (amct_pytorch/experimental/quantization/DeepSeekV3.2/deploy.py)
def ckpt_block_dequant(weight_fp8, scale, block_size=128, out_dtype=torch.bfloat16):
    """E4M3 weight [M, N] times one fp32 scale per block_size x block_size tile -> out_dtype [M, N]."""
    _need_cuda(weight_fp8, scale)
    if weight_fp8.dim() != 2 or weight_fp8.element_size() != 1:
        raise ValueError('weight must be a 2-D tensor of one-byte E4M3 values')
    m, n = weight_fp8.shape
    if tuple(scale.shape) != ((m + block_size - 1) // block_size, (n + block_size - 1) // block_size):
        raise AssertionError('Mismatch in scale shape and weight shape.')          # deploy.py:70-73
    w = weight_fp8.contiguous().view(torch.uint8)
    s = scale.to(torch.float32).contiguous()
    out = torch.empty((m, n), dtype=out_dtype, device=w.device)
    rc = _l.load().amct_ckpt_block_dequant(_p(w), c_int64(m), c_int64(n), c_int64(n), _p(s), c_int64(s.shape[1]),
                                           c_int(block_size), _p(out), c_int(_DT[out_dtype]), c_int64(n), _stream())
    _l.check(rc, 'amct_ckpt_block_dequant')
    COUNTERS['launches'] += 1
    return out


def ckpt_rowquant(weight, bits=8, clip_factor=None):
    """Per-row symmetric codes in the weight's dtype.  bits=8 -> (int8 [N, K], fp32 [N, 1], None);
    bits=4 -> (packed int8 [N / 2, K], uint64 [N, 1], fp32 bias [N])."""
    _need_cuda(weight)
    if weight.dim() != 2:
        raise AssertionError('weight must be 2-D')                                   # deploy.py:129
    if bits not in (8, 4):
        raise ValueError('bits must be 8 or 4')
    w2, rows, k, ld = _rows2d(weight)
    if bits == 4 and rows % 2:
        raise ValueError('INT4 packing pairs output channels: the row count must be even')
    dev = weight.device
    codes = torch.empty((rows if bits == 8 else rows // 2, k), dtype=torch.int8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float32 if bits == 8 else torch.int64, device=dev)
    bias = torch.empty(rows, dtype=torch.float32, device=dev) if bits == 4 else None
    use_clip = clip_factor is not None
    rc = _l.load().amct_ckpt_rowquant(_p(w2), c_int(_dt(w2)), c_int64(rows), c_int64(k), c_int64(ld), c_int(bits),
                                      c_int(int(use_clip)), ctypes.c_float(float(clip_factor) if use_clip else 1.0),
                                      _p(codes), c_int64(k), _p(scale), _p(bias), _stream())
    _l.check(rc, 'amct_ckpt_rowquant')
    COUNTERS['launches'] += 1
    if bits == 4:
        scale = scale.view(torch.uint64)
    return codes, scale, bias


def ckpt_dequant_rowquant(weight_fp8, block_scale, bits=8, clip_factor=None, block_size=128, dtype=torch.bfloat16):
    """ckpt_rowquant(ckpt_block_dequant(weight_fp8, block_scale)) in one pass over the FP8 weight; same results."""
    _need_cuda(weight_fp8, block_scale)
    if weight_fp8.dim() != 2 or weight_fp8.element_size() != 1:
        raise ValueError('weight must be a 2-D tensor of one-byte E4M3 values')
    if bits not in (8, 4):
        raise ValueError('bits must be 8 or 4')
    rows, k = weight_fp8.shape
    if tuple(block_scale.shape) != ((rows + block_size - 1) // block_size, (k + block_size - 1) // block_size):
        raise AssertionError('Mismatch in scale shape and weight shape.')          # deploy.py:70-73
    if bits == 4 and rows % 2:
        raise ValueError('INT4 packing pairs output channels: the row count must be even')
    w = weight_fp8.contiguous().view(torch.uint8)
    s = block_scale.to(torch.float32).contiguous()
    dev = w.device
    codes = torch.empty((rows if bits == 8 else rows // 2, k), dtype=torch.int8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float32 if bits == 8 else torch.int64, device=dev)
    bias = torch.empty(rows, dtype=torch.float32, device=dev) if bits == 4 else None
    use_clip = clip_factor is not None
    rc = _l.load().amct_ckpt_dequant_rowquant(
        _p(w), c_int64(rows), c_int64(k), c_int64(k), _p(s), c_int64(s.shape[1]), c_int(block_size), c_int(_DT[dtype]),
        c_int(bits), c_int(int(use_clip)), ctypes.c_float(float(clip_factor) if use_clip else 1.0),
        _p(codes), c_int64(k), _p(scale), _p(bias), _stream())
    _l.check(rc, 'amct_ckpt_dequant_rowquant')
    COUNTERS['launches'] += 1
    if bits == 4:
        scale = scale.view(torch.uint64)
    return codes, scale, bias


def ckpt_pack4_rows(codes):
    """int8 [N, K] of 4-bit values, N even -> int8 [N / 2, K] (row 2j low nibble, row 2j + 1 high nibble)."""
    _need_cuda(codes)
    assert codes.dtype == torch.int8 and codes.dim() == 2                           # deploy.py:113
    if codes.shape[0] % 2:
        raise ValueError('INT4 packing pairs output channels: the row count must be even')
    c = codes.contiguous()
    rows, k = c.shape
    out = torch.empty((rows // 2, k), dtype=torch.int8, device=c.device)
    rc = _l.load().amct_ckpt_pack4_rows(_p(c), c_int64(rows), c_int64(k), c_int64(k), _p(out), c_int64(k), _stream())
    _l.check(rc, 'amct_ckpt_pack4_rows')
    COUNTERS['launches'] += 1
    return out


def ckpt_int4_bias(codes, scale):
    """fp32 [N]: sum over a row of scale * code * 8 with every product rounded to scale's dtype."""
    _need_cuda(codes, scale)
    assert codes.dtype == torch.int8 and codes.dim() == 2 and scale.dim() == 2 and scale.shape[0] == codes.shape[0]
    c = codes.contiguous()
    s = scale.contiguous()
    rows, k = c.shape
    groups = s.shape[1]
    if groups == 0 or k % groups:
        raise ValueError('the scale columns must divide the code columns')
    bias = torch.empty(rows, dtype=torch.float32, device=c.device)
    rc = _l.load().amct_ckpt_int4_bias(_p(c), c_int64(rows), c_int64(k), c_int64(k), _p(s), c_int(_dt(s)),
                                       c_int64(groups), _p(bias), _stream())
    _l.check(rc, 'amct_ckpt_int4_bias')
    COUNTERS['launches'] += 1
    return bias


def hadamard_pow2(n, norm=True, dtype=torch.bfloat16, device='cuda'):
    """Sylvester Hadamard matrix [n, n]; with norm, log2(n) divisions by sqrt(2) each rounded to dtype."""
    if n <= 0 or n & (n - 1):
        raise ValueError(f'n must be a positive power of 2, got{n}')                 # deploy.py:37-38
    out = torch.empty((n, n), dtype=dtype, device=device)
    _need_cuda(out)
    with torch.cuda.device(out.device):
        rc = _l.load().amct_hadamard_pow2(c_int(n), c_int(int(bool(norm))), c_int(_DT[dtype]), _p(out), _stream())
    _l.check(rc, 'amct_hadamard_pow2')
    COUNTERS['launches'] += 1
    return out


# ---------------------------------------------------------------------------
# KV-cache / indexer activations (amct_pytorch/experimental/quantization/DeepSeekV3.2/cores)
def dsa_rotate_fakequant(x, rotate=False, out_dtype=None, bits=8, symmetric=True, clip_max_sigmoid=None,
                         clip_min_sigmoid=None, clip_ratio=None, static=None, static_fp32=False):
    """Optional Hadamard rotation of the last axis, optional cast, fake quantization (bits=16: none) in one pass.

    Per token and dynamic by default.  clip_max_sigmoid (and, asymmetric, clip_min_sigmoid): learned clipping, fp32
    arithmetic as torch promotes.  clip_ratio: both bounds times a plain ratio.  static=(scale, zero): one given
    scale and zero point for the whole tensor; static_fp32 says whether torch would promote that arithmetic to fp32.
    """
    _need_cuda(x)
    out_dtype = out_dtype or x.dtype
    x2, rows, k, ld = _rows2d(x)
    out = torch.empty((rows, k), dtype=out_dtype, device=x.device)
    chosen = [clip_max_sigmoid is not None, clip_ratio is not None, static is not None]
    if sum(chosen) > 1:
        raise ValueError('learned clipping, clip_ratio and a static scale exclude one another')
    mode, a, b = _l.DSA_DYNAMIC, 1.0, 1.0
    if clip_max_sigmoid is not None:
        if not symmetric and clip_min_sigmoid is None:
            raise ValueError('the asymmetric rule with learned clipping needs both sigmoids')
        mode, a = _l.DSA_LEARNED_CLIP, float(clip_max_sigmoid)
        b = float(clip_min_sigmoid) if clip_min_sigmoid is not None else 1.0
    elif clip_ratio is not None:
        mode, a = _l.DSA_CLIP_RATIO, float(clip_ratio)
    elif static is not None:
        mode, a, b = (_l.DSA_STATIC_F32 if static_fp32 else _l.DSA_STATIC), float(static[0]), float(static[1])
    rc = _l.load().amct_dsa_rotate_fakequant(
        _p(x2), c_int(_dt(x2)), c_int64(rows), c_int64(k), c_int64(ld), c_int(int(bool(rotate))), c_int(_DT[out_dtype]),
        c_int(bits), c_int(int(bool(symmetric))), c_int(mode), ctypes.c_float(a), ctypes.c_float(b),
        _p(out), c_int64(k), _stream())
    _l.check(rc, 'amct_dsa_rotate_fakequant')
    COUNTERS['launches'] += 1
    return out.reshape(x.shape)
