"""Per-kernel roofline measurements (one JSON line per case).

    python bench_kernels.py [--only SUBSTR] [--reps 20] [--out FILE]
    python bench_kernels.py --only SUBSTR --steady SECONDS [--library-refs]

Every case: 3 warm-up launches, then `reps` launches each preceded by an L2 flush
(a 512 MiB buffer is overwritten, untimed), each launch bracketed by CUDA events on
the launching stream.  Reported: median and best time, algorithmic bytes or
operations per launch, achieved GB/s or TOP/s and the fraction of the measured peak
(MEASURED_PEAKS.json when present: HBM copy bandwidth; 2x the bf16 burst figure for
INT8 and FP8, 4x for FP4, since a kernel is timed alone here).

--steady S runs each selected case back to back for S seconds instead (no L2 flush), samples
the SM clock and the board power through NVML every 50 ms, and reports the rate of the first
10 launches and of the last quarter of the run: the figure that holds at the power limit.
--library-refs adds cuBLASLt INT8 (torch._int_mm) and cuBLAS bf16 (torch.matmul) lines for
context; they are never part of this repository's path.
"""
import argparse
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from amct_b200.backend import ops  # noqa: E402


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return p['hbm_gbs'], p['bf16_tflops'], 'measured'
    return 6650.0, 1590.0, 'fallback'


HBM, BF16, SRC = peaks()
_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(512 << 20, dtype=torch.uint8, device='cuda')
    _flush.fill_(1)


def time_case(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times), min(times)


def steady_case(name, fn, secs, nops=None, nbytes=None, out=None):
    import threading
    import time
    import pynvml
    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    samples, stop = [], []

    def sampler():
        while not stop:
            samples.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM), pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0))
            time.sleep(0.05)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    th = threading.Thread(target=sampler)
    th.start()
    t0, evs = time.time(), []
    while time.time() - t0 < secs:
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
    stop.append(1)
    th.join()
    ms = [a.elapsed_time(b) for a, b in evs]
    last, ls = ms[len(ms) * 3 // 4:], samples[len(samples) * 3 // 4:]
    work, unit = (nops, 'TOP/s') if nops is not None else (nbytes, 'TB/s')
    rec = {'case': name, 'mode': f'steady {secs}s', 'launches': len(ms), 'unit': unit,
           'first10': round(work / statistics.median(ms[:10]) / 1e9, 1), 'steady': round(work / statistics.median(last) / 1e9, 1),
           'sm_mhz_steady': statistics.median([c for c, _ in ls]) if ls else None,
           'power_w_steady': round(statistics.median([w for _, w in ls])) if ls else None,
           'variant': os.environ.get('AMCT_GEMM_VARIANT', 'auto')}
    line = json.dumps(rec)
    print(line, flush=True)
    if out:
        out.write(line + '\n')
        out.flush()


def report(name, med, best, nbytes=None, nops=None, out=None, peak_mult=1.0, extra=None):
    rec = {'case': name, 'ms_median': round(med, 5), 'ms_best': round(best, 5)}
    if extra:
        rec['cpu_baseline'] = extra
    if nbytes is not None:
        gbs = nbytes / (med * 1e-3) / 1e9
        rec.update(bound='hbm', bytes=nbytes, achieved=round(gbs, 1), unit='GB/s', peak=HBM, frac=round(gbs / HBM, 4))
    if nops is not None:
        tops = nops / (med * 1e-3) / 1e12
        pk = BF16 * peak_mult
        rec.update(bound='tensor', ops=nops, achieved=round(tops, 1), unit='TOP/s', peak=pk, frac=round(tops / pk, 4))
    rec['peak_source'] = SRC
    line = json.dumps(rec)
    print(line, flush=True)
    if out:
        out.write(line + '\n')
        out.flush()


def mma_peak_lines(out):
    """The MMA-only kernel for every kind, 3 s each, with the SM clock sampled through NVML: TOP/s and TOP/s per MHz."""
    import threading
    import time
    import pynvml
    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    for kind in ('bf16', 'i8', 'mxf8', 'mxf4'):
        steps = 20000
        for _ in range(2):
            nops = ops.mma_peak(kind, steps, status=status)
        torch.cuda.synchronize()
        samples, stop = [], []

        def sampler():
            while not stop:
                samples.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM), pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0))
                time.sleep(0.02)
        th = threading.Thread(target=sampler)
        th.start()
        times, t_end = [], time.time() + 3.0
        while time.time() < t_end:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.mma_peak(kind, steps, status=status)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        stop.append(1)
        th.join()
        ops.raise_if_timed_out(status)
        clk = statistics.median(c for c, _ in samples) if samples else None
        first, last = min(times[:3]), statistics.median(times[len(times) // 2:])
        rec = {'case': f'mma_peak {kind} (tcgen05.mma only, operands resident in shared memory)', 'launches': len(times),
               'burst_tops': round(nops / (first * 1e-3) / 1e12, 1), 'sustained_tops': round(nops / (last * 1e-3) / 1e12, 1),
               'sm_mhz_median': clk, 'power_w_max': max((p for _, p in samples), default=None),
               'sustained_tops_per_mhz': round(nops / (last * 1e-3) / 1e12 / clk, 3) if clk else None,
               'measured_bf16_burst': BF16, 'convention_multiple': {'bf16': 1, 'i8': 2, 'mxf8': 2, 'mxf4': 4}[kind]}
        line = json.dumps(rec)
        print(line, flush=True)
        if out:
            out.write(line + '\n')
            out.flush()


def c4_layer_line(out):
    """Config 4: one Llama-3-8B decoder layer, SmoothQuant a = 0.5 from a 128 x 2048-token random calibration pass, then
    HiFloat8 weights and activations on all seven Linears; evaluation batch 8 x 2048 (seed 3).  Tokens/s of the layer."""
    from amct_b200.workloads import llama_hif8
    os.environ.setdefault('AMCT_LOG_LEVEL', 'warning')
    work = llama_hif8.build(calib_sequences=128, calib_seq=2048, calib_batch=8)
    ids = torch.randint(0, work.layer.shape.vocab, (8, 2048), generator=torch.Generator().manual_seed(3)).cuda()
    for _ in range(3):
        work(ids)
    torch.cuda.synchronize()
    times = []
    for _ in range(10):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        work(ids)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    med = statistics.median(times)
    flops = work.linear_flops_per_token() * ids.numel()
    rec = {'case': 'c4 llama3-8b layer, SmoothQuant 0.5 + HiFloat8 on 7 Linears, batch 8 x 2048', 'ms_median': round(med, 4),
           'tokens_per_s': round(ids.numel() / (med * 1e-3), 1), 'linear_tflops': round(flops / (med * 1e-3) / 1e12, 1),
           'frac_of_bf16_peak': round(flops / (med * 1e-3) / 1e12 / BF16, 4), 'calibration': 'L_cal = 2048, 128 sequences, 16 batches of 8',
           'peak_source': SRC}
    line = json.dumps(rec)
    print(line, flush=True)
    if out:
        out.write(line + '\n')


_REF = {}


def reference_package():
    """The reference package from baseline/_ref (None when it is not installed)."""
    if 'mod' not in _REF:
        ref_dir = os.path.join(ROOT, 'baseline', '_ref')
        _REF['mod'] = None
        if os.path.isdir(os.path.join(ref_dir, 'amct_pytorch')):
            import tempfile
            cwd = os.getcwd()
            os.chdir(tempfile.mkdtemp(prefix='amct_ref_'))
            sys.path.insert(0, ref_dir)
            try:
                import amct_pytorch.quantize_op.utils as qu
                import amct_pytorch.utils.quant_util as qutil
                _REF['mod'] = (qu, qutil)
            except Exception:                                   # noqa: BLE001 -- no reference, no CPU line
                pass
            finally:
                sys.path.remove(ref_dir)
                os.chdir(cwd)
    return _REF['mod']


def cpu_baseline_for(name):
    """The reference's own function for a kernel line, timed on the host cores on a bounded sample (rows cut so that one
    call takes about a second); MX and HiFloat8 have no reference code: the CPU oracle stands in (kind 'port')."""
    import time
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    g = torch.Generator().manual_seed(0)

    def timed(fn, unit_bytes, rows, what, kind):
        fn()
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        return {'value': round(unit_bytes * rows / dt / 1e9, 3), 'unit': 'GB/s', 'cores': torch.get_num_threads(), 'kind': kind,
                'sample': f'{what}, {rows} rows, {dt:.3f} s'}
    ref = reference_package()
    if name.startswith('quant_dynamic_pertoken') and ref:
        qu, qutil = ref
        k = 8192
        x = torch.randn(16384, k, generator=g).to(torch.bfloat16)

        def fn():
            mx, mn = x.amax(1, keepdim=True), x.amin(1, keepdim=True)
            s, _ = qu.calculate_scale_offset(mx, mn, True, 'int8')
            return qutil.convert_dtype(x / s, 'int8')
        return timed(fn, k * 3 + 4, x.shape[0], 'reference amax/amin + calculate_scale_offset + convert_dtype', 'reference')
    if (name.startswith('weight_quant_i4') or name.startswith('weight_codes_i4')) and ref:
        qu, qutil = ref
        w = (torch.randn(16384, 4096, generator=g) * 0.02).to(torch.bfloat16)

        def fn():
            mn, mx = qu.get_weight_min_max_by_granularity(w, {'weights_cfg': {'strategy': 'group', 'group_size': 128}})
            s, o = qu.calculate_scale_offset(mx, mn, False, 'int4')
            return qutil.quant_weight(w, 'int4', s, o, 128)
        try:
            return timed(fn, 4096 * 2.5, w.shape[0], 'reference group min/max + calculate_scale_offset + quant_weight', 'reference')
        except Exception:                                       # noqa: BLE001
            return None
    if name.startswith('fake_quant') and ref:
        qu, qutil = ref
        from oracle import intq
        w = (torch.randn(16384, 4096, generator=g) * 0.02).to(torch.bfloat16)
        s, o = intq.weight_scale_offset(w, 'int4', False, 'group', 128)
        qp = {'weights_cfg': {'quant_type': 'int4', 'group_size': 128}}
        return timed(lambda: qutil.quant_dequant_weight(w, qp, s, o), 4096 * 4, w.shape[0], 'reference quant_dequant_weight', 'reference')
    if name.startswith('mx_quant'):
        from oracle import mx
        fmt = 'fp8' if ' fp8 ' in name else 'fp4'
        x = torch.randn(4096 if fmt == 'fp8' else 1024, 8192, generator=g).to(torch.bfloat16)
        return timed(lambda: mx.quantize(x, fmt), 8192 * (3 if fmt == 'fp8' else 2.5), x.shape[0], 'CPU oracle mx.quantize', 'port')
    if name.startswith('hif8_encode'):
        from oracle import hif8
        x = torch.randn(256, 14336, generator=g).float().numpy()
        return timed(lambda: hif8.encode(x), 14336 * 3, x.shape[0], 'CPU oracle hif8.encode', 'port')
    return None


def cases():
    g = torch.Generator(device='cuda').manual_seed(0)

    def randn(r, k, dtype, std=1.0):
        return (torch.randn(r, k, device='cuda', generator=g, dtype=torch.float32 if dtype == torch.float32 else torch.bfloat16) * std).to(dtype)

    # ---- dynamic per-token activation quantization
    for r, k, dt, tag in ((2048, 4096, torch.float32, 'c1'), (65536, 8192, torch.bfloat16, 'c5-h'),
                          (65536, 28672, torch.bfloat16, 'c5-ffn'), (65536, 4096, torch.float32, 'c1-1GiB')):
        es = 4 if dt == torch.float32 else 2
        yield (f'quant_dynamic_pertoken {tag} [{r}x{k}] {str(dt)[6:]}', lambda r=r, k=k, dt=dt: randn(r, k, dt),
               lambda x: (lambda: ops.quant_dynamic_per_token(x)), dict(nbytes=r * k * es + r * k + r * 4))
    # ---- decoder-layer glue: add + RMSNorm + quant in one pass; rotary embedding in place
    def setup_an():
        return randn(65536, 8192, torch.bfloat16), randn(65536, 8192, torch.bfloat16), torch.ones(8192, device='cuda', dtype=torch.bfloat16)
    yield ('addnorm_quant c5-h [65536x8192] bf16 (+residual)', setup_an,
           lambda t: (lambda: ops.addnorm_quant_per_token(t[0], t[2], 1e-5, residual=t[1])),
           dict(nbytes=65536 * 8192 * (2 + 2 + 2 + 1) + 65536 * 4))

    def setup_rope():
        ang = torch.rand(2048, 64, device='cuda') * 6.28
        return randn(65536, 10240, torch.bfloat16), ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    yield ('rope_inplace c5 qkv [65536x10240], 72 heads of 128, bf16', setup_rope,
           lambda t: (lambda: ops.rope_inplace(t[0], 72, 128, t[1], t[2])), dict(nbytes=65536 * 72 * 128 * 2 * 2))
    # ---- static quantize
    yield ('quantize_static per-tensor [65536x8192] bf16', lambda: randn(65536, 8192, torch.bfloat16),
           lambda x: (lambda s=torch.tensor([30.0], device='cuda', dtype=torch.bfloat16): ops.quantize_static(x, s, None)),
           dict(nbytes=65536 * 8192 * 3))
    # ---- weight quantization, fused min/max + codes
    for n, k, dt, tag in ((4096, 4096, torch.float32, 'c1'), (28672, 8192, torch.bfloat16, 'c5 gate/up shard')):
        es = 4 if dt == torch.float32 else 2
        yield (f'weight_quant_i8 channel {tag} [{n}x{k}] {str(dt)[6:]}', lambda n=n, k=k, dt=dt: randn(n, k, dt, 0.02),
               lambda w: (lambda: ops.quant_rows(w, 'int8', True, 'channel', out='i8', check=False)),
               dict(nbytes=n * k * es + n * k + n * 4))
    yield ('weight_quant_i4 g128 asym pack c2 [11008x4096] bf16', lambda: randn(11008, 4096, torch.bfloat16, 0.02),
           lambda w: (lambda: ops.quant_rows(w, 'int4', False, 'group', 128, out='pack4', check=False)),
           dict(nbytes=11008 * 4096 * 2 + 11008 * 4096 // 2 + 11008 * 32 * 8))
    yield ('fake_quant i4 g128 asym [11008x4096] bf16', lambda: randn(11008, 4096, torch.bfloat16, 0.02),
           lambda w: (lambda: ops.quant_rows(w, 'int4', False, 'group', 128, out='fake', check=False)),
           dict(nbytes=11008 * 4096 * 4 + 11008 * 32 * 8))
    yield ('weight_quant_i4 g128 asym pack c5 gate/up [57344x8192] bf16', lambda: randn(57344, 8192, torch.bfloat16, 0.02),
           lambda w: (lambda: ops.quant_rows(w, 'int4', False, 'group', 128, out='pack4', check=False)),
           dict(nbytes=57344 * 8192 * 2 + 57344 * 8192 // 2 + 57344 * 64 * 8))
    def setup_given():
        w = randn(57344, 8192, torch.bfloat16, 0.02)
        sc, off, _ = ops.quant_rows(w, 'int4', False, 'group', 128, out='none', check=False)
        return w, sc, off
    yield ('weight_codes_i4 g128 asym pack, given scales, c5 gate/up [57344x8192] bf16', setup_given,
           lambda t: (lambda: ops.quant_rows(t[0], 'int4', False, 'group', 128, scale=t[1], offset=t[2], out='pack4', check=False)),
           dict(nbytes=57344 * 8192 * 2 + 57344 * 8192 // 2 + 57344 * 64 * 8))
    yield ('fake_quant_awq i4 g128 asym c5 gate/up [57344x8192] bf16', lambda: randn(57344, 8192, torch.bfloat16, 0.02),
           lambda w: (lambda: ops.quant_rows(w, 'int4', False, 'group', 128, out='fake_awq', check=False)),
           dict(nbytes=57344 * 8192 * 4 + 57344 * 64 * 8))
    # ---- observers
    yield ('minmax column [65536x8192] bf16', lambda: randn(65536, 8192, torch.bfloat16),
           lambda x: (lambda: ops.minmax(x, 'column')), dict(nbytes=65536 * 8192 * 2))
    yield ('minmax tensor [65536x8192] bf16', lambda: randn(65536, 8192, torch.bfloat16),
           lambda x: (lambda: ops.minmax(x, 'tensor')), dict(nbytes=65536 * 8192 * 2))
    # ---- W8A8 GEMM
    for m, n, k, od, tag in ((2048, 4096, 4096, torch.float32, 'c1'), (8192, 8192, 8192, torch.bfloat16, 'square'),
                             (16384, 8192, 8192, torch.bfloat16, 'mid'), (65536, 10240, 8192, torch.bfloat16, 'c5 qkv'), (65536, 8192, 8192, torch.bfloat16, 'c5 o'),
                             (65536, 57344, 8192, torch.bfloat16, 'c5 gate+up'), (65536, 8192, 28672, torch.bfloat16, 'c5 down'),
                             (64, 8192, 8192, torch.bfloat16, 'c5 decode o')):
        def setup(m=m, n=n, k=k, od=od):
            a = torch.randint(-128, 128, (m, k), device='cuda', dtype=torch.int8)
            b = torch.randint(-128, 128, (n, k), device='cuda', dtype=torch.int8)
            return (a, b, torch.rand(n, device='cuda') * 1e-3, torch.rand(m, device='cuda'),
                    torch.empty(m, n, device='cuda', dtype=od))
        # M <= 128 streams the weight once: that launch is bound by HBM, not by the tensor cores
        kw = dict(nops=2 * m * n * k, peak_mult=2.0) if m > 128 else dict(nbytes=n * k + m * k + m * n * (4 if od == torch.float32 else 2))
        yield (f'gemm_w8a8 {tag} {m}x{n}x{k} -> {str(od)[6:]}', setup,
               lambda t: (lambda: ops.gemm_w8a8(t[0], t[1], t[2], t[3], None, out=t[4])), kw)
    # ---- W8A8 gate/up GEMM with the SwiGLU epilogue (the dominant launch of the 70B prefill step; the 8192-row case is
    #      the one small enough for a profiler capture, its DRAM traffic scales with the rows)
    for m in (8192, 65536):
        def setup_sw(m=m):
            a = torch.randint(-128, 128, (m, 8192), device='cuda', dtype=torch.int8)
            b = torch.randint(-128, 128, (57344, 8192), device='cuda', dtype=torch.int8)
            # scales that put the gate values at a few units, as in a model: with random INT8 operands the accumulators
            # are of the order of 5e5, and gates of +-100 would send every exp / division of the epilogue down its
            # out-of-range path
            return (a, b, torch.rand(57344, device='cuda') * 1e-5, torch.rand(m, device='cuda'),
                    torch.empty(m, 28672, device='cuda', dtype=torch.bfloat16))
        yield (f'gemm_w8a8 swiglu c5 gate+up {m}x57344x8192 -> bf16 [{m}x28672]', setup_sw,
               lambda t: (lambda: ops.gemm_w8a8_swiglu(t[0], t[1], t[2], t[3], None, out=t[4])),
               dict(nops=2 * m * 57344 * 8192, peak_mult=2.0))
    # ---- 16-bit GEMM
    for m, n, k, tag in ((8192, 8192, 8192, 'square'), (4096, 11008, 4096, 'c2 M=4096'), (128, 11008, 4096, 'c2 M=128'),
                         (16384, 14336, 4096, 'c4 gate')):
        def setup16(m=m, n=n, k=k):
            return (randn(m, k, torch.bfloat16), randn(n, k, torch.bfloat16, 0.02), torch.empty(m, n, device='cuda', dtype=torch.bfloat16))
        kw = dict(nops=2 * m * n * k, peak_mult=1.0) if m > 128 else dict(nbytes=2 * (n * k + m * k + m * n))
        yield (f'gemm_f16 bf16 {tag} {m}x{n}x{k}', setup16, lambda t: (lambda: ops.gemm_f16(t[0], t[1], out=t[2])), kw)
    # ---- W4A16 Linear, one kernel (dequant in shared memory ahead of the MMA): config 2 sweep over M
    for m in (1, 16, 128, 1024, 4096):
        def setup_w4(m=m):
            n, k = 11008, 4096
            codes = torch.randint(0, 256, (n, k // 2), device='cuda', dtype=torch.uint8)
            sc = (torch.rand(k // 128, n, device='cuda') * 0.01 + 0.002).to(torch.bfloat16)
            off = torch.randint(-8, 8, (k // 128, n), device='cuda').to(torch.bfloat16)
            return randn(m, k, torch.bfloat16), codes, sc, off, torch.empty(m, n, device='cuda', dtype=torch.bfloat16)
        nbytes = 11008 * 2048 + 2 * 32 * 11008 * 2 + m * 4096 * 2 + m * 11008 * 2
        kw = dict(nbytes=nbytes) if m <= 128 else dict(nops=2 * m * 11008 * 4096, peak_mult=1.0)
        yield (f'gemm_w4a16 fused c2 M={m} {m}x11008x4096 g128 bf16', setup_w4,
               lambda t: (lambda: ops.gemm_w4a16(t[0], t[1], 4, t[2], t[3], 128, out=t[4])), kw)
    # ---- the same Linear through the shim's routing for many tokens: dequantize once, then the 16-bit GEMM
    for m in (1024, 4096):
        def setup_w4r(m=m):
            n, k = 11008, 4096
            codes = torch.randint(0, 256, (n, k // 2), device='cuda', dtype=torch.uint8)
            sc = (torch.rand(k // 128, n, device='cuda') * 0.01 + 0.002).to(torch.bfloat16)
            off = torch.randint(-8, 8, (k // 128, n), device='cuda').to(torch.bfloat16)
            return randn(m, k, torch.bfloat16), codes, sc, off
        from amct_b200 import torch_npu_shim
        yield (f'w4a16 linear (dequant + gemm, the route for M > 128) c2 M={m} {m}x11008x4096 g128 bf16', setup_w4r,
               lambda t: (lambda: torch_npu_shim.weight_quant_matmul(t[0], t[1], 4, t[2], t[3], None, 128)),
               dict(nops=2 * m * 11008 * 4096, peak_mult=1.0))
    # ---- MX quantization and block-scaled GEMM (config 3 shapes)
    for fmt, pb in (('fp8', 1.0), ('fp4', 0.5)):
        for r, k, opnd, tag in ((8192, 8192, 'a', 'c3 act'), (28672, 8192, 'b', 'c3 weight')):
            yield (f'mx_quant {fmt} {tag} [{r}x{k}] bf16', lambda r=r, k=k, s=(1.0 if opnd == 'a' else 0.015): randn(r, k, torch.bfloat16, s),
                   lambda x, fmt=fmt, opnd=opnd: (lambda: ops.mx_quant(x, fmt, operand=opnd)),
                   dict(nbytes=int(r * k * (2 + pb) + 2 * r * k // 32)))
    for fmt, mult in (('fp8', 2.0), ('fp4', 4.0)):
        def setup_mx(fmt=fmt):
            a = randn(8192, 8192, torch.bfloat16)
            b = randn(28672, 8192, torch.bfloat16, 0.015)
            ap, _, at = ops.mx_quant(a, fmt, operand='a', rowmajor=False)
            bp, _, bt = ops.mx_quant(b, fmt, operand='b', rowmajor=False)
            return ap, at, bp, bt, torch.empty(8192, 28672, device='cuda', dtype=torch.bfloat16)
        yield (f'gemm_mx {fmt} c3 8192x28672x8192 -> bf16', setup_mx,
               lambda t, fmt=fmt: (lambda: ops.gemm_mx(t[0], t[1], t[2], t[3], fmt, out=t[4])),
               dict(nops=2 * 8192 * 28672 * 8192, peak_mult=mult))
    # ---- HiFloat8
    yield ('hif8_encode [16384x14336] bf16', lambda: randn(16384, 14336, torch.bfloat16),
           lambda x: (lambda: ops.hif8_encode(x)), dict(nbytes=16384 * 14336 * 3))
    yield ('hif8_fake_quant [16384x4096] bf16', lambda: randn(16384, 4096, torch.bfloat16),
           lambda x: (lambda: ops.hif8_fake_quant(x)), dict(nbytes=16384 * 4096 * 4))
    yield ('hif8_decode [14336x4096] -> bf16', lambda: torch.randint(0, 256, (14336, 4096), device='cuda', dtype=torch.uint8),
           lambda c: (lambda: ops.hif8_decode(c)), dict(nbytes=14336 * 4096 * 3))
    # ---- HiFloat8 Linear (config 4 shapes, 16384 tokens): weight codes decoded ahead of the bf16 MMA.  Timed: the whole
    # weight side of HiFloat8Linear.forward for an already fake-quantized activation: decode the codes, multiply.
    for n, k, tag in ((4096, 4096, 'q / o'), (14336, 4096, 'gate / up'), (4096, 14336, 'down')):
        def setup_h(n=n, k=k):
            w = randn(n, k, torch.bfloat16, 0.02)
            return ops.hif8_fake_quant(randn(16384, k, torch.bfloat16)), ops.hif8_encode(w), torch.empty(16384, n, device='cuda', dtype=torch.bfloat16)
        yield (f'hif8 linear (decode + gemm) c4 {tag} 16384x{n}x{k} bf16', setup_h,
               lambda t: (lambda: ops.gemm_f16(t[0], ops.hif8_decode(t[1], dtype=torch.bfloat16), out=t[2])),
               dict(nops=2 * 16384 * n * k, peak_mult=1.0))
    def setup_lut():
        return randn(256, 4096, torch.bfloat16), ops.hif8_encode(randn(14336, 4096, torch.bfloat16, 0.02)), torch.empty(256, 14336, device='cuda', dtype=torch.bfloat16)
    yield ('gemm_lut8 (hif8 codes decoded in shared memory) c4 gate 256x14336x4096 bf16', setup_lut,
           lambda t: (lambda: ops.gemm_hif8_weight(t[0], t[1], out=t[2])), dict(nops=2 * 256 * 14336 * 4096, peak_mult=1.0))
    # ---- weight dequant (stage 1 of the weight-only Linear)
    def setup_dq():
        codes = torch.randint(0, 256, (11008, 2048), device='cuda', dtype=torch.uint8)
        s = (torch.rand(32, 11008, device='cuda') * 0.01).to(torch.bfloat16)
        o = torch.randint(-8, 8, (32, 11008), device='cuda').to(torch.bfloat16)
        return codes, s, o, torch.empty(11008, 4096, device='cuda', dtype=torch.bfloat16)
    yield ('dequant_weight i4 g128 c2 [11008x4096] -> bf16', setup_dq,
           lambda t: (lambda: ops.dequant_weight(t[0], 4, t[1], t[2], 128, out=t[3])),
           dict(nbytes=11008 * 2048 + 11008 * 4096 * 2 + 2 * 32 * 11008 * 2))
    # ---- offline checkpoint formats: 64 routed experts' up projections of a DeepSeek-V3-sized MoE layer at once
    def setup_fp8():
        w = torch.randint(0, 0x77, (64 * 2048, 7168), device='cuda', dtype=torch.uint8).view(torch.float8_e4m3fn)
        return w, torch.rand(64 * 16, 56, device='cuda') * 0.01 + 1e-3
    yield ('ckpt_block_dequant fp8 -> bf16 [131072x7168], 128x128 scales', setup_fp8,
           lambda t: (lambda: ops.ckpt_block_dequant(t[0], t[1])), dict(nbytes=131072 * 7168 * 3))
    for bits in (8, 4):
        yield (f'ckpt_rowquant int{bits} per channel [131072x7168] bf16', lambda: randn(131072, 7168, torch.bfloat16, 0.02),
               lambda w, bits=bits: (lambda: ops.ckpt_rowquant(w, bits)),
               dict(nbytes=131072 * 7168 * 2 + 131072 * 7168 * bits // 8 + 131072 * (4 if bits == 8 else 12)))
    for bits in (8, 4):
        yield (f'ckpt_dequant_rowquant fp8 -> int{bits} in one pass [131072x7168]', setup_fp8,
               lambda t, bits=bits: (lambda: ops.ckpt_dequant_rowquant(t[0], t[1], bits)),
               dict(nbytes=131072 * 7168 + 131072 * 7168 * bits // 8 + 131072 * (4 if bits == 8 else 12)))
    # ---- KV-cache / indexer activations: 4096 tokens x 64 indexer heads of 128; attention output rows of 16384
    yield ('dsa rotate + half + fake_quant [262144x128] bf16 -> fp16', lambda: randn(262144, 128, torch.bfloat16),
           lambda x: (lambda: ops.dsa_rotate_fakequant(x, rotate=True, out_dtype=torch.float16)),
           dict(nbytes=262144 * 128 * 4))
    yield ('dsa fake_quant per token [16384x16384] bf16', lambda: randn(16384, 16384, torch.bfloat16),
           lambda x: (lambda: ops.dsa_rotate_fakequant(x)), dict(nbytes=16384 * 16384 * 4))
    yield ('dsa fake_quant asym + learned clip [65536x512] bf16', lambda: randn(65536, 512, torch.bfloat16),
           lambda x: (lambda: ops.dsa_rotate_fakequant(x, symmetric=False, clip_max_sigmoid=0.9, clip_min_sigmoid=0.8)),
           dict(nbytes=65536 * 512 * 4))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--only', default='')
    ap.add_argument('--reps', type=int, default=20)
    ap.add_argument('--out', default='')
    ap.add_argument('--steady', type=float, default=0.0, help='seconds of back-to-back launches per case')
    ap.add_argument('--library-refs', action='store_true', help='add cuBLASLt / cuBLAS reference lines (context only)')
    ap.add_argument('--mma-peak', action='store_true', help='only the MMA-only tensor-core peak measurement (all four kinds)')
    ap.add_argument('--c4-layer', action='store_true', help='only the SmoothQuant + HiFloat8 Llama-3-8B layer (config 4): tokens/s')
    ap.add_argument('--gemm-variant', default='auto', choices=['auto', 'single', 'pair'],
                    help='pin the kernel that takes GEMMs with more than 128 rows (one-CTA or CTA-pair) for a comparison')
    ap.add_argument('--cpu', action='store_true', help='add a cpu_baseline (the reference function on the host cores, bounded sample) to the lines that have one')
    args = ap.parse_args()
    out = open(args.out, 'w') if args.out else None
    if args.mma_peak:
        return mma_peak_lines(out)
    if args.c4_layer:
        return c4_layer_line(out)
    ops.set_gemm_variant(args.gemm_variant)
    todo = list(cases())
    if args.library_refs:
        for m, n, k in ((16384, 8192, 8192),):
            def setup_ref(m=m, n=n, k=k):
                return (torch.randint(-128, 128, (m, k), device='cuda', dtype=torch.int8),
                        torch.randint(-128, 128, (n, k), device='cuda', dtype=torch.int8).t(),
                        torch.randn(m, k, device='cuda', dtype=torch.bfloat16), torch.randn(n, k, device='cuda', dtype=torch.bfloat16).t())
            todo.append((f'library ref cublaslt int8 {m}x{n}x{k} -> int32', setup_ref, lambda t: (lambda: torch._int_mm(t[0], t[1])),
                         dict(nops=2 * m * n * k, peak_mult=2.0)))
            todo.append((f'library ref cublas bf16 {m}x{n}x{k}', setup_ref, lambda t: (lambda: torch.matmul(t[2], t[3])),
                         dict(nops=2 * m * n * k, peak_mult=1.0)))
    for name, setup, make, kw in todo:
        if args.only and args.only not in name:
            continue
        data = setup()
        fn = make(data)
        if args.steady > 0:
            steady_case(name, fn, args.steady, nops=kw.get('nops'), nbytes=kw.get('nbytes'), out=out)
            del data, fn
            torch.cuda.empty_cache()
            continue
        med, best = time_case(fn, args.reps)
        extra = cpu_baseline_for(name) if args.cpu else None
        report(name, med, best, out=out, extra=extra, **kw)
        del data, fn
        torch.cuda.empty_cache()


if __name__ == '__main__':
    main()
