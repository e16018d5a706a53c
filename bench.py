"""Benchmark of the W8A8 deploy path on a Llama-3-70B-shaped stack (prefill).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one prefill forward of batch 32 x seq 2048 random tokens through 80
decoder layers whose Linears are NpuQuantizationLinear deploy modules (dynamic
per-token INT8 activation quantization + tcgen05 INT8 GEMM + dequant epilogue),
tensor-parallel over the N ranks with a token-sharded residual stream: the row-parallel
GEMMs store their partial tiles into the owning rank's peer-mapped buffer and the add +
norm + quant kernel stores its codes to every rank (--comm push), or NCCL reduce-scatter /
all-gather (--comm nccl).  Total work is fixed as N grows (strong scaling).  Weights are
random-init, data synthetic.

Prints ONE JSON line on rank 0.  Keys beyond the basic contract:
  e2e           same metric with the token ids copied from pinned host memory and the
                logits read back to the host inside the timed region
  roofline      the dominant kernel (INT8 GEMM): achieved = algorithmic 2*M*N*K of every
                launch / its CUDA-event duration, measured live in a separate profiled
                pass of the same step; peak = 2 x the measured bf16 tensor peak
  cpu_baseline  the reference package's own Linear path on the host cores, bounded sample (rank 0, N=1)
  clocks        SM clock / throttle reasons sampled with nvidia-smi during the timed region
  gpu_launches  launches of this repository's kernels inside the timed region
"""
import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
# 320 Linears are converted per rank: keep the per-layer progress lines out of the output
os.environ.setdefault('AMCT_LOG_LEVEL', 'warning')

METRIC = 'w8a8_llama3_70b_prefill_tokens_per_s'
UNIT = 'tokens/s'
BATCH, SEQ = 32, 2048
SEED = 4


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--layers', type=int, default=80, help='debug only: fewer layers is not the benchmark')
    ap.add_argument('--batch', type=int, default=BATCH)
    ap.add_argument('--seq', type=int, default=SEQ)
    ap.add_argument('--cpu-sample-tokens', type=int, default=2048)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--mode', default='prefill', choices=['prefill', 'decode'],
                    help='decode: one new token for 64 sequences against a 2048-token KV cache (not the headline metric)')
    ap.add_argument('--no-cuda-graph', action='store_true')
    ap.add_argument('--comm', choices=('auto', 'nccl', 'push'), default='auto',
                    help="collectives of the token-sharded prefill: NCCL kernels, or the compute kernels' own stores into "
                         "peer-mapped buffers (auto: the latter when N > 1, NCCL if one of its barriers times out)")
    ap.add_argument('--micro-batches', type=int, default=0, help='0 = automatic (one stream)')
    ap.add_argument('--kernel-totals', default=None, metavar='FILE',
                    help='after the measurement, run one more step under torch.profiler (CUDA activities) and write '
                         "rank 0's per-kernel totals to FILE")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p.get('hbm_gbs', 6650.0), p.get('bf16_tflops', 1590.0), p.get('bf16_tflops_sustained', 1400.0), 'measured'
    return 6650.0, 1590.0, 1400.0, 'fallback'


# ----------------------------------------------------------------------------- CPU arm
REF_DIR = os.path.join(ROOT, 'baseline', '_ref')


def _register_cpu_torch_npu():
    """``torch_npu`` for the reference on a machine without an NPU: the four ops of its deploy path as the CPU
    statement in oracle/npu_ops.py gives them (INT8 GEMM through torch's CPU int8 kernel, all host threads)."""
    import types
    from oracle import npu_ops
    mod = types.ModuleType('torch_npu')
    mod.npu_quantize = npu_ops.npu_quantize
    mod.npu_quant_matmul = lambda x1, x2, scale=None, pertoken_scale=None, bias=None, output_dtype=torch.bfloat16, **kw: \
        npu_ops.npu_quant_matmul(x1, x2, scale, pertoken_scale, bias, output_dtype, fast=True)
    mod.npu_weight_quant_batchmatmul = npu_ops.npu_weight_quant_batchmatmul
    mod.npu_convert_weight_to_int4pack = lambda w, inner_k_tiles=0: npu_ops.npu_convert_weight_to_int4pack(w)
    mod.npu = types.SimpleNamespace(is_available=lambda: False, empty_cache=lambda: None)
    sys.modules['torch_npu'] = mod
    if not hasattr(torch.Tensor, 'npu'):
        torch.Tensor.npu = lambda self, *a, **k: self


class _LayerLinears(torch.nn.Module):
    """The four quantized Linears of one decoder layer at TP = 1 (fused q/k/v and gate/up as the GPU arm has them),
    each fed its own input: what the reference's quantize() / convert() operate on."""

    def __init__(self, shape, gen):
        super().__init__()
        dims = {'qkv_proj': (shape.hidden, (shape.n_heads + 2 * shape.n_kv_heads) * shape.head_dim),
                'o_proj': (shape.n_heads * shape.head_dim, shape.hidden),
                'gate_up_proj': (shape.hidden, 2 * shape.intermediate),
                'down_proj': (shape.intermediate, shape.hidden)}
        for name, (k, n) in dims.items():
            lin = torch.nn.Linear(k, n, bias=False, dtype=torch.bfloat16)
            lin.weight.data = torch.empty(n, k).normal_(0, 0.02, generator=gen).to(torch.bfloat16)
            setattr(self, name, lin)

    def forward(self, x_hidden, x_inter):
        return (self.qkv_proj(x_hidden), self.o_proj(x_hidden), self.gate_up_proj(x_hidden), self.down_proj(x_inter))


class ReferenceLinearPath:
    """The reference's own W8A8 deploy path on the host cores: ``amct_pytorch.quantize`` (MinMaxQuant, per-channel INT8
    weights, per-token INT8 activations) -> one calibration forward -> ``amct_pytorch.convert`` ->
    ``NpuQuantizationLinear.forward`` (amct_pytorch/deploy_op/npu_quantization_linear.py:89-103), imported unmodified
    from baseline/_ref.  The package's calls into torch_npu land in oracle/npu_ops.py (the reference ships no
    implementation of them).  One step = the four Linears of one layer over `tokens` rows; a prefill step of the
    benchmark is 80 layers x 65536 rows of exactly this work plus attention and norms, which are left out."""

    def __init__(self, tokens):
        if not os.path.isdir(os.path.join(REF_DIR, 'amct_pytorch')):
            raise FileNotFoundError(f'{REF_DIR}/amct_pytorch missing: install the reference with pip --target baseline/_ref')
        torch.set_num_threads(len(os.sched_getaffinity(0)))      # a launcher may have pinned OMP_NUM_THREADS=1
        _register_cpu_torch_npu()
        os.environ.setdefault('AMCT_LOG_LEVEL', 'warning')
        cwd = os.getcwd()
        import tempfile
        os.chdir(tempfile.mkdtemp(prefix='amct_ref_'))           # the reference writes its log directory into the cwd
        try:
            sys.path.insert(0, REF_DIR)
            import amct_pytorch
        finally:
            sys.path.remove(REF_DIR)
            os.chdir(cwd)
        from amct_b200.workloads.llama_tp import LLAMA3_70B as sh
        g = torch.Generator().manual_seed(SEED)
        self.tokens = tokens
        self.model = _LayerLinears(sh, g)
        self.x_hidden = torch.randn(tokens, sh.hidden, generator=g).to(torch.bfloat16)
        self.x_inter = torch.randn(tokens, sh.intermediate, generator=g).to(torch.bfloat16)
        cfg = {'batch_num': 1, 'quant_cfg': {'weights': {'type': 'int8', 'symmetric': True, 'strategy': 'channel'},
                                             'inputs': {'type': 'int8', 'symmetric': True, 'strategy': 'token'}},
               'algorithm': {'minmax'}}
        amct_pytorch.quantize(self.model, cfg)
        with torch.no_grad():
            self.model(self.x_hidden, self.x_inter)              # calibration
        amct_pytorch.convert(self.model)
        kinds = {type(m).__name__ for m in self.model.children()}
        if kinds != {'NpuQuantizationLinear'}:
            raise RuntimeError(f'the reference left {kinds} after convert()')

    def step(self):
        t0 = time.perf_counter()
        with torch.no_grad():
            self.model(self.x_hidden, self.x_inter)
        return time.perf_counter() - t0


def cpu_baseline(tokens, n_layers):
    path = ReferenceLinearPath(tokens)
    path.step()
    sec_per_layer = path.step()
    tok_s = tokens / (sec_per_layer * n_layers)
    return {'value': tok_s, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'reference',
            'sample': f'the reference package (baseline/_ref) quantize -> convert -> NpuQuantizationLinear.forward, torch_npu '
                      f'ops from the CPU oracle (INT8 GEMM via torch._int_mm), 4 Linears of one decoder layer over {tokens} '
                      f'tokens: {sec_per_layer:.3f} s; scaled x{n_layers} layers; attention/norms excluded',
            'host_cpus': os.cpu_count()}


def run_reference(args):
    """--impl reference: the reference's own CPU path on the host cores, a bounded sample per step (rank 0 only)."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    tokens = args.cpu_sample_tokens
    try:
        path = ReferenceLinearPath(tokens)
    except Exception as exc:                                     # noqa: BLE001 -- reported, not hidden
        print(json.dumps({'impl': 'reference', 'unavailable': f'{type(exc).__name__}: {exc}'[:300]}), flush=True)
        return
    for _ in range(args.warmup):
        path.step()
    times = [path.step() for _ in range(args.steps)]
    sec = statistics.mean(times)
    tok_s = tokens / (sec * 80)
    sample = (f'reference package from baseline/_ref, 4 quantized Linears of one decoder layer (TP=1 shapes) over {tokens} tokens '
              f'per step ({sec:.3f} s), scaled x80 layers; attention / norms excluded; torch_npu ops from the CPU oracle')
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': tok_s, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': (BATCH * SEQ) / tok_s * 1e3, 'higher_is_better': True, 'scaling': 'strong',
        'vs_baseline': None, 'dtype': 'int8', 'data': 'synthetic',
        'config': {'workload': 'llama3-70b W8A8 prefill, batch 32 x seq 2048, 80 layers (Linear path only on CPU)',
                   'parallelism': 'cpu'},
        'cpu_baseline': {'value': tok_s, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'reference', 'sample': sample},
        'e2e': {'value': tok_s, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
class ClockSampler:
    FIELDS = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={index}', f'--query-gpu={self.FIELDS}',
                                          '--format=csv,noheader,nounits', '-lms', '200'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        sm, smax, reasons = [], None, set()
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': smax, 'reasons': sorted(reasons),
                'samples': len(sm)}


def main():
    args = parse()
    if args.impl == 'reference':
        return run_reference(args)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device (no CPU fallback); use --impl reference for the CPU arm')
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    import torch.distributed as dist
    group = None
    if world > 1:
        # a stalled collective ends the run after a minute instead of holding the GPUs
        dist.init_process_group('nccl', device_id=dev, timeout=datetime.timedelta(seconds=60))
        group = dist.group.WORLD

    from amct_b200.backend import ops
    from amct_b200.workloads.llama_tp import LlamaW8A8, LLAMA3_70B

    comm = args.comm
    if comm == 'auto':
        comm = 'push' if (world > 1 and args.mode == 'prefill') else 'nccl'
    t_build = time.time()
    model = LlamaW8A8(LLAMA3_70B, tp=world, rank=rank, group=group, device=dev, seed=SEED, n_layers=args.layers, comm=comm)
    torch.cuda.synchronize()
    t_build = time.time() - t_build

    gen = torch.Generator().manual_seed(SEED)
    kv_caches = None
    if args.mode == 'decode':
        args.batch, args.seq, past = 64, 1, 2048
        sh = LLAMA3_70B
        dgen = torch.Generator(device=dev).manual_seed(SEED + 1)
        kv_caches = [(torch.randn(args.batch, sh.n_kv_heads // world, past + 1, sh.head_dim, device=dev, dtype=torch.bfloat16, generator=dgen),
                      torch.randn(args.batch, sh.n_kv_heads // world, past + 1, sh.head_dim, device=dev, dtype=torch.bfloat16, generator=dgen),
                      past) for _ in range(args.layers)]
    ids_host = torch.randint(0, LLAMA3_70B.vocab, (args.batch, args.seq), generator=gen).pin_memory()
    ids_dev = ids_host.to(dev)
    logits_host = torch.empty((args.batch, LLAMA3_70B.vocab), dtype=torch.float32).pin_memory()
    tokens = args.batch * args.seq

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    mb = args.micro_batches or None

    def comm_failed():
        """True on every rank if a barrier of the push collectives gave up waiting on any rank."""
        return world > 1 and model.comm_failed_anywhere()

    def fall_back(when):
        nonlocal mb
        if rank == 0:
            print(f'bench.py: a barrier of the push collectives timed out {when}; measuring with NCCL instead',
                  file=sys.stderr, flush=True)
        model.comm, mb = 'nccl', (args.micro_batches or None)
        for _ in range(args.warmup):
            step_resident()

    def step_resident():
        return model(ids_dev, kv_caches=kv_caches, past_len=2048 if kv_caches else 0, micro_batches=mb)

    def step_e2e():
        ids = ids_host.to(dev, non_blocking=True)
        logits_host.copy_(model(ids, kv_caches=kv_caches, past_len=2048 if kv_caches else 0, micro_batches=mb), non_blocking=True)

    for _ in range(args.warmup):
        step_resident()
    if comm_failed():
        fall_back('during warm-up')
    graph = None
    if args.mode == 'decode' and not args.no_cuda_graph:
        # the decode step is launch-bound (hundreds of small kernels): replay it as one CUDA graph
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        ops.COUNTERS['launches'] = 0
        with torch.cuda.graph(graph):
            graph_logits = step_resident()
        launches_per_replay = ops.COUNTERS['launches']
        eager_resident = step_resident

        def step_resident():
            graph.replay()
            return graph_logits

        def step_e2e():
            ids_dev.copy_(ids_host, non_blocking=True)
            graph.replay()
            logits_host.copy_(graph_logits, non_blocking=True)
        for _ in range(2):
            step_resident()

    def measure():
        sampler = ClockSampler(local) if rank == 0 else None
        ops.COUNTERS['launches'] = 0
        ms = timed(step_resident, args.steps)
        n_launch = ops.COUNTERS['launches'] if graph is None else launches_per_replay * args.steps
        clk = sampler.stop() if sampler else None
        return ms, n_launch, clk, timed(step_e2e, args.steps)

    ms_total, launches, clocks, ms_e2e = measure()
    if comm_failed():
        fall_back('in the timed region')
        ms_total, launches, clocks, ms_e2e = measure()

    # roofline of the dominant kernel: one more step with CUDA events around every GEMM launch
    ops.GEMM_PROFILE = []
    (eager_resident if graph is not None else step_resident)()
    torch.cuda.synchronize()
    # per stream: launches of one stream do not overlap each other, launches of different streams do (their event
    # intervals then include waiting for the other stream's kernel), so only a single-stream step gives a kernel rate
    per_stream = {}
    for e0, e1, _, stream in ops.GEMM_PROFILE:
        per_stream[stream] = per_stream.get(stream, 0.0) + e0.elapsed_time(e1)
    gemm_ms = max(per_stream.values()) if per_stream else 0.0
    gemm_ops = sum(rec[2] for rec in ops.GEMM_PROFILE) / max(len(per_stream), 1)
    n_gemm = len(ops.GEMM_PROFILE)
    gemm_streams = len(per_stream)
    ops.GEMM_PROFILE = None

    if args.kernel_totals:
        # per-kernel device time of one step (rank 0's view; every rank runs the step).  Not a timing run: the profiler
        # skews the ranks against each other, so waiting inside barriers and collectives reads longer than it is.
        from torch.profiler import ProfilerActivity, profile
        barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            (eager_resident if graph is not None else step_resident)()
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.kernel_totals, 'w') as f:
                f.write(f'{args.mode}, {args.layers} layers, tp{world}, collectives {model.comm if world > 1 else None}: '
                        f'{ms_total / args.steps:.2f} ms per step outside the profiler\n')
                f.write(prof.key_averages().table(sort_by='cuda_time_total', row_limit=20, max_name_column_width=60))
        barrier()

    # the tensor pipe's own INT8 rate on this GPU, measured after the timed region: the MMA-only kernel (no loads, no
    # stores) back to back for about two seconds, rate of the second half (at the power limit, like the step above)
    mma_only = None
    if world == 1:
        st_word = torch.zeros(1, dtype=torch.int32, device=dev)
        ops.mma_peak('i8', 20000, status=st_word)
        torch.cuda.synchronize()
        rates, t_end = [], time.time() + 2.0
        while time.time() < t_end:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            n_ops = ops.mma_peak('i8', 20000, status=st_word)
            e1.record()
            torch.cuda.synchronize()
            rates.append(n_ops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        if not int(st_word.item()) & 2:
            mma_only = statistics.median(rates[len(rates) // 2:])

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    hbm, bf16_burst, bf16_sus, src = measured_peaks()
    value = tokens * args.steps / (ms_total / 1e3)
    achieved = gemm_ops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else None
    peak = 2 * bf16_sus
    # DRAM traffic of the dominant launch (the gate/up GEMM, 57344 x 8192 weights).  The full launch (65536 token rows,
    # 25 ms, 4.7 GB of operands) is too large for a multi-pass profiler capture; dram__bytes_read + dram__bytes_write
    # was captured for 8192 token rows (`bench_kernels.py --only "gemm_w8a8 swiglu c5 gate+up 8192x"`): 1.022 GB read,
    # 0.457 GB written.  The B operand is re-streamed once per 4096-row group of m-tiles and A / C grow with the rows,
    # so a launch's traffic is proportional to its rows.  Only quoted for the unsharded prefill shape it was captured on.
    traffic, traffic_note = None, None
    if world == 1 and args.mode == 'prefill':
        rows = args.batch * args.seq
        traffic = (1.022e9 + 0.457e9) * rows / 8192.0
        traffic_note = ('bytes per gate/up GEMM launch: ncu dram read + write of the 8192-row case scaled by rows; '
                        'algorithmic A + B + C of that launch is %.3g' % (rows * 8192.0 + 57344 * 8192.0 + rows * 28672 * 2.0))
    line = {
        'metric': METRIC if args.mode == 'prefill' else METRIC.replace('prefill', 'decode'), 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': ms_total / args.steps, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
        'dtype': 'int8', 'data': 'synthetic',
        'config': {'workload': f'llama3-70b W8A8 {args.mode}, batch {args.batch} x seq {args.seq}, {args.layers} layers, '
                               'per-channel INT8 weights, dynamic per-token INT8 activations',
                   'parallelism': f'tp{world}', 'collectives': model.comm if world > 1 else None, 'micro_batches': mb or 1, 'l2': 'per-step working set (>70 GB of weights) exceeds L2; no flush needed',
                   'build_s': round(t_build, 1)},
        'e2e': {'value': tokens * args.steps / (ms_e2e / 1e3), 'unit': UNIT,
                'h2d_bytes_per_step': ids_host.numel() * ids_host.element_size(),
                'd2h_bytes_per_step': logits_host.numel() * logits_host.element_size()},
        'gpu_launches': launches,
        'roofline': {'bound': 'tensor', 'kernel': 'gemm_tcgen05_kernel (kind::i8)', 'achieved': achieved, 'peak': peak,
                     'unit': 'TOP/s', 'frac': (achieved / peak) if achieved else None, 'traffic': traffic,
                     'traffic_note': traffic_note, 'launches_per_step': n_gemm, 'gemm_ms_per_step': gemm_ms,
                     'gemm_streams': gemm_streams,
                     'peak_source': f'2 x bf16_tflops_sustained ({bf16_sus}) of {src}',
                     'mma_only_int8_tops': mma_only,
                     'frac_of_mma_only': (achieved / mma_only) if (achieved and mma_only) else None,
                     'mma_only_note': 'tcgen05.mma kind::i8 issued back to back by one CTA per SM on operands resident in shared '
                                      'memory (no loads, no stores), sustained for 2 s on this GPU after the timed region'},
        'clocks': clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        line['cpu_baseline'] = cpu_baseline(args.cpu_sample_tokens, args.layers)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
