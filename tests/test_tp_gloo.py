"""Tensor-parallel sharding of the W8A8 Linear pair, checked on CPU with two gloo ranks.

The GPU kernels cannot run here; what is tested is the sharding arithmetic itself, with
the CPU oracle standing in for each rank's kernels: column-parallel then row-parallel
W8A8 Linears with per-shard dynamic activation scales and one all-reduce reproduce the
unsharded result within the bf16 tolerance, and each shard's codes are bit-identical to
the oracle run on the same slice."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import intq, npu_ops


def _w8a8(x, w):
    """Oracle W8A8 Linear with dynamic per-token activation quantization -> bf16."""
    sw, _ = intq.weight_scale_offset(w, 'int8', True, 'channel')
    wq = intq.w8a8_weight_codes(w, sw.reshape(-1))
    q, s = intq.dynamic_per_token(x)
    return npu_ops.npu_quant_matmul(q, wq.t(), sw.reshape(-1), s, None, torch.bfloat16), q


def _worker(rank, world, port, ret):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(24, 64, generator=g).to(torch.bfloat16)
    w_up = (torch.randn(96, 64, generator=g) * 0.1).to(torch.bfloat16)      # column-parallel: split N
    w_down = (torch.randn(64, 96, generator=g) * 0.1).to(torch.bfloat16)    # row-parallel: split K
    n_loc = 96 // world
    up_loc = w_up[rank * n_loc:(rank + 1) * n_loc]
    down_loc = w_down[:, rank * n_loc:(rank + 1) * n_loc]
    h_loc, q_in = _w8a8(x, up_loc)
    part, q_mid = _w8a8(h_loc, down_loc)
    total = part.float()
    dist.all_reduce(total)
    # unsharded reference on every rank
    h_full, q_in_full = _w8a8(x, w_up)
    ref, _ = _w8a8(h_full, w_down)
    ok_codes = torch.equal(q_in, q_in_full)                                  # replicated input: identical codes
    ok_cols = torch.equal(h_loc, h_full[:, rank * n_loc:(rank + 1) * n_loc])  # column shard = slice of the full output
    _, q_slice = _w8a8(h_full[:, rank * n_loc:(rank + 1) * n_loc].contiguous(), down_loc)
    ok_slice = torch.equal(q_mid, q_slice)                                   # per-shard codes = oracle on the same slice
    err = ((total - ref.float()).abs().max() / ref.float().abs().max()).item()
    ret[rank] = (ok_codes, ok_cols, ok_slice, err)
    dist.destroy_process_group()


def test_column_then_row_parallel_w8a8_two_ranks():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        for rank in range(world):
            ok_codes, ok_cols, ok_slice, err = ret[rank]
            assert ok_codes and ok_cols and ok_slice
            assert err < 3e-2, err          # two chained 8-bit quantizations with per-shard scales vs unsharded


def _sp_worker(rank, world, port, ret):
    """Sequence-parallel dataflow of one decoder block with the oracle as each rank's kernels:
    local rows -> add + RMSNorm + quant -> all-gather of codes and scales -> column-parallel W8A8
    -> row-parallel W8A8 partial -> sum over ranks, local rows kept."""
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    g = torch.Generator().manual_seed(1)
    t, hid, inter = 16, 64, 96
    x = torch.randn(t, hid, generator=g).to(torch.bfloat16)
    res = torch.randn(t, hid, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(hid, generator=g)).to(torch.bfloat16)
    w_up = (torch.randn(inter, hid, generator=g) * 0.1).to(torch.bfloat16)
    w_down = (torch.randn(hid, inter, generator=g) * 0.1).to(torch.bfloat16)
    rows, n_loc = t // world, inter // world
    sl = slice(rank * rows, (rank + 1) * rows)
    # token-sharded glue
    h_loc, _, q_loc, s_loc = intq.addnorm_dynamic_per_token(x[sl], gamma, 1e-5, res[sl])
    q_all = torch.empty(t, hid, dtype=torch.int8)
    s_all = torch.empty(t, dtype=torch.float32)
    dist.all_gather_into_tensor(q_all, q_loc.contiguous())
    dist.all_gather_into_tensor(s_all, s_loc.contiguous())
    # the same on all rows at once (what a replicated rank would compute)
    h_full, _, q_full, s_full = intq.addnorm_dynamic_per_token(x, gamma, 1e-5, res)
    ok_gather = torch.equal(q_all, q_full) and torch.equal(s_all, s_full) and torch.equal(h_loc, h_full[sl])
    # column-parallel then row-parallel Linear on the gathered codes
    up_loc, down_loc = w_up[rank * n_loc:(rank + 1) * n_loc], w_down[:, rank * n_loc:(rank + 1) * n_loc]
    sw, _ = intq.weight_scale_offset(up_loc, 'int8', True, 'channel')
    mid = npu_ops.npu_quant_matmul(q_all, intq.w8a8_weight_codes(up_loc, sw.reshape(-1)).t(), sw.reshape(-1), s_all, None, torch.bfloat16)
    part, _ = _w8a8(mid, down_loc)
    total = part.float()
    dist.all_reduce(total)                                   # gloo has no reduce-scatter: sum, then keep the local rows
    mine = total[sl]
    # reference: the replicated (all-reduce) variant gives the same rows
    ok_rows = mine.shape == (rows, hid)
    ret[rank] = (ok_gather, ok_rows, mine.clone(), total.clone())
    dist.destroy_process_group()


def test_sequence_parallel_dataflow_two_ranks():
    world = 2
    port = 31500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_sp_worker, args=(world, port, ret), nprocs=world, join=True)
        full = ret[0][3]
        for rank in range(world):
            ok_gather, ok_rows, mine, total = ret[rank]
            assert ok_gather            # per-token quantization commutes with sharding the token rows: bit-identical
            assert ok_rows
            assert torch.equal(total, full)
            assert torch.equal(mine, full[rank * (16 // world):(rank + 1) * (16 // world)])


def test_shard_dims():
    from amct_b200.workloads.llama_tp import shard_dims, LLAMA3_70B
    d1, d8 = shard_dims(LLAMA3_70B, 1), shard_dims(LLAMA3_70B, 8)
    assert d1 == {'qkv_proj': (8192, 10240), 'o_proj': (8192, 8192), 'gate_up_proj': (8192, 57344), 'down_proj': (28672, 8192)}
    assert d8 == {'qkv_proj': (8192, 1280), 'o_proj': (1024, 8192), 'gate_up_proj': (8192, 7168), 'down_proj': (3584, 8192)}
    with pytest.raises(ValueError):
        shard_dims(LLAMA3_70B, 3)
    # total Linear work is independent of tp
    work = lambda d: sum(k * n for k, n in d.values())
    assert work(d1) == 8 * work(d8)


def _agree_worker(rank, world, port, ret):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    from amct_b200.workloads import llama_tp

    class Model:                                            # the two attributes and the method the agreement uses
        tp, comm, group = world, 'push', dist.group.WORLD
        embed = torch.zeros(1)

        def __init__(self, failed):
            self.failed = failed

        def check_comm(self):
            if self.failed:
                raise RuntimeError('a device-side wait timed out')

    out = []
    for failing_rank in (None, 1, 0):
        m = Model(failed=(rank == failing_rank))
        out.append(llama_tp.LlamaW8A8.comm_failed_anywhere(m))
    m = Model(failed=True)
    m.comm = 'nccl'                                         # nothing to agree on without the push collectives
    out.append(llama_tp.LlamaW8A8.comm_failed_anywhere(m))
    ret[rank] = out
    dist.destroy_process_group()


def test_every_rank_learns_of_a_barrier_timeout_on_any_rank():
    """The switch from the push collectives to NCCL (bench.py) must be taken by all ranks or by none: a time-out seen by
    one rank, forced here on the host, is reported on both."""
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_agree_worker, args=(world, 29533, ret), nprocs=world, join=True)
    for rank in range(world):
        assert ret[rank] == [False, True, True, False], (rank, ret[rank])
