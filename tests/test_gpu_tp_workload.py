"""Multi-GPU check of the tensor-parallel workload at a toy shape, for every world size the visible GPUs allow
(2, 4, 8): the token-sharded prefill with NCCL collectives and with the push collectives (GEMM epilogue and
add + norm + quant kernel storing into peer-mapped buffers) against the replicated all-reduce prefill on the same
shards.  Ranks are child processes over NCCL on 127.0.0.1; every device-side wait is bounded and the process group
has a short time-out, so a stall ends as a failed test."""
import datetime
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank),
                            timeout=datetime.timedelta(seconds=60))
    from amct_b200.workloads.llama_tp import LlamaW8A8, LlamaShape
    shape = LlamaShape(hidden=1024, n_heads=8, n_kv_heads=8, head_dim=128, intermediate=2048, n_layers=3, vocab=512)
    ids = torch.randint(0, 512, (4, 32), generator=torch.Generator().manual_seed(3)).cuda()
    out = {}
    for name, kw in {'sp': dict(seq_parallel=True), 'ar': dict(seq_parallel=False),
                     'push': dict(seq_parallel=True, comm='push')}.items():
        m = LlamaW8A8(shape, tp=world, rank=rank, group=dist.group.WORLD, device=f'cuda:{rank}', seed=11, **kw)
        out[name] = m(ids, micro_batches=1).cpu()
        out[name + '_again'] = m(ids, micro_batches=1).cpu()              # buffers are reused without a trailing barrier
        out[name + '_mb2'] = m(ids, micro_batches=2).cpu()
        m.check_comm()
    ret[rank] = out
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 4, 8])
def test_seq_parallel_prefill_matches_all_reduce_prefill(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    import torch.multiprocessing as mp
    port = 32500 + (os.getpid() + 7 * world) % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        r0 = ret[0]
        for r in range(1, world):
            for key in r0:
                assert torch.equal(r0[key], ret[r][key]), (key, r)        # logits are replicated
        ref = r0['ar']
        scale = ref.abs().max()
        # The variants see the same activations up to the rounding of the sum over ranks (and the one-ulp freedom of
        # the normalisation's fp32 sum).  With two ranks the sum is the same however it is formed; with more, a
        # one-ulp difference of a bf16 partial sum can move an INT8 code of the next Linear by one step (1 / 127 of the
        # row's range), and the logits of this three-layer toy model carry a few of those: NCCL's own reduce-scatter
        # and all-reduce prefills differ by 2.2e-2 of the largest logit at four ranks.  Stated bound: 2e-2 at two
        # ranks, 5e-2 beyond.
        errors = {key: float((r0[key] - ref).abs().max() / scale) for key in r0}
        for key in ('sp', 'sp_mb2', 'ar_mb2', 'push', 'push_mb2'):
            assert errors[key] < (2e-2 if world == 2 else 5e-2), errors
        # this library's own collectives are deterministic, and safe to run twice (buffers are reused without a trailing barrier)
        assert torch.equal(r0['push'], r0['push_again']), errors
        if world == 2:
            # the sum of two bf16 partials rounds once whichever way it is formed: bit-identical to NCCL's
            assert torch.equal(r0['push'], r0['sp']) and torch.equal(r0['push_mb2'], r0['sp_mb2'])
        assert r0['sp'].shape == (4, 512)
