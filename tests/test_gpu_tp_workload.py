"""Two-GPU check of the tensor-parallel workload: the token-sharded (reduce-scatter + INT8
all-gather) prefill against the replicated (all-reduce) one on the same shards.  Needs two
visible GPUs; skipped otherwise.  Ranks are child processes over NCCL on 127.0.0.1."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    from amct_b200.workloads.llama_tp import LlamaW8A8, LlamaShape
    shape = LlamaShape(hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, intermediate=2048, n_layers=2, vocab=512)
    ids = torch.randint(0, 512, (4, 32), generator=torch.Generator().manual_seed(3)).cuda()
    out = {}
    for name, kw in {'sp': dict(seq_parallel=True), 'ar': dict(seq_parallel=False), 'ce': dict(seq_parallel=True, comm='ce')}.items():
        m = LlamaW8A8(shape, tp=world, rank=rank, group=dist.group.WORLD, device=f'cuda:{rank}', seed=11, **kw)
        out[name] = m(ids, micro_batches=1).cpu()
        out[name + '_mb2'] = m(ids, micro_batches=2).cpu()
        m.check_comm()
    ret[rank] = out
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_seq_parallel_prefill_matches_all_reduce_prefill():
    import torch.multiprocessing as mp
    world, port = 2, 32500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        r0, r1 = ret[0], ret[1]
        for key in r0:
            assert torch.equal(r0[key], r1[key]), key                   # logits are replicated
        ref = r0['ar']
        scale = ref.abs().max()
        # a sum of two partials does not depend on its order, so the two variants see the same
        # activations up to the one-ulp freedom of the normalisation's fp32 sum
        for key in ('sp', 'sp_mb2', 'ar_mb2'):
            assert float((r0[key] - ref).abs().max() / scale) < 2e-2, key
        # copy-engine collectives: the sum of two bf16 partials rounds once whichever way it is formed
        assert torch.equal(r0['ce'], r0['sp']) and torch.equal(r0['ce_mb2'], r0['sp_mb2'])
        assert r0['sp'].shape == (4, 512)
