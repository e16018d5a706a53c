"""Llama-architecture decoder stack whose Linears are W8A8 deploy modules, sharded
tensor-parallel (column / row) over the ranks of one node.

This is the sharded deploy workload: every Linear goes through
amct_b200.quantize() / convert() with dynamic per-token activation quantization,
i.e. NpuQuantizationLinear.forward = one activation-quant kernel + one tcgen05
INT8 GEMM with the dequant epilogue.  With ``fused_glue`` (the default) the residual
add, the RMSNorm and the activation quantization in front of the qkv and gate/up
projections are one kernel (ops.addnorm_quant_per_token), the rotary embedding is one
in-place kernel on the qkv output, and SwiGLU runs in the gate/up GEMM's epilogue;
attention, embedding and lm_head are plain torch.

Sharding (the reference has none; amct_pytorch/deploy_op/npu_quantization_linear.py
is the unit being sharded):
  column-parallel  q/k/v (fused) and gate/up (fused): each rank owns N/tp output
                   channels with their weight scales; the input is replicated, so
                   per-token activation scales are identical on every rank;
  row-parallel     o_proj and down_proj: each rank owns K/tp input channels; the
                   per-token scale is computed on the local K slice, the local
                   partial is dequantized to bf16 and summed over the ranks.
Two ways to do that sum.  `seq_parallel` (prefill default for tp > 1): the residual stream
is kept token-sharded -- rank r owns rows [r T/tp, (r+1) T/tp) -- so the partials are
REDUCE-SCATTERED, the add + RMSNorm + quant kernel runs on the local rows only, and what is
ALL-GATHERED in front of the column-parallel Linears is the INT8 codes and their fp32
per-token scales: 1 byte per element instead of 2, and no replicated glue work.  Per layer
and rank that moves 2 x (2 + 1) x T x hidden x (tp-1)/tp bytes instead of the 2 x 4 of two
bf16 all-reduces.  Otherwise (decode, or T not divisible by tp): one NCCL all-reduce per
row-parallel Linear on replicated activations.

The token-sharded collectives come in two forms (``comm``).  'nccl': reduce_scatter_tensor / all_gather_into_tensor.
'push': the compute kernels do the transfers with their own stores into peer-mapped buffers (PeerBuffers): the
row-parallel GEMM's epilogue writes each partial tile straight into the owning rank's staging slot, so the
reduce-scatter's bytes cross NVLink tile by tile while the GEMM runs; the add + RMSNorm + quant kernel sums the staged
partials in fp32 and stores its codes and scales into every rank's buffer, which is the all-gather.  Between them one
barrier kernel per transfer; no communication library kernel, no copy, no staging sum.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

import amct_b200 as amct
from amct_b200.backend import ops

W8A8_DYNAMIC_CFG = {
    'batch_num': 1,
    'quant_cfg': {
        'weights': {'type': 'int8', 'symmetric': True, 'strategy': 'channel'},
        'inputs': {'type': 'int8', 'symmetric': True, 'strategy': 'token', 'dynamic': True},
    },
    'algorithm': {'minmax'},
}


@dataclass
class LlamaShape:
    hidden: int = 8192
    n_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 28672
    n_layers: int = 80
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5


LLAMA3_70B = LlamaShape()
LLAMA3_8B = LlamaShape(hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, intermediate=14336, n_layers=32)


def shard_dims(shape, tp):
    """(K, N) of the four Linears one rank holds: fused q/k/v and gate/up are split along N
    (column-parallel), o_proj and down_proj along K (row-parallel)."""
    if shape.n_kv_heads % tp or shape.n_heads % tp or shape.intermediate % tp:
        raise ValueError(f'tp={tp} does not divide the head / intermediate sizes')
    h = shape.hidden
    return {
        'qkv_proj': (h, (shape.n_heads + 2 * shape.n_kv_heads) * shape.head_dim // tp),
        'o_proj': (shape.n_heads * shape.head_dim // tp, h),
        'gate_up_proj': (h, 2 * shape.intermediate // tp),
        'down_proj': (shape.intermediate // tp, h),
    }


class _Shard(nn.Module):
    """The float Linears of one rank's slice of a decoder layer (before quantization)."""

    def __init__(self, shape, tp, device, gen, std=0.02):
        super().__init__()
        dims = shard_dims(shape, tp)

        def lin(name):
            k, n = dims[name]
            m = nn.Linear(k, n, bias=False, device='meta', dtype=torch.bfloat16)
            m.weight = nn.Parameter(torch.empty(n, k, dtype=torch.bfloat16, device=device).normal_(0, std, generator=gen),
                                    requires_grad=False)
            return m

        self.qkv_proj = lin('qkv_proj')
        self.o_proj = lin('o_proj')
        self.gate_up_proj = lin('gate_up_proj')
        self.down_proj = lin('down_proj')


def rotary_tables(shape, positions, device):
    inv = 1.0 / (shape.rope_theta ** (torch.arange(0, shape.head_dim, 2, device=device, dtype=torch.float32) / shape.head_dim))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)


def apply_rotary(x, cos, sin):
    """x [B, S, H, D]; rotate-half convention."""
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


class PeerBuffers:
    """Peer-mapped buffers and the barrier of the 'push' collectives of one (micro-)batch of `rows_total` token rows.

    Every rank holds, in memory all ranks have mapped (torch symmetric memory, plain mappings, multicast off):
      stage[i]   [tp, rows, hidden] bf16   slot j = rank j's partial sums of THIS rank's rows, written by rank j's
                                           row-parallel GEMM epilogue (i = 0: o_proj, 1: down_proj)
      codes[i]   [rows_total, hidden] int8 all ranks' codes, slice j written by rank j's add + norm + quant kernel
      scales[i]  [rows_total] fp32         (i = 0: in front of qkv, 1: in front of gate/up)
      flags      [tp] int32                barrier words
    A transfer is complete for its readers after ONE barrier (amct_peer_barrier: release / acquire at system scope,
    bounded wait, status bit 1 on time-out).  No second barrier is needed before a buffer is written again: between
    a rank's last read of a buffer and any peer's next write into it lies a later barrier which that rank signals only
    after the read (two buffers of each kind, four barriers per layer; the argument is spelled out at `barrier`).
    All ranks call the methods in the same order, on one stream per instance."""

    def __init__(self, group, rows_total, hidden, device, dtype=torch.bfloat16):
        import os
        os.environ.setdefault('TORCH_SYMM_MEM_DISABLE_MULTICAST', '1')      # plain peer mappings only: nothing here uses multimem
        import torch.distributed._symmetric_memory as symm
        dist = torch.distributed
        self.tp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.hidden = rows_total // self.tp, hidden
        self.stage = [symm.empty((self.tp, self.rows, hidden), dtype=dtype, device=device) for _ in range(2)]
        self.codes = [symm.empty((rows_total, hidden), dtype=torch.int8, device=device) for _ in range(2)]
        self.scales = [symm.empty((rows_total,), dtype=torch.float32, device=device) for _ in range(2)]
        self.flags = symm.empty((self.tp,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)

        def peer_pointers(t):
            handle = symm.rendezvous(t, group)
            self._handles.append(handle)
            return [int(p_) for p_ in handle.buffer_ptrs]

        self._handles = []
        # device addresses of every rank's buffers through this process's mappings of them
        self.stage_ptrs = [peer_pointers(t) for t in self.stage]
        self.code_ptrs = [peer_pointers(t) for t in self.codes]
        self.scale_ptrs = [peer_pointers(t) for t in self.scales]
        self.flag_ptrs = peer_pointers(self.flags)
        self.seq = 0
        dist.barrier(group)                                                   # every rank's flags are zero before anyone signals

    def barrier(self):
        """Everything this rank's stream wrote into peers' buffers before this point is visible to the peers' kernels
        after it, and vice versa.  Reuse without a trailing barrier, per layer L (B1..B4 = the four barriers of a layer:
        after the o_proj scatter, after the post-attention codes, after the down_proj scatter, after the next layer's
        pre-attention codes): a peer writes stage[0] in o_proj(L) only after it passed B4(L-1), which this rank signals
        after its pre-attention kernel of layer L, i.e. after it read stage[0] in layer L-1; codes[0] is written by the
        peers' pre-attention kernel of L+1 after B3(L), signalled after this rank's qkv GEMM of L; codes[1] by their
        post-attention kernel of L+1 after B1(L+1), signalled after this rank's gate/up GEMM of L; stage[1] in
        down_proj(L+1) after B2(L+1), signalled after this rank's pre-attention kernel of L+1, which read it."""
        self.seq += 1
        ops.peer_barrier(self.flag_ptrs, self.rank, self.seq, self.status)

    def check(self):
        """Raise if a barrier of this instance ever gave up waiting (synchronizes the device)."""
        ops.raise_if_timed_out(self.status)


def any_rank(flag, group, device):
    """Logical OR of a per-rank flag over the group, the same answer on every rank."""
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
    return bool(t.item())


# stands for "the rows are the partial sums lying in the peer-mapped staging buffer" (push collectives)
STAGED = object()


def sum_staged(parts):
    """fp32 sum of staged partial sums [tp, rows, hidden] in rank order, rounded once: what the add + norm + quant
    kernel computes from them (used once per step, for the last layer's MLP output)."""
    acc = parts[0].float()
    for j in range(1, parts.shape[0]):
        acc = acc + parts[j].float()
    return acc.to(parts.dtype)


class DecoderLayer(nn.Module):
    def __init__(self, shape, tp, group, device, gen, fused_swiglu=True, fused_glue=True):
        super().__init__()
        self.shape, self.tp, self.group = shape, tp, group
        self.fused_glue = fused_glue
        self.heads = shape.n_heads // tp
        self.kv_heads = shape.n_kv_heads // tp
        self.linears = _Shard(shape, tp, device, gen)
        amct.quantize(self.linears, W8A8_DYNAMIC_CFG)
        amct.convert(self.linears)
        # the random gate/up rows are taken to be interleaved in blocks of 128, so SwiGLU runs in the GEMM epilogue
        self.fused_swiglu = fused_swiglu and (shape.intermediate // tp) % 128 == 0
        if self.fused_swiglu:
            self.linears.gate_up_proj.fused_act = 'swiglu'
        self.input_norm = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)
        self.post_norm = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)

    def _reduce(self, t):
        if self.tp > 1:
            torch.distributed.all_reduce(t, group=self.group)
        return t

    def _reduce_scatter(self, t):
        """Sum [T, H] partials over the ranks; this rank keeps rows [rank T/tp, (rank+1) T/tp)."""
        dist = torch.distributed
        tp, rank = self.tp, dist.get_rank(self.group)
        rows = t.shape[0] // tp
        if dist.get_backend(self.group) == 'nccl':
            out = torch.empty((rows, t.shape[1]), dtype=t.dtype, device=t.device)
            dist.reduce_scatter_tensor(out, t, group=self.group)
            return out
        dist.all_reduce(t, group=self.group)                     # backends without reduce-scatter
        return t[rank * rows:(rank + 1) * rows].contiguous()

    def _addnorm_quant_gather(self, x_loc, gamma, residual_loc, peers=None, half=0):
        """Local rows -> (codes [T, H] int8, scales [T] fp32 of ALL rows, new local residual).  With `peers` (push
        collectives) x_loc is STAGED when the rows to normalise are the partial sums lying in peers.stage[1 - half]
        (half 0: in front of qkv, the previous layer's down_proj; half 1: in front of gate/up, this layer's o_proj)."""
        if peers is not None:
            if x_loc is STAGED:
                parts = peers.stage[1 - half]
            else:
                parts = x_loc.unsqueeze(0)
            h = ops.addnorm_quant_per_token_tp(parts, gamma, self.shape.rms_eps, peers.code_ptrs[half], peers.scale_ptrs[half],
                                               peers.rank * peers.rows, residual=residual_loc)
            peers.barrier()
            return peers.codes[half], peers.scales[half], (h if h is not None else x_loc)
        dist = torch.distributed
        tp, rank = self.tp, dist.get_rank(self.group)
        rows, hid = x_loc.shape
        q_all = torch.empty((tp * rows, hid), dtype=torch.int8, device=x_loc.device)
        s_all = torch.empty(tp * rows, dtype=torch.float32, device=x_loc.device)
        q_loc, s_loc = q_all[rank * rows:(rank + 1) * rows], s_all[rank * rows:(rank + 1) * rows]
        _, _, h, _ = ops.addnorm_quant_per_token(x_loc, gamma, self.shape.rms_eps, residual=residual_loc, out_q=q_loc, out_scale=s_loc)
        dist.all_gather_into_tensor(q_all, q_loc, group=self.group)
        dist.all_gather_into_tensor(s_all, s_loc, group=self.group)
        return q_all, s_all, (h if h is not None else x_loc)

    def _row_parallel(self, linear, x, peers, half):
        """A row-parallel Linear followed by the sum over ranks, local rows kept.  With `peers` the partial sums are
        left in the owners' staging buffers (the next add + norm + quant kernel sums them) and STAGED is returned."""
        if peers is None:
            return self._reduce_scatter(linear(x))
        linear.forward_scatter(x, peers.stage_ptrs[half], peers.rank, peers.rows, peers.hidden)
        peers.barrier()
        return STAGED

    def sp_attention_half(self, x_loc, cos, sin, branch_loc, b, s, peers=None):
        """First half of a token-sharded prefill layer: (previous MLP output + residual) -> norm ->
        quant -> all-gather -> qkv -> rotary -> attention -> o_proj -> reduce-scatter.
        x_loc / branch_loc: this rank's [b s / tp, hidden] rows.  Returns (x_loc, o_loc)."""
        shp, lin = self.shape, self.linears
        if branch_loc is None:
            q8, ps, x_loc = self._addnorm_quant_gather(x_loc, self.input_norm, None, peers, 0)
        else:
            q8, ps, x_loc = self._addnorm_quant_gather(branch_loc, self.input_norm, x_loc, peers, 0)
        qkv = lin.qkv_proj.forward_quantized(q8, ps).reshape(b, s, -1)
        ops.rope_inplace(qkv, self.heads + self.kv_heads, shp.head_dim, cos, sin)
        q, k, v = qkv.split((self.heads * shp.head_dim, self.kv_heads * shp.head_dim, self.kv_heads * shp.head_dim), dim=-1)
        q = q.reshape(b, s, self.heads, shp.head_dim).transpose(1, 2)
        k = k.reshape(b, s, self.kv_heads, shp.head_dim).transpose(1, 2)
        v = v.reshape(b, s, self.kv_heads, shp.head_dim).transpose(1, 2)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        attn = attn.transpose(1, 2).reshape(b * s, self.heads * shp.head_dim)
        return x_loc, self._row_parallel(lin.o_proj, attn, peers, 0)

    def sp_mlp_half(self, x_loc, o_loc, peers=None):
        """Second half: (attention output + residual) -> norm -> quant -> all-gather -> gate/up with
        SwiGLU -> down_proj -> reduce-scatter.  Returns (x_loc, branch_loc)."""
        lin = self.linears
        q8, ps, x_loc = self._addnorm_quant_gather(o_loc, self.post_norm, x_loc, peers, 1)
        act = lin.gate_up_proj.forward_quantized(q8, ps)
        if not self.fused_swiglu:
            gate, up = act.chunk(2, dim=-1)
            act = F.silu(gate) * up
        return x_loc, self._row_parallel(lin.down_proj, act, peers, 1)

    def forward_seq_parallel(self, x_loc, cos, sin, branch_loc, b, s, peers=None):
        """Prefill with a token-sharded residual stream: x_loc / branch_loc are this rank's
        [b s / tp, hidden] rows.  Returns (x_loc, branch_loc) like forward() with fused_glue."""
        x_loc, o_loc = self.sp_attention_half(x_loc, cos, sin, branch_loc, b, s, peers)
        return self.sp_mlp_half(x_loc, o_loc, peers)

    def forward(self, x, cos, sin, kv_cache=None, branch=None):
        """x [B, S, hidden] bf16 (the residual stream).  kv_cache: None (prefill, causal) or (k, v, past)
        with k, v [B, kvh, >= past + S, D] holding `past` keys/values (decode: S new tokens attend to
        past + S).  With fused_glue the layer returns (x, branch): the residual stream BEFORE the MLP
        output `branch` is added -- the next layer's first kernel does that add."""
        shp, lin = self.shape, self.linears
        b, s, _ = x.shape
        if self.fused_glue:
            q8, ps, h, _ = ops.addnorm_quant_per_token(x if branch is None else branch, self.input_norm, shp.rms_eps,
                                                       residual=None if branch is None else x)
            if h is not None:
                x = h
            qkv = lin.qkv_proj.forward_quantized(q8, ps)
            ops.rope_inplace(qkv, self.heads + self.kv_heads, shp.head_dim, cos, sin)
            q, k, v = qkv.split((self.heads * shp.head_dim, self.kv_heads * shp.head_dim, self.kv_heads * shp.head_dim), dim=-1)
            q = q.reshape(b, s, self.heads, shp.head_dim).transpose(1, 2)
            k = k.reshape(b, s, self.kv_heads, shp.head_dim).transpose(1, 2)
        else:
            hn = F.rms_norm(x, (shp.hidden,), self.input_norm, shp.rms_eps)
            qkv = lin.qkv_proj(hn)
            q, k, v = qkv.split((self.heads * shp.head_dim, self.kv_heads * shp.head_dim, self.kv_heads * shp.head_dim), dim=-1)
            q = apply_rotary(q.reshape(b, s, self.heads, shp.head_dim), cos, sin).transpose(1, 2)
            k = apply_rotary(k.reshape(b, s, self.kv_heads, shp.head_dim), cos, sin).transpose(1, 2)
        v = v.reshape(b, s, self.kv_heads, shp.head_dim).transpose(1, 2)
        if kv_cache is not None:
            # kv_cache = (k, v, past): buffers [B, kvh, past + S, D] whose first `past` positions are filled;
            # the new keys / values are written in place behind them
            kc, vc, past = kv_cache
            kc[:, :, past:past + s].copy_(k)
            vc[:, :, past:past + s].copy_(v)
            if past == 0:
                attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            elif s == 1:
                attn = F.scaled_dot_product_attention(q, kc[:, :, :past + 1], vc[:, :, :past + 1], is_causal=False, enable_gqa=True)
            else:
                # new token i sees the cached positions and new tokens 0..i
                mask = torch.ones(s, past + s, dtype=torch.bool, device=x.device).tril(diagonal=past)
                attn = F.scaled_dot_product_attention(q, kc[:, :, :past + s], vc[:, :, :past + s], attn_mask=mask, enable_gqa=True)
        else:
            attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        attn = attn.transpose(1, 2).reshape(b, s, self.heads * shp.head_dim)
        if self.fused_glue:
            o = self._reduce(lin.o_proj(attn))
            q8, ps, x, _ = ops.addnorm_quant_per_token(o, self.post_norm, shp.rms_eps, residual=x)
            act = lin.gate_up_proj.forward_quantized(q8, ps)
            if not self.fused_swiglu:
                gate, up = act.chunk(2, dim=-1)
                act = F.silu(gate) * up
            return x, self._reduce(lin.down_proj(act))
        x = x + self._reduce(lin.o_proj(attn))
        hn = F.rms_norm(x, (shp.hidden,), self.post_norm, shp.rms_eps)
        if self.fused_swiglu:
            act = lin.gate_up_proj(hn)
        else:
            gate, up = lin.gate_up_proj(hn).chunk(2, dim=-1)
            act = F.silu(gate) * up
        x = x + self._reduce(lin.down_proj(act))
        return x


class LlamaW8A8(nn.Module):
    """Random-initialised Llama stack; rank `rank` of `tp` holds its shard of every layer."""

    def __init__(self, shape=LLAMA3_70B, tp=1, rank=0, group=None, device='cuda', seed=4, n_layers=None, fused_swiglu=True,
                 fused_glue=True, seq_parallel=True, comm='nccl'):
        """comm: collectives of the token-sharded prefill: 'nccl' (reduce-scatter / all-gather kernels) or 'push' (the
        GEMM epilogue and the add + norm + quant kernel store into peer-mapped buffers themselves, see PeerBuffers)."""
        super().__init__()
        if comm not in ('nccl', 'push'):
            raise ValueError(f'comm={comm!r}')
        self.comm, self._peers = comm, {}
        if shape.n_kv_heads % tp or shape.n_heads % tp or shape.intermediate % tp:
            raise ValueError(f'tp={tp} does not divide the head / intermediate sizes')
        self.shape, self.tp = shape, tp
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
        shared = torch.Generator(device=device).manual_seed(seed)            # replicated tensors: same on every rank
        self.embed = torch.empty(shape.vocab, shape.hidden, dtype=torch.bfloat16, device=device).normal_(0, 0.02, generator=shared)
        self.lm_head = torch.empty(shape.vocab, shape.hidden, dtype=torch.bfloat16, device=device).normal_(0, 0.02, generator=shared)
        self.final_norm = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)
        self.fused_glue = fused_glue
        self.seq_parallel = seq_parallel and fused_glue and tp > 1
        self.group, self.rank = group, rank
        self.layers = nn.ModuleList(DecoderLayer(shape, tp, group, device, gen, fused_swiglu, fused_glue)
                                    for _ in range(n_layers if n_layers is not None else shape.n_layers))

    def _peer_buffers(self, j, rows_total, device):
        if self.comm != 'push':
            return None
        key = (j, rows_total)
        if key not in self._peers:
            self._peers[key] = PeerBuffers(self.group, rows_total, self.shape.hidden, device)
        return self._peers[key]

    def check_comm(self):
        """Raise if any barrier of the push collectives timed out since the model was built (synchronizes)."""
        for peers in self._peers.values():
            peers.check()

    def comm_failed_anywhere(self):
        """True on EVERY rank if a barrier of the push collectives gave up waiting on ANY rank: the ranks must agree
        before one of them changes the sequence of collectives it issues (switching to NCCL, repeating a step)."""
        if self.tp == 1 or self.comm != 'push':
            return False
        try:
            self.check_comm()
            failed = False
        except RuntimeError:
            failed = True
        return any_rank(failed, self.group, self.embed.device)

    @torch.no_grad()
    def forward(self, token_ids, kv_caches=None, past_len=0, micro_batches=None):
        """token_ids [B, S] -> logits of the last position [B, vocab] (fp32).

        micro_batches > 1 (tp > 1) cuts the batch into micro-batches that run on separate CUDA
        streams, half layer by half layer, so that one micro-batch's collective can run while
        the other one computes."""
        b, s = token_ids.shape
        if micro_batches is None:
            # one micro-batch by default: with two (two CUDA streams, ping-pong order) the collectives of one ran next to
            # the GEMMs of the other only on paper (a persistent GEMM fills every SM): measured 27.4 vs 27.9 k tokens/s
            # at 2 GPUs, 68.0 vs 69.8 k at 8 with NCCL
            micro_batches = 1
        if self.comm == 'push' and micro_batches > 2:
            # more streams than two put spinning barrier blocks of one stream in front of another stream's work
            raise ValueError("comm='push' runs at most two micro-batch streams")
        pos = torch.arange(past_len, past_len + s, device=token_ids.device)
        cos, sin = rotary_tables(self.shape, pos, token_ids.device)
        sp = self.seq_parallel and kv_caches is None and (b // micro_batches) * s % self.tp == 0 and b % micro_batches == 0
        if micro_batches == 1:
            if sp:
                x = self._stack_seq_parallel(token_ids, cos, sin)
            else:
                x = self._stack(F.embedding(token_ids, self.embed), cos, sin, kv_caches)
        elif sp:
            main = torch.cuda.current_stream()
            if getattr(self, '_streams', None) is None or len(self._streams) != micro_batches:
                self._streams = [torch.cuda.Stream(device=token_ids.device) for _ in range(micro_batches)]
            parts = list(token_ids.chunk(micro_batches, dim=0))
            rows = [p_.numel() // self.tp for p_ in parts]
            xs, branches = [None] * len(parts), [None] * len(parts)
            for st in self._streams:
                st.wait_stream(main)
            for j, ids in enumerate(parts):
                with torch.cuda.stream(self._streams[j]):
                    xs[j] = F.embedding(ids.reshape(-1)[self.rank * rows[j]:(self.rank + 1) * rows[j]], self.embed)
            # ping-pong: the collectives of one micro-batch's half layer are queued right behind that
            # half's kernels, so on NCCL's in-order stream each one waits only for work issued just
            # before it, and runs while the other micro-batch computes
            outs = [None] * len(parts)
            peers = [self._peer_buffers(j, ids.numel(), token_ids.device) for j, ids in enumerate(parts)]
            for layer in self.layers:
                for j, ids in enumerate(parts):
                    with torch.cuda.stream(self._streams[j]):
                        xs[j], outs[j] = layer.sp_attention_half(xs[j], cos, sin, branches[j], ids.shape[0], s, peers[j])
                for j in range(len(parts)):
                    with torch.cuda.stream(self._streams[j]):
                        xs[j], branches[j] = layer.sp_mlp_half(xs[j], outs[j], peers[j])
            for j, ids in enumerate(parts):
                with torch.cuda.stream(self._streams[j]):
                    loc = xs[j] + (sum_staged(peers[j].stage[1]) if branches[j] is STAGED else branches[j])
                    full = torch.empty((ids.numel(), loc.shape[1]), dtype=loc.dtype, device=loc.device)
                    torch.distributed.all_gather_into_tensor(full, loc, group=self.group)
                    xs[j] = full.reshape(ids.shape[0], s, -1)[:, -1:]
            for j, st in enumerate(self._streams[:len(parts)]):
                main.wait_stream(st)
                xs[j].record_stream(main)
            x = torch.cat(xs, dim=0)
        else:
            main = torch.cuda.current_stream()
            if getattr(self, '_streams', None) is None or len(self._streams) != micro_batches:
                self._streams = [torch.cuda.Stream(device=token_ids.device) for _ in range(micro_batches)]
            parts = list(token_ids.chunk(micro_batches, dim=0))
            xs = [None] * len(parts)
            for st in self._streams:
                st.wait_stream(main)
            for j, ids in enumerate(parts):
                with torch.cuda.stream(self._streams[j]):
                    xs[j] = F.embedding(ids, self.embed)
            branches = [None] * len(parts)
            for layer in self.layers:
                for j in range(len(parts)):
                    with torch.cuda.stream(self._streams[j]):
                        if self.fused_glue:
                            xs[j], branches[j] = layer(xs[j], cos, sin, None, branches[j])
                        else:
                            xs[j] = layer(xs[j], cos, sin, None)
            if self.fused_glue:
                for j in range(len(parts)):
                    with torch.cuda.stream(self._streams[j]):
                        xs[j] = xs[j][:, -1:] + branches[j][:, -1:]
            for j, st in enumerate(self._streams[:len(parts)]):
                main.wait_stream(st)
                xs[j].record_stream(main)
            x = torch.cat([t[:, -1:] for t in xs], dim=0)
        x = F.rms_norm(x[:, -1], (self.shape.hidden,), self.final_norm, self.shape.rms_eps)
        return (x @ self.lm_head.t()).float()

    def _stack_seq_parallel(self, token_ids, cos, sin):
        """Prefill of [b, s] token ids with the residual stream sharded by token rows over the ranks;
        returns the last position's hidden state [b, 1, hidden] (replicated)."""
        b, s = token_ids.shape
        rows = b * s // self.tp
        ids_loc = token_ids.reshape(-1)[self.rank * rows:(self.rank + 1) * rows]
        x_loc, branch_loc = F.embedding(ids_loc, self.embed), None
        peers = self._peer_buffers(0, b * s, token_ids.device)
        for layer in self.layers:
            x_loc, branch_loc = layer.forward_seq_parallel(x_loc, cos, sin, branch_loc, b, s, peers)
        if branch_loc is not None:
            x_loc = x_loc + (sum_staged(peers.stage[1]) if branch_loc is STAGED else branch_loc)
        full = torch.empty((b * s, x_loc.shape[1]), dtype=x_loc.dtype, device=x_loc.device)
        torch.distributed.all_gather_into_tensor(full, x_loc.contiguous(), group=self.group)
        return full.reshape(b, s, -1)[:, -1:]

    def _stack(self, x, cos, sin, kv_caches):
        """All decoder layers on one stream; returns the final residual stream."""
        branch = None
        for i, layer in enumerate(self.layers):
            cache = None if kv_caches is None else kv_caches[i]
            if self.fused_glue:
                x, branch = layer(x, cos, sin, cache, branch)
            else:
                x = layer(x, cos, sin, cache)
        if branch is not None:
            x = x[:, -1:] + branch[:, -1:]          # only the last position feeds the logits
        return x

    def linear_ops_per_token(self):
        """2*K*N summed over the quantized Linears of all layers (whole model, all ranks)."""
        sh = self.shape
        per_layer = 2 * (sh.hidden * (sh.n_heads + 2 * sh.n_kv_heads) * sh.head_dim + sh.n_heads * sh.head_dim * sh.hidden
                         + sh.hidden * 2 * sh.intermediate + sh.intermediate * sh.hidden)
        return per_layer * len(self.layers)
