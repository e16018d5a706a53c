"""AWQ and GPTQ calibration through the public API on the GPU.

Their search loops are host control flow around the fake-quant kernel, and their floating-point
reductions (layer outputs, Cholesky) are not bit-reproducible between CPU and GPU, so these are
behavioural tests: module classes, factor shapes, and that each algorithm does what it is for --
the calibrated layer's output error is not worse than plain min-max quantization of the same layer."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


class Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc = torch.nn.Linear(256, 128)
        self.lm_head = torch.nn.Linear(128, 8)

    def forward(self, x):
        return self.lm_head(self.fc(x))


def make(seed=0):
    torch.manual_seed(seed)
    net = Net().to(torch.bfloat16).cuda()
    x = torch.randn(96, 256, device='cuda').to(torch.bfloat16)
    x[:, ::17] *= 8                                   # a few salient input channels
    return net, x


def layer_error(net, ref_net, x):
    return (net.fc(x).float() - ref_net.fc(x).float()).pow(2).mean().item()


def minmax_error(ref_net, x, weights):
    import amct_b200 as amct
    net = copy.deepcopy(ref_net)
    amct.quantize(net, {'batch_num': 1, 'quant_cfg': {'weights': weights}, 'algorithm': 'minmax', 'skip_layers': {'lm_head'}})
    net(x)
    amct.convert(net)
    return layer_error(net, ref_net, x)


@pytest.mark.parametrize('weights', [{'type': 'int4', 'symmetric': True, 'strategy': 'channel'},
                                     {'type': 'int4', 'symmetric': False, 'strategy': 'group', 'group_size': 32}])
def test_awq_flow(weights):
    import amct_b200 as amct
    ref_net, x = make(1)
    net = copy.deepcopy(ref_net)
    amct.quantize(net, {'batch_num': 1, 'quant_cfg': {'weights': weights}, 'algorithm': {'awq': {'grids_num': 8}},
                        'skip_layers': {'lm_head'}})
    assert type(net.fc).__name__ == 'LinearAWQuant' and type(net.lm_head).__name__ == 'Linear'
    net(x)
    assert net.fc.scale.shape == (1, 256) and net.fc.scale_w is not None
    amct.convert(net)
    assert type(net.fc).__name__ == 'NpuWeightQuantizedLinear'
    assert net.fc.scale_factor.shape == (1, 256) and net.fc.quantized_weight.dtype == torch.int32
    err = layer_error(net, ref_net, x)
    assert err <= minmax_error(ref_net, x, weights) * 1.05      # grid point 0 is plain min-max: AWQ cannot be worse


def test_awq_preset_runs():
    import amct_b200 as amct
    net, x = make(2)
    amct.quantize(net, amct.INT4_AWQ_WEIGHT_QUANT_CFG)
    net(x)
    amct.convert(net)
    assert type(net.fc).__name__ == 'NpuWeightQuantizedLinear' and type(net.lm_head).__name__ == 'Linear'
    assert torch.isfinite(net(x).float()).all()


@pytest.mark.parametrize('weights', [{'type': 'int4', 'symmetric': True, 'strategy': 'channel'},
                                     {'type': 'int8', 'symmetric': False, 'strategy': 'group', 'group_size': 64}])
def test_gptq_flow(weights):
    import amct_b200 as amct
    ref_net, x = make(3)
    net = copy.deepcopy(ref_net)
    amct.quantize(net, {'batch_num': 2, 'quant_cfg': {'weights': weights}, 'algorithm': {'gptq'}, 'skip_layers': {'lm_head'}})
    assert type(net.fc).__name__ == 'GPTQuant'
    net(x[:48])
    assert net.fc.scale_w is None                    # factors appear once batch_num batches were seen
    net(x[48:])
    assert net.fc.scale_w is not None
    amct.convert(net)
    assert type(net.fc).__name__ == 'NpuWeightQuantizedLinear'
    err = layer_error(net, ref_net, x)
    assert err <= minmax_error(ref_net, x, weights) * 1.02     # error feedback must not lose to round-to-nearest


GPTQ_BLOCK_CASES = [(40, 128, 'int4', False, 32), (9, 70, 'int8', True, 0), (130, 33, 'int4', True, 16), (5, 128, 'int8', False, 0)]


@pytest.mark.parametrize('n,b,qt,sym,group', GPTQ_BLOCK_CASES)
def test_gptq_block_kernel_matches_column_loop(n, b, qt, sym, group):
    """amct_gptq_block against the column loop written out with tensor ops (the reference's
    amct_pytorch/quantize_op/gptq_module.py:137-151 with the oracle's fake quantization): fp32, same operation order,
    so the updated block and the errors agree bit for bit."""
    from amct_b200.backend import ops
    from oracle import intq
    g = torch.Generator().manual_seed(n + b)
    w = torch.randn(n, b, generator=g) * 0.05
    a = torch.randn(b, b, generator=g)
    hinv = torch.linalg.cholesky(a @ a.t() + b * torch.eye(b), upper=True).contiguous()
    groups = 4 if group else 1
    per_row = group != 0 or n % 2 == 0                     # per-channel factors, or (odd n, no groups) one factor for all rows
    rows = n if per_row else 1
    scale = torch.rand(rows, groups, generator=g) * 0.01 + 0.004
    offset = None if sym else torch.randint(-3, 4, (rows, groups), generator=g, dtype=torch.int32)
    col_group = torch.randint(0, groups, (b,), generator=g, dtype=torch.int32)
    want_w, want_e = w.clone(), torch.zeros(n, b)
    for i in range(b):
        col = want_w[:, i].clone()
        s = scale[:, col_group[i]].reshape(-1, 1)
        o = None if offset is None else offset[:, col_group[i]].reshape(-1, 1)
        q = intq.fake_quant(col.reshape(-1, 1), qt, s, o).reshape(-1)
        e = (col - q) / hinv[i, i]
        want_w[:, i:] = want_w[:, i:] - e.unsqueeze(1) * hinv[i, i:].unsqueeze(0)
        want_e[:, i] = e
    got_w = w.clone().cuda()
    got_e = ops.gptq_block(got_w, hinv.cuda(), scale.cuda(), None if offset is None else offset.cuda(), col_group.cuda(),
                           4 if qt == 'int4' else 8)
    assert torch.equal(got_e.cpu(), want_e) and torch.equal(got_w.cpu(), want_w)
