"""Host-side logic that needs no GPU: config schema, registry, type checks, the
C-ABI library's exported symbols, and the loud failure on CPU tensors."""
import ctypes
import os

import pytest
import torch
import torch.nn as nn

import amct_b200 as amct
from amct_b200.algorithm import AlgorithmRegistry
from amct_b200.backend import lib
from amct_b200.config import parse_config
from amct_b200.quantize_op.base_quant_module import BaseQuantizeModule


class Net(nn.Module):
    def __init__(self, dtype=torch.bfloat16):
        super().__init__()
        self.linear1 = nn.Linear(64, 64).to(dtype)
        self.linear2 = nn.Linear(64, 32).to(dtype)
        self.lm_head = nn.Linear(32, 1).to(dtype)

    def forward(self, x):
        return self.lm_head(self.linear2(self.linear1(x)))


def cfg(weights, inputs=None, algorithm='minmax', **kw):
    c = {'batch_num': 1, 'quant_cfg': {'weights': weights}, 'algorithm': algorithm}
    if inputs is not None:
        c['quant_cfg']['inputs'] = inputs
    c.update(kw)
    return c


W8 = {'type': 'int8', 'symmetric': True, 'strategy': 'channel'}
A8 = {'type': 'int8', 'symmetric': True, 'strategy': 'tensor'}


def test_library_exports_every_declared_symbol():
    from amct_b200.csrc import build
    build.build()
    names = lib.declared_symbols()
    assert len(names) >= 12
    handle = ctypes.CDLL(lib.LIB_PATH)
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, missing
    assert handle.amct_abi_version() >= 1


def test_cpu_tensors_fail_loudly():
    with pytest.raises(lib.BackendError, match='no CPU fallback'):
        amct.quantize(Net(), cfg(W8))


@pytest.mark.parametrize('bad,msg', [
    ({'batch_num': 0}, 'Batch num only support positive int'),
    ({'batch_num': 1.5}, 'Batch num only support positive int'),
    ({'skip_layers': [1]}, 'Skip layers must be str'),
    ({'algorithm': 'nonexistent'}, 'Not support algorithm nonexistent'),
    ({'algorithm': {'minmax', 'smoothquant'}}, 'Algorithm only support 1 str'),
])
def test_top_level_field_errors(bad, msg):
    c = cfg(W8)
    c.update(bad)
    with pytest.raises(ValueError, match=msg):
        parse_config(Net(), c, AlgorithmRegistry)


@pytest.mark.parametrize('weights,msg', [
    ({'type': 'int2', 'symmetric': True, 'strategy': 'channel'}, 'Weights quant_dtype only support'),
    ({'type': 'int8', 'symmetric': 1.5, 'strategy': 'channel'}, 'Weights symmetric only support bool'),
    ({'type': 'int8', 'symmetric': True, 'strategy': 'row'}, 'Weights strategy only support'),
    ({'type': 'int8', 'symmetric': True, 'strategy': 'channel', 'group_size': 32}, 'group_size only support strategy group'),
    ({'type': 'int8', 'symmetric': True, 'strategy': 'group'}, 'group_size is necessary'),
    ({'type': 'int8', 'symmetric': True, 'strategy': 'group', 'group_size': -32}, 'group_size only support positive int'),
    ({'type': 'int4', 'symmetric': True, 'strategy': 'group', 'group_size': 48}, 'integer multiple of 32'),
    ({'type': 'int4', 'symmetric': True, 'strategy': 'group', 'group_size': 16}, 'integer multiple of 32'),
])
def test_weight_field_errors(weights, msg):
    with pytest.raises(ValueError, match=msg):
        parse_config(Net(), cfg(weights), AlgorithmRegistry)


@pytest.mark.parametrize('inputs,msg', [
    ({'type': 'int4', 'symmetric': True, 'strategy': 'tensor'}, 'Inputs quant_dtype only support'),
    ({'type': 'int8', 'symmetric': None, 'strategy': 'tensor'}, 'Inputs symmetric only support bool'),
    ({'type': 'int8', 'symmetric': True, 'strategy': 'channel'}, 'Inputs strategy only support'),
    ({'type': 'int8', 'symmetric': False, 'strategy': 'token'}, 'do not support asymmetric'),
])
def test_input_field_errors(inputs, msg):
    with pytest.raises(ValueError, match=msg):
        parse_config(Net(), cfg(W8, inputs), AlgorithmRegistry)


def test_combination_rules():
    with pytest.raises(ValueError, match='do not support weight quant strategy group'):
        parse_config(Net(), cfg({'type': 'int8', 'symmetric': True, 'strategy': 'group', 'group_size': 32}, A8),
                     AlgorithmRegistry)
    with pytest.raises(ValueError, match='Do not support combination int8 int4'):
        parse_config(Net(), cfg({'type': 'int4', 'symmetric': True, 'strategy': 'channel'}, A8), AlgorithmRegistry)
    with pytest.raises(ValueError, match='Algorithm smoothquant do not support'):
        parse_config(Net(), cfg(W8, None, {'smoothquant': {'smooth_strength': 0.5}}), AlgorithmRegistry)
    with pytest.raises(ValueError, match='smooth_strength only support float'):
        parse_config(Net(), cfg(W8, A8, {'smoothquant': {'smooth_strength': 1}}), AlgorithmRegistry)
    with pytest.raises(ValueError, match='smooth_strength is necessary'):
        parse_config(Net(), cfg(W8, A8, {'smoothquant': {}}), AlgorithmRegistry)


def test_layer_selection_and_detail_config():
    detail = parse_config(Net(), cfg(W8, skip_layers={'lm_head'}), AlgorithmRegistry)
    assert sorted(detail) == ['linear1', 'linear2']
    assert detail['linear1'] == {'batch_num': 1, 'weights_cfg': {'quant_type': 'int8', 'symmetric': True,
                                 'strategy': 'channel'}, 'inputs_cfg': {'enable_quant': False},
                                 'algorithm': {'minmax'}}
    # int4 needs cin and cout divisible by 8: lm_head (32 -> 1) drops out; group_size must be < cin
    d4 = parse_config(Net(), cfg({'type': 'int4', 'symmetric': False, 'strategy': 'group', 'group_size': 32}),
                      AlgorithmRegistry)
    assert sorted(d4) == ['linear1', 'linear2']
    # W8A8 is refused for fp32 layers unless opted in
    assert parse_config(Net(torch.float32), cfg(W8, A8), AlgorithmRegistry) == {}
    assert len(parse_config(Net(torch.float32), cfg(W8, A8, allow_fp32=True), AlgorithmRegistry)) == 3
    # algorithm spelled as str / set / dict
    for alg in ('minmax', {'minmax'}):
        assert len(parse_config(Net(), cfg(W8, algorithm=alg), AlgorithmRegistry)) == 3


def test_default_config_is_int8_minmax():
    from amct_b200.config import set_default_config
    assert set_default_config() is amct.INT8_MINMAX_WEIGHT_QUANT_CFG
    assert amct.INT8_SMOOTHQUANT_CFG['algorithm'] == {'smoothquant': {'smooth_strength': 0.5}}
    assert amct.INT4_AWQ_WEIGHT_QUANT_CFG['algorithm'] == {'awq': {'grids_num': 20}}


def test_public_api_type_checks():
    with pytest.raises(TypeError, match='argument model must be'):
        amct.quantize('not a model')
    with pytest.raises(TypeError, match='argument config must be'):
        amct.quantize(Net(), config=[1])
    with pytest.raises(TypeError, match='argument model must be'):
        amct.convert(3)
    with pytest.raises(TypeError, match='argument quant_op must be'):
        amct.algorithm_register('x', 'Linear', nn.Linear, None)


def test_registry_custom_algorithm_and_duplicates():
    class MyQuant(BaseQuantizeModule):
        def __init__(self, ori_module, layer_name, quant_config):
            super().__init__(ori_module, layer_name, quant_config)
            self.ori_module = ori_module
            self.seen_config = quant_config

        def forward(self, x):
            return self.ori_module(x)

    name = 'custom_host_test'
    amct.algorithm_register(name, 'Linear', MyQuant, None)
    with pytest.raises(ValueError, match=f'{name} is already registered'):
        amct.algorithm_register(name, 'Linear', MyQuant, None)
    net = Net()
    amct.quantize(net, cfg(W8, algorithm={name: {'k': 1}}))
    assert type(net.linear1).__name__ == 'MyQuant' and net.linear1.seen_config['algorithm'] == {name: {'k': 1}}
    with pytest.raises(RuntimeError, match='The deploy_op for MyQuant is None'):
        amct.convert(net)


def test_logger_tolerates_readonly_cwd(tmp_path, monkeypatch):
    from amct_b200.utils.log import _Logger
    ro = tmp_path / 'ro'
    ro.mkdir()
    os.chmod(ro, 0o500)
    monkeypatch.chdir(ro)
    _Logger().logi('x' * 1200, 'test')


def test_dynamic_inputs_key_is_passed_through():
    dyn = {'type': 'int8', 'symmetric': True, 'strategy': 'token', 'dynamic': True}
    detail = parse_config(Net(), cfg(W8, dyn), AlgorithmRegistry)
    assert detail['linear1']['inputs_cfg'] == {'quant_type': 'int8', 'symmetric': True, 'strategy': 'token', 'dynamic': True}
    with pytest.raises(ValueError, match='dynamic quantization only support strategy token'):
        parse_config(Net(), cfg(W8, {'type': 'int8', 'symmetric': True, 'strategy': 'tensor', 'dynamic': True}), AlgorithmRegistry)


def test_quant_util_names_layout_and_errors():
    """amct_b200.utils.quant_util carries the names of amct_pytorch/utils/quant_util.py; layout helpers and argument
    errors work without a device, the arithmetic refuses CPU tensors."""
    from amct_b200.backend.lib import BackendError
    from amct_b200.utils import quant_util as U
    for name in ('pad_zero_by_group', 'convert_to_per_group_shape', 'convert_dtype', 'quant_weight', 'apply_smooth_weight',
                 'check_scale_offset_shape', 'apply_awq_quantize_weight', 'quant_dequant_weight'):
        assert callable(getattr(U, name))
    w = torch.arange(10, dtype=torch.float32).reshape(2, 5)
    assert U.pad_zero_by_group(w, 4).shape == (2, 8) and float(U.pad_zero_by_group(w, 4)[0, 5:].abs().sum()) == 0
    assert U.convert_to_per_group_shape(w, 4).shape == (2, 2, 4)
    assert torch.equal(U.apply_smooth_weight(torch.full((1, 5), 2.0), w), w * 2)
    assert torch.equal(U.apply_awq_quantize_weight(w, torch.full((1, 5), 2.0), 4), w / 2)
    with pytest.raises(RuntimeError, match='smooth_factor shape should be'):
        U.apply_smooth_weight(torch.ones(5), w)
    with pytest.raises(RuntimeError, match='AWQ params scale.shape should be'):
        U.apply_awq_quantize_weight(w, torch.ones(5), 4)
    with pytest.raises(ValueError, match='Not supported quant_dtype'):
        U.convert_dtype(w, 'int2')
    with pytest.raises(RuntimeError, match='scale.shape should be equal to 1 or cout'):
        U.check_scale_offset_shape(w, torch.ones(3, 1))
    with pytest.raises(BackendError):
        U.quant_weight(w, 'int8', torch.ones(2, 1))


def test_scale_rule_helpers_by_the_reference_names():
    from amct_b200.quantize_op import utils as U
    assert U.get_int_quant_scope('int8', True) == 127 and U.get_int_quant_scope('int8', True, True) == 128
    assert U.get_int_quant_scope('int4', False) == 15
    scale, offset = U.process_scale(torch.tensor([1e-9, 0.5]), torch.tensor([3.0, 4.0]), False, 8)
    assert scale.tolist() == [1.0, 0.5] and offset.tolist() == [-128.0, 4.0]
    scale, offset = U.process_scale(torch.tensor([1e-9, 0.5]), None, True)
    assert scale.tolist() == [1.0, 0.5] and offset is None
    with pytest.raises(RuntimeError, match='Param scale has invalid value inf, nan or zeros!'):
        U.check_scale_offset(torch.tensor([float('inf')]), None)
    with pytest.raises(RuntimeError, match='Param offset has invalid value inf or nan!'):
        U.check_scale_offset(torch.tensor([1.0]), torch.tensor([float('nan')]))
    assert U.convert_to_dst_shape(torch.zeros(2, 3, 4), (2, 10)).shape == (2, 10)
    from amct_b200.algorithm import awq
    for name in ('search_scale', 'process_weights_for_layers', 'calculate_scale_offset_by_granularity', 'apply_scale'):
        assert callable(getattr(awq, name))
    from amct_b200.utils.data_utils import convert_precision
    with pytest.raises(RuntimeError, match='only support float32/float16/bfloat16'):
        convert_precision(torch.zeros(2, 2, dtype=torch.float64), 'int8')


def test_int4_buffer_forms_and_conversions():
    """The INT4 ``quantized_weight`` contract: int32 [K, N / 8] as the device op packs the reference's [K, N] codes,
    the kernels' K-major payload beside it, and every form a checkpoint may hold converted back to the same codes."""
    from amct_b200.utils import int4pack
    from oracle import npu_ops
    g = torch.Generator().manual_seed(5)
    q = torch.randint(-8, 8, (12, 24), generator=g, dtype=torch.int32)                 # [K, N]
    packed = int4pack.to_int4pack(q)
    assert packed.dtype == torch.int32 and packed.shape == (12, 3)
    assert torch.equal(packed, npu_ops.npu_convert_weight_to_int4pack(q))               # the oracle's statement of the op
    word = sum((int(q[5, 8 + i]) & 0xF) << (4 * i) for i in range(8))
    assert (int(packed[5, 1]) & 0xFFFFFFFF) == word
    assert torch.equal(int4pack.from_int4pack(packed).to(torch.int32), q)
    payload = int4pack.to_payload(q.t().contiguous())                                   # [N, K / 2]
    assert torch.equal(payload, npu_ops.pack_int4_along_k(q).t().contiguous())
    assert torch.equal(int4pack.from_payload(payload).to(torch.int32), q.t())
    for stored in (packed, q, q.to(torch.int8), payload.t()):
        assert torch.equal(int4pack.codes_from_buffer(stored, 24).to(torch.int32), q)
    with pytest.raises(ValueError):
        int4pack.to_int4pack(q[:, :20])
    with pytest.raises(RuntimeError):
        int4pack.codes_from_buffer(packed, 16)


def test_int4_deploy_module_loads_every_checkpoint_form():
    """A deployed INT4 Linear takes a state dict written by this package (int32 [K, N / 8]), by the reference under
    its test double (int32 [K, N]) or by an earlier version of this package (uint8 [K / 2, N]); it stores the int4pack
    form and rebuilds the kernels' payload, which is not part of the state dict."""
    from amct_b200.deploy_op.weight_npu_quant_module import NpuWeightQuantizedLinear
    from amct_b200.utils import int4pack
    g = torch.Generator().manual_seed(6)
    k, n, group = 64, 16, 32
    q = torch.randint(-8, 8, (k, n), generator=g, dtype=torch.int32)
    m = NpuWeightQuantizedLinear.__new__(NpuWeightQuantizedLinear)
    torch.nn.Module.__init__(m)
    m.wts_bits, m.group_size, m.scale_factor, m.bias, m.offset_w = 4, group, None, None, None
    m.register_buffer('quantized_weight', torch.zeros(k, n // 8, dtype=torch.int32))
    m.register_buffer('weight_payload', torch.zeros(n, k // 2, dtype=torch.uint8), persistent=False)
    m.register_buffer('scale_w', torch.ones(k // group, n, dtype=torch.bfloat16))
    assert sorted(m.state_dict()) == ['quantized_weight', 'scale_w']
    for stored in (int4pack.to_int4pack(q), q, int4pack.to_payload(q.t().contiguous()).t()):
        m.load_state_dict({'quantized_weight': stored, 'scale_w': m.scale_w})
        assert m.quantized_weight.dtype == torch.int32 and torch.equal(m.quantized_weight, int4pack.to_int4pack(q))
        assert torch.equal(m.weight_payload, int4pack.to_payload(q.t().contiguous()))
