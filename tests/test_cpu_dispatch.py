"""CPU tests of the scheme surface: config, wrapper-tensor routing (boundary functions replaced
by recorders, as in the reference's tests/unittest/nvfp4/test_nvfp_dispatch_guards.py:69-241),
``swap_params`` and ``LowPrecisionTrainingModifier``.  No kernel is launched."""
import pickle

import pytest
import torch
from torch import nn

import alto_b200.dispatch as D
from alto_b200.dispatch import (MXFP4TrainingWeightWrapperTensor, MXFP8TrainingWeightWrapperTensor,
                                NVFP4TrainingWeightWrapperTensor, TrainingOpConfig, swap_params)
from alto_b200.lpt import LowPrecisionTrainingModifier


def _cfg(**kw):
    base = dict(precision="nvfp4", use_2dblock_x=False, use_2dblock_w=False, use_hadamard=False, use_sr_grad=False,
                use_dge=False)
    base.update(kw)
    return TrainingOpConfig(**base)


def test_config_is_hashable_keyword_only_and_picklable():
    a, b = _cfg(), _cfg()
    assert a == b and hash(a) == hash(b) and {a: 1}[b] == 1
    with pytest.raises(TypeError):
        TrainingOpConfig("nvfp4", False, False, False, False, False)
    assert a.clip_mode == "none" and a.two_level_scaling == "none" and a.use_uos is False
    assert pickle.loads(pickle.dumps(a)) == a
    with pytest.raises(AttributeError):
        a.not_a_field = 1  # slots


class _Recorder:
    def __init__(self, out_features_from="b"):
        self.calls = []

    def __call__(self, a, b, *args, **kwargs):
        self.calls.append((a, b, args, kwargs))
        return torch.zeros(*a.shape[:-1], b.shape[0])


@pytest.mark.parametrize("two_level,expect_outer", [("none", False), ("tensorwise", True)])
def test_nvfp4_linear_routing_passes_flags(monkeypatch, two_level, expect_outer):
    rec = _Recorder()
    monkeypatch.setattr(D, "_to_nvfp4_then_scaled_mm", rec)
    cfg = _cfg(use_2dblock_w=True, use_hadamard=True, use_sr_grad=True, two_level_scaling=two_level)
    w = NVFP4TrainingWeightWrapperTensor(torch.randn(8, 16), cfg)
    x = torch.randn(4, 16)
    bias = torch.ones(8)
    y = torch.nn.functional.linear(x, w, bias)
    assert len(rec.calls) == 1
    a, b, _, kw = rec.calls[0]
    assert a is x and isinstance(b, NVFP4TrainingWeightWrapperTensor) and b.shape == (8, 16)
    assert kw == dict(use_2dblock_x=False, use_2dblock_w=True, use_sr_grad=True, use_outer_scale=expect_outer,
                      use_hadamard=True, use_dge=False)
    assert torch.equal(y, torch.ones(4, 8))  # bias is added after the boundary function
    # matmul passes the weight as [K, N]; the boundary function always receives [N, K]
    rec.calls.clear()
    torch.matmul(x, w.t())
    torch.ops.aten.mm.default(x, w.t())
    assert [c[1].shape for c in rec.calls] == [(8, 16), (8, 16)]
    # like the reference, the Python-level torch.mm ("mm", not "mm.default") is not intercepted and
    # ends in __torch_dispatch__, which refuses GEMMs (alto/kernels/dispatch/tensor.py:50,120-123)
    with pytest.raises(ValueError, match="__torch_dispatch__"):
        torch.mm(x, w.t())


def test_mxfp4_and_mxfp8_routing(monkeypatch):
    rec4, rec8 = _Recorder(), _Recorder()
    monkeypatch.setattr(D, "_to_mxfp4_then_scaled_mm", rec4)
    monkeypatch.setattr(D, "_to_mxfp8_then_scaled_mm", rec8)
    x = torch.randn(4, 32)
    w4 = MXFP4TrainingWeightWrapperTensor(torch.randn(8, 32),
                                          _cfg(precision="mxfp4", two_level_scaling="blockwise", clip_mode="static"))
    torch.nn.functional.linear(x, w4)
    kw = rec4.calls[0][3]
    assert kw["use_macro_block_scaling"] is True and kw["clip_mode"] == "static" and kw["use_uos"] is False
    w8 = MXFP8TrainingWeightWrapperTensor(torch.randn(8, 32), _cfg(precision="mxfp8_e5m2", use_2dblock_w=True))
    torch.nn.functional.linear(x, w8)
    assert rec8.calls[0][3] == dict(fp8_variant="e5m2", use_sr_grad=False, use_2dblock_x=False, use_2dblock_w=True)
    with pytest.raises(AssertionError):
        torch.nn.functional.linear(x, MXFP8TrainingWeightWrapperTensor(torch.randn(8, 32),
                                                                       _cfg(precision="mxfp8_e4m3", use_hadamard=True)))
    with pytest.raises(AssertionError):  # config of another family on the wrong wrapper
        torch.nn.functional.linear(x, MXFP4TrainingWeightWrapperTensor(torch.randn(8, 32), _cfg(precision="nvfp4")))
    with pytest.raises(NotImplementedError):
        torch.nn.functional.linear(x, NVFP4TrainingWeightWrapperTensor(torch.randn(8, 32), _cfg(precision="amdfp4")))


def test_grouped_mm_routing(monkeypatch):
    calls = []

    def rec(A, B, **kw):
        calls.append((A, B, kw))
        return torch.zeros(A.shape[0], B.shape[-1])

    monkeypatch.setattr(D, "_quantize_then_nvfp4_scaled_grouped_mm", rec)
    cfg = _cfg(two_level_scaling="tensorwise", use_2dblock_w=True)
    W = NVFP4TrainingWeightWrapperTensor(torch.randn(2, 16, 32), cfg)  # [E, N, K] storage
    A = torch.randn(256, 32)
    offs = torch.tensor([128, 256], dtype=torch.int32)
    try:
        out = torch._grouped_mm(A, W.transpose(-2, -1), offs=offs)
    except (RuntimeError, NotImplementedError) as e:  # builds of torch without a CPU _grouped_mm schema
        pytest.skip(f"torch._grouped_mm not callable here: {e}")
    assert out.shape == (256, 16)
    A_, B_, kw = calls[0]
    assert B_.shape == (2, 32, 16) and kw["offs"] is offs and kw["use_outer_scale"] is True


def test_wrapper_tensor_housekeeping():
    cfg = _cfg()
    w = NVFP4TrainingWeightWrapperTensor(torch.randn(8, 16), cfg)
    assert isinstance(w.detach(), NVFP4TrainingWeightWrapperTensor) and w.detach().config == cfg
    assert isinstance(w.t(), NVFP4TrainingWeightWrapperTensor)
    assert isinstance(w.clone(), NVFP4TrainingWeightWrapperTensor)
    assert isinstance(w.to(torch.bfloat16), NVFP4TrainingWeightWrapperTensor)
    s = w + 1.0  # ordinary ops return plain tensors
    assert type(s) is torch.Tensor
    inner, meta = w.__tensor_flatten__()
    assert inner == ["_data"] and meta == {"config": cfg}
    r = NVFP4TrainingWeightWrapperTensor.__tensor_unflatten__({"_data": w._data}, meta, None, None)
    assert torch.equal(r._data, w._data)
    with pytest.raises(ValueError, match="__torch_dispatch__"):
        NVFP4TrainingWeightWrapperTensor.__torch_dispatch__(torch.ops.aten.mm.default, (), (torch.randn(2, 16), w.t()))
    # gradients reach the wrapped leaf (reference: test_nvfp_dispatch_guards.py:243-297)
    p = nn.Parameter(NVFP4TrainingWeightWrapperTensor(torch.randn(4, 4), cfg))
    (p * 2.0).sum().backward()
    assert p.grad is not None and p.grad.shape == (4, 4)


class _GroupedExperts(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1 = nn.Parameter(torch.randn(2, 8, 16))
        self.w2 = nn.Parameter(torch.randn(2, 16, 8))


class _Model(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc = nn.Linear(16, 8, bias=True)
        self.experts = _GroupedExperts()
        self.output = nn.Linear(8, 4)


def test_swap_params_wraps_weights_not_biases():
    m = _Model()
    cfg = _cfg(precision="mxfp4")
    swap_params(m.fc, config=cfg, module_name="fc")
    assert isinstance(m.fc.weight.data, MXFP4TrainingWeightWrapperTensor)
    assert not isinstance(m.fc.bias.data, D.TrainingWeightWrapperBaseTensor)
    assert "mxfp4" in m.fc._get_name()
    swap_params(m.fc, config=cfg)  # idempotent
    swap_params(m.experts, config=cfg, target_parameter_name="w1")
    assert isinstance(m.experts.w1.data, MXFP4TrainingWeightWrapperTensor)
    assert not isinstance(m.experts.w2.data, D.TrainingWeightWrapperBaseTensor)
    with pytest.raises(ValueError):
        swap_params(m.fc, config=None)
    p = swap_params(nn.Parameter(torch.randn(4, 4)), config=_cfg(precision="mxfp8_e4m3"))
    assert isinstance(p.data, MXFP8TrainingWeightWrapperTensor)


def test_modifier_validation_and_conversion():
    with pytest.raises(ValueError):
        LowPrecisionTrainingModifier(scheme="fp3")
    with pytest.raises(ValueError):
        LowPrecisionTrainingModifier(scheme="nvfp4", lora_rank=8)
    with pytest.raises(ValueError):
        LowPrecisionTrainingModifier(scheme="mxfp4", deosc_period=0)
    mod = LowPrecisionTrainingModifier(scheme="nvfp4", targets="Linear", two_level_scaling="tensorwise",
                                       use_hadamard=True, use_sr_grad=True)
    assert mod.targets == ["Linear"] and mod.ignore == ["output"] and mod.use_2dblock_w is True
    (cfg, targets), = mod.resolved_config.items()
    assert cfg == TrainingOpConfig(precision="nvfp4", use_2dblock_x=False, use_2dblock_w=True, use_hadamard=True,
                                   use_sr_grad=True, use_dge=False, two_level_scaling="tensorwise")
    assert targets == ["Linear"]
    m = _Model()
    assert mod.convert(m) is True
    assert isinstance(m.fc.weight.data, NVFP4TrainingWeightWrapperTensor)
    assert not isinstance(m.output.weight.data, D.TrainingWeightWrapperBaseTensor)  # ignored by default
    # dict scheme: different recipes for different targets
    mod2 = LowPrecisionTrainingModifier(scheme={"mxfp4": ["_GroupedExperts"], "mxfp8_e4m3": "Linear"}, ignore=[])
    m2 = _Model()
    mod2.convert(m2)
    assert isinstance(m2.experts.w1.data, MXFP4TrainingWeightWrapperTensor)
    assert isinstance(m2.output.weight.data, MXFP8TrainingWeightWrapperTensor)
    # lifecycle
    with pytest.raises(RuntimeError):
        mod.pre_step([m])
    mod.initialize([m])
    mod.pre_step([m])
    mod.post_step([m])
    mod.finalize([m])
    with pytest.raises(RuntimeError):
        mod.finalize([m])
    assert mod.convert_config(object()) is True and mod.token_alignment == 128
    with pytest.raises(NotImplementedError):
        LowPrecisionTrainingModifier(scheme="amdfp4").convert(_Model())
    with pytest.raises(NotImplementedError):
        LowPrecisionTrainingModifier(scheme="nvfp4", lora_rank=16).convert(_Model())
