"""Weight de-oscillation hook (reference: alto/components/optimizer.py:43-413).

CPU: configuration, eligibility, hook registration and the modifier's wiring (no kernel runs).
GPU: a short training loop with the hook against a restatement of the reference's per-step tensor
expressions built on the same quantizer ops, bit for bit, including a period end with resets."""
import pytest
import torch
from torch import nn

from alto_b200.deosc import (DeOscillationConfig, _DeOscillationHook, _infer_reduction_axis, _peel_to_fp4_wrapper,
                             enable_de_oscillation)
from alto_b200.dispatch import (MXFP8TrainingWeightWrapperTensor, NVFP4TrainingWeightWrapperTensor, TrainingOpConfig,
                                swap_params)
from alto_b200.lpt import LowPrecisionTrainingModifier


def _cfg(precision="nvfp4", **kw):
    base = dict(precision=precision, use_2dblock_x=False, use_2dblock_w=True, use_hadamard=False, use_sr_grad=False,
                use_dge=False)
    base.update(kw)
    return TrainingOpConfig(**base)


def test_config_eligibility_and_registration():
    with pytest.raises(TypeError):
        DeOscillationConfig(True)  # keyword only
    c = DeOscillationConfig(enable=True, period=3, ratio_threshold=4.0)
    assert (c.period, c.ratio_threshold, c.log_freq) == (3, 4.0, 0)
    assert _infer_reduction_axis(torch.zeros(4, 4)) == -1 and _infer_reduction_axis(torch.zeros(2, 4, 4)) == -2
    with pytest.raises(ValueError):
        _infer_reduction_axis(torch.zeros(4))
    p4 = nn.Parameter(NVFP4TrainingWeightWrapperTensor(torch.randn(16, 16), _cfg()))
    p8 = nn.Parameter(MXFP8TrainingWeightWrapperTensor(torch.randn(32, 32), _cfg("mxfp8_e4m3")))
    plain = nn.Parameter(torch.randn(4, 4))
    assert _peel_to_fp4_wrapper(p4) is not None and _peel_to_fp4_wrapper(p8) is None
    hook = _DeOscillationHook(c)
    assert hook._wrapper_if_eligible(p4) is not None
    assert hook._wrapper_if_eligible(p8) is None and hook._wrapper_if_eligible(plain) is None
    frozen = nn.Parameter(NVFP4TrainingWeightWrapperTensor(torch.randn(16, 16), _cfg()), requires_grad=False)
    assert hook._wrapper_if_eligible(frozen) is None
    opt = torch.optim.SGD([plain], lr=0.1)
    enable_de_oscillation(opt, DeOscillationConfig(enable=False))
    assert len(opt._optimizer_step_post_hooks) == 0
    enable_de_oscillation([opt], c)
    enable_de_oscillation(opt, c)  # once per optimizer
    assert len(opt._optimizer_step_post_hooks) == 1
    plain.grad = torch.ones_like(plain)
    opt.step()  # no eligible parameter: the hook is a no-op


def test_modifier_installs_the_hook_from_deosc_step_on():
    class Trainer:
        def __init__(self, opt):
            self.step, self.optimizers = 0, [opt]

    lin = nn.Linear(16, 16)
    opt = torch.optim.SGD(lin.parameters(), lr=0.1)
    mod = LowPrecisionTrainingModifier(scheme="nvfp4", deosc_step=2, deosc_period=5, deosc_ratio=8.0)
    mod.initialize([lin])
    with pytest.raises(ValueError, match="Trainer"):
        mod.pre_step([lin])
    tr = Trainer(opt)
    tr.step = 1
    mod.pre_step([lin], trainer=tr)
    assert len(opt._optimizer_step_post_hooks) == 0
    tr.step = 2
    mod.pre_step([lin], trainer=tr)
    mod.pre_step([lin], trainer=tr)
    (hook,) = opt._optimizer_step_post_hooks.values()
    assert hook._cfg.period == 5 and hook._cfg.ratio_threshold == 8.0


@pytest.mark.gpu
@pytest.mark.parametrize("precision,kw,dtype", [("nvfp4", dict(two_level_scaling="tensorwise"), torch.float32),
                                                ("mxfp4", dict(use_uos=True), torch.bfloat16),
                                                ("nvfp4", dict(use_2dblock_w=False), torch.float32)])
def test_hook_matches_the_reference_expressions(precision, kw, dtype):
    from alto_b200 import mxfp4, nvfp4
    d = torch.device("cuda")
    cfg = _cfg(precision, **kw)
    torch.manual_seed(0)
    lin = nn.Linear(64, 48, bias=False).to(d).to(dtype)      # 48 rows: exercises the padding to a whole block
    swap_params(lin, config=cfg, module_name="lin")
    opt = torch.optim.SGD(lin.parameters(), lr=0.05)
    period = 4
    captured = {}
    # hooks run in registration order: this one sees the weight as the optimizer left it
    opt.register_step_post_hook(lambda o, a, k: captured.__setitem__("w", lin.weight.data._data.clone()))
    enable_de_oscillation(opt, DeOscillationConfig(enable=True, period=period, ratio_threshold=1.5))

    def qdq(w):
        blk = 16 if precision == "nvfp4" else 32
        rows = w.shape[0]
        wp = torch.nn.functional.pad(w, (0, 0, 0, (-rows) % blk))
        if precision == "nvfp4":
            outer = torch.empty(1, device=d) if cfg.two_level_scaling == "tensorwise" else None
            q, s = nvfp4.convert_to_nvfp4(wp, is_2d_block=cfg.use_2dblock_w, outer_scale=outer,
                                          update_outer_scale=outer is not None)
            out = nvfp4.convert_from_nvfp4(q, s, output_dtype=w.dtype, is_2d_block=cfg.use_2dblock_w, outer_scale=outer)
        else:
            q, s = mxfp4.convert_to_mxfp4(wp, is_2d_block=cfg.use_2dblock_w, use_uos=cfg.use_uos)
            out = mxfp4.convert_from_mxfp4(q, s, output_dtype=w.dtype, is_2d_block=cfg.use_2dblock_w)
        return out[:rows]

    prev = dist_w = dist_q = None
    step_in_period, resets = 0, []
    g = torch.Generator(device=d).manual_seed(1)
    for it in range(2 * period + 2):
        # gradients that push weights back and forth across bin boundaries
        lin.weight.grad = (torch.randn(48, 64, device=d, generator=g) * (1.0 if it % 2 else -1.0)).to(dtype)
        opt.step()
        raw = lin.weight.data._data
        w_now = captured["w"]
        state = opt.state[lin.weight]
        # ---- the reference's per-step expressions (alto/components/optimizer.py:363-410) ----
        if prev is None:
            prev, dist_w, dist_q = w_now.clone(), torch.zeros_like(w_now), torch.zeros_like(w_now)
        else:
            w_q, p_q = qdq(w_now), qdq(prev)
            dist_w.add_((w_now - prev).abs())
            dist_q.add_((w_q - p_q).abs())
            prev.copy_(w_now)
            step_in_period += 1
            if step_in_period >= period:
                ratio = dist_q / dist_w.clamp(min=1e-30)
                mask = (dist_w > 0) & (ratio >= 1.5)
                resets.append(int(mask.sum()))
                expect = w_now.clone()
                expect[mask] = w_q[mask]
                if mask.any():
                    prev.copy_(expect)
                dist_w.zero_()
                dist_q.zero_()
                step_in_period = 0
                assert torch.equal(raw, expect)
        assert torch.equal(state["osci_prev_weight"], prev)
        assert torch.equal(state["osci_dist_w"], dist_w) and torch.equal(state["osci_dist_w_qdq"], dist_q)
        assert state["osci_step_in_period"] == step_in_period
    assert len(resets) == 2 and sum(resets) > 0
