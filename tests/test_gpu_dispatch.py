"""GPU tests of the scheme surface end to end: a model converted by the modifier runs its linears
and grouped experts through the CUDA path, gradients reach the wrapped parameters, and a toy
training run behaves (reference: tests/unittest/nvfp4/test_nvfp_dispatch_guards.py:243-297,
tests/unittest/mxfp8/test_e2e_moe.py:56-83)."""
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


@pytest.mark.parametrize("scheme,kw", [("nvfp4", dict(two_level_scaling="tensorwise", use_hadamard=True)),
                                       ("mxfp4", dict(use_hadamard=True)), ("mxfp8_e4m3", {})])
def test_converted_linear_matches_boundary_function(scheme, kw):
    from alto_b200 import mxfp4, mxfp8, nvfp4
    from alto_b200.dispatch import TrainingWeightWrapperBaseTensor
    from alto_b200.hadamard import HadamardFactory
    from alto_b200.lpt import LowPrecisionTrainingModifier
    d = _dev()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 128, bias=True)).to(d).bfloat16()
    ref_w = model[0].weight.detach().clone()
    ref_b = model[0].bias.detach().clone()
    LowPrecisionTrainingModifier(scheme=scheme, targets="Linear", **kw).convert(model)
    assert isinstance(model[0].weight.data, TrainingWeightWrapperBaseTensor)
    x = torch.randn(4, 32, 256, device=d, dtype=torch.bfloat16, requires_grad=True)
    HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=7)
    y = model(x)
    y.float().pow(2).sum().backward()
    assert y.shape == (4, 32, 128) and y.dtype == torch.bfloat16
    assert model[0].weight.grad is not None and model[0].weight.grad.shape == (128, 256)
    assert x.grad is not None and torch.isfinite(x.grad).all()
    # same transform draws -> identical forward through the boundary function called directly
    HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=7)
    if scheme == "nvfp4":
        y2 = nvfp4._to_nvfp4_then_scaled_mm(x.detach(), ref_w, False, True, False, use_outer_scale=True,
                                            use_hadamard=True)
    elif scheme == "mxfp4":
        y2 = mxfp4._to_mxfp4_then_scaled_mm(x.detach(), ref_w, False, True, False, False, "none", True)
    else:
        y2 = mxfp8._to_mxfp8_then_scaled_mm(x.detach(), ref_w, "e4m3", False, False, True)
    assert torch.equal(y, y2 + ref_b)


def test_registered_torch_ops_run_the_cuda_path():
    from alto_b200 import mxfp4, nvfp4, torch_ops
    torch_ops.register()
    d = _dev()
    x = torch.randn(64, 128, device=d).bfloat16()
    q, s = torch.ops.alto_b200.convert_to_mxfp4(x, axis=0)
    q2, s2 = mxfp4.convert_to_mxfp4(x, axis=0)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    dq = torch.ops.alto_b200.convert_from_mxfp4(q, s, torch.bfloat16, axis=0)
    assert torch.equal(dq, mxfp4.convert_from_mxfp4(q2, s2, torch.bfloat16, axis=0))
    outer = torch.zeros(1, device=d)
    qn, sn = torch.ops.alto_b200.convert_to_nvfp4(x, outer_scale=outer)
    assert outer.item() > 0                      # refreshed in place, as the reference op does
    assert torch.equal(qn, nvfp4.convert_to_nvfp4(x, outer_scale=outer, update_outer_scale=False)[0])


class _Experts(nn.Module):
    """Minimal stand-in for TorchTitan's GroupedExperts: w1 [E, hidden, dim] used as x @ w1^T."""

    def __init__(self, n_exp, dim, hidden):
        super().__init__()
        self.w1 = nn.Parameter(torch.randn(n_exp, hidden, dim) * 0.05)
        self.w2 = nn.Parameter(torch.randn(n_exp, dim, hidden) * 0.05)

    def forward(self, x, offs):
        h = torch._grouped_mm(x, self.w1.transpose(-2, -1), offs=offs)
        h = torch.nn.functional.silu(h)
        return torch._grouped_mm(h, self.w2.transpose(-2, -1), offs=offs)


class ToyGroupedExperts(_Experts):
    pass


def test_toy_moe_trains_under_mxfp8():
    from alto_b200.lpt import LowPrecisionTrainingModifier
    d = _dev()
    torch.manual_seed(0)
    n_exp, dim, hidden, tokens = 4, 128, 256, 512
    teacher = ToyGroupedExperts(n_exp, dim, hidden).to(d)  # fp32 master weights, as in mixed-precision training
    student = ToyGroupedExperts(n_exp, dim, hidden).to(d)
    LowPrecisionTrainingModifier(scheme="mxfp8_e4m3", targets=["ToyGroupedExperts"], ignore=[]).convert(student)
    offs = torch.tensor([128, 256, 384, 512], dtype=torch.int32, device=d)
    opt = torch.optim.Adam(student.parameters(), lr=3e-3)
    losses = []
    for step in range(60):
        x = torch.randn(tokens, dim, device=d)
        with torch.no_grad():
            target = teacher(x, offs)
        out = student(x, offs)
        loss = (out.float() - target.float()).pow(2).mean()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert all(torch.isfinite(torch.tensor(losses)))
    assert sum(losses[-5:]) < 0.7 * sum(losses[:5]), losses
