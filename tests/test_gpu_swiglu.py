"""Fused SwiGLU kernels against the tensor-op form silu(h[:, :H]) * h[:, H:] and its autograd on the
same device: the kernels keep that form's bf16 roundings, so values are compared bit for bit (a
mismatch of one bf16 unit would come from a different exp; none is tolerated in the forward, and the
gate gradient is held to one unit in the last place)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,H", [(1, 8), (300, 2880), (4096, 5760), (129, 64)])
def test_swiglu_matches_tensor_ops(rows, H):
    from alto_b200.swiglu import swiglu
    d = torch.device("cuda")
    g = torch.Generator(device=d).manual_seed(rows + H)
    h = (torch.randn(rows, 2 * H, generator=g, device=d) * 3).bfloat16()
    h[0, :4] = torch.tensor([0.0, -0.0, 40.0, -40.0], dtype=torch.bfloat16, device=d)
    go = torch.randn(rows, H, generator=g, device=d).bfloat16()
    a = h.clone().requires_grad_(True)
    b = h.clone().requires_grad_(True)
    ya = swiglu(a)
    yb = torch.nn.functional.silu(b[:, :H]) * b[:, H:]
    assert torch.equal(ya, yb)
    ya.backward(go)
    yb.backward(go)
    # up half: one multiply of two bf16 values, identical; gate half: same expression, at most one unit
    assert torch.equal(a.grad[:, H:], b.grad[:, H:])
    ga, gb = a.grad[:, :H].float(), b.grad[:, :H].float()
    assert torch.all((ga - gb).abs() <= gb.abs() * 2.0 ** -7 + 1e-38)
    assert (ga != gb).float().mean().item() < 0.01


def test_swiglu_rejects_what_it_cannot_take():
    from alto_b200.swiglu import swiglu
    d = torch.device("cuda")
    with pytest.raises(ValueError):
        swiglu(torch.zeros(4, 24, dtype=torch.bfloat16, device=d))
    with pytest.raises(TypeError):
        swiglu(torch.zeros(4, 32, dtype=torch.float32, device=d))
    with pytest.raises(RuntimeError):
        swiglu(torch.zeros(4, 32, dtype=torch.bfloat16))
