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


@pytest.mark.parametrize("T,k,D", [(64, 4, 2880), (5, 1, 64), (300, 2, 1024)])
def test_fused_combine_matches_gather_multiply_sum(T, k, D):
    """`altob200_combine_rows` / `altob200_spread_rows` against the tensor-op form of the end of the MoE
    token path: gather the routed rows, multiply by the scores in bf16, sum over k; forward within one
    bf16 unit of the fp32-accumulated sum's rounding (the order of a k-term fp32 sum is the only
    freedom), row gradients bit for bit, score gradients against their fp32 value."""
    from alto_b200 import distributed as Dd
    d = torch.device("cuda")
    g = torch.Generator(device=d).manual_seed(T * 7 + k)
    rows = torch.randn(T * k, D, generator=g, device=d).bfloat16()
    order = torch.randperm(T * k, generator=g, device=d)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(T * k, device=d)
    inv32, ord32 = inv.to(torch.int32), order.to(torch.int32)
    scores = torch.rand(T, k, generator=g, device=d).bfloat16()
    go = torch.randn(T, D, generator=g, device=d).bfloat16()
    ra, rb = rows.clone().requires_grad_(True), rows.clone().requires_grad_(True)
    sa, sb = scores.clone().requires_grad_(True), scores.clone().requires_grad_(True)
    ya = Dd._CombineRows.apply(ra, inv32, ord32, sa, T, k)
    routed = Dd._GatherRows.apply(rb, inv32, ord32).view(T, k, D)
    yb = (routed * sb.unsqueeze(-1)).sum(1)
    assert torch.all((ya.float() - yb.float()).abs() <= yb.float().abs() * 2.0 ** -7 + 1e-30)
    assert (ya != yb).float().mean().item() < 0.02
    ya.backward(go)
    yb.backward(go)
    assert torch.equal(ra.grad, rb.grad)
    # score gradients: dot products over D; the tensor-op form rounds every product to bf16 first, the fused
    # backward accumulates fp32 products, so both are held to the fp32 value in norm
    ref = (rows[inv].view(T, k, D).float() * go.float().unsqueeze(1)).sum(-1)
    for got in (sa.grad, sb.grad):
        assert ((got.float() - ref).norm() / ref.norm()).item() < 1e-2
    # without scores: a plain gather-and-sum
    yc = Dd._CombineRows.apply(rows, inv32, ord32, None, T, k)
    yd = rows[inv].view(T, k, D).sum(1)
    assert torch.all((yc.float() - yd.float()).abs() <= yd.float().abs() * 2.0 ** -7 + 1e-30)
