"""The benchmark configurations at their full sizes, through properties that do not need a full-size
CPU oracle run:

* sampled exactness -- a random sample of rows of every quantizer output (codes, scales) is compared
  bit for bit with the oracle run on just those rows (row-wise blocks are row-local; column-wise
  blocks are column-local), and a random sample of GEMM outputs with fp32 dot products of the
  dequantised operand rows (relative error <= 1e-3, the stated tolerance);
* idempotence -- quantising a dequantised tensor reproduces the same codes and scales (RTN);
* linearity of the grouped GEMM in the expert assignment -- rows of one expert do not depend on the
  rows of any other.

Shapes: C1 MXFP4 2048^3 (checked against the oracle in full), C2 NVFP4 Llama-3-8B MLP-up with the
recipe of the headline benchmark, C3 MXFP8 8192 x 4096 x 4096, C4 MXFP4 MoE 32 experts x 2880."""
import numpy as np
import pytest
import torch

from oracle import alto_oracle as O

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _gen(shape, seed, scale=1.0):
    g = torch.Generator(device=_dev()).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=_dev(), dtype=torch.float32) * scale).bfloat16()


def _sample(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(n, generator=g)[:k].sort().values


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp(min=1e-30)).item()


def test_c1_mxfp4_quantize_and_gemm_match_oracle_in_full():
    from alto_b200 import mxfp4 as MX
    x, w = _gen((2048, 2048), 0), _gen((2048, 2048), 1)
    xq, xs = MX.convert_to_mxfp4(x)
    wq, ws = MX.convert_to_mxfp4(w)
    xo, xso = O.quantize_mxfp4(x.cpu())
    wo, wso = O.quantize_mxfp4(w.cpu())
    assert torch.equal(xq.cpu().view(torch.uint8), xo) and torch.equal(xs.cpu(), xso)
    assert torch.equal(wq.cpu().view(torch.uint8), wo) and torch.equal(ws.cpu(), wso)
    y = MX.blockwise_mxfp4_gemm(xq, xs, wq, ws, trans_b=True, output_dtype=torch.bfloat16)
    ref = O.dequantize_mxfp4(xo, xso) @ O.dequantize_mxfp4(wo, wso).t()
    assert _rel(y.float().cpu(), ref.bfloat16().float()) <= 1e-3


def test_c2_nvfp4_quantizers_sampled_exactness_and_idempotence():
    from alto_b200 import nvfp4 as NV
    M, K, N = 8192, 4096, 14336
    dy = _gen((M, N), 2, 1e-3)
    outer = NV.compute_dynamic_outer_scale(dy)
    assert outer.item() == O.compute_dynamic_outer_scale(dy.cpu()).item()
    # row-wise (dgrad operand), RTN: sampled rows against the oracle
    q, s = NV.convert_to_nvfp4(dy, outer_scale=outer, update_outer_scale=False)
    rows = _sample(M, 48, 3)
    qo, so = O.quantize_nvfp4(dy[rows.to(_dev())].cpu(), 16, -1, False, outer.cpu())
    assert torch.equal(q[rows.to(_dev())].cpu().view(torch.uint8), qo) and torch.equal(s[rows.to(_dev())].cpu(), so)
    # idempotence of quantise(dequantise(.)) with the same outer scale
    dq = NV.convert_from_nvfp4(q, s, torch.bfloat16, outer_scale=outer)
    q2, s2 = NV.convert_to_nvfp4(dq, outer_scale=outer, update_outer_scale=False)
    assert torch.equal(q2, q) and torch.equal(s2, s)
    # column-wise (wgrad operand) with stochastic rounding from (seed, offset): sampled columns
    cols = _sample(N, 32, 4)
    qc, sc = NV.convert_to_nvfp4(dy, axis=0, outer_scale=outer, update_outer_scale=False, use_sr=True,
                                 philox_seed=11, philox_offset=22)
    # the table repeats every 64 rows of the axis-last view (its rows are the original columns)
    planes = O.reference_sr_planes(11, 22, 64, M)[:, cols % 64]
    qo, so = O.quantize_nvfp4(dy[:, cols.to(_dev())].cpu(), 16, 0, False, outer.cpu(), planes)
    assert torch.equal(qc[:, cols.to(_dev())].cpu().view(torch.uint8), qo)
    assert torch.equal(sc[:, cols.to(_dev())].cpu(), so)


def test_c2_nvfp4_linear_sampled_outputs():
    """Forward, dgrad and wgrad of the headline recipe (without stochastic rounding, so that the operands
    can be rebuilt by the standalone quantizers): sampled outputs against fp32 dot products of the
    dequantised operands."""
    from alto_b200 import nvfp4 as NV
    M, K, N = 8192, 4096, 14336
    NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
    x, w, dy = _gen((M, K), 5), _gen((N, K), 6, 0.02), _gen((M, N), 7, 1e-3)
    xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = NV._to_nvfp4_then_scaled_mm(xd, wd, False, True, False, use_outer_scale=True, use_hadamard=True)
    y.backward(dy)
    NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
    had = NV.HadamardFactory.create_transform(device=_dev())

    def qdq(t, axis, is2d):
        outer = NV.compute_dynamic_outer_scale(t)
        q, s = NV.convert_to_nvfp4(t, axis=axis, is_2d_block=is2d, outer_scale=outer, update_outer_scale=False)
        return NV.convert_from_nvfp4(q, s, torch.float32, axis=axis, is_2d_block=is2d, outer_scale=outer)

    rm, rn, rk = (_sample(M, 40, 8).to(_dev()), _sample(N, 40, 9).to(_dev()), _sample(K, 40, 10).to(_dev()))
    x_dq, w_dq, g_dq = qdq(x, -1, False), qdq(w, -1, True), qdq(dy, -1, False)
    assert _rel(y[rm][:, rn].float(), (x_dq[rm].double() @ w_dq[rn].double().t()).float().bfloat16().float()) <= 1e-3
    assert _rel(xd.grad[rm][:, rk].float(),
                (g_dq[rm].double() @ w_dq[:, rk].double()).float().bfloat16().float()) <= 1e-3
    xh_dq, gh_dq = qdq(had(x, left_mul=True), 0, False), qdq(had(dy, left_mul=True), 0, False)
    assert _rel(wd.grad[rn][:, rk].float(),
                (gh_dq[:, rn].double().t() @ xh_dq[:, rk].double()).float().bfloat16().float()) <= 1e-3


def test_c3_mxfp8_linear_sampled_outputs():
    from alto_b200 import mxfp8 as M8
    M, K, N = 8192, 4096, 4096
    x, w, dy = _gen((M, K), 11), _gen((N, K), 12, 0.02), _gen((M, N), 13, 1e-3)
    xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = M8._to_mxfp8_then_scaled_mm(xd, wd, "e4m3", False, False, True)
    y.backward(dy)

    def qdq(t, axis, is2d):
        q, s = M8.convert_to_mxfp8(t, mxfp_format="e4m3", axis=axis, is_2d_block=is2d)
        return M8.convert_from_mxfp8(q, s, torch.float32, axis=axis, is_2d_block=is2d)

    rm, rn, rk = (_sample(M, 40, 14).to(_dev()), _sample(N, 40, 15).to(_dev()), _sample(K, 40, 16).to(_dev()))
    x_dq, w_dq, g_dq = qdq(x, -1, False), qdq(w, -1, True), qdq(dy, -1, False)
    assert _rel(y[rm][:, rn].float(), (x_dq[rm].double() @ w_dq[rn].double().t()).float().bfloat16().float()) <= 1e-3
    assert _rel(xd.grad[rm][:, rk].float(),
                (g_dq[rm].double() @ w_dq[:, rk].double()).float().bfloat16().float()) <= 1e-3
    x0, g0 = qdq(x, 0, False), qdq(dy, 0, False)
    assert _rel(wd.grad[rn][:, rk].float(), (g0[:, rn].double().t() @ x0[:, rk].double()).float().bfloat16().float()) <= 1e-3
    # sampled rows of the row-wise quantizer against the oracle
    q, s = M8.convert_to_mxfp8(x, mxfp_format="e4m3")
    qo, so = O.quantize_mxfp8(x[rm].cpu(), 32, "e4m3")
    assert torch.equal(q[rm].cpu().view(torch.uint8), qo.view(torch.uint8)) and torch.equal(s[rm].cpu(), so)


def test_c4_mxfp4_grouped_gemm_at_moe_shape():
    """GPT-OSS-20B expert shapes: 32 experts, 16384 tokens x top-4, hidden 2880, gate+up 5760.  Every
    expert's rows equal the dense linear of those rows with that expert's weight (another kernel: the
    CTA-pair GEMM), padding rows are zero, and routed rows do not depend on other experts' rows."""
    from alto_b200 import mxfp4 as MX
    from alto_b200.grouped import _quantize_then_mxfp_scaled_grouped_mm as gmm
    E, D, H, T, k = 32, 2880, 5760, 16384, 4
    d = _dev()
    g = torch.Generator(device=d).manual_seed(0)
    logits = torch.randn(T, E, generator=g, device=d)
    ids = torch.topk(torch.softmax(logits, -1), k, dim=-1).indices.reshape(-1)
    counts = torch.bincount(ids, minlength=E)
    padded = (counts + 127) // 128 * 128
    offs = torch.cumsum(padded, 0).to(torch.int32)
    m_pad = int(offs[-1])
    x = torch.zeros(m_pad, D, dtype=torch.bfloat16, device=d)
    start = torch.cumsum(padded, 0) - padded
    valid = torch.zeros(m_pad, dtype=torch.bool, device=d)
    for e in range(E):
        n = int(counts[e])
        x[int(start[e]):int(start[e]) + n] = _gen((n, D), 100 + e)
        valid[int(start[e]):int(start[e]) + n] = True
    W = _gen((E, H, D), 17, 0.02)
    y = gmm(x, W.transpose(-2, -1), offs, False, True, False, False, False, "none", False)
    assert y.shape == (m_pad, H) and torch.isfinite(y).all()
    assert torch.count_nonzero(y[~valid]) == 0
    for e in (0, 7, 31):
        lo, hi = int(start[e]), int(start[e] + padded[e])
        dense = MX._to_mxfp4_then_scaled_mm(x[lo:hi], W[e], False, True, False, False, "none", False)
        assert _rel(y[lo:hi].float(), dense.float()) <= 1e-3
    # changing another expert's rows leaves this expert's output untouched
    x2 = x.clone()
    x2[int(start[3]):int(start[3]) + 128] = 0
    y2 = gmm(x2, W.transpose(-2, -1), offs, False, True, False, False, False, "none", False)
    lo, hi = int(start[5]), int(start[5] + padded[5])
    assert torch.equal(y2[lo:hi], y[lo:hi])


def test_c4_two_level_recipe_forward_dgrad_wgrad_at_moe_shape():
    """The MoE configuration as the benchmark definition states it: MXFP4, 2-D weight blocks with the 128
    macro-block two-level scale, Hadamard rotation of the token-axis operands, stochastic rounding of the
    gradients, 32 experts x 65 536 routed rows x 2880 -> 5760.  Forward, dgrad and wgrad run on the
    tensor cores (no dense matmul in the path); checked through properties that need no full-size CPU run:
    sampled outputs of the forward against float64 dot products of the de-quantised, de-scaled operands,
    zero padding rows, finite gradients, an expert's gradient rows equal to the dense two-level linear on
    those rows (another code path: dense tiles, no expert table), and empty gradient for nothing."""
    from alto_b200 import _lib as L
    from alto_b200 import mxfp4 as MX
    from alto_b200.grouped import _quantize_then_mxfp_scaled_grouped_mm as gmm
    from alto_b200.hadamard import HadamardFactory
    from alto_b200.macro_block_scaling import macro_block_descaling, macro_block_scaling
    E, D, H, T, k = 32, 2880, 5760, 16384, 4
    d = _dev()
    g = torch.Generator(device=d).manual_seed(0)
    ids = torch.topk(torch.softmax(torch.randn(T, E, generator=g, device=d), -1), k, dim=-1).indices.reshape(-1)
    counts = torch.bincount(ids, minlength=E)
    padded = (counts + 127) // 128 * 128
    offs = torch.cumsum(padded, 0).to(torch.int32)
    start = torch.cumsum(padded, 0) - padded
    m_pad = int(offs[-1])
    x = _gen((m_pad, D), 21)
    valid = torch.zeros(m_pad, dtype=torch.bool, device=d)
    for e in range(E):
        valid[int(start[e]):int(start[e]) + int(counts[e])] = True
    x[~valid] = 0
    W = _gen((E, H, D), 22, 0.02)
    dy = _gen((m_pad, H), 23, 1e-3)
    dy[~valid] = 0

    def run(xs, ws, offs_, gs):
        HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)
        xa, wa = xs.clone().requires_grad_(True), ws.clone().requires_grad_(True)
        torch.manual_seed(5)                      # the stochastic-rounding streams are drawn from the CPU generator
        y = gmm(xa, wa.transpose(-2, -1), offs_, False, True, True, False, True, "none", True)
        y.backward(gs)
        return y.detach(), xa.grad, wa.grad

    y, dx, dw = run(x, W, offs, dy)
    st, detail = L.status_read()
    assert st == 0, detail
    assert y.shape == (m_pad, H) and torch.isfinite(y).all() and torch.isfinite(dx).all() and torch.isfinite(dw).all()
    assert torch.count_nonzero(y[~valid]) == 0
    # forward samples against the definition: codes x scales / factors, float64 dot products
    def qdq(t, is2d):
        s, mbs = macro_block_scaling(t, axis=-1, use_2d_block=is2d)
        q, sc = MX.convert_to_mxfp4(s, axis=-1, is_2d_block=is2d)
        return macro_block_descaling(MX.convert_from_mxfp4(q, sc, torch.float32, axis=-1, is_2d_block=is2d), mbs,
                                     axis=-1, use_2d_block=is2d)
    x_dq = qdq(x, False)
    for e in (0, 13, 31):
        lo, n = int(start[e]), int(counts[e])
        rows = lo + _sample(n, 24, 30 + e).to(d)
        cols = _sample(H, 40, 60 + e).to(d)
        w_dq = qdq(W[e], True)
        want = (x_dq[rows].double() @ w_dq[cols].double().t()).float().bfloat16().float()
        assert _rel(y[rows][:, cols].float(), want) <= 1e-3
    # one expert alone through the dense two-level linear: same quantisation blocks (runs are multiples of 128
    # rows, stochastic-rounding words repeat with period 64), so dX rows and that expert's dW agree
    e = 7
    lo, hi = int(start[e]), int(start[e] + padded[e])
    HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)
    xe, we = x[lo:hi].clone().requires_grad_(True), W[e].clone().requires_grad_(True)
    torch.manual_seed(5)
    ye = MX._to_mxfp4_then_scaled_mm(xe, we, False, True, True, False, "none", True, True)
    ye.backward(dy[lo:hi])
    assert _rel(y[lo:hi].float(), ye.float()) <= 1e-3
    assert _rel(dx[lo:hi].float(), xe.grad.float()) <= 1e-3
    assert _rel(dw[e].float(), we.grad.float()) <= 2e-3
