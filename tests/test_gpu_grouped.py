"""GPU tests of the MoE grouped GEMM path (forward, dgrad, wgrad) against the oracle's per-expert
loop, including an expert without tokens and padding rows past ``offs[-1]``."""
import numpy as np
import pytest
import torch

from oracle import alto_oracle as O
from tests.helpers import rand_u32, reference_data

pytestmark = pytest.mark.gpu
REL_TOL = 1e-3


def _dev():
    return torch.device("cuda")


def _u32dev(r):
    return torch.from_numpy((r.numpy() & 0xFFFFFFFF).astype(np.uint32).view(np.int32)).to(_dev())


def _rel(got, exp):
    got = got.detach().float().cpu()
    return ((got - exp).norm() / exp.norm().clamp(min=1e-30)).item()


def _case(n_exp=4, K=256, N=384, counts=(256, 0, 128, 384), pad=128, seed=0):
    M = sum(counts) + pad
    x = reference_data((M, K), torch.float32, seed + 1, outliers=False).bfloat16()
    w = (reference_data((n_exp, N, K), torch.float32, seed + 2, outliers=False) * 0.05).bfloat16()
    dy = (reference_data((M, N), torch.float32, seed + 3, outliers=False) * 1e-2).bfloat16()
    offs = torch.tensor(np.cumsum(counts), dtype=torch.int32)
    return x, w, dy, offs, M


@pytest.mark.parametrize("scheme", ["nvfp4", "mxfp4", "mxfp8"])
@pytest.mark.parametrize("use_2dblock_w", [True, False])
def test_grouped_gemm_matches_oracle(scheme, use_2dblock_w):
    from alto_b200 import _linear as E, grouped as G
    from alto_b200.hadamard import HadamardFactory
    x, w, dy, offs, M = _case()
    n_exp, N, K = w.shape
    d = _dev()
    xd = x.to(d).requires_grad_(True)
    B = w.to(d).transpose(-2, -1).contiguous().requires_grad_(True)  # dispatch layout [E, K, N]
    offs_d = offs.to(d)
    if scheme == "nvfp4":
        HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
        W_had, _, _ = O.random_hadamard(16, torch.Generator().manual_seed(0))
        rn, rm = rand_u32((2, M, N // 2), 31), rand_u32((2, N, M // 2), 32)
        yo, dxo, dwo = O.grouped_linear(x, w, offs, dy, fmt="nvfp4", use_2dblock_w=use_2dblock_w, use_outer=True,
                                        W_had=W_had, rand_dy_n=rn, rand_dy_m=rm)
        bits = {"dy_n": _u32dev(rn), "dy_m": _u32dev(rm)}
        with E.explicit_sr_bits(lambda name, shape, dev: bits[name]):
            y = G._quantize_then_nvfp4_scaled_grouped_mm(xd, B, offs_d, False, use_2dblock_w, True,
                                                         use_outer_scale=True, use_hadamard=True)
            y.backward(dy.to(d))
    elif scheme == "mxfp4":
        yo, dxo, dwo = O.grouped_linear(x, w, offs, dy, fmt="mxfp4", use_2dblock_w=use_2dblock_w)
        y = G._quantize_then_mxfp_scaled_grouped_mm(xd, B, offs_d, False, use_2dblock_w, False, False, False, "none",
                                                    False)
        y.backward(dy.to(d))
    else:
        yo, dxo, dwo = O.grouped_linear(x, w, offs, dy, fmt="e4m3", fmt_grad="e5m2", use_2dblock_w=use_2dblock_w)
        y = G._quantize_then_mxfp8_scaled_grouped_mm(xd, B, offs_d, use_2dblock_w=use_2dblock_w,
                                                     bwd_grad_format="e5m2")
        y.backward(dy.to(d))
    from alto_b200 import _lib as L
    st, detail = L.status_read()
    assert st == 0, detail
    assert _rel(y, yo.bfloat16().float()) <= REL_TOL
    assert _rel(xd.grad, dxo.bfloat16().float()) <= REL_TOL
    dw = B.grad.transpose(-2, -1)  # back to [E, N, K]
    assert _rel(dw, dwo.bfloat16().float()) <= REL_TOL
    # exact zeros where nothing was routed (tests/unittest/nvfp4/test_nvfp_grouped_gemm.py:497-543,
    # tests/unittest/mxfp8/test_mxfp8_grouped_gemm.py:202-224)
    last = int(offs[-1])
    assert torch.all(y[last:] == 0) and torch.all(xd.grad[last:] == 0)
    assert torch.all(dw[1] == 0), "an expert without tokens must get a zero weight gradient"


@pytest.mark.parametrize("use_2dblock_x,use_2dblock_w,use_hadamard,use_sr", [
    (False, True, True, True),      # the MoE recipe: 2-D weight blocks, rotated token-axis operands, SR gradients
    (False, False, False, False), (True, True, False, True)])
@pytest.mark.parametrize("K,N", [(256, 384), (320, 288)])
def test_two_level_grouped_gemm_matches_oracle(use_2dblock_x, use_2dblock_w, use_hadamard, use_sr, K, N):
    """MXFP4 grouped forward, dgrad and wgrad with two-level (macro-block) scaling on the tensor cores
    against the oracle's whole-buffer chains and per-expert fp32 contractions
    (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:631-909).  K = 320 and N = 288 end in chunks
    shorter than 128 and in ragged output tiles; one expert has no tokens; rows past offs[-1] are padding."""
    from alto_b200 import _lib as L
    from alto_b200 import _linear as E, grouped as G
    from alto_b200.hadamard import HadamardFactory
    x, w, dy, offs, M = _case(K=K, N=N)
    n_exp = w.shape[0]
    d = _dev()
    xd = x.to(d).requires_grad_(True)
    B = w.to(d).transpose(-2, -1).contiguous().requires_grad_(True)
    W_had = None
    if use_hadamard:
        HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)
        W_had = HadamardFactory.create_transform(device=d).matrix().cpu()
        HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)
    rn = rm = None
    if use_sr:
        rn, rm = rand_u32((2, M, N // 2), 51), rand_u32((2, N, M // 2), 52)
    bits = {"dy_n": None if rn is None else _u32dev(rn), "dy_m": None if rm is None else _u32dev(rm)}
    with E.explicit_sr_bits(lambda name, shape, dev: bits[name]):
        y = G._quantize_then_mxfp_scaled_grouped_mm(xd, B, offs.to(d), use_2dblock_x, use_2dblock_w, use_sr, False,
                                                    use_hadamard, "none", True)
        y.backward(dy.to(d))
    st, detail = L.status_read()
    assert st == 0, detail
    yo, dxo, dwo = O.mxfp4_macro_grouped_linear(x, w, offs, dy, use_2dblock_x=use_2dblock_x,
                                                use_2dblock_w=use_2dblock_w, W_had=W_had,
                                                operand_dtype=torch.float32, rand_dy_n=rn, rand_dy_m=rm)
    dw = B.grad.transpose(-2, -1)
    assert _rel(y, yo.bfloat16().float()) <= REL_TOL
    assert _rel(xd.grad, dxo.bfloat16().float()) <= REL_TOL
    assert _rel(dw, dwo.bfloat16().float()) <= REL_TOL
    last = int(offs[-1])
    assert torch.all(y[last:] == 0) and torch.all(xd.grad[last:] == 0)
    assert torch.all(dw[1] == 0), "an expert without tokens must get a zero weight gradient"


def test_single_expert_equals_dense_linear():
    """tests/unittest/nvfp4/test_nvfp_grouped_gemm.py:384-420."""
    from alto_b200 import grouped as G, nvfp4 as NV
    d = _dev()
    x = reference_data((256, 256), torch.bfloat16, 5, outliers=False).to(d)
    w = (reference_data((1, 128, 256), torch.bfloat16, 6, outliers=False) * 0.05).to(d)
    offs = torch.tensor([256], dtype=torch.int32, device=d)
    y_g = G._quantize_then_nvfp4_scaled_grouped_mm(x, w.transpose(-2, -1), offs, False, True, False)
    y_d = NV._to_nvfp4_then_scaled_mm(x, w[0], False, True, False)
    assert torch.equal(y_g, y_d)


def test_group_ids_from_offsets_without_sync():
    from alto_b200 import grouped as G
    d = _dev()
    offs = torch.tensor([256, 256, 384, 768], dtype=torch.int32, device=d)
    ge = G.group_experts_from_offsets(offs, 768 + 200)
    assert ge.tolist() == [0, 0, 2, 3, 3, 3, -1, -1]
    idx = G.create_indices_from_offsets_nosync(offs)
    assert idx.shape[0] == 768 and idx[255].item() == 0 and idx[256].item() == 2 and idx[-1].item() == 3


def test_unsupported_grouped_options_raise():
    from alto_b200 import grouped as G
    d = _dev()
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device=d)
    B = torch.zeros(1, 64, 64, dtype=torch.bfloat16, device=d)
    offs = torch.tensor([128], dtype=torch.int32, device=d)
    with pytest.raises(ValueError):
        G._quantize_then_mxfp_scaled_grouped_mm(x, B, offs, False, True, False, False, False, "bogus", False)


def _per_expert_dense(x, w, dy, offs, dense_fn):
    """Dense boundary function on every expert's rows: (y, dx, dw) assembled like the grouped outputs."""
    M, n_exp = x.shape[0], w.shape[0]
    y = torch.zeros(M, w.shape[1], dtype=x.dtype, device=x.device)
    dx = torch.zeros_like(x)
    dw = torch.zeros_like(w)
    lo = 0
    for e in range(n_exp):
        hi = int(offs[e])
        if hi > lo:
            xe, we = x[lo:hi].clone().requires_grad_(True), w[e].clone().requires_grad_(True)
            ye = dense_fn(xe, we)
            ye.backward(dy[lo:hi])
            y[lo:hi], dx[lo:hi], dw[e] = ye.detach(), xe.grad, we.grad
        lo = hi
    return y, dx, dw


@pytest.mark.parametrize("opts", [dict(use_uos=True), dict(clip_mode="static"), dict(clip_mode="dynamic"),
                                  dict(use_dge=True), dict(use_dge=True, use_uos=True, clip_mode="static"),
                                  dict(macro=True), dict(macro=True, use_2dblock_w=False, use_hadamard=True),
                                  dict(use_2dblock_x=True), dict(use_2dblock_x=True, use_uos=True, use_dge=True),
                                  dict(macro=True, use_2dblock_x=True),
                                  dict(macro=True, use_uos=True, clip_mode="static", use_dge=True),
                                  dict(macro=True, use_2dblock_w=False, use_dge=True)])
def test_mxfp4_grouped_options_equal_the_dense_function_per_expert(opts):
    """use_uos, clip_mode, use_dge and two-level scaling in the grouped MXFP4 function.  The dense
    function with the same options is pinned to the reference's vectors; every quantisation block of
    the grouped call (32 rows along tokens, 16 / 32-row Hadamard groups, 128-row macro blocks) lies
    inside one expert's run of rows, so each expert's slice must reproduce the dense call on those
    rows: forward and dgrad bit for bit (same operands, row-local), wgrad to GEMM rounding."""
    from alto_b200 import grouped as G
    from alto_b200 import mxfp4 as MX
    d = _dev()
    x, w, dy, offs, M = _case(counts=(256, 0, 128, 384))
    x, w, dy, offs = x.to(d), w.to(d), dy.to(d), offs.to(d)
    macro = opts.get("macro", False)
    w2d, had = opts.get("use_2dblock_w", True), opts.get("use_hadamard", False)
    uos, clip, dgef = opts.get("use_uos", False), opts.get("clip_mode", "none"), opts.get("use_dge", False)
    x2d = opts.get("use_2dblock_x", False)
    MX.HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ya = G._quantize_then_mxfp_scaled_grouped_mm(xa, wa.transpose(-2, -1), offs, x2d, w2d, False, dgef, had, clip,
                                                 macro, uos)
    ya.backward(dy)

    def dense(a, b):
        MX.HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)  # same matrix
        return MX._to_mxfp4_then_scaled_mm(a, b, x2d, w2d, False, dgef, clip, had, macro, uos)

    yb, dxb, dwb = _per_expert_dense(x, w, dy, offs, dense)
    assert torch.equal(ya, yb), _rel(ya, yb.float().cpu())
    assert torch.equal(xa.grad, dxb)
    assert _rel(wa.grad, dwb.float().cpu()) <= 1e-3
    assert torch.count_nonzero(ya[int(offs[-1]):]) == 0 and torch.count_nonzero(wa.grad[1]) == 0


def test_nvfp4_grouped_dge_equals_the_dense_function_per_expert():
    from alto_b200 import grouped as G
    from alto_b200 import nvfp4 as NV
    d = _dev()
    x, w, dy, offs, M = _case(counts=(128, 256, 0, 128))
    x, w, dy, offs = x.to(d), w.to(d), dy.to(d), offs.to(d)
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ya = G._quantize_then_nvfp4_scaled_grouped_mm(xa, wa.transpose(-2, -1), offs, False, True, False, use_dge=True)
    ya.backward(dy)
    yb, dxb, dwb = _per_expert_dense(
        x, w, dy, offs, lambda a, b: NV._to_nvfp4_then_scaled_mm(a, b, False, True, False, use_dge=True))
    assert torch.equal(ya, yb) and torch.equal(xa.grad, dxb)
    assert _rel(wa.grad, dwb.float().cpu()) <= 1e-3
    # the factor is applied: without it the gradient is about five times larger
    xn, wn = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    G._quantize_then_nvfp4_scaled_grouped_mm(xn, wn.transpose(-2, -1), offs, False, True, False).backward(dy)
    ratio = (wn.grad[0].float().norm() / wa.grad[0].float().norm()).item()
    assert 4.5 < ratio < 5.5


@pytest.mark.parametrize("scheme", ["nvfp4", "mxfp8"])
def test_grouped_2d_activation_blocks_equal_the_dense_function_per_expert(scheme):
    from alto_b200 import grouped as G
    from alto_b200 import mxfp8 as M8, nvfp4 as NV
    d = _dev()
    x, w, dy, offs, M = _case(counts=(128, 256, 0, 128))
    x, w, dy, offs = x.to(d), w.to(d), dy.to(d), offs.to(d)
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    if scheme == "nvfp4":
        ya = G._quantize_then_nvfp4_scaled_grouped_mm(xa, wa.transpose(-2, -1), offs, True, True, False)
        dense = lambda a, b: NV._to_nvfp4_then_scaled_mm(a, b, True, True, False)  # noqa: E731
    else:
        ya = G._quantize_then_mxfp8_scaled_grouped_mm(xa, wa.transpose(-2, -1), offs, use_2dblock_x=True)
        dense = lambda a, b: M8._to_mxfp8_then_scaled_mm(a, b, "e4m3", False, True, True)  # noqa: E731
    ya.backward(dy)
    yb, dxb, dwb = _per_expert_dense(x, w, dy, offs, dense)
    assert torch.equal(ya, yb) and torch.equal(xa.grad, dxb)
    assert _rel(wa.grad, dwb.float().cpu()) <= 1e-3


@pytest.mark.parametrize("scheme", ["mxfp4", "mxfp8"])
@pytest.mark.parametrize("use_2dblock_w,trans_weights", [(True, True), (False, True), (True, False)])
def test_prequantized_grouped_forward_op_equals_the_quantize_then_function(scheme, use_2dblock_w, trans_weights):
    """The registered forward ops on quantised operands (reference:
    alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_forward.py:200, alto/kernels/mxfp8/mxfp8_grouped_gemm/cg_forward.py:222)
    fed with the public quantizers' codes and plain scales give the forward of the quantise-then-GEMM
    boundary function bit for bit, zero rows past the routed rows included."""
    from alto_b200 import grouped as G, mxfp4, mxfp8, torch_ops
    torch_ops.register()
    x, w, _, offs, M = _case()
    d = _dev()
    xd, wd, offs_d = x.to(d), w.to(d), offs.to(d)
    idx = G.create_indices_from_offsets_nosync(offs_d)
    if scheme == "mxfp4":
        xq, xs = mxfp4.convert_to_mxfp4(xd, axis=-1)
        wq, ws = mxfp4.convert_to_mxfp4(wd, axis=-1, is_2d_block=use_2dblock_w)
        want = G._quantize_then_mxfp_scaled_grouped_mm(xd, wd.transpose(-2, -1), offs_d, False, use_2dblock_w, False,
                                                       False, False, "none", False)
        op = torch.ops.alto_b200.mxfp4_grouped_gemm_forward
    else:
        xq, xs = mxfp8.convert_to_mxfp8(xd, axis=-1)
        wq, ws = mxfp8.convert_to_mxfp8(wd, axis=-1, is_2d_block=use_2dblock_w)
        want = G._quantize_then_mxfp8_scaled_grouped_mm(xd, wd.transpose(-2, -1), offs_d, use_2dblock_w=use_2dblock_w)
        op = torch.ops.alto_b200.mxfp8_grouped_gemm_forward
    if not trans_weights:
        wq, ws = wq.transpose(-2, -1), ws.transpose(-2, -1)
    got = op(xq, wq, idx, xs, ws, trans_weights=trans_weights, use_2dblock_w=use_2dblock_w)
    assert got.dtype == torch.bfloat16 and got.shape == want.shape
    assert torch.equal(got, want)
    assert int(offs[-1]) < M and not got[int(offs[-1]):].any()
    with pytest.raises(RuntimeError):
        op(xq, wq, idx[:-1], xs, ws, trans_weights=trans_weights, use_2dblock_w=use_2dblock_w)


@pytest.mark.parametrize("scheme", ["mxfp4", "mxfp8"])
@pytest.mark.parametrize("use_2dblock_w,trans_weights", [(True, True), (False, True), (True, False)])
def test_prequantized_grouped_backward_ops_equal_the_autograd_gradients(scheme, use_2dblock_w, trans_weights):
    """The registered backward ops on quantised operands (reference:
    alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:398, 500;
    alto/kernels/mxfp8/mxfp8_grouped_gemm/cg_backward.py:313, 416) fed with the public quantizers' codes and
    plain scales reproduce dX and dW of the quantise-then-GEMM boundary function bit for bit (RTN, no
    Hadamard): the same codes reach the same kernels."""
    from alto_b200 import grouped as G, mxfp4, mxfp8, torch_ops
    torch_ops.register()
    x, w, dy, offs, M = _case()
    d = _dev()
    xd, wd, dyd, offs_d = x.to(d), w.to(d), dy.to(d), offs.to(d)
    n_exp = wd.shape[0]
    idx = G.create_indices_from_offsets_nosync(offs_d)
    xa, wa = xd.clone().requires_grad_(True), wd.clone().requires_grad_(True)
    if scheme == "mxfp4":
        ya = G._quantize_then_mxfp_scaled_grouped_mm(xa, wa.transpose(-2, -1), offs_d, False, use_2dblock_w, False,
                                                     False, False, "none", False)
        conv, ops = mxfp4.convert_to_mxfp4, torch.ops.alto_b200
        dx_op, dw_op = ops.mxfp4_grouped_gemm_backward_inputs, ops.mxfp4_grouped_gemm_backward_weights
    else:
        ya = G._quantize_then_mxfp8_scaled_grouped_mm(xa, wa.transpose(-2, -1), offs_d, use_2dblock_w=use_2dblock_w)
        conv, ops = mxfp8.convert_to_mxfp8, torch.ops.alto_b200
        dx_op, dw_op = ops.mxfp8_grouped_gemm_backward_inputs, ops.mxfp8_grouped_gemm_backward_weights
    ya.backward(dyd)
    # dgrad operands: dY along N; W along N (axis -2 of [E, N, K]), or its 2-D quantisation
    gq, gs = conv(dyd, axis=-1)
    wq, ws = conv(wd, axis=-2, is_2d_block=use_2dblock_w)
    if not trans_weights:
        wq, ws = wq.transpose(-2, -1), ws.transpose(-2, -1)
    dx = dx_op(gq, wq, idx, gs, ws, trans_weights=trans_weights, use_2dblock_w=use_2dblock_w)
    assert dx.dtype == torch.bfloat16 and torch.equal(dx, xa.grad)
    # wgrad operands: dY and X along the token axis
    gmq, gms = conv(dyd, axis=0)
    xmq, xms = conv(xd, axis=0)
    dw = dw_op(gmq, xmq, idx, n_exp, gms, xms, trans_weights=trans_weights, use_2dblock_x=False)
    want = wa.grad if trans_weights else wa.grad.transpose(-2, -1)
    assert dw.shape == want.shape and torch.equal(dw, want)
    assert not dx[int(offs[-1]):].any() and not wa.grad[1].any()
    if scheme == "mxfp4":
        with pytest.raises(NotImplementedError):
            dx_op(gq, wq, idx, gs, ws, trans_weights=trans_weights, use_2dblock_w=use_2dblock_w, k_pack_w=False)
