"""Macro-block (128) two-level scaling: the oracle against the reference kernel's outputs (CPU), and
the CUDA kernels against both (GPU).  Everything is bit-exact.  Cases and properties follow the
reference's tests/unittest/mxfp4/test_macro_block_scaling.py:36-58 (shapes with ragged blocks,
axis -1 / -2, 1-D and 2-D blocks, bf16 and fp32, factor in [1, 2], round trip)."""
import numpy as np
import pytest
import torch

from oracle import alto_oracle as O
from tests.helpers import bits_equal, case_input, macro_cases

_IDS = lambda v: v[0] if isinstance(v, tuple) else ""  # noqa: E731


@pytest.mark.parametrize("z,m", list(macro_cases()), ids=_IDS)
def test_oracle_matches_reference_kernel(z, m):
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m)
    y, s = O.macro_block_scaling(x, axis, is2d)
    assert bits_equal(s, z[tag + "_s"])
    assert bits_equal(y, z[tag + "_y"])
    xr = O.macro_block_descaling(y, s, axis, is2d)
    assert bits_equal(xr, z[tag + "_xr"])


def test_scale_shape_rule():
    from alto_b200.macro_block_scaling import macro_scale_shape
    assert macro_scale_shape((513, 385), -1, False) == (513, 4)
    assert macro_scale_shape((513, 385), -2, False) == (385, 5)
    assert macro_scale_shape((513, 385), -2, True) == (4, 5)
    assert macro_scale_shape((2, 513, 385), -1, True) == (2, 5, 4)
    assert macro_scale_shape((2, 513, 385), -2, False) == (2, 385, 5)


@pytest.mark.gpu
@pytest.mark.parametrize("z,m", list(macro_cases()), ids=_IDS)
def test_cuda_matches_reference_kernel(z, m):
    from alto_b200.macro_block_scaling import macro_block_descaling, macro_block_scaling
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m).cuda()
    y, s = macro_block_scaling(x, axis=axis, use_2d_block=is2d)
    assert y.dtype == x.dtype and s.dtype == torch.uint8
    assert bits_equal(s, z[tag + "_s"])
    assert bits_equal(y, z[tag + "_y"])
    xr = macro_block_descaling(y, s, axis=axis, use_2d_block=is2d)
    assert bits_equal(xr, z[tag + "_xr"])


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1024, 2048), (513, 385), (2, 513, 385)])
@pytest.mark.parametrize("axis", [-1, -2])
@pytest.mark.parametrize("is2d", [False, True])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_cuda_matches_oracle_and_round_trips(shape, axis, is2d, dt):
    from alto_b200.macro_block_scaling import macro_block_descaling, macro_block_scaling, macro_scale_shape
    g = torch.Generator().manual_seed(hash((shape, axis, is2d)) & 0xFFFF)
    x = torch.randn(shape, generator=g).to(dt)
    y, s = macro_block_scaling(x.cuda(), axis=axis, use_2d_block=is2d)
    assert y.shape == x.shape and tuple(s.shape) == macro_scale_shape(shape, axis, is2d)
    y_o, s_o = O.macro_block_scaling(x, axis, is2d)
    assert torch.equal(s.cpu(), s_o)
    assert torch.equal(y.cpu().view(torch.int16 if dt == torch.bfloat16 else torch.int32),
                       y_o.view(torch.int16 if dt == torch.bfloat16 else torch.int32))
    factor = ((s.to(torch.int32) << 15) + (127 << 23)).view(torch.float32)
    assert torch.all(factor >= 1) and torch.all(factor <= 2)
    xr = macro_block_descaling(y, s, axis=axis, use_2d_block=is2d)
    assert xr.dtype == x.dtype and xr.shape == x.shape
    assert torch.equal(xr.cpu(), O.macro_block_descaling(y_o, s_o, axis, is2d))
    if dt == torch.bfloat16:
        assert torch.allclose(xr.cpu(), x, rtol=1e-2, atol=1e-3)
    else:
        assert torch.allclose(xr.cpu(), x, rtol=1e-6, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("axis,is2d", [(-1, False), (0, False), (-1, True)])
def test_macro_qdq_chain_is_bit_exact(axis, is2d):
    """scale -> quantise -> dequantise -> descale through the public ops equals the oracle's chain."""
    from alto_b200.mxfp4 import _macro_qdq
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(256, 384, generator=g) * torch.exp(torch.randn(256, 1, generator=g))).to(torch.bfloat16)
    got = _macro_qdq(x.cuda(), axis, is2d).cpu()
    want = O.macro_qdq(x, axis, is2d)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def _rel(a, b):
    return ((a.detach().float().cpu() - b).norm() / b.norm()).item()


def _u32dev(r):
    return torch.from_numpy((r.numpy() & 0xFFFFFFFF).astype(np.uint32).view(np.int32)).cuda()


# Two tolerances.  1e-3: against the dequantise-to-fp32, descale-in-fp32, fp32-matmul definition of the
# contraction (the bar for every block-scaled GEMM of this library); the kernel folds exact chunk sums
# with fp32 reciprocal factors, so what is left is fp32 rounding and the bf16 output.  1e-2: against the
# reference's emulation of the recipe, which rounds every de-scaled operand to bf16 before its matmul
# (alto/kernels/fp4/mxfp4/mxfp_linear.py:337-356); that rounding alone moves the result by about 2e-3,
# and the reference's own test of this recipe uses rtol 1e-2.
TOL_FP32_DEFINITION = 1e-3
TOL_BF16_EMULATION = 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(256, 384, 128), (256, 320, 160), (384, 576, 288)])
@pytest.mark.parametrize("use_2dblock_x,use_2dblock_w,use_hadamard,use_sr", [
    (False, True, True, False), (False, False, False, False), (True, True, False, False),
    (False, True, True, True), (True, False, False, True)])
def test_two_level_blockwise_linear_matches_oracle(shape, use_2dblock_x, use_2dblock_w, use_hadamard, use_sr):
    """two_level_scaling='blockwise' on the tensor cores: forward, dgrad and wgrad against the oracle.
    Shapes include reduction axes that end in a chunk shorter than 128 (320, 576, 160, 288) and
    outputs whose last 128 x 128 tile is ragged."""
    from alto_b200 import _lib as L
    from alto_b200 import _linear as E
    from alto_b200 import mxfp4 as MX
    from alto_b200.hadamard import HadamardFactory
    from tests.helpers import rand_u32
    M, K, N = shape
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g))).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=3)
    xd = x.cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    rn = rm = None
    if use_sr:
        rn, rm = rand_u32((2, M, N // 2), 41), rand_u32((2, N, M // 2), 42)
    bits = {"dy_n": None if rn is None else _u32dev(rn), "dy_m": None if rm is None else _u32dev(rm)}
    with E.explicit_sr_bits(lambda name, shp, dev: bits[name]):
        y = MX._to_mxfp4_then_scaled_mm(xd, wd, use_2dblock_x, use_2dblock_w, use_sr, False, "none", use_hadamard,
                                        use_macro_block_scaling=True)
        y.backward(dy.cuda())
    st, detail = L.status_read()
    assert st == 0, detail
    W_had = None
    if use_hadamard:
        HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=3)
        W_had = HadamardFactory.create_transform(device=torch.device("cuda")).matrix().cpu()
    kw = dict(use_2dblock_x=use_2dblock_x, use_2dblock_w=use_2dblock_w, W_had=W_had, rand_dy_n=rn, rand_dy_m=rm)
    assert y.dtype == torch.bfloat16 and y.shape == (M, N)
    yo, dxo, dwo = O.mxfp4_macro_linear(x, w, dy, operand_dtype=torch.float32, **kw)
    assert _rel(y, yo.bfloat16().float()) <= TOL_FP32_DEFINITION
    assert _rel(xd.grad, dxo.bfloat16().float()) <= TOL_FP32_DEFINITION
    assert _rel(wd.grad, dwo.bfloat16().float()) <= TOL_FP32_DEFINITION
    yo, dxo, dwo = O.mxfp4_macro_linear(x, w, dy, **kw)
    assert _rel(y, yo) <= TOL_BF16_EMULATION and _rel(xd.grad, dxo) <= TOL_BF16_EMULATION
    assert _rel(wd.grad, dwo) <= TOL_BF16_EMULATION


@pytest.mark.gpu
def test_two_level_gemm_fp32_output_and_factor_layouts():
    """The C-ABI GEMM alone with fp32 output, factor codes per row on one side and per 128 x 128 tile
    (read through the transposed strides) on the other, against float64 arithmetic on the codes."""
    from alto_b200 import _lib as L
    from alto_b200 import _two_level as T
    g = torch.Generator().manual_seed(21)
    M, K, N = 200 + 56, 448, 320
    a = (torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g))).bfloat16()
    b = torch.randn(K, N, generator=g).bfloat16()          # B^T is the operand: rows n, reduction k
    a_op = T.rows_operand(a.cuda(), False)
    _, b_op = T.tiles_operands(b.cuda(), False)              # operand [N, K] of the 2-D quantised [K, N] tensor
    out = torch.empty(M, N, dtype=torch.float32, device="cuda")
    L.gemm_mxfp4_two_level(M, N, K, a_op.codes, a_op.scales, a_op.macro, b_op.codes, b_op.scales, b_op.macro, out,
                           out_scale=0.5)
    a_dq = O.macro_qdq(a, -1, False, out_dtype=torch.float32).double()
    b_dq = O.macro_qdq(b, -1, True, out_dtype=torch.float32).double()
    want = 0.5 * (a_dq @ b_dq)
    assert ((out.cpu().double() - want).norm() / want.norm()).item() <= 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("clip_mode,use_uos", [("static", False), ("none", True), ("static", True)])
def test_two_level_blockwise_linear_with_clip_uos_and_dge(clip_mode, use_uos):
    """clip_mode / use_uos inside the two-level flow against the oracle, and the DGE factor on top."""
    from alto_b200 import dge
    from alto_b200 import mxfp4 as MX
    M, K, N = 256, 384, 128
    g = torch.Generator().manual_seed(12)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    y = MX._to_mxfp4_then_scaled_mm(xd, wd, False, True, False, False, clip_mode, False, True, use_uos)
    y.backward(dy.cuda())
    yo, dxo, dwo = O.mxfp4_macro_linear(x, w, dy, use_2dblock_x=False, use_2dblock_w=True, clip_mode=clip_mode,
                                        use_uos=use_uos, operand_dtype=torch.float32)
    assert _rel(y, yo.bfloat16().float()) <= TOL_FP32_DEFINITION
    assert _rel(xd.grad, dxo.bfloat16().float()) <= TOL_FP32_DEFINITION
    assert _rel(wd.grad, dwo.bfloat16().float()) <= TOL_FP32_DEFINITION
    # with use_dge the weight gradient is multiplied by the table entry of each weight code (all about 1/5)
    x2, w2 = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    MX._to_mxfp4_then_scaled_mm(x2, w2, False, True, False, True, clip_mode, False, True, use_uos).backward(dy.cuda())
    table = torch.tensor(dge.fp4_bin_table(torch.device("cuda"), torch.bfloat16))
    assert 0.19 < float(table.min()) and float(table.max()) < 0.21
    nz = wd.grad.float().abs() > 1e-3
    ratio = (w2.grad.float()[nz] / wd.grad.float()[nz])
    assert torch.allclose(ratio, torch.full_like(ratio, 0.2), rtol=2e-2)
    assert torch.equal(x2.grad, xd.grad)


@pytest.mark.gpu
def test_refusals():
    from alto_b200.macro_block_scaling import macro_block_descaling, macro_block_scaling
    x = torch.randn(2, 4, 128, 128, device="cuda")
    with pytest.raises(AssertionError):
        macro_block_scaling(x)
    x3 = torch.randn(2, 128, 128, device="cuda")
    with pytest.raises(NotImplementedError):
        macro_block_scaling(x3, axis=0)
    y, s = macro_block_scaling(x3)
    with pytest.raises(AssertionError, match="Unexpected scale shape"):
        macro_block_descaling(y, s, use_2d_block=True)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        macro_block_scaling(torch.randn(128, 128))
