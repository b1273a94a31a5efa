"""GPU parity tests of the quantizer kernels: CUDA path (through the C ABI) vs the CPU oracle and
the committed reference vectors.  Codes, scales and packed layouts are compared bit for bit."""
import numpy as np
import pytest
import torch

from oracle import alto_oracle as O
from tests.helpers import case_input, golden_cases, load_golden, rand_u32, reference_data, tensor_from_bits

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _u32dev(r):
    return torch.from_numpy((r.numpy() & 0xFFFFFFFF).astype(np.uint32).view(np.int32)).to(_dev())


def _same(got: torch.Tensor, exp, what=""):
    got = got.detach().cpu()
    if isinstance(exp, np.ndarray):
        exp = torch.from_numpy(exp.copy())
    if got.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        got = got.view(torch.uint8)
    if exp.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        exp = exp.view(torch.uint8)
    assert tuple(got.shape) == tuple(exp.shape), f"{what}: shape {tuple(got.shape)} vs {tuple(exp.shape)}"
    if got.dtype.is_floating_point:
        bad = ~((got == exp) | (got.isnan() & exp.isnan()))
    else:
        bad = got != exp.to(got.dtype)
    assert int(bad.sum()) == 0, f"{what}: {int(bad.sum())} of {got.numel()} entries differ"


# ------------------------------------------------------------------------------------------
# committed reference vectors (outputs of the reference's own code)
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("z,m", list(golden_cases("nvfp4")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_nvfp4_kernel_matches_reference_vectors(z, m):
    from alto_b200 import nvfp4 as NV
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m).to(_dev())
    outer = z[tag + "_outer"]
    outer_d = torch.from_numpy(outer.copy()).to(_dev()) if outer.size else None
    if outer_d is not None:
        _same(NV.compute_dynamic_outer_scale(x), outer, "outer scale")
        buf = torch.zeros(1, dtype=torch.float32, device=_dev())
        q, s = NV.convert_to_nvfp4(x, axis=axis, is_2d_block=is2d, outer_scale=buf, update_outer_scale=True)
        _same(buf, outer, "outer scale refreshed in place")
    else:
        q, s = NV.convert_to_nvfp4(x, axis=axis, is_2d_block=is2d, update_outer_scale=False)
    _same(s, z[tag + "_s"], "scales")
    nan_in = torch.isnan(x.float()).cpu()
    if nan_in.any():
        # The code emitted for a NaN ELEMENT is an accident of the NaN payload that survives the
        # division (the reference's kernel and its CPU emulation differ there); what the reference
        # tests for NaN input is finite scales and a finite dequantisation.
        keep = ~(nan_in[..., 0::2] | nan_in[..., 1::2])
        assert torch.equal(q.cpu()[keep], torch.from_numpy(z[tag + "_q"].copy())[keep])
        assert torch.isfinite(NV.convert_from_nvfp4(q, s, torch.float32, outer_scale=outer_d)).all()
        return
    _same(q, z[tag + "_q"], "codes")
    dq = NV.convert_from_nvfp4(q, s, torch.float32, axis=axis, is_2d_block=is2d, outer_scale=outer_d)
    _same(dq, z[tag + "_dq"], "dequantised")


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp4")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_mxfp4_kernel_matches_reference_vectors(z, m):
    from alto_b200 import mxfp4 as MX
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m).to(_dev())
    q, s = MX.convert_to_mxfp4(x, axis=axis, is_2d_block=is2d)
    _same(s, z[tag + "_s"], "scales")
    _same(q, z[tag + "_q"], "codes")
    _same(MX.convert_from_mxfp4(q, s, torch.float32, axis=axis, is_2d_block=is2d), z[tag + "_dq"], "dequantised")


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp4sr")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_mxfp4_stochastic_rounding_matches_reference_kernel(z, m):
    """Same random words as the reference's Triton kernel consumed -> same codes."""
    from alto_b200 import mxfp4 as MX
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m).to(_dev())
    rand = torch.from_numpy(z[tag + "_rand"].view(np.int32).copy()).to(_dev())
    q, s = MX.convert_to_mxfp4(x, axis=axis, use_sr=True, rand_bits=rand)
    _same(s, z[tag + "_s"], "scales")
    _same(q, z[tag + "_q"], "codes")


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp8")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_mxfp8_kernel_matches_reference_vectors(z, m):
    from alto_b200 import mxfp8 as M8
    tag, shape, dt, axis, is2d, fmt = m
    x = case_input(z, m).to(_dev())
    q, s = M8.convert_to_mxfp8(x, mxfp_format=fmt, axis=axis, is_2d_block=is2d)
    _same(s, z[tag + "_s"], "scales")
    _same(q, z[tag + "_q"], "codes")
    _same(M8.convert_from_mxfp8(q, s, torch.float32, axis=axis, is_2d_block=is2d), z[tag + "_dq"], "dequantised")
    _same(M8.calculate_mxfp8_scales(x, mxfp_format=fmt, axis=axis, is_2d_block=is2d), z[tag + "_s"], "scale op")


def test_hadamard_kernel_matches_reference_vectors():
    from alto_b200 import _lib as L
    z, _ = load_golden()
    W = torch.from_numpy(z["rht16_W"])
    g = torch.Generator().manual_seed(0)
    W2, perm, sign = O.random_hadamard(16, g)
    assert torch.equal(W, W2)
    x = tensor_from_bits(z["rht16_x"], torch.bfloat16).to(_dev())
    y = torch.empty_like(x)
    L.rht_apply(x, y, L.Rht(16, perm.tolist(), [int(v) for v in sign.tolist()]))
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), z["rht16_y"])


def test_hadamard_factory_matches_reference_draws():
    from alto_b200.hadamard import HadamardFactory
    z, _ = load_golden()
    HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
    t = HadamardFactory.create_transform(device=_dev())
    assert torch.equal(t.matrix().cpu(), torch.from_numpy(z["rht16_W"]))
    x = tensor_from_bits(z["rht16_x"], torch.bfloat16).to(_dev())
    y = t(x, left_mul=True)
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), z["rht16_y"])
    HadamardFactory.configure(block_size=16)


@pytest.mark.parametrize("n", [16, 32])
def test_dense_hadamard_kernel(n):
    """The reference's default block size 32 uses a table matrix that is not of Sylvester type: the
    dense transform kernel must give what the reference's own tensor ops give on this GPU (fp32 matmul,
    division by the 0-dim sqrt(n) tensor, cast), bit for bit, and the oracle's restatement of it."""
    from alto_b200 import _lib as L
    from alto_b200.hadamard import HadamardFactory
    z, _ = load_golden()
    HadamardFactory.configure(block_size=n, randomized=True, dtype=torch.float32, seed=0)
    t = HadamardFactory.create_transform(device=_dev())
    W = torch.from_numpy(z[f"rht{n}_W"])
    assert torch.equal(t.matrix().cpu(), W)
    assert t.is_fused == (n == 16)
    x = tensor_from_bits(z[f"rht{n}_x"], torch.bfloat16).to(_dev())
    y = torch.empty_like(x)
    L.rht_dense(x, y, W.to(_dev()))
    want = O.rht_apply(x.cpu(), W)
    assert torch.equal(y.cpu().view(torch.int16), want.view(torch.int16))
    assert torch.equal(t(x, left_mul=True), y)   # fused butterfly (16) or dense kernel (32): same values
    # the reference's formula with PyTorch's own CUDA kernels (transform.py:133-141)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        scale = torch.tensor(n, dtype=torch.float64).sqrt()
        M_, N_ = x.shape
        ref = ((W.to(_dev()).float() @ x.float().view(M_ // n, n, N_)) / scale).view(M_, N_).to(x.dtype)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert torch.equal(y, ref)
    # vectors made on CPU (true division): identical for 16, within one bf16 ulp in rare places for 32
    gold = tensor_from_bits(z[f"rht{n}_y"], torch.bfloat16)
    d = (y.cpu().view(torch.int16).int() - gold.view(torch.int16).int()).abs()
    assert d.max().item() <= (0 if n == 16 else 1) and (d != 0).float().mean().item() < 1e-3
    HadamardFactory.configure(block_size=16)
    # fp32 input and a ragged last column
    xf = torch.randn(64, 37, device=_dev())
    yf = torch.empty_like(xf)
    L.rht_dense(xf, yf, W.to(_dev()))
    assert torch.allclose(yf.cpu(), O.rht_apply(xf.cpu(), W), rtol=1e-6, atol=1e-6)
    # bf16 at the shapes that take the tensor-core form of the 32-point transform (rows of whole 16-byte
    # chunks; a last column tile that is not full; in place) and at one that does not (odd width)
    for shape in ((96, 264), (64, 2880), (32, 8), (64, 36)):
        xb = reference_data(shape, torch.bfloat16, 4321 + shape[1]).to(_dev())
        yb = torch.empty_like(xb)
        L.rht_dense(xb, yb, W.to(_dev()))
        want = O.rht_apply(xb.cpu(), W)
        assert torch.equal(yb.cpu().view(torch.int16), want.view(torch.int16)), shape
        L.rht_dense(xb, xb, W.to(_dev()))
        assert torch.equal(xb, yb), shape
    HadamardFactory.configure(block_size=16, seed=0)


# ------------------------------------------------------------------------------------------
# oracle parity at the reference tests' shapes and at larger, ragged and special inputs
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(128, 64), (2048, 2048), (4, 128, 64), (150, 64), (96, 2880)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("outer", [False, True])
def test_nvfp4_rowwise(shape, dtype, outer):
    from alto_b200 import nvfp4 as NV
    x = reference_data(shape, dtype, 1234)
    oc = O.compute_dynamic_outer_scale(x) if outer else None
    qo, so = O.quantize_nvfp4(x, 16, -1, False, oc)
    q, s = NV.convert_to_nvfp4(x.to(_dev()), update_outer_scale=outer)
    _same(s, so, "scales")
    _same(q, qo, "codes")


@pytest.mark.parametrize("fmt", ["mxfp4", "e4m3", "e5m2"])
@pytest.mark.parametrize("shape,axis,is2d", [((128, 64), -1, False), ((2048, 2048), -1, False), ((4, 128, 64), -2, False),
                                             ((2048, 2048), 0, False), ((2048, 2048), -1, True), ((256, 2880), -1, False),
                                             ((2048, 1024), 0, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_mx_formats(fmt, shape, axis, is2d, dtype):
    from alto_b200 import mxfp4 as MX, mxfp8 as M8
    x = reference_data(shape, dtype, 1234)
    if fmt == "mxfp4":
        qo, so = O.quantize_mxfp4(x, 32, axis, is2d)
        q, s = MX.convert_to_mxfp4(x.to(_dev()), axis=axis, is_2d_block=is2d)
    else:
        qo, so = O.quantize_mxfp8(x, 32, fmt, axis, is2d)
        q, s = M8.convert_to_mxfp8(x.to(_dev()), mxfp_format=fmt, axis=axis, is_2d_block=is2d)
    _same(s, so, "scales")
    _same(q, qo, "codes")


@pytest.mark.parametrize("shape", [(128, 64), (2048, 1024), (512, 200)])
@pytest.mark.parametrize("mode", ["rtn", "sr_bits", "sr_philox"])
@pytest.mark.parametrize("use_rht", [False, True])
def test_nvfp4_colwise_with_hadamard_and_sr(shape, mode, use_rht):
    """Axis-0 quantisation, optionally after the 16-point randomised Hadamard transform, with
    round-to-nearest, explicit random bits, and in-kernel Philox."""
    from alto_b200 import _lib as L
    M, N = shape
    x = reference_data(shape, torch.bfloat16, 7, outliers=False)
    g = torch.Generator().manual_seed(3)
    W, perm, sign = O.random_hadamard(16, g)
    rht = L.Rht(16, perm.tolist(), [int(v) for v in sign.tolist()]) if use_rht else None
    xin = O.rht_apply(x, W) if use_rht else x
    outer = O.compute_dynamic_outer_scale(xin)
    rand, kw = None, {}
    if mode == "sr_bits":
        rand = rand_u32((2, N, M // 2), 11)
        kw = dict(rounding=L.ROUND_SR_BITS, rand_bits=_u32dev(rand))
    elif mode == "sr_philox":
        seed, off = 0x1234567890AB, 77
        ctr = torch.arange(N * (M // 2) // 2, dtype=torch.int64) + off
        zz = torch.zeros_like(ctr)
        o = O.philox4x32_10(ctr & 0xFFFFFFFF, ctr >> 32, zz, zz, torch.full_like(ctr, seed & 0xFFFFFFFF),
                            torch.full_like(ctr, seed >> 32))
        # call q feeds pairs 2q (words 0,1) and 2q+1 (words 2,3); word parity = element parity
        rand = torch.stack([torch.stack([o[0], o[2]], 1).reshape(N, M // 2),
                            torch.stack([o[1], o[3]], 1).reshape(N, M // 2)])
        kw = dict(rounding=L.ROUND_SR_PHILOX, philox=(seed, off))
    qo, so = O.quantize_nvfp4(xin, 16, 0, False, outer, rand)
    xd = x.to(_dev())
    codes = torch.empty(N, M // 2, dtype=torch.uint8, device=_dev())
    plain = torch.empty(N, M // 16, dtype=torch.float32, device=_dev())
    packed = torch.full((L.packed_scale_bytes(N, M // 16),), 0xAB, dtype=torch.uint8, device=_dev())
    L.quantize_colwise(xd, L.FMT_NVFP4, codes, plain, packed, outer_scale=outer.to(_dev()), rht=rht, **kw)
    _same(plain, so.t(), "scales")
    _same(codes, qo.t(), "codes")
    _same(packed, O.pack_scale_bytes(O.e4m3_byte(so.t().contiguous())), "packed scales")


def test_nvfp4_rowwise_stochastic_rounding_bits_and_philox():
    from alto_b200 import nvfp4 as NV
    x = reference_data((256, 512), torch.bfloat16, 4)
    r = rand_u32((2, 256, 256), 5)
    qo, _ = O.quantize_nvfp4(x, 16, -1, False, None, r)
    q, _ = NV.convert_to_nvfp4(x.to(_dev()), update_outer_scale=False, use_sr=True, rand_bits=_u32dev(r))
    _same(q, qo, "explicit bits")
    q_rtn, _ = O.quantize_nvfp4(x, 16, -1, False, None)
    assert (q_rtn != qo).float().mean() > 0.05
    # (seed, offset): the reference kernel's words in the reference kernel's layout
    seed, off = 987654321, 12345
    rp = O.reference_sr_planes(seed, off, 256, 512)
    qo, _ = O.quantize_nvfp4(x, 16, -1, False, None, rp)
    q, _ = NV.convert_to_nvfp4(x.to(_dev()), update_outer_scale=False, use_sr=True, philox_seed=seed,
                               philox_offset=off)
    _same(q, qo, "philox")
    # along the token axis: the view is the transposed matrix [512, 256]
    qo, _ = O.quantize_nvfp4(x, 16, 0, False, None, O.reference_sr_planes(seed, off, 512, 256))
    q, _ = NV.convert_to_nvfp4(x.to(_dev()), axis=0, update_outer_scale=False, use_sr=True, philox_seed=seed,
                               philox_offset=off)
    _same(q, qo, "philox, axis 0")


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp4sr")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_mxfp4_stochastic_rounding_from_seed_and_offset_matches_reference_kernel(z, m):
    """Same (philox_seed, philox_offset) as the reference's Triton kernel was run with -> same codes."""
    from alto_b200 import mxfp4 as MX
    tag, shape, dt, axis, is2d = m
    seed, off = [int(v) for v in z["philox_seed_offset"]]
    x = case_input(z, m).to(_dev())
    q, s = MX.convert_to_mxfp4(x, axis=axis, use_sr=True, philox_seed=seed, philox_offset=off)
    _same(s, z[tag + "_s"], "scales")
    _same(q, z[tag + "_q"], "codes")


@pytest.mark.parametrize("shape", [(128, 64), (256, 320), (1024, 2048), (144, 80)])
def test_nvfp4_2d_dual_packing_and_packed_scales(shape):
    from alto_b200 import _lib as L
    R, Cc = shape
    x = (reference_data(shape, torch.bfloat16, 9, outliers=False) * 0.02).to(torch.bfloat16)
    oc = O.compute_dynamic_outer_scale(x)
    d = _dev()
    ck = torch.empty(R, Cc // 2, dtype=torch.uint8, device=d)
    ct = torch.empty(Cc, R // 2, dtype=torch.uint8, device=d)
    plain = torch.empty(R // 16, Cc // 16, dtype=torch.float32, device=d)
    pk = torch.full((L.packed_scale_bytes(R, Cc // 16),), 0xAB, dtype=torch.uint8, device=d)
    pt = torch.full((L.packed_scale_bytes(Cc, R // 16),), 0xAB, dtype=torch.uint8, device=d)
    L.quantize_2d(x.to(d), L.FMT_NVFP4, ck, ct, plain, pk, pt, outer_scale=oc.to(d))
    qo, so = O.quantize_nvfp4(x, 16, -1, True, oc)
    qt, _ = O.quantize_nvfp4(x, 16, 0, True, oc)
    _same(plain, so, "scales")
    _same(ck, qo, "codes packed along columns")
    _same(ct, qt.t(), "codes packed along rows")
    sb = O.e4m3_byte(so)
    _same(pk, O.pack_scale_bytes(sb.repeat_interleave(16, 0)), "packed scales (row operand)")
    _same(pt, O.pack_scale_bytes(sb.t().repeat_interleave(16, 0)), "packed scales (transposed operand)")


def test_nvfp4_special_values():
    """The reference's edge cases (tests/unittest/nvfp4/test_nvfp_quantization.py:167-339)."""
    from alto_b200 import nvfp4 as NV
    d = _dev()
    zeros = torch.zeros(64, 64, dtype=torch.bfloat16, device=d)
    q, s = NV.convert_to_nvfp4(zeros, update_outer_scale=False)
    assert torch.all(s == 2.0 ** -6) and torch.all(q == 0)
    big = torch.full((64, 64), 5000.0, dtype=torch.bfloat16, device=d)
    q, s = NV.convert_to_nvfp4(big, update_outer_scale=False)
    assert torch.all(s == 448.0) and torch.all(q == 0x77)
    buf = torch.zeros(1, dtype=torch.float32, device=d)
    q, s = NV.convert_to_nvfp4(zeros, outer_scale=buf)
    assert buf.item() == pytest.approx(1e-30) and (s * buf).min().item() > 1.17e-38
    x = torch.randn(64, 64, device=d).bfloat16()
    x.view(-1)[7] = float("nan")
    q, s = NV.convert_to_nvfp4(x, update_outer_scale=False)
    assert torch.isfinite(s).all()
    assert torch.isfinite(NV.convert_from_nvfp4(q, s)).all()
    assert NV.compute_dynamic_outer_scale(x).item() == pytest.approx(1e-30)
    neg0 = torch.full((16, 16), -0.0, dtype=torch.bfloat16, device=d)
    q, _ = NV.convert_to_nvfp4(neg0, update_outer_scale=False)
    assert torch.all(q == 0x88)


def test_contract_violations_raise_before_launch():
    from alto_b200 import _lib as L, mxfp8 as M8, nvfp4 as NV
    d = _dev()
    with pytest.raises(RuntimeError):
        NV.convert_to_nvfp4(torch.zeros(16, 24, dtype=torch.bfloat16, device=d))
    with pytest.raises(AssertionError):
        NV.convert_to_nvfp4(torch.zeros(16, 32, dtype=torch.float16, device=d))
    with pytest.raises(NotImplementedError):
        NV.convert_to_nvfp4(torch.zeros(16, 32, dtype=torch.bfloat16, device=d), scale_format="ue5m3")
    with pytest.raises(AssertionError):
        M8.convert_to_mxfp8(torch.zeros(32, 32, dtype=torch.bfloat16, device=d), use_sr=True)
    with pytest.raises(RuntimeError):
        NV.convert_to_nvfp4(torch.zeros(16, 32, dtype=torch.bfloat16))  # CPU tensor: no fallback
    x = torch.zeros(64, 64, dtype=torch.bfloat16, device=d)
    with pytest.raises(L.Altob200Error) as e:
        L.quantize_rowwise(x[:, 1:33], L.FMT_NVFP4, torch.empty(64, 16, dtype=torch.uint8, device=d))
    assert e.value.status == L.E_ALIGN


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("shape", [(256, 512), (96, 160)])
def test_2d_blocks_with_stochastic_rounding(fmt, shape):
    """2-D blocks quantised once with stochastic rounding (the gradient of a `use_2dblock_x` linear,
    alto/kernels/fp4/nvfp4/nvfp_linear.py:176-186): explicit words and (seed, offset), both packings."""
    from alto_b200 import _lib as L
    from alto_b200 import mxfp4 as MX, nvfp4 as NV
    R, Cc = shape
    if fmt == "mxfp4" and (R % 32 or Cc % 32):
        pytest.skip("32 x 32 blocks")
    x = reference_data(shape, torch.bfloat16, 14)
    r = rand_u32((2, R, Cc // 2), 15)
    seed, off = 24680, 1357
    rp = O.reference_sr_planes(seed, off, R, Cc)
    if fmt == "nvfp4":
        qo, so = O.quantize_nvfp4(x, 16, -1, True, None, r)
        q, s = NV.convert_to_nvfp4(x.to(_dev()), is_2d_block=True, update_outer_scale=False, use_sr=True,
                                   rand_bits=_u32dev(r))
        qp_o, _ = O.quantize_nvfp4(x, 16, -1, True, None, rp)
        qp, _ = NV.convert_to_nvfp4(x.to(_dev()), is_2d_block=True, update_outer_scale=False, use_sr=True,
                                    philox_seed=seed, philox_offset=off)
        q_rtn, _ = O.quantize_nvfp4(x, 16, -1, True, None)
    else:
        qo, so = O.quantize_mxfp4(x, 32, -1, True, r)
        q, s = MX.convert_to_mxfp4(x.to(_dev()), is_2d_block=True, use_sr=True, rand_bits=_u32dev(r))
        qp_o, _ = O.quantize_mxfp4(x, 32, -1, True, rp)
        qp, _ = MX.convert_to_mxfp4(x.to(_dev()), is_2d_block=True, use_sr=True, philox_seed=seed, philox_offset=off)
        q_rtn, _ = O.quantize_mxfp4(x, 32, -1, True)
    _same(s, so, "scales")
    _same(q, qo, "explicit bits")
    _same(qp, qp_o, "philox")
    assert (q_rtn != qo).float().mean() > 0.05
    # the second packing holds the same codes transposed
    fid = L.FMT_NVFP4 if fmt == "nvfp4" else L.FMT_MXFP4
    d = _dev()
    ck = torch.empty(R, Cc // 2, dtype=torch.uint8, device=d)
    ct = torch.empty(Cc, R // 2, dtype=torch.uint8, device=d)
    L.quantize_2d(x.to(d), fid, ck, ct, rounding=L.ROUND_SR_BITS, rand_bits=_u32dev(r))
    _same(ck, qo, "K packing")
    want_t = O.pack_nibbles(O.unpack_nibbles(qo.view(torch.uint8)).t().contiguous())
    _same(ct, want_t, "N packing")
    # along axis 0 the words belong to the transposed view: the same codes as quantising x^T along its last axis
    rt = rand_u32((2, Cc, R // 2), 78)
    qa, sa = NV.convert_to_nvfp4(x.to(d), axis=0, is_2d_block=True, update_outer_scale=False, use_sr=True,
                                 rand_bits=_u32dev(rt)) if fmt == "nvfp4" else \
        MX.convert_to_mxfp4(x.to(d), axis=0, is_2d_block=True, use_sr=True, rand_bits=_u32dev(rt))
    if fmt == "nvfp4":
        qr, sr_ = O.quantize_nvfp4(x, 16, 0, True, None, rt)
    else:
        qr, sr_ = O.quantize_mxfp4(x, 32, 0, True, rt)
    _same(qa.contiguous(), qr.contiguous(), "axis-0 codes")
    _same(sa.contiguous(), sr_.contiguous(), "axis-0 scales")


def test_mxfp4_2d_blocks_with_seeded_stochastic_rounding_match_the_reference_kernel():
    import ast
    from pathlib import Path
    from alto_b200 import mxfp4 as MX
    z = np.load(Path(__file__).resolve().parent / "golden" / "sr2d_vectors.npz")
    seed, off = [int(v) for v in z["philox_seed_offset"]]
    for tag, shape, axis in ast.literal_eval(str(z["meta"])):
        x = torch.from_numpy(z[tag + "_x"].view(np.int16)).view(torch.bfloat16).reshape(shape).to(_dev())
        q, s = MX.convert_to_mxfp4(x, axis=axis, is_2d_block=True, use_sr=True, philox_seed=seed, philox_offset=off)
        _same(s.contiguous(), z[tag + "_s"], tag + " scales")
        _same(q.contiguous(), z[tag + "_q"], tag + " codes")


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "mxfp8"])
def test_2d_batched_launch_equals_one_launch_per_matrix(fmt):
    """`altob200_quantize_2d_batched` (all experts of a MoE weight in one launch) against per-matrix calls,
    every output, and batched stochastic rounding against the oracle's flattened view."""
    from alto_b200 import _lib as L
    from alto_b200 import mxfp4 as MX
    fid = {"nvfp4": L.FMT_NVFP4, "mxfp4": L.FMT_MXFP4, "mxfp8": L.FMT_MXFP8_E4M3}[fmt]
    b = L.block_of(fid)
    nb, R, Cc = 3, 160, 96
    if b == 32:
        R, Cc = 160, 96
    d = _dev()
    x = reference_data((nb, R, Cc), torch.bfloat16, 21).to(d)
    cc, rc = (Cc // 2, R // 2) if L.is_fp4(fid) else (Cc, R)
    sdt = torch.float32 if fmt == "nvfp4" else torch.uint8

    def bufs(n):
        return (torch.empty(n, R, cc, dtype=torch.uint8, device=d), torch.empty(n, Cc, rc, dtype=torch.uint8, device=d),
                torch.empty(n, R // b, Cc // b, dtype=sdt, device=d),
                torch.zeros(n, L.packed_scale_bytes(R, Cc // b), dtype=torch.uint8, device=d),
                torch.zeros(n, L.packed_scale_bytes(Cc, R // b), dtype=torch.uint8, device=d))

    ck, ct, sp, pk, pt = bufs(nb)
    L.quantize_2d_batched(x, fid, ck, ct, sp, pk.view(-1), pt.view(-1))
    for i in range(nb):
        ck1, ct1, sp1, pk1, pt1 = bufs(1)
        L.quantize_2d(x[i], fid, ck1[0], ct1[0], sp1[0], pk1[0], pt1[0])
        for got, exp, what in ((ck[i], ck1[0], "codes_k"), (ct[i], ct1[0], "codes_t"), (sp[i], sp1[0], "scales"),
                               (pk[i], pk1[0], "packed_k"), (pt[i], pt1[0], "packed_t")):
            _same(got, exp.cpu(), f"{what}[{i}]")
    if fmt == "mxfp4":
        r = rand_u32((2, nb * R, Cc // 2), 22)
        qo, so = O.quantize_mxfp4(x.cpu(), 32, -1, True, r)
        q, s = MX.convert_to_mxfp4(x, is_2d_block=True, use_sr=True, rand_bits=_u32dev(r))
        _same(s, so, "batched SR scales")
        _same(q, qo, "batched SR codes")


def _sweep_shapes(seed, n, block):
    """Seeded ragged shapes: rows and columns are multiples of the block, otherwise arbitrary (not
    multiples of the kernels' 4-row tasks, 64 / 256-row tiles or 512-column chunks)."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        r = int(torch.randint(1, 24, (1,), generator=g)) * block
        c = int(torch.randint(1, 40, (1,), generator=g)) * block
        out.append((r, c))
    return out


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "mxfp8"])
def test_ragged_shape_sweep_all_layouts(fmt):
    """Every quantizer layout (1-D along the last axis, 1-D along the token axis, 2-D) on a seeded
    sweep of ragged shapes, round to nearest and (FP4) stochastic rounding from (seed, offset), bit for
    bit against the oracle.  Covers the tile edges of the row-wise (4 rows x 512 columns per task),
    column-wise (256 x 64 tiles) and 2-D (64 x 64 / 32 x 128 warp tiles) kernels."""
    from alto_b200 import mxfp4 as MX, mxfp8 as M8, nvfp4 as NV
    block = 16 if fmt == "nvfp4" else 32
    d = _dev()
    for i, (R, Cc) in enumerate(_sweep_shapes({"nvfp4": 1, "mxfp4": 2, "mxfp8": 3}[fmt], 10, block)):
        x = reference_data((R, Cc), torch.bfloat16, 500 + i)
        xd = x.to(d)
        x_all, xd_all, R_all = x, xd, R
        for axis, is2d in ((-1, False), (0, False), (-1, True), (0, True)):
            x, xd, R = x_all, xd_all, R_all
            if axis == 0 and not is2d and R % 32:
                # the token-axis quantizer writes 16-byte aligned output rows: 32 tokens per FP4 row
                if R < 48:
                    continue
                R = R - 16
                x, xd = x_all[:R].contiguous(), xd_all[:R].contiguous()
            tag = f"{fmt} {R}x{Cc} axis={axis} 2d={is2d}"
            if fmt == "nvfp4":
                outer = O.compute_dynamic_outer_scale(x)
                qo, so = O.quantize_nvfp4(x, 16, axis, is2d, outer)
                q, s = NV.convert_to_nvfp4(xd, axis=axis, is_2d_block=is2d, outer_scale=outer.to(d),
                                           update_outer_scale=False)
            elif fmt == "mxfp4":
                qo, so = O.quantize_mxfp4(x, 32, axis, is2d)
                q, s = MX.convert_to_mxfp4(xd, axis=axis, is_2d_block=is2d)
            else:
                qo, so = O.quantize_mxfp8(x, 32, "e4m3", axis, is2d)
                q, s = M8.convert_to_mxfp8(xd, mxfp_format="e4m3", axis=axis, is_2d_block=is2d)
            _same(s, so, tag + " scales")
            _same(q, qo, tag + " codes")
            if fmt == "mxfp8" or (is2d and axis == 0):
                continue
            seed, off = 1000 + i, 77 * i
            vr, vc = (R, Cc) if axis == -1 else (Cc, R)
            rp = O.reference_sr_planes(seed, off, vr, vc)
            if fmt == "nvfp4":
                qo, _ = O.quantize_nvfp4(x, 16, axis, is2d, outer, rp)
                q, _ = NV.convert_to_nvfp4(xd, axis=axis, is_2d_block=is2d, outer_scale=outer.to(d),
                                           update_outer_scale=False, use_sr=True, philox_seed=seed, philox_offset=off)
            else:
                qo, _ = O.quantize_mxfp4(x, 32, axis, is2d, rp)
                q, _ = MX.convert_to_mxfp4(xd, axis=axis, is_2d_block=is2d, use_sr=True, philox_seed=seed,
                                           philox_offset=off)
            _same(q, qo, tag + " SR codes")


@pytest.mark.parametrize("special", ["none", "nan", "inf", "huge"])
def test_hadamard_amax_equals_amax_of_the_materialised_transform(special):
    """One read of x yields the outer scales of x and of bf16(H x) (the wgrad operand): both equal
    ``compute_dynamic_outer_scale`` (alto/kernels/fp4/nvfp4/nvfp_quantization.py:460-487) of x and of the
    transform's own bf16 output bit for bit -- also when a NaN, an infinity (Inf - Inf inside the
    butterfly) or an overflowing sum makes the maximum non-finite."""
    from alto_b200 import _linear as E, nvfp4 as NV
    from alto_b200.hadamard import HadamardFactory
    d = _dev()
    g = torch.Generator(device=d).manual_seed(11)
    x = torch.randn(256, 192, generator=g, device=d).bfloat16()
    if special == "nan":
        x[37, 5] = float("nan")
    elif special == "inf":
        x[100, 64], x[101, 64] = float("inf"), float("-inf")
    elif special == "huge":
        x[32:48, 7] = 3.0e38
    HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=3)
    had = HadamardFactory.create_transform(device=d)
    assert had.is_fused
    got = E.outer_scales(x, True, had.device_params())
    hx = had(x, left_mul=True)
    assert hx.dtype == torch.bfloat16
    want = torch.cat([NV.compute_dynamic_outer_scale(x), NV.compute_dynamic_outer_scale(hx)])
    assert torch.equal(got, want), (got, want)
    # the reference's expression, evaluated on the CPU (a correctly rounded division; on a CUDA device
    # PyTorch evaluates tensor / python-scalar as a multiplication by the reciprocal, one ulp off at times)
    ref = [torch.nan_to_num(t.float().cpu().abs().max(), nan=0.0) / (448.0 * 6.0) for t in (x, hx)]
    ref = torch.stack([r.clamp(min=1e-30) for r in ref])
    assert torch.equal(want.cpu(), ref.to(torch.float32)), (want, ref)
