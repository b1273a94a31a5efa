"""GPU tests of the tcgen05 block-scaled GEMM and of the three linear autograd functions.

GEMM results are compared with the oracle's dequantize-then-fp32-matmul definition:
relative Frobenius error <= 1e-3 (the tolerance the task states); in practice the fp32-output
kernel agrees to ~1e-7 because products of FP4/FP8 codes and block scales are exact and only
the fp32 accumulation order differs."""
import numpy as np
import pytest
import torch

from oracle import alto_oracle as O
from tests.helpers import load_golden, rand_u32, reference_data

pytestmark = pytest.mark.gpu
REL_TOL = 1e-3


def _dev():
    return torch.device("cuda")


def _u32dev(r):
    return torch.from_numpy((r.numpy() & 0xFFFFFFFF).astype(np.uint32).view(np.int32)).to(_dev())


def _rel(got, exp):
    got = got.detach().float().cpu()
    return ((got - exp).norm() / exp.norm().clamp(min=1e-30)).item()


def _snr(got, ref):
    got = got.detach().float().cpu()
    ref = ref.float()
    return (10 * torch.log10(ref.pow(2).sum() / (got - ref).pow(2).sum().clamp(min=1e-30))).item()


# ------------------------------------------------------------------------------------------
# raw GEMM on synthetic codes and scales
# ------------------------------------------------------------------------------------------

def _operand(rows, K, kind, seed):
    """Random codes and scale bytes; returns (codes bytes [rows, K/2 or K], scale bytes [rows, K/block],
    dequantised fp32 [rows, K])."""
    g = torch.Generator().manual_seed(seed)
    if kind == "nvfp4":
        c = torch.randint(0, 16, (rows, K), generator=g, dtype=torch.uint8)
        sf = torch.randint(0x20, 0x48, (rows, K // 16), generator=g, dtype=torch.uint8)
        dq = O.e2m1_decode(c) * sf.view(torch.float8_e4m3fn).float().repeat_interleave(16, 1)
        return O.pack_nibbles(c), sf, dq
    if kind == "mxfp4":
        c = torch.randint(0, 16, (rows, K), generator=g, dtype=torch.uint8)
        sf = torch.randint(120, 134, (rows, K // 32), generator=g, dtype=torch.uint8)
        dq = O.e2m1_decode(c) * (sf.to(torch.int32) << 23).view(torch.float32).repeat_interleave(32, 1)
        return O.pack_nibbles(c), sf, dq
    dt = torch.float8_e4m3fn if kind == "e4m3" else torch.float8_e5m2
    v = (torch.randn(rows, K, generator=g) * 4).to(dt)
    sf = torch.randint(120, 134, (rows, K // 32), generator=g, dtype=torch.uint8)
    dq = v.float() * (sf.to(torch.int32) << 23).view(torch.float32).repeat_interleave(32, 1)
    return v.view(torch.uint8), sf, dq


_FMT = {"nvfp4": 0, "mxfp4": 1, "e4m3": 2, "e5m2": 3}


@pytest.mark.parametrize("kind", ["nvfp4", "mxfp4", "e4m3", "e5m2"])
@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 256, 1024), (256, 512, 2048), (160, 96, 512),
                                   (384, 640, 768), (2048, 2048, 2048), (512, 1024, 2880)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_matches_dequantised_fp32_matmul(kind, M, N, K, out_dtype):
    from alto_b200 import _lib as L
    if kind != "nvfp4" and K % 32:
        pytest.skip("K must be a multiple of the block")
    if out_dtype == torch.bfloat16 and (M, N, K) not in [(256, 512, 2048), (160, 96, 512)]:
        pytest.skip("bf16 output checked on two shapes")
    ac, asf, adq = _operand(M, K, kind, 1)
    bc, bsf, bdq = _operand(N, K, kind, 2)
    ref = O.gemm_nt_fp32(adq, bdq)
    d = _dev()
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=d)
    alpha = torch.tensor([0.5], device=d)
    L.gemm_blockscaled(_FMT[kind], _FMT[kind], M, N, K, ac.to(d), O.pack_scale_bytes(asf).to(d), bc.to(d),
                       O.pack_scale_bytes(bsf).to(d), out, alpha, None)
    st, detail = L.status_read()
    assert st == 0, f"device status {st} {detail}"
    ref = ref * 0.5
    if out_dtype == torch.bfloat16:
        ref = ref.bfloat16().float()
    assert not torch.isnan(out).any()
    assert _rel(out, ref) <= REL_TOL


def test_gemm_mixed_fp8_formats():
    """Forward operands E4M3 with E5M2 gradients (one operand of each format in a GEMM)."""
    from alto_b200 import _lib as L
    M, N, K = 256, 384, 1024
    ac, asf, adq = _operand(M, K, "e5m2", 3)
    bc, bsf, bdq = _operand(N, K, "e4m3", 4)
    d = _dev()
    out = torch.empty(M, N, dtype=torch.float32, device=d)
    L.gemm_blockscaled(3, 2, M, N, K, ac.to(d), O.pack_scale_bytes(asf).to(d), bc.to(d),
                       O.pack_scale_bytes(bsf).to(d), out)
    assert _rel(out, O.gemm_nt_fp32(adq, bdq)) <= REL_TOL


def test_gemm_rejects_bad_arguments():
    from alto_b200 import _lib as L
    d = _dev()
    a = torch.zeros(128, 64, dtype=torch.uint8, device=d)
    s = torch.zeros(512 * 2, dtype=torch.uint8, device=d)
    out = torch.empty(128, 128, dtype=torch.float32, device=d)
    with pytest.raises(L.Altob200Error) as e:
        L.gemm_blockscaled(0, 0, 128, 128, 144, a, s, a, s, out)  # K not a multiple of 32
    assert e.value.status == L.E_SHAPE
    with pytest.raises(L.Altob200Error) as e:
        L.gemm_blockscaled(0, 1, 128, 128, 128, a, s, a, s, out)  # NVFP4 x MXFP4
    assert e.value.status == L.E_UNSUPPORTED


def test_public_gemm_ops_with_plain_scales():
    """blockwise_mxfp4_gemm / blockwise_mxfp8_gemm take the reference's plain scale layouts."""
    from alto_b200 import mxfp4 as MX, mxfp8 as M8
    d = _dev()
    x = reference_data((256, 512), torch.bfloat16, 1).to(d)
    w = reference_data((384, 512), torch.bfloat16, 2).to(d)
    for is2d_w in (False, True):
        xq, xs = MX.convert_to_mxfp4(x)
        wq, ws = MX.convert_to_mxfp4(w, is_2d_block=is2d_w)
        y = MX.blockwise_mxfp4_gemm(xq, xs, wq, ws, trans_b=True, use_2dblock_b=is2d_w)
        ref = MX.convert_from_mxfp4(xq, xs).cpu() @ MX.convert_from_mxfp4(wq, ws, is_2d_block=is2d_w).cpu().t()
        assert _rel(y, ref) <= REL_TOL
        xq, xs = M8.convert_to_mxfp8(x)
        wq, ws = M8.convert_to_mxfp8(w, is_2d_block=is2d_w)
        y = M8.blockwise_mxfp8_gemm(xq, xs, wq, ws, trans_b=True, use_2dblock_b=is2d_w)
        ref = M8.convert_from_mxfp8(xq, xs).cpu() @ M8.convert_from_mxfp8(wq, ws, is_2d_block=is2d_w).cpu().t()
        assert _rel(y, ref) <= REL_TOL
    # wgrad form: both operands quantised along axis 0 (transposed views), trans_a
    g = reference_data((256, 384), torch.bfloat16, 3).to(d)
    gq, gs = M8.convert_to_mxfp8(g, axis=0)
    xq, xs = M8.convert_to_mxfp8(x, axis=0)
    dw = M8.blockwise_mxfp8_gemm(gq, gs, xq, xs, trans_a=True)
    ref = M8.convert_from_mxfp8(gq, gs, axis=0).cpu().t() @ M8.convert_from_mxfp8(xq, xs, axis=0).cpu()
    assert _rel(dw, ref) <= REL_TOL


# ------------------------------------------------------------------------------------------
# linear autograd functions against the oracle orchestration
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("M,K,N", [(256, 512, 384), (1024, 2048, 1536)])
@pytest.mark.parametrize("use_2dblock_w", [True, False])
def test_nvfp4_linear_matches_oracle(M, K, N, use_2dblock_w):
    """The recipe of the headline benchmark: 1D activations, tensorwise outer scale, 16-point
    randomised Hadamard on the wgrad operands, stochastic rounding of gradients from explicit
    random bits.  fp32 inputs make the function return fp32, so the comparison is not limited by
    the bf16 rounding of the outputs."""
    from alto_b200 import nvfp4 as NV
    NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
    g = torch.Generator().manual_seed(0)
    W, perm, sign = O.random_hadamard(16, g)
    x = reference_data((M, K), torch.float32, 21, outliers=False).bfloat16().float()
    w = (reference_data((N, K), torch.float32, 22, outliers=False) * 0.02).bfloat16().float()
    dy = (reference_data((M, N), torch.float32, 23, outliers=False) * 1e-3).bfloat16().float()
    rn, rm = rand_u32((2, M, N // 2), 31), rand_u32((2, N, M // 2), 32)
    # bf16-valued inputs keep the Hadamard sums exact, so the oracle's dot products and the
    # kernel's butterfly agree bit for bit and every operand is identical on both sides
    yo, dxo, dwo = O.nvfp4_linear(x.bfloat16(), w.bfloat16(), dy.bfloat16(), use_2dblock_w=use_2dblock_w, W_had=W,
                                  rand_dy_n=rn, rand_dy_m=rm)
    d = _dev()
    xd = x.bfloat16().to(d).requires_grad_(True)
    wd = w.bfloat16().to(d).requires_grad_(True)
    bits = {"dy_n": _u32dev(rn), "dy_m": _u32dev(rm)}
    with NV.explicit_sr_bits(lambda name, shape, dev: bits[name]):
        y = NV._to_nvfp4_then_scaled_mm(xd, wd, False, use_2dblock_w, True, use_outer_scale=True, use_hadamard=True)
        y.backward(dy.bfloat16().to(d))
    # outputs are bf16: compare with the oracle rounded the same way
    assert _rel(y, yo.bfloat16().float()) <= REL_TOL
    assert _rel(xd.grad, dxo.bfloat16().float()) <= REL_TOL
    assert _rel(wd.grad, dwo.bfloat16().float()) <= REL_TOL


def test_nvfp4_linear_with_default_hadamard_size_32():
    """The reference's default HadamardFactory block size is 32, whose table matrix is not of
    Sylvester type: the rotation runs as the dense kernel and materialises bf16(H x) like the
    reference; everything downstream is identical to the oracle's operands."""
    from alto_b200 import nvfp4 as NV
    M, K, N = 256, 512, 384
    NV.HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)
    try:
        z, _ = load_golden()
        W = torch.from_numpy(z["rht32_W"])
        x = reference_data((M, K), torch.float32, 41, outliers=False).bfloat16()
        w = (reference_data((N, K), torch.float32, 42, outliers=False) * 0.02).bfloat16()
        dy = (reference_data((M, N), torch.float32, 43, outliers=False) * 1e-3).bfloat16()
        rn, rm = rand_u32((2, M, N // 2), 51), rand_u32((2, N, M // 2), 52)
        yo, dxo, dwo = O.nvfp4_linear(x, w, dy, use_2dblock_w=True, W_had=W, rand_dy_n=rn, rand_dy_m=rm)
        d = _dev()
        xd = x.to(d).requires_grad_(True)
        wd = w.to(d).requires_grad_(True)
        bits = {"dy_n": _u32dev(rn), "dy_m": _u32dev(rm)}
        with NV.explicit_sr_bits(lambda name, shape, dev: bits[name]):
            y = NV._to_nvfp4_then_scaled_mm(xd, wd, False, True, True, use_outer_scale=True, use_hadamard=True)
            y.backward(dy.to(d))
        assert _rel(y, yo.bfloat16().float()) <= REL_TOL
        assert _rel(xd.grad, dxo.bfloat16().float()) <= REL_TOL
        assert _rel(wd.grad, dwo.bfloat16().float()) <= REL_TOL
    finally:
        NV.HadamardFactory.configure(block_size=16)


@pytest.mark.parametrize("scheme", ["nvfp4", "mxfp4", "mxfp8_e4m3", "mxfp8_e5m2"])
def test_linear_snr_against_high_precision(scheme):
    """SNR floors of the reference's own autograd tests (tests/unittest/mxfp4/test_mxfp_linear.py:189-197,
    tests/unittest/mxfp8/test_mxfp8_linear.py:177-186, alto/kernels/fp4/testing_utils.py:53-103)."""
    from alto_b200 import mxfp4 as MX, mxfp8 as M8, nvfp4 as NV
    M, K, N = 512, 1024, 768
    d = _dev()
    torch.manual_seed(0)
    x = torch.randn(M, K, device=d, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, K, device=d, dtype=torch.bfloat16) * 0.05).requires_grad_(True)
    dy = torch.randn(M, N, device=d, dtype=torch.bfloat16)
    NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
    if scheme == "nvfp4":
        y = NV._to_nvfp4_then_scaled_mm(x, w, False, True, False, use_outer_scale=True, use_hadamard=True)
        floors = (12.0, 12.0, 12.0)
    elif scheme == "mxfp4":
        y = MX._to_mxfp4_then_scaled_mm(x, w, False, True, False, False, "none", True)
        floors = (8.4, 8.4, 8.4)
    else:
        v = scheme.split("_")[1]
        y = M8._to_mxfp8_then_scaled_mm(x, w, v, False, False, True)
        floors = (24.0, 15.0, 15.0) if v == "e4m3" else (19.0, 12.0, 12.0)
    y.backward(dy)
    xf, wf, dyf = x.detach().float().cpu(), w.detach().float().cpu(), dy.float().cpu()
    assert _snr(y, xf @ wf.t()) > floors[0]
    assert _snr(x.grad, dyf @ wf) > floors[1]
    assert _snr(w.grad, dyf.t() @ xf) > floors[2]


@pytest.mark.parametrize("scheme", ["nvfp4", "mxfp4"])
def test_dge_scales_the_weight_gradient_like_the_reference(scheme):
    """use_dge multiplies dW by dge_bwd(FP4 bin values of W) (alto/kernels/dge/dge.py:81-93;
    alto/kernels/fp4/nvfp4/nvfp_linear.py:250-268).  On bin values the reference's formula gives one
    number, 1/k = 0.2, for all sixteen codes; dX and Y are untouched."""
    from alto_b200 import dge, mxfp4 as MX, nvfp4 as NV
    d = _dev()
    table = dge.fp4_bin_table(d, torch.bfloat16)
    assert len(table) == 16 and all(abs(t - 0.2) < 1e-6 for t in table)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(128, 256, generator=g).bfloat16().to(d)
    w = (torch.randn(192, 256, generator=g) * 0.05).bfloat16().to(d)
    dy = torch.randn(128, 192, generator=g).bfloat16().to(d)
    outs = []
    for use_dge in (False, True):
        xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        if scheme == "nvfp4":
            y = NV._to_nvfp4_then_scaled_mm(xd, wd, False, True, False, use_outer_scale=True, use_dge=use_dge)
        else:
            y = MX._to_mxfp4_then_scaled_mm(xd, wd, False, True, False, use_dge, "none", False)
        y.backward(dy)
        outs.append((y.detach(), xd.grad, wd.grad))
    (y0, dx0, dw0), (y1, dx1, dw1) = outs
    assert torch.equal(y0, y1) and torch.equal(dx0, dx1)
    # the reference's expression with tensor ops on this device: decode W's codes with unit scales in
    # the gradient's dtype, dge_bwd on them, multiply
    if scheme == "nvfp4":
        q, _ = NV.convert_to_nvfp4(w, is_2d_block=True, outer_scale=NV.compute_dynamic_outer_scale(w))
    else:
        q, _ = MX.convert_to_mxfp4(w, is_2d_block=True)
    codes = q.view(torch.uint8)
    nib = torch.stack((codes & 0xF, codes >> 4), dim=-1).reshape(codes.shape[0], -1).long()
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], device=d)
    w_fp4_values = lut[nib].to(torch.bfloat16)
    want = (dw0 * dge.dge_bwd_fp4(w_fp4_values)).to(torch.bfloat16)
    assert torch.equal(dw1, want)


def test_linear_shape_contracts():
    from alto_b200 import nvfp4 as NV
    d = _dev()
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device=d)
    with pytest.raises(RuntimeError):
        NV._to_nvfp4_then_scaled_mm(torch.zeros(24, 64, dtype=torch.bfloat16, device=d), w, False, True, False)
    with pytest.raises(NotImplementedError):
        NV._to_nvfp4_then_scaled_mm(torch.zeros(32, 64, dtype=torch.bfloat16, device=d), w, False, True, False,
                                    scale_format="ue5m3")
    x3 = torch.randn(2, 32, 64, dtype=torch.bfloat16, device=d)
    y = NV._to_nvfp4_then_scaled_mm(x3, w, False, True, False)
    assert y.shape == (2, 32, 64) and y.dtype == torch.bfloat16


def test_nvfp4_linear_2d_activation_blocks_with_stochastic_rounding():
    """`use_2dblock_x=True` with `use_sr_grad=True`: the gradient is quantised once in 16 x 16 blocks
    with stochastic rounding and feeds both backward GEMMs (alto/kernels/fp4/nvfp4/nvfp_linear.py:176-186)."""
    from alto_b200 import nvfp4 as NV
    M, K, N = 256, 512, 384
    x = reference_data((M, K), torch.float32, 61, outliers=False).bfloat16()
    w = (reference_data((N, K), torch.float32, 62, outliers=False) * 0.02).bfloat16()
    dy = (reference_data((M, N), torch.float32, 63, outliers=False) * 1e-3).bfloat16()
    rn = rand_u32((2, M, N // 2), 64)
    yo, dxo, dwo = O.nvfp4_linear(x, w, dy, use_2dblock_x=True, use_2dblock_w=True, rand_dy_n=rn)
    d = _dev()
    xd, wd = x.to(d).requires_grad_(True), w.to(d).requires_grad_(True)
    with NV.explicit_sr_bits(lambda name, shape, dev: {"dy_n": _u32dev(rn)}[name]):
        y = NV._to_nvfp4_then_scaled_mm(xd, wd, True, True, True, use_outer_scale=True)
        y.backward(dy.to(d))
    assert _rel(y, yo.bfloat16().float()) <= REL_TOL
    assert _rel(xd.grad, dxo.bfloat16().float()) <= REL_TOL
    assert _rel(wd.grad, dwo.bfloat16().float()) <= REL_TOL
    # and it differs from round-to-nearest
    x2, w2 = x.to(d).requires_grad_(True), w.to(d).requires_grad_(True)
    NV._to_nvfp4_then_scaled_mm(x2, w2, True, True, False, use_outer_scale=True).backward(dy.to(d))
    assert not torch.equal(x2.grad, xd.grad)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(4224, 5792, 384), (2176, 2912, 256)])
def test_gemm_ragged_tiles_over_many_waves(M, N, K, out_dtype):
    """Output extents that end inside a tile (rows inside a 256-row CTA-pair tile, columns inside a
    256-column tile and inside a 64-column store unit) with a short K, so that every CTA runs many
    store-heavy tiles back to back: the shape class in which a skipped store unit once let a staging
    buffer be refilled under a store in flight.  Checked on the device against an fp32 matmul of the
    dequantised operands, twice (the failure was a race)."""
    from alto_b200 import _lib as L
    ac, asf, adq = _operand(M, K, "nvfp4", 11)
    bc, bsf, bdq = _operand(N, K, "nvfp4", 12)
    d = _dev()
    ref = adq.to(d) @ bdq.to(d).t()
    if out_dtype == torch.bfloat16:
        ref = ref.bfloat16().float()
    args = (ac.to(d), O.pack_scale_bytes(asf).to(d), bc.to(d), O.pack_scale_bytes(bsf).to(d))
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=d)
        L.gemm_blockscaled(0, 0, M, N, K, *args, out, None, None)
        assert not torch.isnan(out).any()
        # fp32: accumulation order only; bf16: at most one unit in the last place of the rounded output
        diff = (out.float() - ref).abs()
        tol = 1e-5 * ref.abs().max() if out_dtype == torch.float32 else ref.abs() * 2.0 ** -7 + 1e-30
        bad = diff > tol
        assert int(bad.sum()) == 0, f"{int(bad.sum())} entries differ, first at {torch.nonzero(bad)[:4].tolist()}"


def test_bounded_device_wait_times_out_and_is_reported():
    """Failure detection without a fault: a kernel whose only wait can never be satisfied (an mbarrier
    nobody arrives on) gives up after its limit, leaves through its normal exit, and the status word
    reports ETIMEOUT with {kernel, block, site}; the word is sticky until read, then clear; the
    context stays usable."""
    from alto_b200 import _lib as L
    st, _ = L.status_read()
    assert st == 0
    L.selftest_wait_timeout(1_000_000)          # 1 ms
    st, detail = L.status_read()
    assert st == L.E_TIMEOUT, (st, detail)
    assert detail[:3] == [9, 0, 99]
    assert "wait" in L.status_string(st) or "time" in L.status_string(st).lower()
    st, detail = L.status_read()
    assert st == 0 and detail[:3] == [0, 0, 0]
    # the context is intact: a real GEMM still runs and the limit can be changed and restored
    L.set_wait_limit_ns(2_000_000_000)
    a = torch.randn(128, 128, device="cuda").bfloat16()
    from alto_b200 import mxfp4 as MX
    y = MX._to_mxfp4_then_scaled_mm(a, a, False, True, False, False, "none", False)
    assert torch.isfinite(y.float()).all()
    L.set_wait_limit_ns(4_000_000_000)
    assert L.status_read()[0] == 0
    with pytest.raises(L.Altob200Error):
        L.selftest_wait_timeout(5_000_000_000)  # limits above one second are refused


def test_pair_tile_of_192_columns_with_two_accumulator_stages():
    """The CTA-pair kernel also exists with a 256 x 192 tile and two accumulator stages (scale columns of
    B then start at word 0 or word 2 of a 128-row block, 64-byte store rows for bf16).  It is slower
    than the 256 x 256 tile on every measured shape and is not the default; ALTOB200_PAIR_BN=192 selects
    it when the library is loaded, so the raw-GEMM and ragged-tile cases are re-run in a child process."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, ALTOB200_PAIR_BN="192")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_gemm.py", "-q", "-x", "-m", "gpu", "-k",
                        "matches_dequantised_fp32_matmul or ragged_tiles or mixed_fp8"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout


def test_plain_launches_give_the_same_results():
    """Kernels are normally launched with programmatic stream serialisation (each waits for its
    predecessor when it first touches global memory); ALTOB200_PDL=0 launches them the plain way.  The
    linear and quantizer parity cases are re-run that way in a child process."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, ALTOB200_PDL="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_gemm.py", "tests/test_gpu_quantizers.py", "-q", "-x",
                        "-m", "gpu", "-k", "linear_matches_oracle or rowwise or colwise or ragged_tiles"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
