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
    with pytest.raises(NotImplementedError):
        G._quantize_then_mxfp_scaled_grouped_mm(x, B, offs, False, True, False, False, False, "none", True)
    with pytest.raises(NotImplementedError):
        G._quantize_then_nvfp4_scaled_grouped_mm(x, B, offs, False, True, False, use_dge=True)
