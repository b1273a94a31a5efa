"""MXFP4 quantizer options `clip_mode` (static / dynamic) and `use_uos`: the oracle against the
reference emulation's outputs (CPU) and the CUDA quantizers against both (GPU).  Scales and codes
are compared bit for bit, as the reference's own test does for every case generated here
(tests/unittest/mxfp4/test_mxfp_quantization.py:29-100); dynamic clipping with bf16 inputs is only
held to a mean dequantisation error there, and so it is here."""
import ast
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import alto_oracle as O
from tests.helpers import bits_equal, tensor_from_bits

_NPZ = Path(__file__).resolve().parent / "golden" / "mxfp4_options_vectors.npz"
_DT = {"torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}


def _cases():
    z = np.load(_NPZ, allow_pickle=False)
    for m in ast.literal_eval(str(z["meta"])):
        yield z, m


_IDS = lambda v: "-".join(str(t) for t in (v[0], v[5], "uos" if v[6] else "")) if isinstance(v, tuple) else ""  # noqa: E731


@pytest.mark.parametrize("z,m", list(_cases()), ids=_IDS)
def test_oracle_matches_reference_emulation(z, m):
    tag, shape, dt, axis, is2d, clip, uos = m
    x = tensor_from_bits(z[tag + "_x"], _DT[dt])
    q, s = O.quantize_mxfp4(x, 32, axis, is2d, None, clip, uos)
    assert bits_equal(s, z[tag + "_s"])
    assert bits_equal(q, z[tag + "_q"])
    for odt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        dq = O.dequantize_mxfp4(q, s, odt, 32, axis, is2d, clip)
        assert bits_equal(dq, z[tag + "_dq_" + name])


@pytest.mark.gpu
@pytest.mark.parametrize("z,m", list(_cases()), ids=_IDS)
def test_cuda_matches_reference_emulation(z, m):
    from alto_b200 import mxfp4 as MX
    tag, shape, dt, axis, is2d, clip, uos = m
    x = tensor_from_bits(z[tag + "_x"], _DT[dt]).cuda()
    q, s = MX.convert_to_mxfp4(x, axis=axis, is_2d_block=is2d, clip_mode=clip, use_uos=uos)
    assert bits_equal(s, z[tag + "_s"])
    assert bits_equal(q.view(torch.uint8), z[tag + "_q"])
    for odt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        dq = MX.convert_from_mxfp4(q, s, odt, axis=axis, is_2d_block=is2d, clip_mode=clip)
        assert bits_equal(dq, z[tag + "_dq_" + name])


@pytest.mark.gpu
def test_dynamic_clip_bf16_mean_error_and_refusals():
    from alto_b200 import mxfp4 as MX
    g = torch.Generator().manual_seed(2)
    x = torch.randn(128, 256, generator=g).bfloat16()
    q, s = MX.convert_to_mxfp4(x.cuda(), clip_mode="dynamic")
    qo, so = O.quantize_mxfp4(x, 32, -1, False, None, "dynamic", False)
    assert (s.cpu().int() - so.int()).abs().max().item() <= 1          # scale bytes may differ by one step
    dq = MX.convert_from_mxfp4(q, s, torch.bfloat16, clip_mode="dynamic").cpu()
    dqo = O.dequantize_mxfp4(qo, so, torch.bfloat16, 32, -1, False, "dynamic")
    assert (dq.float() - dqo.float()).abs().mean().item() < 0.5
    # 2-D blocks: the statistics run over the 32 x 32 tile
    q2, s2 = MX.convert_to_mxfp4(x.cuda(), is_2d_block=True, clip_mode="dynamic")
    q2o, s2o = O.quantize_mxfp4(x, 32, -1, True, None, "dynamic", False)
    assert (s2.cpu().int() - s2o.int()).abs().max().item() <= 1
    dq2 = MX.convert_from_mxfp4(q2, s2, torch.bfloat16, is_2d_block=True, clip_mode="dynamic").cpu()
    dq2o = O.dequantize_mxfp4(q2o, s2o, torch.bfloat16, 32, -1, True, "dynamic")
    assert (dq2.float() - dq2o.float()).abs().mean().item() < 0.5
    with pytest.raises(ValueError):
        MX.convert_to_mxfp4(x.cuda(), clip_mode="sometimes")


@pytest.mark.gpu
@pytest.mark.parametrize("clip,uos", [("static", False), ("none", True), ("static", True)])
def test_mxfp4_linear_with_options_matches_oracle(clip, uos):
    """The linear applies use_uos to every quantisation and clip_mode to the two token-axis (wgrad)
    operands, and rescales dW by 16/9 for the static clip (alto/kernels/fp4/mxfp4/mxfp_linear.py:
    301-411, 436-545)."""
    from alto_b200 import mxfp4 as MX
    M, K, N = 256, 512, 384
    g = torch.Generator().manual_seed(8)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    dy = torch.randn(M, N, generator=g).bfloat16()
    xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    y = MX._to_mxfp4_then_scaled_mm(xd, wd, False, True, False, False, clip, False, False, uos)
    y.backward(dy.cuda())

    def qdq(t, axis, is2d, c="none"):
        q, s = O.quantize_mxfp4(t, 32, axis, is2d, None, c, uos)
        return O.dequantize_mxfp4(q, s, torch.float32, 32, axis, is2d)   # codes x scale, no 4/3 factor

    yo = qdq(x, -1, False) @ qdq(w, -1, True).t()
    dxo = qdq(dy, -1, False) @ qdq(w, -1, True)
    dwo = qdq(dy, 0, False, clip).t() @ qdq(x, 0, False, clip)
    if clip == "static":
        dwo = dwo.bfloat16().float() * (16.0 / 9.0)

    def rel(a, b):
        return ((a.float().cpu() - b).norm() / b.norm()).item()

    assert rel(y, yo.bfloat16().float()) <= 1e-3
    assert rel(xd.grad, dxo.bfloat16().float()) <= 1e-3
    assert rel(wd.grad, dwo.bfloat16().float()) <= 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("grouped", [False, True])
def test_static_clip_with_2d_activation_blocks_leaves_the_weight_gradient_unscaled(grouped):
    """With use_2dblock_x the activations and gradients are quantised once in 32 x 32 blocks and no
    operand takes the clip mode (alto/kernels/fp4/mxfp4/mxfp_linear.py:310-315, 436-452), so the
    16/9 that undoes the static clip of the 1-D token-axis operands must not be applied to dW."""
    from alto_b200 import grouped as G
    from alto_b200 import mxfp4 as MX
    M, K, N = 256, 256, 128
    g = torch.Generator().manual_seed(9)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    dy = torch.randn(M, N, generator=g).bfloat16()
    xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    if grouped:
        offs = torch.tensor([M], dtype=torch.int32, device="cuda")
        B = wd.unsqueeze(0).transpose(-2, -1)
        y = G._quantize_then_mxfp_scaled_grouped_mm(xd, B, offs, True, True, False, False, False, "static", False)
    else:
        y = MX._to_mxfp4_then_scaled_mm(xd, wd, True, True, False, False, "static", False, False, False)
    y.backward(dy.cuda())

    def qdq(t):
        q, s = O.quantize_mxfp4(t, 32, -1, True)
        return O.dequantize_mxfp4(q, s, torch.float32, 32, -1, True)

    dwo = qdq(dy).t() @ qdq(x)
    rel = ((wd.grad.float().cpu() - dwo.bfloat16().float()).norm() / dwo.norm()).item()
    assert rel <= 1e-3, rel
