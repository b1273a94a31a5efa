"""torch.ops registration of the quantizer / GEMM ops: the ops exist and their shape functions give
the reference's output shapes and dtypes (checked on meta tensors; no kernel runs).  Reference:
``register_fake`` functions next to each triton_op, e.g. alto/kernels/fp4/mxfp4/mxfp_quantization.py:548-585."""
import pytest
import torch

from alto_b200 import torch_ops


@pytest.fixture(scope="module", autouse=True)
def _registered():
    torch_ops.register()
    torch_ops.register()  # idempotent


def _meta(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, dtype=dtype, device="meta")


@pytest.mark.parametrize("axis,is2d,cshape,sshape", [(-1, False, (64, 64), (64, 4)), (0, False, (32, 128), (2, 128)),
                                                     (-1, True, (64, 64), (2, 4))])
def test_mxfp4_shapes(axis, is2d, cshape, sshape):
    ops = torch.ops.alto_b200
    x = _meta(64, 128)
    q, s = ops.convert_to_mxfp4(x, axis=axis, is_2d_block=is2d)
    assert tuple(q.shape) == cshape and q.dtype == torch.uint8
    assert tuple(s.shape) == sshape and s.dtype == torch.uint8
    dq = ops.convert_from_mxfp4(q, s, torch.bfloat16, axis=axis, is_2d_block=is2d)
    assert tuple(dq.shape) == (64, 128) and dq.dtype == torch.bfloat16


def test_nvfp4_and_mxfp8_shapes():
    ops = torch.ops.alto_b200
    x = _meta(2, 64, 128)
    q, s = ops.convert_to_nvfp4(x, axis=-2)
    assert tuple(q.shape) == (2, 32, 128) and tuple(s.shape) == (2, 4, 128) and s.dtype == torch.float32
    assert tuple(ops.convert_from_nvfp4(q, s, axis=-2).shape) == (2, 64, 128)
    q, s = ops.convert_to_mxfp8(x, mxfp_format="e5m2")
    assert q.dtype == torch.float8_e5m2 and tuple(q.shape) == (2, 64, 128) and tuple(s.shape) == (2, 64, 4)
    assert ops.convert_from_mxfp8(q, s, torch.bfloat16).dtype == torch.bfloat16
    assert tuple(ops.calculate_mxfp8_scales(x, is_2d_block=True).shape) == (2, 2, 4)


def test_gemm_shapes():
    ops = torch.ops.alto_b200
    a, a_s = _meta(96, 64, dtype=torch.uint8), _meta(96, 4, dtype=torch.uint8)
    b, b_s = _meta(160, 64, dtype=torch.uint8), _meta(160, 4, dtype=torch.uint8)
    assert tuple(ops.blockwise_mxfp4_gemm(a, a_s, b, b_s, trans_b=True).shape) == (96, 160)
    assert tuple(ops.blockwise_mxfp4_gemm(a, a_s, b.t(), b_s.t()).shape) == (96, 160)
    out = ops.blockwise_mxfp8_gemm(a.t(), a_s.t(), b.t(), b_s.t(), trans_a=True, output_dtype=torch.bfloat16)
    assert tuple(out.shape) == (96, 160) and out.dtype == torch.bfloat16   # a given as [K, M], b as [K, N]


def test_grouped_forward_shapes():
    ops = torch.ops.alto_b200
    x, xs = _meta(384, 64, dtype=torch.uint8), _meta(384, 4, dtype=torch.uint8)
    w, ws = _meta(4, 160, 64, dtype=torch.uint8), _meta(4, 5, 4, dtype=torch.uint8)
    idx = _meta(256, dtype=torch.int32)
    out = ops.mxfp4_grouped_gemm_forward(x, w, idx, xs, ws)
    assert tuple(out.shape) == (384, 160) and out.dtype == torch.bfloat16
    out = ops.mxfp4_grouped_gemm_forward(x, w.transpose(-2, -1), idx, xs, ws.transpose(-2, -1), trans_weights=False)
    assert tuple(out.shape) == (384, 160)
    x8, w8 = _meta(384, 128, dtype=torch.float8_e4m3fn), _meta(4, 160, 128, dtype=torch.float8_e4m3fn)
    out = ops.mxfp8_grouped_gemm_forward(x8, w8, idx, xs, ws, output_dtype=torch.float32)
    assert tuple(out.shape) == (384, 160) and out.dtype == torch.float32


def test_grouped_backward_shapes():
    ops = torch.ops.alto_b200
    idx = _meta(256, dtype=torch.int32)
    go8, x8 = _meta(384, 160, dtype=torch.float8_e4m3fn), _meta(384, 128, dtype=torch.float8_e4m3fn)
    w8 = _meta(4, 160, 128, dtype=torch.float8_e4m3fn)
    out = ops.mxfp8_grouped_gemm_backward_inputs(go8, w8, idx, _meta(384, 5, dtype=torch.uint8),
                                                 _meta(4, 5, 4, dtype=torch.uint8))
    assert tuple(out.shape) == (384, 128) and out.dtype == torch.bfloat16
    out = ops.mxfp8_grouped_gemm_backward_weights(go8, x8, idx, 4, _meta(12, 160, dtype=torch.uint8),
                                                  _meta(12, 128, dtype=torch.uint8))
    assert tuple(out.shape) == (4, 160, 128)
    out = ops.mxfp8_grouped_gemm_backward_weights(go8, x8, idx, 4, _meta(12, 160, dtype=torch.uint8),
                                                  _meta(12, 128, dtype=torch.uint8), trans_weights=False)
    assert tuple(out.shape) == (4, 128, 160)
    go4, w4 = _meta(384, 80, dtype=torch.uint8), _meta(4, 80, 128, dtype=torch.uint8)    # packed along N
    out = ops.mxfp4_grouped_gemm_backward_inputs(go4, w4, idx, _meta(384, 5, dtype=torch.uint8),
                                                 _meta(4, 5, 4, dtype=torch.uint8))
    assert tuple(out.shape) == (384, 128)
    gom, xm = _meta(192, 160, dtype=torch.uint8), _meta(192, 128, dtype=torch.uint8)      # packed along tokens
    out = ops.mxfp4_grouped_gemm_backward_weights(gom, xm, idx, 4, _meta(12, 160, dtype=torch.uint8),
                                                  _meta(12, 128, dtype=torch.uint8), use_2dblock_x=False)
    assert tuple(out.shape) == (4, 160, 128)


def test_ops_refuse_cpu_tensors():
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        torch.ops.alto_b200.convert_to_mxfp4(torch.zeros(32, 32, dtype=torch.bfloat16))
