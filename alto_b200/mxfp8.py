"""MXFP8 quantizers, block-scaled GEMM and the MXFP8 linear on B200.

Public surface mirrors the reference:
  convert_to_mxfp8 / convert_from_mxfp8 / calculate_mxfp8_scales
      (alto/kernels/mxfp8/mxfp8_quantization.py:483-857)
  blockwise_mxfp8_gemm / MXFP8LinearFunction / _to_mxfp8_then_scaled_mm
      (alto/kernels/mxfp8/mxfp8_linear.py:153-456)
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L
from . import _linear as E
from . import _quant as Q
from .nvfp4 import unwrap_weight_wrapper

BLOCK_SIZE_DEFAULT = 32
SUPPORTED_FORMATS = ["e4m3", "e5m2"]
FORMAT_TO_TARGET_MAX = {"e4m3": 8, "e5m2": 15}
FORMAT_TO_MBITS = {"e4m3": 3, "e5m2": 2}
_FMT = {"e4m3": L.FMT_MXFP8_E4M3, "e5m2": L.FMT_MXFP8_E5M2}
_FMT_OF_DTYPE = {torch.float8_e4m3fn: L.FMT_MXFP8_E4M3, torch.float8_e5m2: L.FMT_MXFP8_E5M2}


@L.traced("convert_to_mxfp8")
def convert_to_mxfp8(
    data_hp: torch.Tensor,
    block_size: int = BLOCK_SIZE_DEFAULT,
    mxfp_format: str = "e4m3",
    axis: int = -1,
    is_2d_block: bool = False,
    use_sr: bool = False,
    use_asm: Optional[bool] = None,
    philox_seed: Optional[int] = None,
    philox_offset: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    torch._check(data_hp.shape[axis] % block_size == 0,
                 lambda: f"tensor shape ({data_hp.shape}) at axis={axis} is not divisible by {block_size}")
    assert mxfp_format in SUPPORTED_FORMATS, f"Unsupported format: {mxfp_format}. Supported: {SUPPORTED_FORMATS}"
    assert data_hp.dtype in [torch.float32, torch.bfloat16]
    assert block_size == BLOCK_SIZE_DEFAULT, f"MXFP8 kernels are built for block_size 32, got {block_size}"
    # the reference offers stochastic rounding for MXFP8 only through gfx950 instructions
    assert not use_sr, "use_sr=True requires use_asm=True (CDNA4 only); MXFP8 stochastic rounding is not available"
    if is_2d_block:
        torch._check(data_hp.shape[-2] % block_size == 0 and data_hp.shape[-1] % block_size == 0,
                     lambda: f"tensor shape ({data_hp.shape}) is not divisible by {block_size} for 2D block")
    return Q.quantize(data_hp, _FMT[mxfp_format], axis, is_2d_block)


def convert_from_mxfp8(
    data_lp: torch.Tensor,
    scales: torch.Tensor,
    output_dtype: torch.dtype = torch.float32,
    block_size: int = BLOCK_SIZE_DEFAULT,
    axis: int = -1,
    is_2d_block: bool = False,
    use_asm: Optional[bool] = None,
) -> torch.Tensor:
    assert output_dtype in [torch.float32, torch.bfloat16]
    assert block_size == BLOCK_SIZE_DEFAULT
    if data_lp.dtype not in _FMT_OF_DTYPE:
        raise ValueError(f"Unsupported FP8 dtype: {data_lp.dtype}")
    return Q.dequantize(data_lp, scales, _FMT_OF_DTYPE[data_lp.dtype], axis, is_2d_block, output_dtype)


def calculate_mxfp8_scales(
    data_hp: torch.Tensor,
    block_size: int = BLOCK_SIZE_DEFAULT,
    mxfp_format: str = "e4m3",
    axis: int = -1,
    is_2d_block: bool = False,
) -> torch.Tensor:
    """Block scales alone (the quantizer kernel computes them together with the codes)."""
    return convert_to_mxfp8(data_hp, block_size, mxfp_format, axis, is_2d_block)[1]


def blockwise_mxfp8_gemm(
    a: torch.Tensor,
    a_s: torch.Tensor,
    b: torch.Tensor,
    b_s: torch.Tensor,
    trans_a: bool = False,
    trans_b: bool = False,
    use_2dblock_a: bool = False,
    use_2dblock_b: bool = False,
    block_size: int = BLOCK_SIZE_DEFAULT,
    output_dtype: torch.dtype = torch.float32,
    use_dot_scaled: Optional[bool] = None,
    debug_print: bool = False,
) -> torch.Tensor:
    """C = A @ B with per-block E8M0 scales; scale layouts as in the reference
    (A: [M, K/32] or [K/32, M] with trans_a; B: [N, K/32] with trans_b or [K/32, N])."""
    assert a.dim() == 2 and b.dim() == 2
    if a.dtype != b.dtype:
        raise ValueError(f"A/B FP8 dtypes must match, got a.dtype={a.dtype}, b.dtype={b.dtype}")
    if a.dtype not in _FMT_OF_DTYPE:
        raise ValueError(f"Unsupported FP8 dtype: {a.dtype}")
    fmt = _FMT_OF_DTYPE[a.dtype]
    am = a.t() if trans_a else a
    bn = b if trans_b else b.t()
    asm_ = a_s.t() if trans_a else a_s
    bsn = b_s if trans_b else b_s.t()
    M, K = am.shape
    N = bn.shape[0]
    if K % block_size != 0:
        raise ValueError(f"K={K} must be divisible by block_size={block_size}")
    if bn.shape[1] != K:
        raise ValueError(f"inner dimensions differ: {K} vs {bn.shape[1]}")
    am, bn = E.as_2d_rows(am.view(torch.uint8)), E.as_2d_rows(bn.view(torch.uint8))
    sa = E.pack_plain_scales(asm_, M, use_2dblock_a, block_size)
    sb = E.pack_plain_scales(bsn, N, use_2dblock_b, block_size)
    out = torch.empty(M, N, dtype=output_dtype, device=a.device)
    L.gemm_blockscaled(fmt, fmt, M, N, K, am, sa, bn, sb, out)
    return out


class MXFP8LinearFunction(torch.autograd.Function):
    """Same argument list as the reference (alto/kernels/mxfp8/mxfp8_linear.py:305-314): one
    ``fp8_variant`` for all six operands."""

    @staticmethod
    def forward(ctx, x, weight, fp8_variant: str = "e4m3", use_sr_grad: bool = False,
                use_2dblock_x: bool = False, use_2dblock_w: bool = False):
        weight = unwrap_weight_wrapper(weight)
        if fp8_variant not in SUPPORTED_FORMATS:
            raise ValueError(f"Unsupported FP8 variant: {fp8_variant}. Supported: {SUPPORTED_FORMATS}")
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"x dtype must be float32/bfloat16, got {x.dtype}")
        if weight.dtype != x.dtype:
            raise ValueError(f"weight dtype ({weight.dtype}) must match x dtype ({x.dtype})")
        if use_sr_grad:
            raise NotImplementedError("MXFP8 stochastic rounding exists only as gfx950 instructions in the reference")
        return E.linear_forward(ctx, "MXFP8LinearFunction", x, weight, _FMT[fp8_variant],
                                use_2dblock_x=use_2dblock_x, use_2dblock_w=use_2dblock_w, use_sr_grad=False,
                                use_outer_scale=False, hadamard_transform=None)

    @staticmethod
    def backward(ctx, grad_output):
        gi, gw = E.linear_backward(ctx, grad_output)
        return gi, gw, None, None, None, None


@L.traced("mxfp8_linear")
def _to_mxfp8_then_scaled_mm(
    a: torch.Tensor,
    b: torch.Tensor,
    fp8_variant: str = "e4m3",
    use_sr_grad: bool = False,
    use_2dblock_x: bool = False,
    use_2dblock_w: bool = False,
) -> torch.Tensor:
    return MXFP8LinearFunction.apply(a, b, fp8_variant, use_sr_grad, use_2dblock_x, use_2dblock_w)
