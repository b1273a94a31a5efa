"""MXFP4 quantizers, block-scaled GEMM and the MXFP4 linear on B200.

Public surface mirrors the reference:
  convert_to_mxfp4 / convert_from_mxfp4  (alto/kernels/fp4/mxfp4/mxfp_quantization.py:411-545)
  blockwise_mxfp4_gemm                   (alto/kernels/fp4/mxfp4/mxfp_linear.py:143-255)
  MXFP4LinearFunction / _to_mxfp4_then_scaled_mm (alto/kernels/fp4/mxfp4/mxfp_linear.py:259-602)
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L
from . import _linear as E
from . import _quant as Q
from . import _two_level as T
from .hadamard import HadamardFactory, HadamardTransform
from .macro_block_scaling import macro_block_descaling, macro_block_scaling
from .nvfp4 import unwrap_weight_wrapper

BLOCK_SIZE_DEFAULT = 32


def _check_options(clip_mode: str, use_uos: bool, is_2d_block: bool = False) -> None:
    if clip_mode not in ("none", "static", "dynamic"):
        raise ValueError(f"Invalid clip mode: {clip_mode}")


@L.traced("convert_to_mxfp4")
def convert_to_mxfp4(
    data_hp: torch.Tensor,
    block_size: int = BLOCK_SIZE_DEFAULT,
    axis: int = -1,
    is_2d_block: bool = False,
    use_sr: bool = False,
    use_asm: Optional[bool] = None,
    philox_seed: Optional[int] = None,
    philox_offset: Optional[int] = None,
    clip_mode: str = "none",
    use_uos: bool = False,
    rand_bits: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """E2M1 codes packed two per byte along ``axis`` plus one E8M0 exponent per 32 elements
    (or per 32x32 tile).  ``rand_bits`` (extension): explicit random words for ``use_sr``."""
    torch._check(data_hp.shape[axis] % block_size == 0)
    assert not is_2d_block or data_hp.size(-2) % block_size == 0
    assert data_hp.dtype in [torch.float32, torch.bfloat16]
    assert block_size == BLOCK_SIZE_DEFAULT, f"MXFP4 kernels are built for block_size 32, got {block_size}"
    _check_options(clip_mode, use_uos, is_2d_block)
    rounding, philox = L.ROUND_RTN, (0, 0)
    if use_sr:
        if rand_bits is not None:
            rounding = L.ROUND_SR_BITS
        else:
            rounding = L.ROUND_SR_PHILOX
            drawn = E.draw_philox()
            philox = (drawn[0] if philox_seed is None else philox_seed,
                      drawn[1] if philox_offset is None else philox_offset)
    return Q.quantize(data_hp, L.FMT_MXFP4, axis, is_2d_block, rounding=rounding,
                      rand_bits=rand_bits if use_sr else None, philox=philox, clip_mode=clip_mode, use_uos=use_uos)


def convert_from_mxfp4(
    data_lp: torch.Tensor,
    scales: torch.Tensor,
    output_dtype: torch.dtype = torch.float32,
    block_size: int = BLOCK_SIZE_DEFAULT,
    axis: int = -1,
    is_2d_block: bool = False,
    use_asm: Optional[bool] = None,
    clip_mode: str = "none",
) -> torch.Tensor:
    assert output_dtype in [torch.float32, torch.bfloat16]
    assert block_size == BLOCK_SIZE_DEFAULT
    _check_options(clip_mode, False)
    return Q.dequantize(data_lp, scales, L.FMT_MXFP4, axis, is_2d_block, output_dtype,
                        static_clip=clip_mode == "static")


def blockwise_mxfp4_gemm(
    a: torch.Tensor,
    a_s: torch.Tensor,
    b: torch.Tensor,
    b_s: torch.Tensor,
    use_2dblock_a: bool = False,
    use_2dblock_b: bool = False,
    k_pack_a: bool = True,
    k_pack_b: bool = True,
    trans_a: bool = False,
    trans_b: bool = False,
    block_size: int = BLOCK_SIZE_DEFAULT,
    output_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """C = A @ B over packed E2M1 operands with E8M0 block scales.

    ``a`` is [M, K/2] (or, with ``trans_a``, the [K/2, M] transposed view an axis-0 quantisation
    returns); ``b`` is [K/2, N] as a view of a K-contiguous [N, K/2] tensor (``trans_b`` gives it
    as [N, K/2] directly).  Both operands must be packed along K: the tensor cores read FP4
    operands with the reduction axis contiguous."""
    if not (k_pack_a and k_pack_b):
        raise NotImplementedError("operands packed along a non-reduction axis cannot feed the tcgen05 FP4 MMA; "
                                  "quantise with is_2d_block=True and take the K-packed copy instead")
    am = a.t() if trans_a else a              # [M, K/2]
    bn = b if trans_b else b.t()              # [N, K/2]
    asm_ = a_s.t() if trans_a else a_s        # [M or M/32, K/32]
    bsn = b_s if trans_b else b_s.t()         # [N or N/32, K/32]
    M, N, K = am.shape[0], bn.shape[0], am.shape[1] * 2
    assert bn.shape[1] * 2 == K, "inner dimensions differ"
    am, bn = E.as_2d_rows(am.view(torch.uint8)), E.as_2d_rows(bn.view(torch.uint8))
    sa = E.pack_plain_scales(asm_, M, use_2dblock_a, block_size)
    sb = E.pack_plain_scales(bsn, N, use_2dblock_b, block_size)
    out = torch.empty(M, N, dtype=output_dtype, device=a.device)
    L.gemm_blockscaled(L.FMT_MXFP4, L.FMT_MXFP4, M, N, K, am, sa, bn, sb, out)
    return out


def _macro_qdq(t: torch.Tensor, axis: int, is_2d: bool, use_sr: bool = False, clip_mode: str = "none",
               use_uos: bool = False, return_codes: bool = False):
    """macro-block scale -> MXFP4 quantise -> dequantise -> macro-block descale, in t's dtype: the
    operand values the reference's two-level ("blockwise") MXFP4 recipe feeds its emulation matmuls
    (alto/kernels/fp4/mxfp4/mxfp_linear.py:301-302, 335-354).  Not on the linear path here (the
    two-level GEMM consumes the codes and factors directly); kept as a public composition of the
    four ops.  ``clip_mode`` goes to the quantizer and the dequantizer (the static clip is undone
    there), ``use_uos`` to the quantizer."""
    scaled, mbs = macro_block_scaling(t, axis=axis, use_2d_block=is_2d)
    q, s = convert_to_mxfp4(scaled, axis=axis, is_2d_block=is_2d, use_sr=use_sr, clip_mode=clip_mode, use_uos=use_uos)
    dq = convert_from_mxfp4(q, s, t.dtype, axis=axis, is_2d_block=is_2d, clip_mode=clip_mode)
    out = macro_block_descaling(dq, mbs, axis=axis, use_2d_block=is_2d)
    return (out, q) if return_codes else out


class MXFP4LinearFunction(torch.autograd.Function):
    """Same argument list as the reference's autograd function
    (alto/kernels/fp4/mxfp4/mxfp_linear.py:266-284)."""

    @staticmethod
    def forward(ctx, x, weight, use_2dblock_x, use_2dblock_w, use_sr_grad, use_dge, clip_mode,
                use_macro_block_scaling, hadamard_transform: Optional[HadamardTransform] = None,
                use_uos: bool = False):
        _check_options(clip_mode, use_uos)
        weight = unwrap_weight_wrapper(weight)
        if weight.dtype != x.dtype:
            weight = weight.to(dtype=x.dtype)
        ctx.macro = False
        if use_macro_block_scaling:
            ctx.macro = True
            return T.linear_forward(ctx, x, weight, bool(use_2dblock_x), bool(use_2dblock_w), bool(use_sr_grad),
                                    hadamard_transform, clip_mode, bool(use_uos), bool(use_dge))
        return E.linear_forward(ctx, "MXFP4LinearFunction", x, weight, L.FMT_MXFP4, use_2dblock_x=use_2dblock_x,
                                use_2dblock_w=use_2dblock_w, use_sr_grad=bool(use_sr_grad), use_outer_scale=False,
                                hadamard_transform=hadamard_transform, use_uos=bool(use_uos), clip_mode=clip_mode,
                                use_dge=bool(use_dge))

    @staticmethod
    def backward(ctx, grad_output):
        gi, gw = T.linear_backward(ctx, grad_output) if ctx.macro else E.linear_backward(ctx, grad_output)
        return gi, gw, None, None, None, None, None, None, None, None


@L.traced("mxfp4_linear")
def _to_mxfp4_then_scaled_mm(
    a: torch.Tensor,
    b: torch.Tensor,
    use_2dblock_x: bool,
    use_2dblock_w: bool,
    use_sr_grad: int,
    use_dge: bool,
    clip_mode: str,
    use_hadamard: bool,
    use_macro_block_scaling: bool = False,
    use_uos: bool = False,
) -> torch.Tensor:
    if use_hadamard:
        with torch.no_grad():
            hadamard_transform = HadamardFactory.create_transform(device=b.device)
    else:
        hadamard_transform = None
    return MXFP4LinearFunction.apply(a, b, use_2dblock_x, use_2dblock_w, use_sr_grad, use_dge, clip_mode,
                                     use_macro_block_scaling, hadamard_transform, use_uos)
