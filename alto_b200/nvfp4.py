"""NVFP4 quantizers and the NVFP4 linear (forward, dgrad, wgrad) on B200.

Public surface mirrors the reference:
  convert_to_nvfp4 / convert_from_nvfp4 / compute_dynamic_outer_scale / _qdq
      (alto/kernels/fp4/nvfp4/nvfp_quantization.py:460-812)
  NVFP4LinearFunction / _to_nvfp4_then_scaled_mm
      (alto/kernels/fp4/nvfp4/nvfp_linear.py:20-314)

Where the reference emulates the GEMMs (quantize -> dequantize -> bf16 matmul), this
module keeps the operands in FP4 and runs the three contractions on the tcgen05
block-scaled MMA; the tensorwise outer scales are applied once in the GEMM epilogue.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Optional, Tuple, Union

import torch

from . import _lib as L
from . import _linear as E
from . import _quant as Q
from .hadamard import HadamardFactory, HadamardTransform

BLOCK_SIZE_DEFAULT = 16
F4_E2M1_MAX = 6.0
F8E4M3_MAX = 448.0
E4M3_EPS = 2.0 ** -6
SUPPORTED_SCALE_FORMATS = ("e4m3",)
_OUTER_SCALE_DIVZERO_FLOOR = 1.0e-30


def _check_scale_format(scale_format: str) -> None:
    if scale_format == "ue5m3":
        raise NotImplementedError(
            "scale_format='ue5m3' (AMD-FP4 inner scales) is not part of the B200 path; use 'e4m3'")
    if scale_format not in SUPPORTED_SCALE_FORMATS:
        raise NotImplementedError(
            f"scale_format={scale_format!r} is not supported. Currently supported: {SUPPORTED_SCALE_FORMATS}")


def unwrap_weight_wrapper(weight: torch.Tensor) -> torch.Tensor:
    """alto/kernels/fp4/fp4_common/tensor_wrappers.py:8-30."""
    if type(weight) is torch.Tensor:
        return weight
    pre = getattr(weight, "_prequant", None)
    if pre is not None:          # a wrapper that holds only the quantised operands (quantised all-gather)
        return pre
    if hasattr(weight, "_data"):
        return weight._data
    return weight.as_subclass(torch.Tensor)


from ._linear import amax_scratch as _amax_scratch, draw_philox as _draw_philox, explicit_sr_bits  # noqa: E402,F401

# ---------------------------------------------------------------------------------------
# public quantizer ops
# ---------------------------------------------------------------------------------------

def compute_dynamic_outer_scale(data_hp: torch.Tensor, scale_format: str = "e4m3") -> torch.Tensor:
    """FP32 outer scale ``max(nan_to_num(amax) / (448 * 6), 1e-30)`` as a 1-element tensor."""
    _check_scale_format(scale_format)
    if not data_hp.is_cuda:
        raise RuntimeError("alto_b200 kernels run on CUDA tensors only (no CPU fallback)")
    x = data_hp.reshape(-1, data_hp.shape[-1])
    if x.stride(-1) != 1 or (x.stride(0) * x.element_size()) % 16 != 0 or x.dtype not in (torch.bfloat16, torch.float32):
        x = x.contiguous() if x.dtype in (torch.bfloat16, torch.float32) else x.float().contiguous()
    amax_bits = torch.empty(2, dtype=torch.int32, device=x.device)
    outer = torch.empty(2, dtype=torch.float32, device=x.device)
    L.amax(x, amax_bits, outer, _amax_scratch(x.device))
    return outer[:1]


@L.traced("convert_to_nvfp4")
def convert_to_nvfp4(
    data_hp: torch.Tensor,
    block_size: int = BLOCK_SIZE_DEFAULT,
    axis: int = -1,
    is_2d_block: bool = False,
    outer_scale: Optional[torch.Tensor] = None,
    update_outer_scale: bool = True,
    scale_format: str = "e4m3",
    use_sr: bool = False,
    philox_seed: Optional[int] = None,
    philox_offset: Optional[int] = None,
    use_asm: Optional[bool] = None,
    rand_bits: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantize to NVFP4; same contract as the reference op, including the in-place refresh of a
    caller-supplied ``outer_scale`` buffer when ``update_outer_scale`` is set.

    ``rand_bits`` (extension): explicit 32-bit random words [2, rows, cols/2] for ``use_sr``.
    With ``use_sr`` and no ``rand_bits`` the words are the reference's: Philox-4x32-10 words of
    (philox_seed, philox_offset) laid out as its kernel lays them out (one table per launch,
    repeated over the 64 x 64 tiles of the quantisation-axis-last view).
    """
    torch._check(
        data_hp.shape[axis] % block_size == 0,
        lambda: f"tensor shape ({data_hp.shape}) at axis={axis} is not divisible by {block_size}",
    )
    assert data_hp.dtype in [torch.float32, torch.bfloat16]
    assert block_size == BLOCK_SIZE_DEFAULT, f"NVFP4 kernels are built for block_size 16, got {block_size}"
    assert not is_2d_block or data_hp.size(-2) % block_size == 0, (
        f"2D block requires dim -2 ({data_hp.size(-2)}) divisible by block_size ({block_size})")
    _check_scale_format(scale_format)

    if outer_scale is not None:
        assert outer_scale.numel() == 1, "outer_scale must be a scalar tensor"
        assert outer_scale.dtype == torch.float32, "outer_scale must be float32"
        assert outer_scale.device == data_hp.device, (
            f"outer_scale device ({outer_scale.device}) must match data_hp device ({data_hp.device})")
        if update_outer_scale:
            outer_scale.copy_(compute_dynamic_outer_scale(data_hp, scale_format).reshape_as(outer_scale))
        outer_buf = outer_scale.reshape(1)
    elif update_outer_scale:
        outer_buf = compute_dynamic_outer_scale(data_hp, scale_format)
    else:
        outer_buf = None

    rounding, philox = L.ROUND_RTN, (0, 0)
    if use_sr:
        if rand_bits is not None:
            rounding = L.ROUND_SR_BITS
        else:
            rounding = L.ROUND_SR_PHILOX
            drawn = _draw_philox()
            philox = (drawn[0] if philox_seed is None else philox_seed,
                      drawn[1] if philox_offset is None else philox_offset)
    return Q.quantize(data_hp, L.FMT_NVFP4, axis, is_2d_block, outer_scale=outer_buf, rounding=rounding,
                      rand_bits=rand_bits if use_sr else None, philox=philox)


def convert_from_nvfp4(
    data_lp: torch.Tensor,
    scales: torch.Tensor,
    output_dtype: torch.dtype = torch.float32,
    block_size: int = BLOCK_SIZE_DEFAULT,
    axis: int = -1,
    is_2d_block: bool = False,
    outer_scale: Optional[torch.Tensor] = None,
    scale_format: str = "e4m3",
    use_asm: Optional[bool] = None,
) -> torch.Tensor:
    assert output_dtype in [torch.float32, torch.bfloat16]
    assert block_size == BLOCK_SIZE_DEFAULT
    if outer_scale is not None:
        assert outer_scale.numel() == 1, "outer_scale must be a scalar tensor"
    return Q.dequantize(data_lp, scales, L.FMT_NVFP4, axis, is_2d_block, output_dtype, outer_scale)


def _qdq(tensor: torch.Tensor, *, axis: int, is_2d_block: bool, use_outer_scale: bool, use_sr: bool = False,
         block_size: int = 16, return_raw: bool = False, scale_format: str = "e4m3",
         ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    """Quantize then dequantize (alto/kernels/fp4/nvfp4/nvfp_quantization.py:758-812)."""
    outer_scale = torch.empty(1, dtype=torch.float32, device=tensor.device) if use_outer_scale else None
    data_lp, scales = convert_to_nvfp4(tensor, block_size=block_size, axis=axis, is_2d_block=is_2d_block,
                                       outer_scale=outer_scale, update_outer_scale=use_outer_scale,
                                       scale_format=scale_format, use_sr=use_sr)
    dq = convert_from_nvfp4(data_lp, scales, output_dtype=tensor.dtype, block_size=block_size, axis=axis,
                            is_2d_block=is_2d_block, outer_scale=outer_scale, scale_format=scale_format)
    if return_raw:
        return dq, data_lp, scales
    return dq


# ---------------------------------------------------------------------------------------
# fused linear
# ---------------------------------------------------------------------------------------

class NVFP4LinearFunction(torch.autograd.Function):
    """y = x W^T with NVFP4 operands; same argument list as the reference's autograd function
    (alto/kernels/fp4/nvfp4/nvfp_linear.py:53-278).

    forward : X quantised along K, W along K (1D or 16x16)         -> fprop GEMM
              saves X quantised along M (after the Hadamard rotation) and W packed along N
    backward: dY quantised along N (SR optional)                    -> dgrad GEMM with W along N
              H dY quantised along M (SR optional)                  -> wgrad GEMM with H X along M
    The tensorwise outer scales multiply the accumulator once, in the GEMM epilogue.
    """

    @staticmethod
    def forward(ctx, x, weight, use_2dblock_x: bool, use_2dblock_w: bool, use_sr_grad: bool,
                use_outer_scale: bool, hadamard_transform: Optional[HadamardTransform] = None,
                use_dge: bool = False, scale_format: str = "e4m3"):
        _check_scale_format(scale_format)
        weight = unwrap_weight_wrapper(weight)
        if weight.dtype != x.dtype:
            weight = weight.to(dtype=x.dtype)
        M = x.numel() // x.shape[-1]
        if not use_2dblock_w:
            torch._check(weight.shape[0] % BLOCK_SIZE_DEFAULT == 0, lambda: (
                f"NVFP4LinearFunction wgrad-axis weight QDQ requires weight.shape[0] ({weight.shape[0]}) divisible "
                f"by BLOCK_SIZE_DEFAULT ({BLOCK_SIZE_DEFAULT}) when use_2dblock_w=False."))
        if not use_2dblock_x:
            torch._check(M % BLOCK_SIZE_DEFAULT == 0, lambda: (
                f"NVFP4LinearFunction wgrad-axis activation QDQ requires x.shape[0] ({M}) divisible by "
                f"BLOCK_SIZE_DEFAULT ({BLOCK_SIZE_DEFAULT}) when use_2dblock_x=False."))
        return E.linear_forward(ctx, "NVFP4LinearFunction", x, weight, L.FMT_NVFP4, use_2dblock_x=use_2dblock_x,
                                use_2dblock_w=use_2dblock_w, use_sr_grad=use_sr_grad,
                                use_outer_scale=use_outer_scale, hadamard_transform=hadamard_transform,
                                use_dge=bool(use_dge))

    @staticmethod
    def backward(ctx, grad_output):
        grad_inputs, grad_weights = E.linear_backward(ctx, grad_output)
        return grad_inputs, grad_weights, None, None, None, None, None, None, None


@L.traced("nvfp4_linear")
def _to_nvfp4_then_scaled_mm(
    a: torch.Tensor,
    b: torch.Tensor,
    use_2dblock_x: bool,
    use_2dblock_w: bool,
    use_sr_grad: bool,
    use_outer_scale: bool = False,
    use_hadamard: bool = False,
    use_dge: bool = False,
    scale_format: str = "e4m3",
) -> torch.Tensor:
    """Boundary function of the dispatch layer (alto/kernels/fp4/nvfp4/nvfp_linear.py:281-314)."""
    hadamard_transform: Optional[HadamardTransform] = None
    if use_hadamard:
        with torch.no_grad():
            hadamard_transform = HadamardFactory.create_transform(device=b.device)
    return NVFP4LinearFunction.apply(a, b, use_2dblock_x, use_2dblock_w, use_sr_grad, use_outer_scale,
                                     hadamard_transform, use_dge, scale_format)
