"""Macro-block (128) two-level scaling for MXFP4: ``macro_block_scaling`` / ``macro_block_descaling``.

Same signatures, shapes and return conventions as the reference's public ops
(alto/kernels/fp4/mxfp4/macro_block_scaling.py:423-437): ``axis`` names the axis the blocks of 128
run along, ``use_2d_block`` selects 128 x 128 tiles, the scaled tensor comes back in the input's
layout and the uint8 scale in the coordinates of the view with ``axis`` moved last
(``[..., rows_of_that_view, ceil(len(axis)/128)]``, or ``[..., ceil/128, ceil/128]`` for tiles).

The reference reaches a non-last axis through a strided transposed view; here the kernel has a
mode for blocks that run down the rows, so no transposed copy is made.  Only the last two axes of
a 2-D or 3-D tensor can carry the blocks.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["MACRO_BLOCK_SIZE", "MAX_FP4", "macro_block_scaling", "macro_block_descaling", "macro_scale_shape"]

MACRO_BLOCK_SIZE = 128
MAX_FP4 = 6.0


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def _plan(t: torch.Tensor, axis: int):
    """-> (3-D contiguous view [batch, rows, cols] of t, along_last: bool)."""
    if t.dim() not in (2, 3):
        raise AssertionError(f"Only support 2D or 3D input, got shape={tuple(t.shape)}")
    ax = axis % t.dim()
    if ax == t.dim() - 1:
        along_last = True
    elif ax == t.dim() - 2:
        along_last = False
    else:
        raise NotImplementedError("macro blocks can run along one of the last two axes only")
    if t.dtype not in (torch.bfloat16, torch.float32):
        raise AssertionError(f"unsupported dtype {t.dtype}")
    t3 = t.contiguous()
    t3 = t3.unsqueeze(0) if t3.dim() == 2 else t3
    return t3, along_last


def macro_scale_shape(shape, axis: int = -1, use_2d_block: bool = False) -> tuple:
    """Shape of the scale tensor for an input of ``shape`` (reference: macro_block_scaling.py:19-31,
    applied to the view with ``axis`` moved last)."""
    shape = list(shape)
    ax = axis % len(shape)
    shape[ax], shape[-1] = shape[-1], shape[ax]
    m, n = shape[-2], shape[-1]
    tail = (_ceil_div(m, MACRO_BLOCK_SIZE), _ceil_div(n, MACRO_BLOCK_SIZE)) if use_2d_block else \
        (m, _ceil_div(n, MACRO_BLOCK_SIZE))
    return (*shape[:-2], *tail)


def macro_block_scaling(x: torch.Tensor, axis: int = -1, use_2d_block: bool = False):
    """-> (y, scale): y = x times a per-block factor in [1, 2) that brings the block amax towards the
    top of an E2M1 binade; scale holds the factor's 8 mantissa bits."""
    x3, along_last = _plan(x, axis)
    b, rows, cols = x3.shape
    y3 = torch.empty_like(x3)
    if use_2d_block:
        s = torch.empty((b, _ceil_div(rows, 128), _ceil_div(cols, 128)), dtype=torch.uint8, device=x.device)
        _lib.macro_block_scaling(x3, y3, s, _lib.MACRO_2D)
        if not along_last:  # the reference indexes tiles of the transposed view
            s = s.transpose(-1, -2).contiguous()
    elif along_last:
        s = torch.empty((b, rows, _ceil_div(cols, 128)), dtype=torch.uint8, device=x.device)
        _lib.macro_block_scaling(x3, y3, s, _lib.MACRO_LAST)
    else:
        s = torch.empty((b, cols, _ceil_div(rows, 128)), dtype=torch.uint8, device=x.device)
        _lib.macro_block_scaling(x3, y3, s, _lib.MACRO_ROWS)
    if x.dim() == 2:
        return y3.squeeze(0), s.squeeze(0)
    return y3, s


def macro_block_descaling(y: torch.Tensor, scale: torch.Tensor, axis: int = -1, use_2d_block: bool = False):
    """Inverse of ``macro_block_scaling``: x = y / factor(scale)."""
    y3, along_last = _plan(y, axis)
    expect = macro_scale_shape(y.shape, axis, use_2d_block)
    assert tuple(scale.shape) == tuple(expect), f"Unexpected scale shape {tuple(scale.shape)}, expected {expect}"
    assert scale.dtype == torch.uint8
    s3 = scale.unsqueeze(0) if y.dim() == 2 else scale
    x3 = torch.empty_like(y3)
    if use_2d_block:
        if not along_last:
            s3 = s3.transpose(-1, -2)
        _lib.macro_block_descaling(y3, s3.contiguous(), x3, _lib.MACRO_2D)
    else:
        _lib.macro_block_descaling(y3, s3.contiguous(), x3, _lib.MACRO_LAST if along_last else _lib.MACRO_ROWS)
    return x3.squeeze(0) if y.dim() == 2 else x3
