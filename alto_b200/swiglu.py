"""SwiGLU of an expert MLP whose gate and up projections are one grouped GEMM: ``swiglu(h)`` with
``h = [gate | up]`` equals ``silu(h[:, :H]) * h[:, H:]`` (same bf16 roundings, forward and backward)
in one kernel per direction instead of eight tensor-op passes over the routed rows.

The module that owns this activation in the reference's setting is ``GroupedExperts`` of its
TorchTitan fork, whose parameters the modifier swaps (alto/modifiers/lpt/base.py:186-187); the
grouped GEMMs on either side are ``alto_b200.grouped``."""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["swiglu"]


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h):
        ctx.save_for_backward(h)
        return _lib.swiglu_forward(h)

    @staticmethod
    def backward(ctx, grad_out):
        (h,) = ctx.saved_tensors
        return _lib.swiglu_backward(h, grad_out.contiguous())


def swiglu(h: torch.Tensor) -> torch.Tensor:
    """h: [rows, 2H] bf16 on a CUDA device, H a multiple of 8 -> [rows, H]."""
    if h.dim() != 2 or h.shape[1] % 16 != 0:
        raise ValueError(f"swiglu expects [rows, 2H] with H a multiple of 8, got {tuple(h.shape)}")
    if h.dtype != torch.bfloat16:
        raise TypeError(f"swiglu expects bfloat16, got {h.dtype}")
    return _SwiGLU.apply(h.contiguous())
