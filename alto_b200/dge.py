"""Differentiable gradient estimator (DGE) factor of the FP4 recipes.

The reference multiplies the weight gradient by ``dge_bwd(w_fp4_values, float4_e2m1fn_x2)``
(alto/kernels/dge/dge.py:81-93; call sites alto/kernels/fp4/nvfp4/nvfp_linear.py:250-268 and
alto/kernels/fp4/mxfp4/mxfp_linear.py:546-566), where ``w_fp4_values`` are the weight's E2M1 codes
decoded with unit scales.  Such a value is one of sixteen numbers, so the factor is a table over the
code: ``fp4_bin_table`` evaluates the reference's expression on the sixteen values once per device
and dtype, with the same tensor ops, and ``apply_to_weight_grad`` hands the table and the packed
weight codes to the CUDA kernel that scales the gradient in place.

Every bin value is an end point of its own interval of the estimator's piecewise function, where
``|x - mid| = half_delta`` and the factor is ``half_delta**(1-1/k) * half_delta**(1/k-1) / k``, i.e.
1/k = 0.2 up to the rounding of the two powers (exactly 0.2 for every bin with the CPU's ``pow``, one
fp32 ulp below for some bins with CUDA's).
"""
from __future__ import annotations

import torch

from . import _lib as L

K = 5
_E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
_BREAK_POINTS = [-6, -4, -3, -2, -1.5, -1, -0.5, 0, 0.5, 1, 1.5, 2, 3, 4, 6]
_cache = {}


def dge_bwd_fp4(x: torch.Tensor) -> torch.Tensor:
    """The reference's ``dge_bwd`` for the E2M1 grid (alto/kernels/dge/dge.py:81-93)."""
    bp = torch.tensor(_BREAK_POINTS, dtype=torch.float32, device=x.device)
    iv = bp[1:] - bp[:-1]
    idx = torch.searchsorted(bp, x.contiguous(), right=False, out_int32=True) - 1
    idx = torch.where(idx < 0, 0, idx)
    idx = torch.where(idx >= len(bp) - 1, len(bp) - 2, idx)
    half = iv[idx] / 2.0
    mid = bp[idx] + half
    return torch.clamp(half ** (1 - 1 / K) * (torch.abs(x - mid) ** (1 / K - 1)) / K, 0, 3.0)


def fp4_bin_table(device, dtype: torch.dtype) -> list:
    """Sixteen fp32 factors indexed by the E2M1 code (sign in bit 3), for code values held in
    ``dtype`` (the dtype of the weight gradient, in which the reference decodes the codes)."""
    key = (str(device), dtype)
    if key not in _cache:
        v = torch.tensor(_E2M1_VALUES + [-t for t in _E2M1_VALUES], dtype=dtype, device=device)
        _cache[key] = [float(t) for t in dge_bwd_fp4(v).float().cpu()]
    return _cache[key]


def apply_to_weight_grad(grad_weights: torch.Tensor, codes_t: torch.Tensor) -> torch.Tensor:
    """grad_weights[n, k] * table[code of W[n, k]], rounded to the gradient's dtype, in place.
    ``codes_t``: packed E2M1 codes of the weight operand of the dgrad GEMM, [K, N/2]."""
    L.dge_scale(grad_weights, codes_t, fp4_bin_table(grad_weights.device, grad_weights.dtype))
    return grad_weights
