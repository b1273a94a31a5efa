"""MXFP4 with two-level ("blockwise" macro-block) scaling on the block-scaled tensor cores.

The recipe (alto/kernels/fp4/mxfp4/mxfp_linear.py:301-303, 359-360, 385-386, 437-440, 467-468,
482-483; grouped: mxfp_grouped_gemm/cg_backward.py:631-635, 692-695, 721-722, 782-785, 812-813,
826-827): before every MXFP4 quantisation each block of 128 elements along the quantisation axis (or
each 128 x 128 tile) is multiplied by a factor in [1, 2) that lifts the block amax towards the top
of an E2M1 binade; the matmul must divide the factor out again.  The reference has no matrix core
that takes the factors, so it de-quantises, de-scales and multiplies in bf16
(mxfp_linear.py:337-356).  Here the operands stay quantised: the GEMM accumulates one 128-wide chunk
of the reduction axis at a time in tensor memory and folds it into the fp32 result with
1 / (factor_a * factor_b) (``csrc/gemm_macro.cuh``).  The contraction is the same; only the
bf16 rounding of the de-scaled operands, which the reference's emulation adds, is absent.

Operand builders return ``_linear.Operand`` objects whose ``macro`` field says where the factor
codes of (operand row, chunk) sit, so the scale tensors ``macro_block_scaling`` returns are used as
they are for every axis and block shape.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L
from . import _linear as E
from . import dge
from .macro_block_scaling import macro_block_scaling

MX = L.FMT_MXFP4
STATIC_CLIP_WGRAD = 16.0 / 9.0


def rows_operand(t2: torch.Tensor, use_uos: bool, sr: Optional[dict] = None) -> E.Operand:
    """t2 [R, C] -> operand [R, C] reduced along C: 1-D macro blocks and MXFP4 blocks along the last axis."""
    ts, mbs = macro_block_scaling(t2, axis=-1, use_2d_block=False)            # mbs [R, ceil(C/128)]
    op = E.quant_rows(ts, MX, None, sr or E.RTN, use_uos)
    op.macro = L.MacroScale(mbs, mbs.shape[-1], 1, 0)
    return op


def cols_operand(t2: torch.Tensor, use_uos: bool, clip_mode: str = "none", sr: Optional[dict] = None) -> E.Operand:
    """t2 [R, C] -> operand [C, R] reduced along R (the token axis): blocks run down the rows of t2."""
    ts, mbs = macro_block_scaling(t2, axis=0, use_2d_block=False)             # mbs [C, ceil(R/128)]
    op = E.quant_cols(ts, MX, None, None, sr or E.RTN, use_uos, clip_mode)
    op.macro = L.MacroScale(mbs, mbs.shape[-1], 1, 0)
    return op


def tiles_operands(t2: torch.Tensor, use_uos: bool, sr: Optional[dict] = None) -> Tuple[E.Operand, E.Operand]:
    """t2 [R, C] in 128 x 128 macro tiles and 32 x 32 MXFP4 blocks, quantised once:
    -> (operand [R, C] reduced along C, operand [C, R] reduced along R)."""
    ts, mbs = macro_block_scaling(t2, axis=-1, use_2d_block=True)             # mbs [ceil(R/128), ceil(C/128)]
    op_k, op_t = E.quant_2d(ts, MX, None, True, use_uos, sr)
    nc = mbs.shape[-1]
    op_k.macro = L.MacroScale(mbs, nc, 1, 7)
    op_t.macro = L.MacroScale(mbs, 1, nc, 7)
    return op_k, op_t


def gemm(a: E.Operand, b: E.Operand, out_dtype: torch.dtype, out_scale: float = 1.0) -> torch.Tensor:
    assert a.k == b.k and a.macro is not None and b.macro is not None
    out = torch.empty(a.rows, b.rows, dtype=out_dtype, device=a.codes.device)
    L.gemm_mxfp4_two_level(a.rows, b.rows, a.k, a.codes, a.scales, a.macro, b.codes, b.scales, b.macro, out, out_scale)
    return out


def _rotate(t2: torch.Tensor, hadamard_transform) -> torch.Tensor:
    # the rotated tensor is materialised in the input dtype, as the reference does before it scales
    return hadamard_transform(t2, left_mul=True) if hadamard_transform is not None else t2


def _save_macro(ctx, x_m: E.Operand, w_t: E.Operand) -> None:
    ctx.save_for_backward(x_m.codes, x_m.scales, x_m.macro.codes, w_t.codes, w_t.scales, w_t.macro.codes)
    ctx.x_macro = (x_m.macro.row_stride, x_m.macro.chunk_stride, x_m.macro.row_shift, x_m.macro.expert_stride)
    ctx.w_macro = (w_t.macro.row_stride, w_t.macro.chunk_stride, w_t.macro.row_shift, w_t.macro.expert_stride)


def _load_macro(ctx, x_shape, w_shape) -> Tuple[E.Operand, E.Operand]:
    xc, xs, xm, wc, ws, wm = ctx.saved_tensors[:6]
    x_m = E.Operand(xc, xs, None, x_shape[0], x_shape[1], MX)
    x_m.macro = L.MacroScale(xm, ctx.x_macro[0], ctx.x_macro[1], ctx.x_macro[2], ctx.x_macro[3])
    w_t = E.Operand(wc, ws, None, w_shape[0], w_shape[1], MX)
    w_t.macro = L.MacroScale(wm, ctx.w_macro[0], ctx.w_macro[1], ctx.w_macro[2], ctx.w_macro[3])
    return x_m, w_t


def _grad_operands(ctx, g2: torch.Tensor, M: int, N: int) -> Tuple[E.Operand, E.Operand]:
    """dY along N for dgrad and (rotated) along the tokens for wgrad (mxfp_linear.py:436-517)."""
    if ctx.use_2dblock_x:
        return tiles_operands(g2, ctx.use_uos, E.sr_args(ctx.use_sr_grad, "dy_n", M, N, g2.device))
    g_n = rows_operand(g2, ctx.use_uos, E.sr_args(ctx.use_sr_grad, "dy_n", M, N, g2.device))
    g_m = cols_operand(_rotate(g2, ctx.hadamard_transform), ctx.use_uos, ctx.clip_mode,
                       E.sr_args(ctx.use_sr_grad, "dy_m", N, M, g2.device))
    return g_n, g_m


def _wgrad_scale(ctx) -> float:
    # both wgrad operands were clipped to 3/4 of their range (mxfp_linear.py:543-544); 2-D activation
    # blocks are never clipped
    return STATIC_CLIP_WGRAD if (ctx.clip_mode == "static" and not ctx.use_2dblock_x) else 1.0


# ---------------------------------------------------------------------------------------------
# dense linear
# ---------------------------------------------------------------------------------------------
def linear_forward(ctx, x, weight, use_2dblock_x: bool, use_2dblock_w: bool, use_sr_grad: bool, hadamard_transform,
                   clip_mode: str = "none", use_uos: bool = False, use_dge: bool = False):
    if not x.is_cuda:
        raise RuntimeError("MXFP4LinearFunction runs on CUDA tensors only (no CPU fallback)")
    original_shape = x.shape
    x2 = E.as_2d_rows(x.detach())
    w2 = E.as_2d_rows(weight.detach())
    M, K = x2.shape
    N = w2.shape[0]
    E.check_dims("MXFP4LinearFunction", M, K, N)
    if use_2dblock_x:
        x_k, x_m = tiles_operands(x2, use_uos)
    else:
        x_k = rows_operand(x2, use_uos)
    if use_2dblock_w:
        w_k, w_t = tiles_operands(w2, use_uos)
    else:
        w_k = rows_operand(w2, use_uos)
    y = gemm(x_k, w_k, x.dtype)
    if not use_2dblock_w:
        w_t = cols_operand(w2, use_uos)
    if not use_2dblock_x:
        x_m = cols_operand(_rotate(x2, hadamard_transform), use_uos, clip_mode)
    _save_macro(ctx, x_m, w_t)
    ctx.dims = (M, K, N)
    ctx.use_2dblock_x, ctx.use_sr_grad, ctx.hadamard_transform = use_2dblock_x, use_sr_grad, hadamard_transform
    ctx.clip_mode, ctx.use_uos, ctx.use_dge = clip_mode, use_uos, use_dge
    return y.view(*original_shape[:-1], N)


def linear_backward(ctx, grad_output):
    E.take_dx_ready_hook()   # this backward does not hand dX over early; a caller's all-reduce follows it
    M, K, N = ctx.dims
    x_m, w_t = _load_macro(ctx, (K, M), (K, N))
    original_shape = grad_output.shape
    g2 = E.as_2d_rows(grad_output)
    g_n, g_m = _grad_operands(ctx, g2, M, N)
    grad_inputs = grad_weights = None
    if ctx.needs_input_grad[0]:
        grad_inputs = gemm(g_n, w_t, grad_output.dtype).view(*original_shape[:-1], K)
    if ctx.needs_input_grad[1]:
        grad_weights = gemm(g_m, x_m, grad_output.dtype, _wgrad_scale(ctx))
        if ctx.use_dge:
            grad_weights = dge.apply_to_weight_grad(grad_weights, w_t.codes)
    return grad_inputs, grad_weights


# ---------------------------------------------------------------------------------------------
# grouped (MoE) linear
# ---------------------------------------------------------------------------------------------
def _weight_stack(w3: torch.Tensor, use_2dblock_w: bool, use_uos: bool) -> Tuple[E.Operand, E.Operand]:
    """[E, N, K] -> (W along K stacked [E*N, K], W along N stacked [E*K, N]) with per-expert factor codes."""
    n_exp, N, K = w3.shape
    if use_2dblock_w:
        ws, mbs = macro_block_scaling(w3, axis=-1, use_2d_block=True)        # mbs [E, ceil(N/128), ceil(K/128)]
        cc = E._code_cols(MX, K)
        ck = torch.empty(n_exp, N, cc, dtype=torch.uint8, device=w3.device)
        ct = torch.empty(n_exp, K, E._code_cols(MX, N), dtype=torch.uint8, device=w3.device)
        sk = torch.empty(n_exp * L.packed_scale_bytes(N, K // 32), dtype=torch.uint8, device=w3.device)
        st = torch.empty(n_exp * L.packed_scale_bytes(K, N // 32), dtype=torch.uint8, device=w3.device)
        L.quantize_2d_batched(ws, MX, ck, ct, None, sk, st, use_uos=use_uos)
        w_k = E.Operand(ck.view(n_exp * N, cc), sk, None, n_exp * N, K, MX)
        w_t = E.Operand(ct.view(n_exp * K, -1), st, None, n_exp * K, N, MX)
        nr, nc = mbs.shape[-2], mbs.shape[-1]
        w_k.macro = L.MacroScale(mbs, nc, 1, 7, nr * nc)
        w_t.macro = L.MacroScale(mbs, 1, nc, 7, nr * nc)
        return w_k, w_t
    ws_k, mbs_k = macro_block_scaling(w3, axis=-1, use_2d_block=False)       # [E, N, ceil(K/128)]
    ws_t, mbs_t = macro_block_scaling(w3, axis=-2, use_2d_block=False)       # [E, K, ceil(N/128)]
    from .grouped import _stack
    w_k = _stack([E.quant_rows(ws_k[e], MX, None, E.RTN, use_uos) for e in range(n_exp)])
    w_t = _stack([E.quant_cols(ws_t[e], MX, None, None, E.RTN, use_uos) for e in range(n_exp)])
    w_k.macro = L.MacroScale(mbs_k, mbs_k.shape[-1], 1, 0, mbs_k.shape[-2] * mbs_k.shape[-1])
    w_t.macro = L.MacroScale(mbs_t, mbs_t.shape[-1], 1, 0, mbs_t.shape[-2] * mbs_t.shape[-1])
    return w_k, w_t


class GroupedTwoLevelFunction(torch.autograd.Function):
    """MXFP4 grouped linear with two-level scaling (mxfp_grouped_gemm/cg_backward.py:600-930 with
    ``use_macro_block_scaling``); ``weights`` is canonical [E, N, K].  Forward and dgrad pick the
    expert's weight tile and factor codes per 128-row group, wgrad reduces over each expert's token
    range; nothing synchronises with the host."""

    @staticmethod
    def forward(ctx, inputs, weights, offs, use_2dblock_w, use_sr_grad, hadamard_transform, use_2dblock_x=False,
                clip_mode="none", use_uos=False, use_dge=False):
        from .grouped import group_experts_from_offsets
        from .nvfp4 import unwrap_weight_wrapper
        if not inputs.is_cuda:
            raise RuntimeError("grouped GEMM runs on CUDA tensors only (no CPU fallback)")
        weights = unwrap_weight_wrapper(weights)
        if weights.dtype != inputs.dtype:
            weights = weights.to(dtype=inputs.dtype)
        assert inputs.dim() == 2 and weights.dim() == 3, "expected inputs [M, K] and weights [E, N, K]"
        M, K = inputs.shape
        n_exp, N, K2 = weights.shape
        assert K == K2, f"inner dimensions differ: {K} vs {K2}"
        torch._check(offs is not None and offs.numel() == n_exp, lambda: "offs must hold one entry per expert")
        E.check_dims("grouped GEMM", M, K, N)
        x2 = E.as_2d_rows(inputs.detach())
        w3 = weights.detach().contiguous()
        offs32 = offs.to(torch.int32).contiguous()
        group_expert = group_experts_from_offsets(offs32, M)
        if use_2dblock_x:
            x_k, x_m = tiles_operands(x2, use_uos)
        else:
            x_k = rows_operand(x2, use_uos)
            x_m = cols_operand(_rotate(x2, hadamard_transform), use_uos, clip_mode)
        w_k, w_t = _weight_stack(w3, use_2dblock_w, use_uos)
        y = torch.empty(M, N, dtype=inputs.dtype, device=inputs.device)
        L.gemm_mxfp4_two_level(M, N, K, x_k.codes, x_k.scales, x_k.macro, w_k.codes, w_k.scales, w_k.macro, y,
                               group_expert=group_expert, num_experts=n_exp)
        ctx.save_for_backward(x_m.codes, x_m.scales, x_m.macro.codes, w_t.codes, w_t.scales, w_t.macro.codes,
                              group_expert, offs32)
        ctx.x_macro = (x_m.macro.row_stride, x_m.macro.chunk_stride, x_m.macro.row_shift, x_m.macro.expert_stride)
        ctx.w_macro = (w_t.macro.row_stride, w_t.macro.chunk_stride, w_t.macro.row_shift, w_t.macro.expert_stride)
        ctx.dims = (M, K, N, n_exp)
        ctx.use_2dblock_x, ctx.use_sr_grad, ctx.hadamard_transform = use_2dblock_x, use_sr_grad, hadamard_transform
        ctx.clip_mode, ctx.use_uos, ctx.use_dge = clip_mode, use_uos, use_dge
        return y

    @staticmethod
    def backward(ctx, grad_output):
        M, K, N, n_exp = ctx.dims
        x_m, w_t = _load_macro(ctx, (K, M), (n_exp * K, N))
        group_expert, offs32 = ctx.saved_tensors[6:8]
        g2 = E.as_2d_rows(grad_output)
        g_n, g_m = _grad_operands(ctx, g2, M, N)
        grad_inputs = grad_weights = None
        if ctx.needs_input_grad[0]:
            grad_inputs = torch.empty(M, K, dtype=grad_output.dtype, device=g2.device)
            L.gemm_mxfp4_two_level(M, K, N, g_n.codes, g_n.scales, g_n.macro, w_t.codes, w_t.scales, w_t.macro,
                                   grad_inputs, group_expert=group_expert, num_experts=n_exp)
        if ctx.needs_input_grad[1]:
            grad_weights = torch.empty(n_exp, N, K, dtype=grad_output.dtype, device=g2.device)
            L.gemm_mxfp4_two_level(N, K, M, g_m.codes, g_m.scales, g_m.macro, x_m.codes, x_m.scales, x_m.macro,
                                   grad_weights, _wgrad_scale(ctx), k_offs=offs32, num_experts=n_exp)
            if ctx.use_dge:
                wt_codes = w_t.codes.view(n_exp, K, -1)
                for e in range(n_exp):
                    dge.apply_to_weight_grad(grad_weights[e], wt_codes[e])
        return grad_inputs, grad_weights, None, None, None, None, None, None, None, None
