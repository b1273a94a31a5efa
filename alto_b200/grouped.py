"""MoE grouped GEMMs with MXFP4 / NVFP4 / MXFP8 operands on B200.

Boundary functions of the dispatch layer, same names and arguments as the reference:
  _quantize_then_mxfp_scaled_grouped_mm   (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/functional.py:11-38)
  _quantize_then_nvfp4_scaled_grouped_mm  (alto/kernels/fp4/nvfp4/nvfp_grouped_gemm/functional.py:134-167)
  _quantize_then_mxfp8_scaled_grouped_mm  (alto/kernels/mxfp8/mxfp8_grouped_gemm/functional.py:48-81)

``A`` is the routed token buffer [M_buf, K], sorted by expert; ``B`` the expert weights in dispatch
layout [E, K, N]; ``offs`` the int32 cumulative token counts per expert, every count a multiple
of 128 (ALIGN_SIZE_M) and ``offs[-1] <= M_buf``.  Rows past ``offs[-1]`` give zero output and zero
gradient.  The three contractions

    Y[m]  = X[m]  . W[e(m)]^T          dX[m] = dY[m] . W[e(m)]          dW[e] = sum_{m in e} dY[m]^T X[m]

run on the block-scaled tensor-core kernel: forward and dgrad pick the expert's weight tile per
128-row group, wgrad reduces over each expert's token range.  Operand preparation is that of
the dense linear (alto/kernels/fp4/nvfp4/nvfp_grouped_gemm/autograd.py:66-250): whole-buffer
quantisation, one tensorwise outer scale for the token buffer and one for the whole weight stack.
Nothing synchronises with the host: expert ids per group are derived from ``offs`` on the device.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib as L
from . import _linear as E
from . import dge
from .hadamard import HadamardFactory, HadamardTransform
from .nvfp4 import _check_scale_format, unwrap_weight_wrapper

ALIGN_SIZE_M = 128


def create_indices_from_offsets_nosync(m_offsets: torch.Tensor) -> torch.Tensor:
    """Expert id of every routed row (alto/kernels/dsgemm_utils.py:97-112).  Unlike the reference's
    helper of the same name this one is kept for API parity only: it needs ``offs[-1]`` on the host."""
    total = int(m_offsets[-1])
    rows = torch.arange(total, device=m_offsets.device, dtype=torch.int32)
    return torch.bucketize(rows, m_offsets, right=True, out_int32=True)


def group_experts_from_offsets(offs: torch.Tensor, m_buf: int) -> torch.Tensor:
    """int32 [ceil(m_buf / 128)]: expert of each 128-row group, -1 for groups past ``offs[-1]``.
    Computed on the device, no host synchronisation."""
    n_groups = (m_buf + ALIGN_SIZE_M - 1) // ALIGN_SIZE_M
    starts = torch.arange(n_groups, device=offs.device, dtype=torch.int32) * ALIGN_SIZE_M
    e = torch.bucketize(starts, offs.to(torch.int32), right=True, out_int32=True)
    return torch.where(e >= offs.numel(), torch.full_like(e, -1), e).contiguous()


def _stack(ops):
    """Per-expert operands -> one operand whose rows are the experts' rows stacked."""
    first = ops[0]
    codes = torch.stack([o.codes for o in ops]).reshape(-1, first.codes.shape[-1])
    scales = torch.cat([o.scales for o in ops])
    return E.Operand(codes, scales, first.outer, first.rows * len(ops), first.k, first.fmt)


def _quant_weight_stack(w3: torch.Tensor, fmt: int, use_2dblock_w: bool, use_outer_scale: bool, use_uos: bool = False):
    """[E, N, K] -> (W along K stacked [E*N, K], W along N stacked [E*K, N]), one outer scale for all."""
    n_exp, N, K = w3.shape
    ow = E.outer_scales(w3.reshape(n_exp * N, K), use_outer_scale, None)
    outer = None if ow is None else ow[0:1]
    if use_2dblock_w:
        # every expert in one launch; the stacked outputs are the operands of the grouped GEMMs as they are
        b = L.block_of(fmt)
        cc = E._code_cols(fmt, K)
        ck = torch.empty(n_exp, N, cc, dtype=torch.uint8, device=w3.device)
        ct = torch.empty(n_exp, K, E._code_cols(fmt, N), dtype=torch.uint8, device=w3.device)
        sk = torch.empty(n_exp * L.packed_scale_bytes(N, K // b), dtype=torch.uint8, device=w3.device)
        st = torch.empty(n_exp * L.packed_scale_bytes(K, N // b), dtype=torch.uint8, device=w3.device)
        L.quantize_2d_batched(w3, fmt, ck, ct, None, sk, st, outer_scale=outer, use_uos=use_uos)
        return (E.Operand(ck.view(n_exp * N, cc), sk, outer, n_exp * N, K, fmt),
                E.Operand(ct.view(n_exp * K, -1), st, outer, n_exp * K, N, fmt))
    ks, ts = [], []
    for e in range(n_exp):
        we = w3[e]
        k_op = E.quant_rows(we, fmt, outer, E.RTN, use_uos)
        t_op = E.quant_cols(we, fmt, outer, None, E.RTN, use_uos)
        ks.append(k_op)
        ts.append(t_op)
    return _stack(ks), _stack(ts)


def _grouped_gemm(a: E.Operand, b_stack: E.Operand, n_out: int, num_experts: int, group_expert, out_dtype):
    out = torch.empty(a.rows, n_out, dtype=out_dtype, device=a.codes.device)
    L.grouped_gemm_blockscaled(a.fmt, b_stack.fmt, a.rows, n_out, a.k, num_experts, a.codes, a.scales, b_stack.codes,
                               b_stack.scales, group_expert, out, a.outer, b_stack.outer)
    return out


class GroupedLinearFunction(torch.autograd.Function):
    """Shared autograd function of the three grouped paths; ``weights`` is canonical [E, N, K]."""

    @staticmethod
    def forward(ctx, inputs, weights, offs, fmt, fmt_grad, use_2dblock_x, use_2dblock_w, use_sr_grad,
                use_outer_scale, hadamard_transform, use_uos=False, clip_mode="none", use_dge=False):
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
        rht, dense = E.split_transform(hadamard_transform, False)

        if use_2dblock_x:
            # 2-D blocks never straddle an expert (runs of rows are multiples of 128): one pass, both packings
            ox = E.outer_scales(x2, use_outer_scale, None)
            x_k, x_m = E.quant_2d(x2, fmt, None if ox is None else ox[0:1], True, use_uos)
        else:
            ox = E.outer_scales(x2, use_outer_scale, rht)
            x_k = E.quant_rows(x2, fmt, None if ox is None else ox[0:1], E.RTN, use_uos)
            x_m = E.cols_operand(x2, fmt, use_outer_scale, ox, rht, dense, E.RTN, use_uos, clip_mode)
        w_k, w_t = _quant_weight_stack(w3, fmt, use_2dblock_w, use_outer_scale, use_uos)
        y = _grouped_gemm(x_k, w_k, N, n_exp, group_expert, inputs.dtype)

        extra_x = [x_m.outer] if x_m.outer is not None else []
        extra_w = [w_t.outer] if w_t.outer is not None else []
        ctx.save_for_backward(x_m.codes, x_m.scales, *extra_x, w_t.codes, w_t.scales, *extra_w, group_expert, offs32)
        ctx.dims = (M, K, N, n_exp)
        ctx.fmt, ctx.fmt_grad = fmt, fmt_grad
        ctx.use_sr_grad, ctx.use_outer_scale, ctx.rht, ctx.dense_transform = use_sr_grad, use_outer_scale, rht, dense
        ctx.use_uos, ctx.clip_mode, ctx.use_dge, ctx.use_2dblock_x = use_uos, clip_mode, use_dge, use_2dblock_x
        return y

    @staticmethod
    def backward(ctx, grad_output):
        M, K, N, n_exp = ctx.dims
        saved = ctx.saved_tensors
        if ctx.use_outer_scale:
            xc, xs, xo, wc, ws, wo, group_expert, offs32 = saved
        else:
            (xc, xs, wc, ws, group_expert, offs32), xo, wo = saved, None, None
        x_m = E.Operand(xc, xs, xo, K, M, ctx.fmt)
        w_t = E.Operand(wc, ws, wo, n_exp * K, N, ctx.fmt)
        g2 = E.as_2d_rows(grad_output)
        if ctx.use_2dblock_x:
            og = E.outer_scales(g2, ctx.use_outer_scale, None)
            g_n, g_m = E.quant_2d(g2, ctx.fmt_grad, None if og is None else og[0:1], True, ctx.use_uos,
                                  E.sr_args(ctx.use_sr_grad and L.is_fp4(ctx.fmt_grad), "dy_n", M, N, g2.device))
        else:
            og = E.outer_scales(g2, ctx.use_outer_scale, ctx.rht)
            g_n = E.quant_rows(g2, ctx.fmt_grad, None if og is None else og[0:1],
                               E.sr_args(ctx.use_sr_grad, "dy_n", M, N, g2.device), ctx.use_uos)
            g_m = E.cols_operand(g2, ctx.fmt_grad, ctx.use_outer_scale, og, ctx.rht, ctx.dense_transform,
                                 E.sr_args(ctx.use_sr_grad, "dy_m", N, M, g2.device), ctx.use_uos, ctx.clip_mode)
        grad_inputs = grad_weights = None
        if ctx.needs_input_grad[0]:
            grad_inputs = _grouped_gemm(g_n, w_t, K, n_exp, group_expert, grad_output.dtype)
        if ctx.needs_input_grad[1]:
            grad_weights = torch.empty(n_exp, N, K, dtype=grad_output.dtype, device=g2.device)
            L.grouped_gemm_wgrad_blockscaled(g_m.fmt, x_m.fmt, N, K, M, n_exp, g_m.codes, g_m.scales, x_m.codes,
                                             x_m.scales, offs32, grad_weights, g_m.outer, x_m.outer)
            if ctx.clip_mode == "static" and not ctx.use_2dblock_x:
                # both wgrad operands were clipped to 3/4 of their range (mxfp_grouped_gemm/cg_backward.py:
                # 893-894); 2-D activation blocks are quantised without a clip mode
                grad_weights *= (16.0 / 9.0)
            if ctx.use_dge:
                # factor from the E2M1 code of every weight element (cg_backward.py:912-929); the codes
                # saved for dgrad are the experts' [K, N/2] packings stacked
                wt_codes = w_t.codes.view(n_exp, K, -1)
                for e in range(n_exp):
                    dge.apply_to_weight_grad(grad_weights[e], wt_codes[e])
        return grad_inputs, grad_weights, None, None, None, None, None, None, None, None, None, None, None


def _hadamard(use_hadamard: bool, use_2dblock_x: bool, device) -> Optional[HadamardTransform]:
    if not use_hadamard:
        return None
    assert not use_2dblock_x, "Hadamard transform can only be applied when use_2dblock_x=False."
    with torch.no_grad():
        return HadamardFactory.create_transform(device=device)


@L.traced("mxfp4_grouped_mm")
def _quantize_then_mxfp_scaled_grouped_mm(A, B, offs, use_2dblock_x: bool, use_2dblock_w: bool, use_sr_grad: bool,
                                          use_dge: bool, use_hadamard: bool, clip_mode: str,
                                          use_macro_block_scaling: bool, use_uos: bool = False) -> torch.Tensor:
    clip_mode = clip_mode or "none"
    if clip_mode not in ("none", "static", "dynamic"):
        raise ValueError(f"unknown clip_mode {clip_mode!r}")
    had = _hadamard(use_hadamard, use_2dblock_x, B.device)
    if use_macro_block_scaling:
        from ._two_level import GroupedTwoLevelFunction
        return GroupedTwoLevelFunction.apply(A, B.transpose(-2, -1), offs, bool(use_2dblock_w), bool(use_sr_grad), had,
                                             bool(use_2dblock_x), clip_mode, bool(use_uos), bool(use_dge))
    return GroupedLinearFunction.apply(A, B.transpose(-2, -1), offs, L.FMT_MXFP4, L.FMT_MXFP4, use_2dblock_x,
                                       use_2dblock_w, bool(use_sr_grad), False, had, bool(use_uos), clip_mode,
                                       bool(use_dge))


@L.traced("nvfp4_grouped_mm")
def _quantize_then_nvfp4_scaled_grouped_mm(A, B, offs, use_2dblock_x: bool, use_2dblock_w: bool, use_sr_grad: bool,
                                           use_outer_scale: bool = False, use_hadamard: bool = False,
                                           use_dge: bool = False, scale_format: str = "e4m3") -> torch.Tensor:
    _check_scale_format(scale_format)
    return GroupedLinearFunction.apply(A, B.transpose(-2, -1), offs, L.FMT_NVFP4, L.FMT_NVFP4, use_2dblock_x,
                                       use_2dblock_w, use_sr_grad, use_outer_scale,
                                       _hadamard(use_hadamard, use_2dblock_x, B.device), False, "none", bool(use_dge))


_FP8 = {"e4m3": L.FMT_MXFP8_E4M3, "e5m2": L.FMT_MXFP8_E5M2}


@L.traced("mxfp8_grouped_mm")
def _quantize_then_mxfp8_scaled_grouped_mm(A, B, offs, *, use_2dblock_x: bool = False, use_2dblock_w: bool = True,
                                           use_sr_grad: bool = False, fwd_format: str = "e4m3",
                                           bwd_grad_format: str = "e4m3") -> torch.Tensor:
    if fwd_format not in _FP8 or bwd_grad_format not in _FP8:
        raise ValueError(f"Unsupported FP8 format: {fwd_format} / {bwd_grad_format}")
    if use_sr_grad:
        raise NotImplementedError("MXFP8 stochastic rounding exists only as gfx950 instructions in the reference")
    return GroupedLinearFunction.apply(A, B.transpose(-2, -1), offs, _FP8[fwd_format], _FP8[bwd_grad_format],
                                       use_2dblock_x, use_2dblock_w, False, False, None)


# ---------------------------------------------------------------------------------------------
# Forward grouped GEMMs on operands that are already quantised
# ---------------------------------------------------------------------------------------------
def _grouped_forward_prequantized(fmt_a: int, fmt_b: int, inputs, expert_weights, expert_indices, input_scales,
                                  weight_scales, trans_weights: bool, use_2dblock_x: bool, use_2dblock_w: bool,
                                  output_dtype: torch.dtype) -> torch.Tensor:
    """Y[m] = X[m] W[expert(m)]^T over quantised operands with plain (reference-layout) block scales.

    ``inputs`` [M_buf, K] codes (FP4: two per byte along K) with scales [M_buf, K/32] (or
    [M_buf/32, K/32] for 2-D blocks); ``expert_weights`` [E, N, K] codes (``trans_weights``) or the
    [E, K, N] view of such a tensor, with scales [E, N, K/32] (or [E, N/32, K/32]); ``expert_indices``
    [M_total] gives every row's expert, constant over groups of 128 rows.  Rows from M_total on are zero."""
    torch._check(inputs.dim() == 2 and expert_weights.dim() == 3, lambda: "inputs must be 2-D, expert_weights 3-D")
    m_buf = inputs.shape[0]
    m_total = expert_indices.numel()
    torch._check(m_total > 0)
    torch._check(m_total % ALIGN_SIZE_M == 0,
                 lambda: f"M_total ({m_total}) must be a multiple of group_size_m ({ALIGN_SIZE_M})")
    torch._check(m_buf >= m_total, lambda: f"M_bufferlen ({m_buf}) must be >= M_total ({m_total})")
    w = expert_weights if trans_weights else expert_weights.transpose(-2, -1)     # [E, N, K codes]
    ws = weight_scales if trans_weights else weight_scales.transpose(-2, -1)      # [E, N or N/32, K/32]
    n_exp, N, kc = w.shape
    torch._check(inputs.shape[1] == kc, lambda: f"Input K ({inputs.shape[1]}) must match weight K ({kc})")
    K = kc * 2 if L.is_fp4(fmt_a) else kc
    block = L.block_of(fmt_a)
    a_codes = E.as_2d_rows(inputs.view(torch.uint8))
    b_codes = w.contiguous().view(torch.uint8).reshape(n_exp * N, kc)
    sa = E.pack_plain_scales(input_scales, m_buf, use_2dblock_x, block)
    sb = torch.cat([E.pack_plain_scales(ws[e], N, use_2dblock_w, block) for e in range(n_exp)])
    n_groups = (m_buf + ALIGN_SIZE_M - 1) // ALIGN_SIZE_M
    group_expert = torch.full((n_groups,), -1, dtype=torch.int32, device=inputs.device)
    group_expert[:m_total // ALIGN_SIZE_M] = expert_indices.to(torch.int32)[::ALIGN_SIZE_M]
    out = torch.empty(m_buf, N, dtype=output_dtype, device=inputs.device)
    L.grouped_gemm_blockscaled(fmt_a, fmt_b, m_buf, N, K, n_exp, a_codes, sa, b_codes, sb, group_expert, out)
    return out


def mxfp4_grouped_gemm_forward(inputs, expert_weights, expert_indices, input_scales, weight_scales,
                               trans_weights: bool = True, use_2dblock_x: bool = False, use_2dblock_w: bool = True,
                               output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The reference's ``torch.ops.torchtitan.mxfp4_grouped_gemm_forward``
    (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_forward.py:200-311) on the block-scaled tensor cores."""
    return _grouped_forward_prequantized(L.FMT_MXFP4, L.FMT_MXFP4, inputs, expert_weights, expert_indices,
                                         input_scales, weight_scales, trans_weights, use_2dblock_x, use_2dblock_w,
                                         output_dtype)


def mxfp8_grouped_gemm_forward(inputs, expert_weights, expert_indices, input_scales, weight_scales,
                               trans_weights: bool = True, use_2dblock_x: bool = False, use_2dblock_w: bool = True,
                               lhs_format_id: int = 0, rhs_format_id: int = 0,
                               output_dtype: torch.dtype = torch.bfloat16,
                               use_dot_scaled: Optional[bool] = None) -> torch.Tensor:
    """The reference's ``torch.ops.alto.mxfp8_grouped_gemm_forward``
    (alto/kernels/mxfp8/mxfp8_grouped_gemm/cg_forward.py:222-330); format ids 0 = e4m3, 1 = e5m2.
    ``use_dot_scaled`` selects between the reference's two Triton code paths and has no meaning here."""
    ids = {0: L.FMT_MXFP8_E4M3, 1: L.FMT_MXFP8_E5M2}
    if lhs_format_id not in ids or rhs_format_id not in ids:
        raise ValueError(f"Unsupported FP8 format id: {lhs_format_id} / {rhs_format_id}")
    return _grouped_forward_prequantized(ids[lhs_format_id], ids[rhs_format_id], inputs, expert_weights,
                                         expert_indices, input_scales, weight_scales, trans_weights, use_2dblock_x,
                                         use_2dblock_w, output_dtype)


# ---------------------------------------------------------------------------------------------
# Backward grouped GEMMs on operands that are already quantised
# ---------------------------------------------------------------------------------------------
def _offsets_from_indices(expert_indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Cumulative rows per expert (int32 [E]) from the per-row expert ids; device ops only."""
    counts = torch.bincount(expert_indices.to(torch.int64), minlength=num_experts)[:num_experts]
    return torch.cumsum(counts, 0).to(torch.int32)


def _check_group_rows(m_buf: int, m_total: int) -> None:
    torch._check(m_total > 0)
    torch._check(m_total % ALIGN_SIZE_M == 0,
                 lambda: f"M_total ({m_total}) must be a multiple of group_size_m ({ALIGN_SIZE_M})")
    torch._check(m_buf >= m_total, lambda: f"M_bufferlen ({m_buf}) must be >= M_total ({m_total})")


def _grouped_backward_inputs_prequantized(fmt_a: int, fmt_b: int, grad_output, expert_weights, expert_indices, go_scales,
                                          expert_weight_scales, trans_weights: bool, use_2dblock_x: bool,
                                          use_2dblock_w: bool, output_dtype: torch.dtype) -> torch.Tensor:
    """dX[m] = dY[m] W[expert(m)] over quantised operands with plain scales.  ``grad_output`` [M_buf, N]
    codes along N; ``expert_weights`` the codes of W quantised along N (the reduction axis of this GEMM):
    [E, N, K] (FP4: [E, N/2, K]) when ``trans_weights``, else the [E, K, N] view of such a tensor, with
    scales [E, N/32, K] (or [E, N/32, K/32] for 2-D blocks).  The tensor cores read operands with the
    reduction axis contiguous, so the weight codes are transposed once here (data movement only)."""
    torch._check(grad_output.dim() == 2 and expert_weights.dim() == 3,
                 lambda: "grad_output must be 2-D, expert_weights 3-D")
    m_buf, m_total = grad_output.shape[0], expert_indices.numel()
    _check_group_rows(m_buf, m_total)
    w = expert_weights if trans_weights else expert_weights.transpose(-2, -1)        # [E, N codes, K]
    ws = expert_weight_scales if trans_weights else expert_weight_scales.transpose(-2, -1)   # [E, N/32, K or K/32]
    n_exp, n_codes, K = w.shape
    fp4 = L.is_fp4(fmt_a)
    N = n_codes * 2 if fp4 else n_codes
    torch._check(grad_output.shape[1] == n_codes,
                 lambda: f"grad_output N ({grad_output.shape[1]}) must match weight N ({n_codes})")
    block = L.block_of(fmt_a)
    a_codes = E.as_2d_rows(grad_output.view(torch.uint8))
    b_codes = w.view(torch.uint8).transpose(-2, -1).contiguous().reshape(n_exp * K, n_codes)   # [E*K, N codes]
    sa = E.pack_plain_scales(go_scales, m_buf, use_2dblock_x, block)
    wst = ws.transpose(-2, -1)                                                        # [E, K or K/32, N/32]
    sb = torch.cat([E.pack_plain_scales(wst[e].contiguous(), K, use_2dblock_w, block) for e in range(n_exp)])
    n_groups = (m_buf + ALIGN_SIZE_M - 1) // ALIGN_SIZE_M
    group_expert = torch.full((n_groups,), -1, dtype=torch.int32, device=grad_output.device)
    group_expert[:m_total // ALIGN_SIZE_M] = expert_indices.to(torch.int32)[::ALIGN_SIZE_M]
    out = torch.empty(m_buf, K, dtype=output_dtype, device=grad_output.device)
    L.grouped_gemm_blockscaled(fmt_a, fmt_b, m_buf, K, N, n_exp, a_codes, sa, b_codes, sb, group_expert, out)
    return out


def _grouped_backward_weights_prequantized(fmt_a: int, fmt_b: int, grad_output, inputs, expert_indices, num_experts: int,
                                           go_scales, input_scales, trans_weights: bool, use_2dblock_go: bool,
                                           use_2dblock_x: bool, output_dtype: torch.dtype) -> torch.Tensor:
    """dW[e] = sum over the rows of expert e of dY[m]^T X[m] over operands quantised along the token axis:
    ``grad_output`` [M_buf, N] and ``inputs`` [M_buf, K] codes (FP4: [M_buf/2, .], two tokens per byte) with
    scales [M_buf/32, N] and [M_buf/32, K] (or [M_buf/32, ./32] for 2-D blocks).  Returns [E, N, K]
    (``trans_weights``) or its [E, K, N] view.  Both code matrices are transposed once so that the token
    axis is contiguous (data movement only); each expert's token range comes from ``expert_indices``."""
    torch._check(grad_output.dim() == 2 and inputs.dim() == 2, lambda: "grad_output and inputs must be 2-D")
    fp4 = L.is_fp4(fmt_a)
    m_codes, N = grad_output.shape
    m_codes_x, K = inputs.shape
    torch._check(m_codes == m_codes_x, lambda: f"inputs M ({m_codes_x}) must match grad_output M ({m_codes})")
    m_buf = m_codes * 2 if fp4 else m_codes
    _check_group_rows(m_buf, expert_indices.numel())
    block = L.block_of(fmt_a)
    a_codes = grad_output.view(torch.uint8).t().contiguous()          # [N, M codes]
    b_codes = inputs.view(torch.uint8).t().contiguous()               # [K, M codes]
    sa = E.pack_plain_scales(go_scales.t().contiguous(), N, use_2dblock_go, block)
    sb = E.pack_plain_scales(input_scales.t().contiguous(), K, use_2dblock_x, block)
    offs = _offsets_from_indices(expert_indices, num_experts)
    out = torch.empty(num_experts, N, K, dtype=output_dtype, device=grad_output.device)
    L.grouped_gemm_wgrad_blockscaled(fmt_a, fmt_b, N, K, m_buf, num_experts, a_codes, sa, b_codes, sb, offs, out)
    return out if trans_weights else out.transpose(-2, -1)


def mxfp4_grouped_gemm_backward_inputs(grad_output, expert_weights, expert_indices, go_scales, expert_weight_scales,
                                       trans_weights: bool = True, use_2dblock_x: bool = False,
                                       use_2dblock_w: bool = True, k_pack_w: bool = True,
                                       output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The reference's ``torch.ops.torchtitan.mxfp4_grouped_gemm_backward_inputs``
    (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:500-597) for weights packed along the
    reduction axis N (``k_pack_w=True``); the other packing cannot feed the FP4 tensor cores."""
    if not k_pack_w:
        raise NotImplementedError("weights packed along a non-reduction axis cannot feed the tcgen05 FP4 MMA; "
                                  "quantise along N (or in 2-D blocks, packed along N) and pass k_pack_w=True")
    return _grouped_backward_inputs_prequantized(L.FMT_MXFP4, L.FMT_MXFP4, grad_output, expert_weights, expert_indices,
                                                 go_scales, expert_weight_scales, trans_weights, use_2dblock_x,
                                                 use_2dblock_w, output_dtype)


def mxfp4_grouped_gemm_backward_weights(grad_output, inputs, expert_indices, num_experts: int, go_scales, input_scales,
                                        trans_weights: bool = True, use_2dblock_go: bool = False,
                                        use_2dblock_x: bool = True, k_pack_go: bool = True, k_pack_x: bool = True,
                                        output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The reference's ``torch.ops.torchtitan.mxfp4_grouped_gemm_backward_weights``
    (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:398-497) for operands packed along the token
    axis (``k_pack_go = k_pack_x = True``)."""
    if not (k_pack_go and k_pack_x):
        raise NotImplementedError("operands packed along a non-reduction axis cannot feed the tcgen05 FP4 MMA; "
                                  "quantise along the token axis and pass k_pack_go = k_pack_x = True")
    return _grouped_backward_weights_prequantized(L.FMT_MXFP4, L.FMT_MXFP4, grad_output, inputs, expert_indices,
                                                  num_experts, go_scales, input_scales, trans_weights, use_2dblock_go,
                                                  use_2dblock_x, output_dtype)


_FP8_IDS = {0: L.FMT_MXFP8_E4M3, 1: L.FMT_MXFP8_E5M2}


def _fp8_ids(lhs_format_id: int, rhs_format_id: int):
    if lhs_format_id not in _FP8_IDS or rhs_format_id not in _FP8_IDS:
        raise ValueError(f"Unsupported FP8 format id: {lhs_format_id} / {rhs_format_id}")
    return _FP8_IDS[lhs_format_id], _FP8_IDS[rhs_format_id]


def mxfp8_grouped_gemm_backward_inputs(grad_output, expert_weights, expert_indices, go_scales, expert_weight_scales,
                                       trans_weights: bool = True, use_2dblock_x: bool = False,
                                       use_2dblock_w: bool = True, lhs_format_id: int = 0, rhs_format_id: int = 0,
                                       output_dtype: torch.dtype = torch.bfloat16,
                                       use_dot_scaled: Optional[bool] = None) -> torch.Tensor:
    """The reference's ``torch.ops.alto.mxfp8_grouped_gemm_backward_inputs``
    (alto/kernels/mxfp8/mxfp8_grouped_gemm/cg_backward.py:313-413); format ids 0 = e4m3, 1 = e5m2."""
    fa, fb = _fp8_ids(lhs_format_id, rhs_format_id)
    return _grouped_backward_inputs_prequantized(fa, fb, grad_output, expert_weights, expert_indices, go_scales,
                                                 expert_weight_scales, trans_weights, use_2dblock_x, use_2dblock_w,
                                                 output_dtype)


def mxfp8_grouped_gemm_backward_weights(grad_output, inputs, expert_indices, num_experts: int, go_scales, input_scales,
                                        trans_weights: bool = True, use_2dblock_go: bool = False,
                                        use_2dblock_x: bool = False, lhs_format_id: int = 0, rhs_format_id: int = 0,
                                        output_dtype: torch.dtype = torch.bfloat16,
                                        use_dot_scaled: Optional[bool] = None) -> torch.Tensor:
    """The reference's ``torch.ops.alto.mxfp8_grouped_gemm_backward_weights``
    (alto/kernels/mxfp8/mxfp8_grouped_gemm/cg_backward.py:416-513)."""
    fa, fb = _fp8_ids(lhs_format_id, rhs_format_id)
    return _grouped_backward_weights_prequantized(fa, fb, grad_output, inputs, expert_indices, num_experts, go_scales,
                                                  input_scales, trans_weights, use_2dblock_go, use_2dblock_x,
                                                  output_dtype)
