"""Format-independent engine of the low-precision linear: operand preparation (one fused
quantize launch per operand use) and the three block-scaled GEMMs.

All three reference autograd functions share this structure
(alto/kernels/fp4/nvfp4/nvfp_linear.py:53-278, alto/kernels/fp4/mxfp4/mxfp_linear.py:266-570,
alto/kernels/mxfp8/mxfp8_linear.py:305-439):

  forward : X along K, W along K                      -> Y  = Xq Wq^T
            saves X along M (after the optional Hadamard rotation) and W along N
  backward: dY along N                                -> dX = dYq Wq       (reduction over N)
            (H) dY along M                            -> dW = dYq^T Xq     (reduction over M)

Every GEMM operand is stored with its reduction axis contiguous and carries its scales in
the packed layout the tensor cores read, so the quantizers write exactly what the GEMM
consumes and nothing is dequantised.
"""
from __future__ import annotations

import contextlib
import os
import threading
from typing import Callable, Optional, Tuple

import torch

from . import _lib as L
from . import dge

# ---------------------------------------------------------------------------------------
# scratch and random-bit plumbing
# ---------------------------------------------------------------------------------------
_scratch = {}


def amax_scratch(device: torch.device) -> torch.Tensor:
    """Zeroed per-(device, stream) scratch of the amax kernel (the kernel leaves it zeroed)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.zeros(L.AMAX_SCRATCH_BYTES // 4, dtype=torch.int32, device=device)
        _scratch[key] = buf
    return buf


_sr_bits_provider: Optional[Callable[[str, Tuple[int, ...], torch.device], torch.Tensor]] = None


@contextlib.contextmanager
def explicit_sr_bits(provider: Callable[[str, Tuple[int, ...], torch.device], torch.Tensor]):
    """Within the context, stochastic rounding inside the linear functions consumes the random
    words returned by ``provider(name, shape, device)`` (int32 tensor of ``shape`` =
    [2, rows, cols/2] in the quantisation-axis-last view; names: "dy_n", "dy_m") instead of
    generating Philox words in the kernel.  Used to check bit parity against the oracle."""
    global _sr_bits_provider
    prev = _sr_bits_provider
    _sr_bits_provider = provider
    try:
        yield
    finally:
        _sr_bits_provider = prev


def draw_philox() -> Tuple[int, int]:
    """Seed and offset from the global CPU generator, as the reference draws them when none is
    given (alto/kernels/fp4/nvfp4/nvfp_quantization.py:587-590)."""
    v = torch.randint(0, 2 ** 31 - 1, (2,))
    return int(v[0]), int(v[1])


def sr_args(use_sr: bool, name: str, rows: int, cols: int, device) -> dict:
    if not use_sr:
        return dict(rounding=L.ROUND_RTN)
    if _sr_bits_provider is not None:
        bits = _sr_bits_provider(name, (2, rows, cols // 2), device)
        return dict(rounding=L.ROUND_SR_BITS, rand_bits=bits.contiguous())
    # The reference's scheme: (seed, offset) drawn from the global CPU generator, one table of
    # Philox words per quantizer launch, repeated over its 64 x 64 tiles (rows x cols is the
    # quantisation-axis-last view).  The table costs one tiny launch and replaces ~15 instructions
    # of Philox per element inside the quantizer by cached loads.
    seed, offset = draw_philox()
    tile = L.sr_tile_dims(rows, cols)
    return dict(rounding=L.ROUND_SR_BITS, rand_bits=L.philox_tile(seed, offset, tile[0], tile[1], device),
                rand_tile=tile)


RTN = dict(rounding=L.ROUND_RTN)

# ---------------------------------------------------------------------------------------
# operands
# ---------------------------------------------------------------------------------------


class Operand:
    """Codes + packed scales (+ NVFP4 outer scale) of one GEMM operand [rows, k], k contiguous.
    ``macro``: the operand's macro-block factor codes (``_lib.MacroScale``) in the two-level MXFP4 flow."""

    __slots__ = ("codes", "scales", "outer", "rows", "k", "fmt", "macro")

    def __init__(self, codes, scales, outer, rows, k, fmt, macro=None):
        self.codes, self.scales, self.outer, self.rows, self.k, self.fmt = codes, scales, outer, rows, k, fmt
        self.macro = macro


def as_2d_rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    return x2


def outer_scales(x2: torch.Tensor, use_outer: bool, rht: Optional[L.Rht]) -> Optional[torch.Tensor]:
    """[outer(x), outer(H x)] from ONE read of x, or None when outer scaling is off."""
    if not use_outer:
        return None
    amax_bits = torch.empty(2, dtype=torch.int32, device=x2.device)
    outer = torch.empty(2, dtype=torch.float32, device=x2.device)
    L.amax(x2, amax_bits, outer, amax_scratch(x2.device), rht)
    return outer


def _packed(rows: int, ncols: int, device) -> torch.Tensor:
    return torch.empty(L.packed_scale_bytes(rows, ncols), dtype=torch.uint8, device=device)


def _code_cols(fmt: int, n: int) -> int:
    return n // 2 if L.is_fp4(fmt) else n


def quant_rows(x2, fmt, outer, sr: dict, use_uos: bool = False) -> Operand:
    R, Cc = x2.shape
    codes = torch.empty(R, _code_cols(fmt, Cc), dtype=torch.uint8, device=x2.device)
    sf = _packed(R, Cc // L.block_of(fmt), x2.device)
    L.quantize_rowwise(x2, fmt, codes, None, sf, outer_scale=outer, use_uos=use_uos, **sr)
    return Operand(codes, sf, outer, R, Cc, fmt)


def quant_cols(x2, fmt, outer, rht, sr: dict, use_uos: bool = False, clip_mode: str = "none") -> Operand:
    R, Cc = x2.shape
    codes = torch.empty(Cc, _code_cols(fmt, R), dtype=torch.uint8, device=x2.device)
    sf = _packed(Cc, R // L.block_of(fmt), x2.device)
    L.quantize_colwise(x2, fmt, codes, None, sf, outer_scale=outer, rht=rht, use_uos=use_uos, clip_mode=clip_mode,
                       **sr)
    return Operand(codes, sf, outer, Cc, R, fmt)


def quant_2d(x2, fmt, outer, want_t: bool, use_uos: bool = False, sr: Optional[dict] = None) -> Tuple[Operand, Optional[Operand]]:
    R, Cc = x2.shape
    b = L.block_of(fmt)
    ck = torch.empty(R, _code_cols(fmt, Cc), dtype=torch.uint8, device=x2.device)
    sk = _packed(R, Cc // b, x2.device)
    ct = torch.empty(Cc, _code_cols(fmt, R), dtype=torch.uint8, device=x2.device) if want_t else None
    stt = _packed(Cc, R // b, x2.device) if want_t else None
    L.quantize_2d(x2, fmt, ck, ct, None, sk, stt, outer_scale=outer, use_uos=use_uos, **(sr or {}))
    return Operand(ck, sk, outer, R, Cc, fmt), (Operand(ct, stt, outer, Cc, R, fmt) if want_t else None)


def gemm(a: Operand, b: Operand, out_dtype: torch.dtype) -> torch.Tensor:
    """D[a.rows, b.rows] = alpha * A B^T, alpha = product of the operands' outer scales."""
    assert a.k == b.k
    out = torch.empty(a.rows, b.rows, dtype=out_dtype, device=a.codes.device)
    L.gemm_blockscaled(a.fmt, b.fmt, a.rows, b.rows, a.k, a.codes, a.scales, b.codes, b.scales, out, a.outer,
                       b.outer)
    return out


def check_dims(name: str, M: int, K: int, N: int) -> None:
    torch._check(K % 32 == 0, lambda: f"{name} on B200 requires in_features ({K}) divisible by 32")
    torch._check(N % 32 == 0, lambda: f"{name} on B200 requires out_features ({N}) divisible by 32")
    torch._check(M % 32 == 0, lambda: (
        f"{name} on B200 requires the token count ({M}) divisible by 32: the wgrad operands are quantised "
        "in blocks along the token axis and stored in 16-byte aligned rows"))


def split_transform(hadamard_transform, use_2dblock_x: bool):
    """-> (rht, dense): launch parameters for the quantizers' fused 16-point butterfly, or the
    transform object itself when it has to run as its own (dense) kernel; both None without one."""
    if hadamard_transform is None or use_2dblock_x:
        return None, None
    if hadamard_transform.is_fused:
        return hadamard_transform.device_params(), None
    return None, hadamard_transform


def cols_operand(t2, fmt, use_outer_scale, o, rht, dense, sr: dict, use_uos: bool = False,
                 clip_mode: str = "none") -> Operand:
    """t2 quantised along its token axis after the optional rotation.  ``o`` = outer_scales(t2, .., rht).
    The MXFP4 clip mode applies to these operands only (alto/kernels/fp4/mxfp4/mxfp_linear.py:383-390, 491-498)."""
    if dense is not None:
        th = dense(t2, left_mul=True)          # bf16(H t), as the reference materialises it
        oh = outer_scales(th, use_outer_scale, None)
        return quant_cols(th, fmt, None if oh is None else oh[0:1], None, sr, use_uos, clip_mode)
    o_m = None if o is None else (o[1:2] if rht is not None else o[0:1])
    return quant_cols(t2, fmt, o_m, rht, sr, use_uos, clip_mode)


class PrequantizedWeight:
    """A weight [N, K] that exists only as its two GEMM operands (W along K for fprop, W along N for dgrad),
    e.g. assembled from an all-gather of quantised shards.  It stands in for the weight tensor inside the
    linear functions: ``shape`` / ``dtype`` describe the weight it was quantised from, ``detach`` and ``to``
    return it unchanged (there is nothing left to convert)."""

    __slots__ = ("w_k", "w_t", "shape", "dtype", "fmt", "is_2d")

    def __init__(self, w_k: Operand, w_t: Operand, shape, dtype, fmt: int, is_2d: bool = True):
        self.w_k, self.w_t, self.shape, self.dtype, self.fmt, self.is_2d = w_k, w_t, tuple(shape), dtype, fmt, is_2d

    def detach(self):
        return self

    def to(self, *args, **kwargs):
        return self

    def dim(self):
        return len(self.shape)


def activation_operands(x2, fmt, *, use_2dblock_x, use_outer_scale, rht, dense=None, use_uos=False, clip_mode="none"):
    """(x_k, x_m): X along K (fprop) and X along M after the optional Hadamard rotation (wgrad)."""
    ox = outer_scales(x2, use_outer_scale, None if use_2dblock_x else rht)
    if use_2dblock_x:
        return quant_2d(x2, fmt, None if ox is None else ox[0:1], True, use_uos)
    x_k = quant_rows(x2, fmt, None if ox is None else ox[0:1], RTN, use_uos)
    x_m = cols_operand(x2, fmt, use_outer_scale, ox, rht, dense, RTN, use_uos, clip_mode)
    return x_k, x_m


def weight_operands(w2, fmt, *, use_2dblock_w, use_outer_scale, use_uos=False):
    """(w_k, w_t): W along K (fprop) and W along N (dgrad)."""
    if isinstance(w2, PrequantizedWeight):
        torch._check(w2.fmt == fmt and w2.is_2d == bool(use_2dblock_w), lambda: (
            "the pre-quantised weight was built for another recipe than the one this linear runs"))
        return w2.w_k, w2.w_t
    ow = outer_scales(w2, use_outer_scale, None)
    if use_2dblock_w:
        return quant_2d(w2, fmt, None if ow is None else ow[0:1], True, use_uos)
    w_k = quant_rows(w2, fmt, None if ow is None else ow[0:1], RTN, use_uos)
    w_t = quant_cols(w2, fmt, None if ow is None else ow[0:1], None, RTN, use_uos)
    return w_k, w_t


def forward_operands(x2, w2, fmt, *, use_2dblock_x, use_2dblock_w, use_outer_scale, rht, dense=None,
                     use_uos=False, clip_mode="none"):
    """Returns (x_k, x_m, w_k, w_t): X along K (fprop), X along M after the optional Hadamard
    rotation (wgrad), W along K (fprop), W along N (dgrad)."""
    # Every pass over one tensor is launched before the first pass over the other: X at the benchmark
    # shapes (64 MiB) stays in the 126 MB L2 between its amax pass and its two quantizers, and W's
    # quantizer finds the tail of W that its amax pass left there.
    x_k, x_m = activation_operands(x2, fmt, use_2dblock_x=use_2dblock_x, use_outer_scale=use_outer_scale, rht=rht,
                                   dense=dense, use_uos=use_uos, clip_mode=clip_mode)
    w_k, w_t = weight_operands(w2, fmt, use_2dblock_w=use_2dblock_w, use_outer_scale=use_outer_scale, use_uos=use_uos)
    return x_k, x_m, w_k, w_t


def backward_operands(g2, fmt, *, use_2dblock_x, use_sr_grad, use_outer_scale, rht, dense=None, use_uos=False,
                      clip_mode="none"):
    """dY along N for dgrad and (after the optional Hadamard rotation) along M for wgrad."""
    M, N = g2.shape
    og = outer_scales(g2, use_outer_scale, None if use_2dblock_x else rht)
    if use_2dblock_x:
        # quantised once; both GEMMs use the same codes (2-D scales are axis-invariant)
        return quant_2d(g2, fmt, None if og is None else og[0:1], True, use_uos,
                        sr_args(use_sr_grad, "dy_n", M, N, g2.device))
    g_n = quant_rows(g2, fmt, None if og is None else og[0:1], sr_args(use_sr_grad, "dy_n", M, N, g2.device),
                     use_uos)
    g_m = cols_operand(g2, fmt, use_outer_scale, og, rht, dense, sr_args(use_sr_grad, "dy_m", N, M, g2.device),
                       use_uos, clip_mode)
    return g_n, g_m


# ---------------------------------------------------------------------------------------
# overlap of quantizers (ALU work) with GEMMs (tensor-core work)
# ---------------------------------------------------------------------------------------
#: With OVERLAP on, the quantizer whose output is not needed by the next GEMM is launched on a side
#: stream right after that GEMM:
#:   forward : fprop GEMM   ||  X along M (needed only in backward)
#:   backward: wgrad GEMM   ||  dY along N (needed by the dgrad GEMM that follows)
#: Results are identical; only the launch order differs.  Off by default (ALTO_B200_OVERLAP=1 turns it
#: on): the CTA-pair GEMM fills every SM, so a concurrent quantizer can only take SMs away from it.
OVERLAP = os.environ.get("ALTO_B200_OVERLAP", "0") == "1"
_side_streams = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    s = _side_streams.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _side_streams[device.index] = s
    return s


# A caller that shards the weight by output features must sum the partial dX of all ranks; it can
# start that all-reduce as soon as the dgrad GEMM has been launched and let it run beside the wgrad
# quantizer and GEMM.  The hook is armed on the autograd thread right before the linear's backward runs
# (``distributed._ArmDxAllReduce``) and taken by that backward; it receives the contiguous dX [M, K].
_dx_hook = threading.local()


def set_dx_ready_hook(fn) -> None:
    _dx_hook.fn = fn


def take_dx_ready_hook():
    fn = getattr(_dx_hook, "fn", None)
    _dx_hook.fn = None
    return fn


def _keep_for(stream, *tensors) -> None:
    """Tell the caching allocator that ``tensors`` are also in use on ``stream``."""
    for t in tensors:
        if t is not None:
            t.record_stream(stream)


def linear_forward(ctx, name: str, x, weight, fmt, *, use_2dblock_x, use_2dblock_w, use_sr_grad, use_outer_scale,
                   hadamard_transform, use_uos: bool = False, clip_mode: str = "none", use_dge: bool = False):
    """Shared body of the three autograd ``forward`` methods."""
    if not x.is_cuda:
        raise RuntimeError(f"{name} runs on CUDA tensors only (no CPU fallback)")
    original_shape = x.shape
    x2 = as_2d_rows(x.detach())
    pre = isinstance(weight, PrequantizedWeight)
    w2 = weight if pre else as_2d_rows(weight.detach())
    M, K = x2.shape
    N = w2.shape[0]
    check_dims(name, M, K, N)
    rht, dense = split_transform(hadamard_transform, use_2dblock_x)
    ctx.xm_ready = None
    plain = not use_uos and clip_mode == "none"
    if OVERLAP and not use_2dblock_x and dense is None and plain and not pre:
        main = torch.cuda.current_stream(x2.device)
        side = _side_stream(x2.device)
        ox = outer_scales(x2, use_outer_scale, rht)
        ow = outer_scales(w2, use_outer_scale, None)
        x_k = quant_rows(x2, fmt, None if ox is None else ox[0:1], RTN)
        if use_2dblock_w:
            w_k, w_t = quant_2d(w2, fmt, None if ow is None else ow[0:1], True)
        else:
            w_k = quant_rows(w2, fmt, None if ow is None else ow[0:1], RTN)
            w_t = quant_cols(w2, fmt, None if ow is None else ow[0:1], None, RTN)
        ready = torch.cuda.Event()
        ready.record(main)
        y = gemm(x_k, w_k, x.dtype)  # submitted first so that its CTAs take the SMs first
        o_m = None if ox is None else (ox[1:2] if rht is not None else ox[0:1])
        side.wait_event(ready)
        with torch.cuda.stream(side):
            x_m = quant_cols(x2, fmt, o_m, rht, RTN)
        ctx.xm_ready = torch.cuda.Event()
        ctx.xm_ready.record(side)
        _keep_for(side, x2, ox)
        _keep_for(main, x_m.codes, x_m.scales)
    else:
        x_k, x_m, w_k, w_t = forward_operands(x2, w2, fmt, use_2dblock_x=use_2dblock_x, use_2dblock_w=use_2dblock_w,
                                              use_outer_scale=use_outer_scale, rht=rht, dense=dense,
                                              use_uos=use_uos, clip_mode=clip_mode)
        y = gemm(x_k, w_k, x.dtype)
    extra_x = [x_m.outer] if x_m.outer is not None else []
    extra_w = [w_t.outer] if w_t.outer is not None else []
    ctx.save_for_backward(x_m.codes, x_m.scales, *extra_x, w_t.codes, w_t.scales, *extra_w)
    ctx.dims = (M, K, N)
    ctx.fmt = fmt
    ctx.use_2dblock_x = use_2dblock_x
    ctx.use_sr_grad = use_sr_grad
    ctx.use_outer_scale = use_outer_scale
    ctx.rht = rht
    ctx.dense_transform = dense
    ctx.use_uos, ctx.clip_mode, ctx.use_dge = use_uos, clip_mode, use_dge
    return y.view(*original_shape[:-1], N)


def linear_backward(ctx, grad_output):
    """Shared body of the three autograd ``backward`` methods; returns (dX, dW)."""
    M, K, N = ctx.dims
    saved = ctx.saved_tensors
    if ctx.use_outer_scale:
        xc, xs, xo, wc, ws, wo = saved
    else:
        (xc, xs, wc, ws), xo, wo = saved, None, None
    x_m = Operand(xc, xs, xo, K, M, ctx.fmt)
    w_t = Operand(wc, ws, wo, K, N, ctx.fmt)
    original_shape = grad_output.shape
    g2 = as_2d_rows(grad_output)
    main = torch.cuda.current_stream(g2.device)
    if ctx.xm_ready is not None:
        main.wait_event(ctx.xm_ready)
    need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    grad_inputs = grad_weights = None
    dx_hook = take_dx_ready_hook()      # always taken here, so that an armed hook never outlives this backward
    plain = not ctx.use_uos and ctx.clip_mode == "none"
    if OVERLAP and not ctx.use_2dblock_x and need_dx and need_dw and ctx.dense_transform is None and plain:
        fmt, rht = ctx.fmt, ctx.rht
        side = _side_stream(g2.device)
        og = outer_scales(g2, ctx.use_outer_scale, rht)
        sr_n = sr_args(ctx.use_sr_grad, "dy_n", M, N, g2.device)  # drawn in the same order as without overlap
        sr_m = sr_args(ctx.use_sr_grad, "dy_m", N, M, g2.device)
        o_m = None if og is None else (og[1:2] if rht is not None else og[0:1])
        g_m = quant_cols(g2, fmt, o_m, rht, sr_m)
        ready = torch.cuda.Event()
        ready.record(main)
        grad_weights = gemm(g_m, x_m, grad_output.dtype)  # wgrad first; dY along N is quantised beside it
        side.wait_event(ready)
        with torch.cuda.stream(side):
            g_n = quant_rows(g2, fmt, None if og is None else og[0:1], sr_n)
        done = torch.cuda.Event()
        done.record(side)
        _keep_for(side, g2, og, sr_n.get("rand_bits"))
        _keep_for(main, g_n.codes, g_n.scales)
        main.wait_event(done)
        grad_inputs = gemm(g_n, w_t, grad_output.dtype).view(*original_shape[:-1], K)
        if ctx.use_dge:
            grad_weights = dge.apply_to_weight_grad(grad_weights, w_t.codes)
        return grad_inputs, grad_weights
    if dx_hook is not None and need_dx and not ctx.use_2dblock_x:
        # dgrad first, with only the operand it needs; the hook (an asynchronous all-reduce of dX) then runs
        # beside the second quantizer of dY and the wgrad GEMM.  Random words are drawn in the usual order.
        og = outer_scales(g2, ctx.use_outer_scale, ctx.rht)
        sr_n = sr_args(ctx.use_sr_grad, "dy_n", M, N, g2.device)
        sr_m = sr_args(ctx.use_sr_grad, "dy_m", N, M, g2.device)
        g_n = quant_rows(g2, ctx.fmt, None if og is None else og[0:1], sr_n, ctx.use_uos)
        dx2 = gemm(g_n, w_t, grad_output.dtype)
        dx_hook(dx2)
        grad_inputs = dx2.view(*original_shape[:-1], K)
        need_dx = False
        g_m = cols_operand(g2, ctx.fmt, ctx.use_outer_scale, og, ctx.rht, ctx.dense_transform, sr_m, ctx.use_uos,
                           ctx.clip_mode) if need_dw else None
    else:
        g_n, g_m = backward_operands(g2, ctx.fmt, use_2dblock_x=ctx.use_2dblock_x, use_sr_grad=ctx.use_sr_grad,
                                     use_outer_scale=ctx.use_outer_scale, rht=ctx.rht, dense=ctx.dense_transform,
                                     use_uos=ctx.use_uos, clip_mode=ctx.clip_mode)
    if need_dx:
        grad_inputs = gemm(g_n, w_t, grad_output.dtype).view(*original_shape[:-1], K)
    if need_dw:
        grad_weights = gemm(g_m, x_m, grad_output.dtype)
        if ctx.clip_mode == "static" and not ctx.use_2dblock_x:
            # both wgrad operands were clipped to 3/4 of their range (alto/kernels/fp4/mxfp4/mxfp_linear.py:
            # 543-544); 2-D activation blocks take no clip mode (:310-315, 444-450), so nothing is undone there
            grad_weights *= (16.0 / 9.0)
        if ctx.use_dge:
            grad_weights = dge.apply_to_weight_grad(grad_weights, w_t.codes)
    return grad_inputs, grad_weights


def pack_plain_scales(scales: torch.Tensor, rows: int, is_2d: bool, block: int) -> torch.Tensor:
    """Plain scales ([rows, K/block], or [rows/block, K/block] when ``is_2d``; uint8 exponents or
    fp32 values on the E4M3 grid) -> the packed layout of the GEMM.  Pure data movement on a
    tensor that is 1/16 or 1/32 of the operand; done with tensor ops."""
    s = scales
    if s.dtype == torch.float32:
        s = s.to(torch.float8_e4m3fn).view(torch.uint8)
    assert s.dtype == torch.uint8
    if is_2d:
        s = s.repeat_interleave(block, dim=0)
    assert s.shape[0] == rows, f"scale rows {s.shape[0]} != operand rows {rows}"
    ncols = s.shape[1]
    rt, ct = (rows + 127) // 128, (ncols + 3) // 4
    buf = torch.zeros(rt * 128, ct * 4, dtype=torch.uint8, device=s.device)
    buf[:rows, :ncols] = s
    return buf.view(rt, 4, 32, ct, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)
