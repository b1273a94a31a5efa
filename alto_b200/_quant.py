"""Shared host logic of the public quantize / dequantize ops.

The reference's ops transpose the quantisation axis last, flatten to 2-D, launch one
Triton kernel and return transposed views (alto/kernels/fp4/mxfp4/mxfp_quantization.py:
439-484).  Here the same logical results come from three kernels that avoid the physical
transpose: row-wise (axis=-1), column-wise (axis=-2 / 0) and 2D-block.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L

_CODE_DTYPE = {L.FMT_NVFP4: torch.uint8, L.FMT_MXFP4: torch.uint8,
               L.FMT_MXFP8_E4M3: torch.float8_e4m3fn, L.FMT_MXFP8_E5M2: torch.float8_e5m2}


def _norm_axis(axis: int, ndim: int) -> int:
    a = axis if axis < 0 else axis - ndim
    if a not in (-1, -2):
        raise ValueError(f"axis must address one of the last two dimensions, got {axis}")
    return a


def _rand_planes(rand_bits: Optional[torch.Tensor], rows: int, cols: int):
    if rand_bits is None:
        return None
    assert rand_bits.dtype in (torch.int32, torch.uint32), "random bits are 32-bit words"
    assert tuple(rand_bits.shape) == (2, rows, cols // 2), (
        f"random bits must be [2, {rows}, {cols // 2}] in the quantisation-axis-last view, got {tuple(rand_bits.shape)}")
    return rand_bits.contiguous()


def quantize(x: torch.Tensor, fmt: int, axis: int, is_2d: bool, *, outer_scale: Optional[torch.Tensor] = None,
             rounding: int = L.ROUND_RTN, rand_bits: Optional[torch.Tensor] = None, philox=(0, 0),
             rht: Optional[L.Rht] = None, clip_mode: str = "none",
             use_uos: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (codes, plain scales) with the reference's logical shapes and transposed views."""
    opts = dict(clip_mode=clip_mode, use_uos=use_uos)
    if not x.is_cuda:
        raise RuntimeError("alto_b200 quantizers run on CUDA tensors only (no CPU fallback)")
    block = L.block_of(fmt)
    fp4 = L.is_fp4(fmt)
    a = _norm_axis(axis, x.dim())
    scale_dtype = torch.float32 if fmt == L.FMT_NVFP4 else torch.uint8
    if x.dim() < 2:
        x = x.reshape(1, -1)
    lead = x.shape[:-2]
    M, N = x.shape[-2], x.shape[-1]
    dev = x.device

    if is_2d:
        x3 = x.reshape(-1, M, N).contiguous()
        nb = x3.shape[0]
        sr = {}
        if rounding != L.ROUND_RTN:
            # words belong to (row, column pair) of the quantisation-axis-last view, leading dimensions
            # flattened into its rows
            if not fp4:
                raise NotImplementedError("stochastic rounding is implemented for the FP4 formats")
            if a == -2:
                # that view is the transposed matrix: quantise a transposed copy along its last axis (2-D
                # blocks are symmetric) and hand the results back as transposed views, which is what the
                # reference does with a strided view (alto/kernels/fp4/mxfp4/mxfp_quantization.py:439, 484)
                ct, st = quantize(x.transpose(-1, -2).contiguous(), fmt, -1, True, outer_scale=outer_scale,
                                  rounding=rounding, rand_bits=rand_bits, philox=philox, clip_mode=clip_mode,
                                  use_uos=use_uos)
                return ct.transpose(-1, -2), st.transpose(-1, -2)
            if rounding == L.ROUND_SR_PHILOX:
                tile = L.sr_tile_dims(nb * M, N)
                sr = dict(rounding=L.ROUND_SR_BITS, rand_tile=tile,
                          rand_bits=L.philox_tile(philox[0], philox[1], tile[0], tile[1], dev))
            else:
                sr = dict(rounding=L.ROUND_SR_BITS, rand_bits=_rand_planes(rand_bits, nb * M, N))
        codes_k = torch.empty(nb, M, N // 2 if fp4 else N, dtype=torch.uint8, device=dev)
        codes_t = torch.empty(nb, N, M // 2 if fp4 else M, dtype=torch.uint8, device=dev) if a == -2 else None
        scales = torch.empty(nb, M // block, N // block, dtype=scale_dtype, device=dev)
        if nb == 1:
            L.quantize_2d(x3[0], fmt, codes_k[0], None if codes_t is None else codes_t[0], scales[0],
                          outer_scale=outer_scale, **opts, **sr)
        else:
            L.quantize_2d_batched(x3, fmt, codes_k, codes_t, scales, outer_scale=outer_scale, **opts, **sr)
        if a == -1:
            codes = codes_k.reshape(*lead, M, codes_k.shape[-1])
        else:  # physical [N, M/2], returned as its transpose like the reference
            codes = codes_t.reshape(*lead, N, codes_t.shape[-1]).transpose(-1, -2)
        scales = scales.reshape(*lead, M // block, N // block)
        return codes.view(_CODE_DTYPE[fmt]), scales

    if a == -1:
        x2 = x.reshape(-1, N)
        if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 != 0:
            x2 = x2.contiguous()
        R = x2.shape[0]
        codes = torch.empty(R, N // 2 if fp4 else N, dtype=torch.uint8, device=dev)
        scales = torch.empty(R, N // block, dtype=scale_dtype, device=dev)
        if rounding == L.ROUND_SR_PHILOX:
            # the reference's words for (seed, offset): one table per launch, repeated over its tiles
            tile = L.sr_tile_dims(R, N)
            L.quantize_rowwise(x2, fmt, codes, scales, None, rounding=L.ROUND_SR_BITS, outer_scale=outer_scale,
                               rand_bits=L.philox_tile(philox[0], philox[1], tile[0], tile[1], dev), rand_tile=tile,
                               **opts)
        else:
            L.quantize_rowwise(x2, fmt, codes, scales, None, rounding=rounding, outer_scale=outer_scale,
                               rand_bits=_rand_planes(rand_bits, R, N), philox=philox, **opts)
        return (codes.reshape(*x.shape[:-1], codes.shape[-1]).view(_CODE_DTYPE[fmt]),
                scales.reshape(*x.shape[:-1], N // block))

    # axis = -2: blocks of consecutive rows; physical output is the transposed matrix
    x3 = x.reshape(-1, M, N)
    nb = x3.shape[0]
    codes = torch.empty(nb, N, M // 2 if fp4 else M, dtype=torch.uint8, device=dev)
    scales = torch.empty(nb, N, M // block, dtype=scale_dtype, device=dev)
    rb = None if rand_bits is None else _rand_planes(rand_bits, nb * N, M).reshape(2, nb, N, M // 2)
    table, tile = None, (0, 0)
    if rounding == L.ROUND_SR_PHILOX:
        # the reference flattens the leading dimensions into the rows of the axis-last view [nb * N, M]
        tile = L.sr_tile_dims(nb * N, M)
        if nb > 1 and N % tile[0] != 0:
            raise NotImplementedError("stochastic rounding of a batched tensor whose rows do not fill whole "
                                      "64-row tiles per batch entry is not implemented")
        table = L.philox_tile(philox[0], philox[1], tile[0], tile[1], dev)
    for b in range(nb):
        xb = x3[b]
        if xb.stride(-1) != 1 or (xb.stride(0) * xb.element_size()) % 16 != 0:
            xb = xb.contiguous()
        if table is not None:
            L.quantize_colwise(xb, fmt, codes[b], scales[b], None, rounding=L.ROUND_SR_BITS, outer_scale=outer_scale,
                               rand_bits=table, rand_tile=tile, rht=rht, **opts)
            continue
        L.quantize_colwise(xb, fmt, codes[b], scales[b], None, rounding=rounding, outer_scale=outer_scale,
                           rand_bits=None if rb is None else rb[:, b].contiguous(), rht=rht,
                           philox=(philox[0], philox[1] + b * (N * M // 4)), **opts)
    codes = codes.reshape(*lead, N, codes.shape[-1]).transpose(-1, -2)
    scales = scales.reshape(*lead, N, M // block).transpose(-1, -2)
    return codes.view(_CODE_DTYPE[fmt]), scales


def dequantize(codes: torch.Tensor, scales: torch.Tensor, fmt: int, axis: int, is_2d: bool, out_dtype: torch.dtype,
               outer_scale: Optional[torch.Tensor] = None, static_clip: bool = False) -> torch.Tensor:
    if not codes.is_cuda:
        raise RuntimeError("alto_b200 dequantizers run on CUDA tensors only (no CPU fallback)")
    assert out_dtype in (torch.float32, torch.bfloat16)
    block = L.block_of(fmt)
    fp4 = L.is_fp4(fmt)
    a = _norm_axis(axis, codes.dim())
    c = codes.transpose(a, -1)
    s = scales.transpose(a, -1)
    shp = c.shape
    cols = shp[-1] * (2 if fp4 else 1)
    if is_2d:
        c3 = c.reshape(-1, shp[-2], shp[-1]).contiguous().view(torch.uint8)
        s3 = s.reshape(-1, shp[-2] // block, cols // block).contiguous()
    else:
        c3 = c.reshape(1, -1, shp[-1]).contiguous().view(torch.uint8)
        s3 = s.reshape(1, -1, cols // block).contiguous()
    if fmt == L.FMT_NVFP4:
        s3 = s3.float()
    out = torch.empty(c3.shape[0], c3.shape[1], cols, dtype=out_dtype, device=codes.device)
    osc = None if outer_scale is None else outer_scale.to(device=codes.device, dtype=torch.float32).reshape(1)
    for b in range(c3.shape[0]):
        L.dequantize(c3[b], s3[b], fmt, is_2d, c3.shape[1], cols, out[b], osc, static_clip)
    return out.reshape(*shp[:-1], cols).transpose(a, -1)
