"""ctypes binding of ``libaltob200.so`` (the C ABI declared in ``include/altob200.h``).

There is no CPU fallback: if the shared library is missing, or a call returns a negative
status, an exception is raised.  Every wrapper takes torch tensors only to read their
device pointers and launches on the calling thread's current CUDA stream, as the
reference's Triton launches do (forward on the caller's thread, backward on the autograd
engine's device thread).
"""
from __future__ import annotations

import ctypes as C
import functools
import os
import threading
from pathlib import Path
from typing import Optional, Sequence

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libaltob200.so"

# enums of include/altob200.h
FMT_NVFP4, FMT_MXFP4, FMT_MXFP8_E4M3, FMT_MXFP8_E5M2 = 0, 1, 2, 3
DT_BF16, DT_F32 = 0, 1
SCALE_PLAIN, SCALE_PACKED = 1, 2
ROUND_RTN, ROUND_SR_BITS, ROUND_SR_PHILOX = 0, 1, 2
AMAX_SCRATCH_BYTES = 16

E_SHAPE, E_ALIGN, E_TIMEOUT, E_CUDA, E_UNSUPPORTED, E_LIMIT = -1, -2, -3, -4, -5, -6

#: every symbol the header declares (checked by the CPU test-suite)
EXPORTED_SYMBOLS = (
    "altob200_version",
    "altob200_status_string",
    "altob200_packed_scale_bytes",
    "altob200_status_read",
    "altob200_amax",
    "altob200_amax_noalloc",
    "altob200_quantize_rowwise",
    "altob200_quantize_colwise",
    "altob200_quantize_2d",
    "altob200_quantize_2d_batched",
    "altob200_dequantize",
    "altob200_philox_tile",
    "altob200_rht",
    "altob200_rht_dense",
    "altob200_macro_block_scaling",
    "altob200_macro_block_descaling",
    "altob200_gather_rows",
    "altob200_combine_rows",
    "altob200_spread_rows",
    "altob200_swiglu_forward",
    "altob200_swiglu_backward",
    "altob200_dge_scale",
    "altob200_deosc_accumulate",
    "altob200_gemm_blockscaled",
    "altob200_grouped_gemm_blockscaled",
    "altob200_grouped_gemm_wgrad_blockscaled",
    "altob200_gemm_mxfp4_two_level",
    "altob200_grouped_gemm_mxfp4_two_level",
    "altob200_grouped_gemm_wgrad_mxfp4_two_level",
    "altob200_set_wait_limit_ns",
    "altob200_selftest_wait_timeout",
)


class QuantParams(C.Structure):
    _fields_ = [
        ("format", C.c_int32),
        ("in_dtype", C.c_int32),
        ("rounding", C.c_int32),
        ("scale_flags", C.c_int32),
        ("outer_scale", C.c_void_p),
        ("rand_bits", C.c_void_p),
        ("philox_seed", C.c_uint64),
        ("philox_offset", C.c_uint64),
        ("rht_n", C.c_int32),
        ("rht_perm", C.POINTER(C.c_int32)),
        ("rht_sign", C.POINTER(C.c_int32)),
        ("clip_mode", C.c_int32),
        ("use_uos", C.c_int32),
        ("rand_tile_rows", C.c_int64),
        ("rand_tile_pairs", C.c_int64),
    ]


# ---------------------------------------------------------------------------------------
# tracing: NVTX ranges around the boundary calls (off unless ALTO_B200_NVTX=1)
# ---------------------------------------------------------------------------------------
NVTX = os.environ.get("ALTO_B200_NVTX", "0") == "1"


def traced(name: str):
    """Decorator: the call runs inside an NVTX range ``alto_b200::<name>`` when tracing is switched on
    (environment variable ALTO_B200_NVTX=1, read at import); otherwise the function is returned as it is,
    so the default path pays nothing.  Ranges nest: a linear shows its quantizers and GEMMs below it in a
    timeline."""
    def wrap(fn):
        if not NVTX:
            return fn

        @functools.wraps(fn)
        def inner(*args, **kwargs):
            torch.cuda.nvtx.range_push(f"alto_b200::{name}")
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()
        return inner
    return wrap


class MacroScaleDesc(C.Structure):
    """``altob200_macro_scale`` of the header: where the macro-block factor codes of an operand sit."""
    _fields_ = [
        ("codes", C.c_void_p),
        ("row_stride", C.c_int64),
        ("chunk_stride", C.c_int64),
        ("expert_stride", C.c_int64),
        ("row_shift", C.c_int32),
    ]


class Altob200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


_lib = None
_lock = threading.Lock()


def _declare(lib):
    vp, i32, i64 = C.c_void_p, C.c_int32, C.c_int64
    lib.altob200_version.restype = C.c_int
    lib.altob200_status_string.restype = C.c_char_p
    lib.altob200_status_string.argtypes = [C.c_int]
    lib.altob200_packed_scale_bytes.restype = C.c_size_t
    lib.altob200_packed_scale_bytes.argtypes = [i64, i64]
    lib.altob200_status_read.restype = C.c_int
    lib.altob200_status_read.argtypes = [vp, C.POINTER(i32)]
    lib.altob200_amax.restype = C.c_int
    lib.altob200_amax.argtypes = [vp, i32, i64, i64, i64, i32, C.POINTER(i32), C.POINTER(i32), vp, vp, vp, vp]
    lib.altob200_amax_noalloc.restype = C.c_int
    lib.altob200_amax_noalloc.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp]
    for name in ("altob200_quantize_rowwise", "altob200_quantize_colwise"):
        f = getattr(lib, name)
        f.restype = C.c_int
        f.argtypes = [vp, i64, i64, i64, C.POINTER(QuantParams), vp, vp, vp, vp]
    lib.altob200_quantize_2d.restype = C.c_int
    lib.altob200_quantize_2d.argtypes = [vp, i64, i64, i64, C.POINTER(QuantParams), vp, vp, vp, vp, vp, vp]
    lib.altob200_quantize_2d_batched.restype = C.c_int
    lib.altob200_quantize_2d_batched.argtypes = [vp, i64, i64, i64, i64, i64, C.POINTER(QuantParams), vp, vp, vp, vp,
                                                 vp, vp]
    lib.altob200_dequantize.restype = C.c_int
    lib.altob200_dequantize.argtypes = [vp, vp, vp, i32, i32, i64, i64, i32, vp, i64, vp]
    lib.altob200_rht.restype = C.c_int
    lib.altob200_rht.argtypes = [vp, i32, i64, i64, i64, i32, C.POINTER(i32), C.POINTER(i32), vp, i64, vp]
    lib.altob200_gemm_blockscaled.restype = C.c_int
    lib.altob200_gemm_blockscaled.argtypes = [i32, i32, i64, i64, i64, vp, vp, vp, vp, vp, vp, i32, vp, i64, vp]
    lib.altob200_grouped_gemm_blockscaled.restype = C.c_int
    lib.altob200_grouped_gemm_blockscaled.argtypes = [i32, i32, i64, i64, i64, i32, vp, vp, vp, vp, vp, vp, vp,
                                                      i32, vp, i64, vp]


def _declare_more(lib):
    vp, i32, i64 = C.c_void_p, C.c_int32, C.c_int64
    lib.altob200_grouped_gemm_wgrad_blockscaled.restype = C.c_int
    lib.altob200_grouped_gemm_wgrad_blockscaled.argtypes = [i32, i32, i64, i64, i64, i32, vp, vp, vp, vp, vp, vp, vp,
                                                            i32, vp, i64, vp]
    lib.altob200_macro_block_scaling.restype = C.c_int
    lib.altob200_macro_block_scaling.argtypes = [vp, i32, i64, i64, i64, i32, vp, vp, vp]
    lib.altob200_macro_block_descaling.restype = C.c_int
    lib.altob200_macro_block_descaling.argtypes = [vp, vp, i32, i64, i64, i64, i32, vp, vp]
    lib.altob200_rht_dense.restype = C.c_int
    lib.altob200_rht_dense.argtypes = [vp, i32, i64, i64, i64, i32, vp, vp, i64, vp]
    lib.altob200_gather_rows.restype = C.c_int
    lib.altob200_gather_rows.argtypes = [vp, i64, i64, vp, i64, vp, vp]
    lib.altob200_combine_rows.restype = C.c_int
    lib.altob200_combine_rows.argtypes = [vp, i64, i64, vp, vp, i64, i32, vp, vp]
    lib.altob200_spread_rows.restype = C.c_int
    lib.altob200_spread_rows.argtypes = [vp, i64, i32, i64, vp, vp, i64, vp, vp]
    lib.altob200_swiglu_forward.restype = C.c_int
    lib.altob200_swiglu_forward.argtypes = [vp, i64, i64, i64, vp, vp]
    lib.altob200_swiglu_backward.restype = C.c_int
    lib.altob200_swiglu_backward.argtypes = [vp, vp, i64, i64, i64, vp, vp]
    lib.altob200_philox_tile.restype = C.c_int
    lib.altob200_philox_tile.argtypes = [C.c_uint64, C.c_uint64, i64, i64, vp, vp]
    lib.altob200_deosc_accumulate.restype = C.c_int
    lib.altob200_deosc_accumulate.argtypes = [vp, vp, vp, vp, vp, vp, i64, i32, vp]
    lib.altob200_dge_scale.restype = C.c_int
    lib.altob200_dge_scale.argtypes = [vp, i32, i64, i64, i64, vp, C.POINTER(C.c_float), vp]
    ms = C.POINTER(MacroScaleDesc)
    lib.altob200_gemm_mxfp4_two_level.restype = C.c_int
    lib.altob200_gemm_mxfp4_two_level.argtypes = [i64, i64, i64, vp, vp, ms, vp, vp, ms, C.c_float, i32, vp, i64, vp]
    for name in ("altob200_grouped_gemm_mxfp4_two_level", "altob200_grouped_gemm_wgrad_mxfp4_two_level"):
        f = getattr(lib, name)
        f.restype = C.c_int
        f.argtypes = [i64, i64, i64, i32, vp, vp, ms, vp, vp, ms, vp, C.c_float, i32, vp, i64, vp]
    lib.altob200_set_wait_limit_ns.restype = C.c_int
    lib.altob200_set_wait_limit_ns.argtypes = [C.c_uint64]
    lib.altob200_selftest_wait_timeout.restype = C.c_int
    lib.altob200_selftest_wait_timeout.argtypes = [C.c_uint64, vp]


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not LIB_PATH.exists():
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m alto_b200.build` "
                        "(there is no CPU or PyTorch fallback for this path)")
                handle = C.CDLL(str(LIB_PATH))
                _declare(handle)
                _declare_more(handle)
                _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().altob200_status_string(int(status)).decode()


def _check(status: int, where: str) -> None:
    if status != 0:
        raise Altob200Error(status, where)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(t: torch.dtype) -> int:
    if t == torch.bfloat16:
        return DT_BF16
    if t == torch.float32:
        return DT_F32
    raise AssertionError(f"unsupported high-precision dtype {t}")


def _require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("alto_b200 kernels run on CUDA tensors only (no CPU fallback)")


def packed_scale_bytes(rows: int, ncols: int) -> int:
    return int(lib().altob200_packed_scale_bytes(rows, ncols))


def block_of(fmt: int) -> int:
    return 16 if fmt == FMT_NVFP4 else 32


def is_fp4(fmt: int) -> bool:
    return fmt in (FMT_NVFP4, FMT_MXFP4)


def _i32_array(v: Optional[Sequence[int]]):
    if v is None:
        return None
    return (C.c_int32 * len(v))(*[int(x) for x in v])


class Rht:
    """Host description of a randomised Hadamard transform W = (diag(sign) H)[perm][:, perm]."""

    def __init__(self, n: int, perm: Sequence[int], sign: Sequence[int]):
        self.n = int(n)
        self.perm = [int(p) for p in perm]
        self.sign = [int(s) for s in sign]
        self._perm_c = _i32_array(self.perm)
        self._sign_c = _i32_array(self.sign)


CLIP_MODES = {"none": 0, "static": 1, "dynamic": 2}


def _params(fmt, x, rounding, outer_scale, rand_bits, rht: Optional[Rht], flags, philox=(0, 0),
            clip_mode: str = "none", use_uos: bool = False, rand_tile=(0, 0)) -> QuantParams:
    p = QuantParams()
    p.clip_mode = CLIP_MODES[clip_mode]
    p.use_uos = 1 if use_uos else 0
    p.rand_tile_rows, p.rand_tile_pairs = int(rand_tile[0]), int(rand_tile[1])
    p.format = fmt
    p.in_dtype = _dt(x.dtype)
    p.rounding = rounding
    p.scale_flags = flags
    p.outer_scale = _ptr(outer_scale)
    p.rand_bits = _ptr(rand_bits)
    p.philox_seed = int(philox[0]) & 0xFFFFFFFFFFFFFFFF
    p.philox_offset = int(philox[1]) & 0xFFFFFFFFFFFFFFFF
    if rht is not None:
        p.rht_n = rht.n
        p.rht_perm = rht._perm_c
        p.rht_sign = rht._sign_c
    else:
        p.rht_n = 0
    return p


def philox_tile(seed: int, offset: int, tile_rows: int, tile_pairs: int, device) -> torch.Tensor:
    """The reference's [2][tile_rows][tile_pairs] table of stochastic-rounding words for (seed, offset)."""
    out = torch.empty(2, tile_rows, tile_pairs, dtype=torch.int32, device=device)
    _require_cuda(out)
    _check(lib().altob200_philox_tile(int(seed) & 0xFFFFFFFFFFFFFFFF, int(offset) & 0xFFFFFFFFFFFFFFFF, tile_rows,
                                      tile_pairs, out.data_ptr(), _stream()), "altob200_philox_tile")
    return out


def sr_tile_dims(view_rows: int, view_cols: int) -> tuple:
    """(BLOCK_M, BLOCK_N / 2) of the reference quantizer launch for a [view_rows, view_cols] axis-last view."""
    return (64 if view_rows >= 64 else view_rows), (64 if view_cols >= 64 else view_cols) // 2


def status_read() -> tuple:
    """Synchronises the current stream and returns (status, [kernel, block, site, 0])."""
    detail = (C.c_int32 * 4)()
    st = lib().altob200_status_read(_stream(), detail)
    return st, list(detail)


def amax(x: torch.Tensor, amax_bits: torch.Tensor, outer_scale: Optional[torch.Tensor], scratch: torch.Tensor,
         rht: Optional[Rht] = None) -> None:
    """x: [rows, cols] (last dim contiguous).  amax_bits: uint32/int32 [2]; outer_scale: float32 [2] or None;
    scratch: zeroed device buffer of AMAX_SCRATCH_BYTES."""
    _require_cuda(x, amax_bits, outer_scale, scratch)
    assert x.dim() == 2 and x.stride(1) == 1
    _check(lib().altob200_amax(x.data_ptr(), _dt(x.dtype), x.shape[0], x.shape[1], x.stride(0),
                               rht.n if rht else 0, rht._perm_c if rht else None, rht._sign_c if rht else None,
                               amax_bits.data_ptr(), _ptr(outer_scale), scratch.data_ptr(), _stream()),
           "altob200_amax")


NOALLOC_MAX_BYTES = 512 << 20


def amax_noalloc(x: torch.Tensor, amax_bits: torch.Tensor, outer_scale: Optional[torch.Tensor]) -> None:
    """Tensor amax (and NVFP4 outer scale) through the entry point that needs no scratch buffer from
    the caller and allocates nothing: its working memory is a fixed array inside the library.  Inputs
    above NOALLOC_MAX_BYTES are refused; calls that may overlap on one GPU must not be issued."""
    _require_cuda(x, amax_bits, outer_scale)
    assert x.dim() == 2 and x.stride(1) == 1
    _check(lib().altob200_amax_noalloc(x.data_ptr(), _dt(x.dtype), x.shape[0], x.shape[1], x.stride(0),
                                       amax_bits.data_ptr(), _ptr(outer_scale), _stream()),
           "altob200_amax_noalloc")


def quantize_rowwise(x, fmt, codes, scale_plain=None, scale_packed=None, *, rounding=ROUND_RTN,
                     outer_scale=None, rand_bits=None, philox=(0, 0), clip_mode="none", use_uos=False,
                     rand_tile=(0, 0)) -> None:
    _require_cuda(x, codes, scale_plain, scale_packed, outer_scale, rand_bits)
    assert x.dim() == 2 and x.stride(1) == 1
    flags = (SCALE_PLAIN if scale_plain is not None else 0) | (SCALE_PACKED if scale_packed is not None else 0)
    p = _params(fmt, x, rounding, outer_scale, rand_bits, None, flags, philox, clip_mode, use_uos, rand_tile)
    _check(lib().altob200_quantize_rowwise(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), C.byref(p),
                                           codes.data_ptr(), _ptr(scale_plain), _ptr(scale_packed), _stream()),
           "altob200_quantize_rowwise")


def quantize_colwise(x, fmt, codes, scale_plain=None, scale_packed=None, *, rounding=ROUND_RTN,
                     outer_scale=None, rand_bits=None, rht: Optional[Rht] = None, philox=(0, 0),
                     clip_mode="none", use_uos=False, rand_tile=(0, 0)) -> None:
    _require_cuda(x, codes, scale_plain, scale_packed, outer_scale, rand_bits)
    assert x.dim() == 2 and x.stride(1) == 1
    flags = (SCALE_PLAIN if scale_plain is not None else 0) | (SCALE_PACKED if scale_packed is not None else 0)
    p = _params(fmt, x, rounding, outer_scale, rand_bits, rht, flags, philox, clip_mode, use_uos, rand_tile)
    _check(lib().altob200_quantize_colwise(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), C.byref(p),
                                           codes.data_ptr(), _ptr(scale_plain), _ptr(scale_packed), _stream()),
           "altob200_quantize_colwise")


def quantize_2d(w, fmt, codes_k, codes_t=None, scale_plain=None, scale_packed_k=None, scale_packed_t=None, *,
                outer_scale=None, clip_mode="none", use_uos=False, rounding=ROUND_RTN, rand_bits=None,
                rand_tile=(0, 0)) -> None:
    """``rounding``: ROUND_RTN, or ROUND_SR_BITS (FP4) with ``rand_bits`` = words by (row, column pair) as in
    ``quantize_rowwise``: [2, rows, cols/2], or the periodic table [2, tile_rows, tile_pairs] with ``rand_tile``."""
    _require_cuda(w, codes_k, codes_t, scale_plain, scale_packed_k, scale_packed_t, outer_scale, rand_bits)
    assert w.dim() == 2 and w.stride(1) == 1
    p = _params(fmt, w, rounding, outer_scale, rand_bits, None, 0, (0, 0), clip_mode, use_uos, rand_tile)
    _check(lib().altob200_quantize_2d(w.data_ptr(), w.shape[0], w.shape[1], w.stride(0), C.byref(p),
                                      codes_k.data_ptr(), _ptr(codes_t), _ptr(scale_plain), _ptr(scale_packed_k),
                                      _ptr(scale_packed_t), _stream()),
           "altob200_quantize_2d")


def quantize_2d_batched(w3, fmt, codes_k, codes_t=None, scale_plain=None, scale_packed_k=None, scale_packed_t=None,
                        *, outer_scale=None, clip_mode="none", use_uos=False, rounding=ROUND_RTN, rand_bits=None,
                        rand_tile=(0, 0)) -> None:
    """``w3`` [batch, rows, cols] (last dim contiguous, equal batch stride): every matrix quantised in 2-D
    blocks by one launch; outputs are the per-matrix outputs of ``quantize_2d`` stacked along a leading
    batch dimension.  Random words, if any, are indexed by the rows of the flattened [batch * rows, cols] view."""
    _require_cuda(w3, codes_k, codes_t, scale_plain, scale_packed_k, scale_packed_t, outer_scale, rand_bits)
    assert w3.dim() == 3 and w3.stride(2) == 1
    p = _params(fmt, w3, rounding, outer_scale, rand_bits, None, 0, (0, 0), clip_mode, use_uos, rand_tile)
    _check(lib().altob200_quantize_2d_batched(w3.data_ptr(), w3.shape[0], w3.stride(0), w3.shape[1], w3.shape[2],
                                              w3.stride(1), C.byref(p), codes_k.data_ptr(), _ptr(codes_t),
                                              _ptr(scale_plain), _ptr(scale_packed_k), _ptr(scale_packed_t), _stream()),
           "altob200_quantize_2d_batched")


def dequantize(codes, scale_plain, fmt, is_2d, rows, cols, out, outer_scale=None, static_clip=False) -> None:
    _require_cuda(codes, scale_plain, out, outer_scale)
    assert out.dim() == 2 and out.stride(1) == 1
    _check(lib().altob200_dequantize(codes.data_ptr(), scale_plain.data_ptr(), _ptr(outer_scale), fmt,
                                     (1 if is_2d else 0) | (2 if static_clip else 0), rows, cols, _dt(out.dtype), out.data_ptr(), out.stride(0),
                                     _stream()),
           "altob200_dequantize")


def rht_apply(x, y, rht: Rht) -> None:
    _require_cuda(x, y)
    assert x.dim() == 2 and x.stride(1) == 1 and y.stride(1) == 1 and x.dtype == y.dtype
    _check(lib().altob200_rht(x.data_ptr(), _dt(x.dtype), x.shape[0], x.shape[1], x.stride(0), rht.n, rht._perm_c,
                              rht._sign_c, y.data_ptr(), y.stride(0), _stream()),
           "altob200_rht")


def rht_dense(x, y, w: torch.Tensor) -> None:
    """y = cast((w @ x_block) / sqrt(n)) over row blocks of n = w.shape[0] in {16, 32, 64}; w: fp32 device."""
    _require_cuda(x, y, w)
    assert x.dim() == 2 and x.stride(1) == 1 and y.stride(1) == 1 and x.dtype == y.dtype
    assert w.dtype == torch.float32 and w.is_contiguous() and w.dim() == 2 and w.shape[0] == w.shape[1]
    _check(lib().altob200_rht_dense(x.data_ptr(), _dt(x.dtype), x.shape[0], x.shape[1], x.stride(0), w.shape[0],
                                    w.data_ptr(), y.data_ptr(), y.stride(0), _stream()), "altob200_rht_dense")


MACRO_LAST, MACRO_2D, MACRO_ROWS = 0, 1, 2


def macro_block_scaling(x, y, scale, mode: int) -> None:
    """x, y: contiguous [batch, rows, cols]; scale: uint8, shaped as the header says for `mode`."""
    _require_cuda(x, y, scale)
    assert x.dim() == 3 and x.is_contiguous() and y.is_contiguous() and x.dtype == y.dtype and x.shape == y.shape
    assert scale.dtype == torch.uint8 and scale.is_contiguous()
    _check(lib().altob200_macro_block_scaling(x.data_ptr(), _dt(x.dtype), x.shape[0], x.shape[1], x.shape[2], mode,
                                              y.data_ptr(), scale.data_ptr(), _stream()),
           "altob200_macro_block_scaling")


def macro_block_descaling(y, scale, x, mode: int) -> None:
    _require_cuda(x, y, scale)
    assert y.dim() == 3 and x.is_contiguous() and y.is_contiguous() and x.dtype == y.dtype and x.shape == y.shape
    assert scale.dtype == torch.uint8 and scale.is_contiguous()
    _check(lib().altob200_macro_block_descaling(y.data_ptr(), scale.data_ptr(), _dt(y.dtype), y.shape[0], y.shape[1],
                                                y.shape[2], mode, x.data_ptr(), _stream()),
           "altob200_macro_block_descaling")


def dge_scale(dw: torch.Tensor, codes_t: torch.Tensor, lut16: Sequence[float]) -> None:
    """In place: dw[n, k] *= lut16[code of W[n, k]], codes_t = packed [K, N/2] weight operand."""
    _require_cuda(dw, codes_t)
    assert dw.dim() == 2 and dw.stride(1) == 1 and codes_t.is_contiguous() and len(lut16) == 16
    N, K = dw.shape
    assert codes_t.numel() == K * (N // 2), "codes_t must be the [K, N/2] packing of the weight"
    lut = (C.c_float * 16)(*[float(v) for v in lut16])
    _check(lib().altob200_dge_scale(dw.data_ptr(), _dt(dw.dtype), N, K, dw.stride(0), codes_t.data_ptr(), lut,
                                    _stream()), "altob200_dge_scale")


def deosc_accumulate(w, prev, w_qdq, prev_qdq, dist_w, dist_qdq) -> None:
    """dist_w += |w - prev|; dist_qdq += |w_qdq - prev_qdq|; prev = w (all contiguous, same dtype and size)."""
    ts = (w, prev, w_qdq, prev_qdq, dist_w, dist_qdq)
    _require_cuda(*ts)
    assert all(t.is_contiguous() and t.dtype == w.dtype and t.numel() == w.numel() for t in ts)
    _check(lib().altob200_deosc_accumulate(w.data_ptr(), prev.data_ptr(), w_qdq.data_ptr(), prev_qdq.data_ptr(),
                                           dist_w.data_ptr(), dist_qdq.data_ptr(), w.numel(), _dt(w.dtype), _stream()),
           "altob200_deosc_accumulate")


def gather_rows(src: torch.Tensor, index: torch.Tensor, out_rows: Optional[int] = None) -> torch.Tensor:
    """out[i] = src[index[i]] for index[i] >= 0, else a zero row.  src: [rows, cols] contiguous with
    rows of a multiple of 16 bytes; index: int32 on the same device."""
    _require_cuda(src, index)
    assert src.dim() == 2 and src.is_contiguous() and index.dtype == torch.int32 and index.is_contiguous()
    n = int(index.numel() if out_rows is None else out_rows)
    out = torch.empty(n, src.shape[1], dtype=src.dtype, device=src.device)
    _check(lib().altob200_gather_rows(src.data_ptr(), src.shape[0], src.shape[1] * src.element_size(),
                                      index.data_ptr(), n, out.data_ptr(), _stream()), "altob200_gather_rows")
    return out


def combine_rows(rows: torch.Tensor, index: torch.Tensor, scores: Optional[torch.Tensor], tokens: int, k: int) -> torch.Tensor:
    """out[t] = sum_j rows[index[t k + j]] * scores[t, j] (bf16 roundings of the tensor-op form); [tokens, D]."""
    _require_cuda(rows, index, scores)
    assert rows.dim() == 2 and rows.is_contiguous() and rows.dtype == torch.bfloat16
    assert index.dtype == torch.int32 and index.is_contiguous() and index.numel() == tokens * k
    assert scores is None or (scores.dtype == torch.bfloat16 and scores.is_contiguous() and scores.numel() == tokens * k)
    out = torch.empty(tokens, rows.shape[1], dtype=rows.dtype, device=rows.device)
    _check(lib().altob200_combine_rows(rows.data_ptr(), rows.shape[0], rows.shape[1] * 2, index.data_ptr(),
                                       None if scores is None else scores.data_ptr(), tokens, k, out.data_ptr(),
                                       _stream()), "altob200_combine_rows")
    return out


def spread_rows(grad_out: torch.Tensor, position: torch.Tensor, scores: Optional[torch.Tensor], k: int) -> torch.Tensor:
    """grad_rows[r] = grad_out[position[r] // k] * scores.flat[position[r]], zero rows where position[r] < 0."""
    _require_cuda(grad_out, position, scores)
    assert grad_out.dim() == 2 and grad_out.is_contiguous() and grad_out.dtype == torch.bfloat16
    assert position.dtype == torch.int32 and position.is_contiguous()
    n = position.numel()
    out = torch.empty(n, grad_out.shape[1], dtype=grad_out.dtype, device=grad_out.device)
    _check(lib().altob200_spread_rows(grad_out.data_ptr(), grad_out.shape[0], k, grad_out.shape[1] * 2,
                                      position.data_ptr(), None if scores is None else scores.data_ptr(), n,
                                      out.data_ptr(), _stream()), "altob200_spread_rows")
    return out


def swiglu_forward(h: torch.Tensor) -> torch.Tensor:
    """h: [rows, 2H] bf16 contiguous (gate | up) -> bf16(bf16(silu(gate)) * up), [rows, H]."""
    _require_cuda(h)
    assert h.dim() == 2 and h.is_contiguous() and h.dtype == torch.bfloat16 and h.shape[1] % 2 == 0
    rows, H = h.shape[0], h.shape[1] // 2
    out = torch.empty(rows, H, dtype=h.dtype, device=h.device)
    _check(lib().altob200_swiglu_forward(h.data_ptr(), rows, H, 2 * H, out.data_ptr(), _stream()),
           "altob200_swiglu_forward")
    return out


def swiglu_backward(h: torch.Tensor, grad_out: torch.Tensor) -> torch.Tensor:
    """Gradient of swiglu_forward with respect to h, [rows, 2H] bf16."""
    _require_cuda(h, grad_out)
    assert h.dim() == 2 and h.is_contiguous() and h.dtype == torch.bfloat16
    rows, H = h.shape[0], h.shape[1] // 2
    assert grad_out.shape == (rows, H) and grad_out.is_contiguous() and grad_out.dtype == torch.bfloat16
    grad_h = torch.empty_like(h)
    _check(lib().altob200_swiglu_backward(h.data_ptr(), grad_out.data_ptr(), rows, H, 2 * H, grad_h.data_ptr(),
                                          _stream()), "altob200_swiglu_backward")
    return grad_h


def gemm_blockscaled(fmt_a, fmt_b, M, N, K, a_codes, a_scales, b_codes, b_scales, out, alpha_a=None,
                     alpha_b=None) -> None:
    _require_cuda(a_codes, a_scales, b_codes, b_scales, out, alpha_a, alpha_b)
    assert out.dim() == 2 and out.stride(1) == 1
    _check(lib().altob200_gemm_blockscaled(fmt_a, fmt_b, M, N, K, a_codes.data_ptr(), a_scales.data_ptr(),
                                           b_codes.data_ptr(), b_scales.data_ptr(), _ptr(alpha_a), _ptr(alpha_b),
                                           _dt(out.dtype), out.data_ptr(), out.stride(0), _stream()),
           "altob200_gemm_blockscaled")


def grouped_gemm_blockscaled(fmt_a, fmt_b, M, N, K, num_experts, a_codes, a_scales, b_codes, b_scales,
                             group_expert, out, alpha_a=None, alpha_b=None) -> None:
    _require_cuda(a_codes, a_scales, b_codes, b_scales, group_expert, out, alpha_a, alpha_b)
    assert out.dim() == 2 and out.stride(1) == 1 and group_expert.dtype == torch.int32
    _check(lib().altob200_grouped_gemm_blockscaled(fmt_a, fmt_b, M, N, K, num_experts, a_codes.data_ptr(),
                                                   a_scales.data_ptr(), b_codes.data_ptr(), b_scales.data_ptr(),
                                                   group_expert.data_ptr(), _ptr(alpha_a), _ptr(alpha_b),
                                                   _dt(out.dtype), out.data_ptr(), out.stride(0), _stream()),
           "altob200_grouped_gemm_blockscaled")


def grouped_gemm_wgrad_blockscaled(fmt_a, fmt_b, M, N, K, num_experts, a_codes, a_scales, b_codes, b_scales, k_offs,
                                   out, alpha_a=None, alpha_b=None) -> None:
    """out[e] = A[:, range_e] @ B[:, range_e]^T with range_e = [k_offs[e-1], k_offs[e]) along the shared
    reduction axis of length K; out is [num_experts, M, N]."""
    _require_cuda(a_codes, a_scales, b_codes, b_scales, k_offs, out, alpha_a, alpha_b)
    assert out.dim() == 3 and out.stride(2) == 1 and out.stride(0) == M * out.stride(1)
    assert k_offs.dtype == torch.int32 and k_offs.numel() == num_experts
    _check(lib().altob200_grouped_gemm_wgrad_blockscaled(
        fmt_a, fmt_b, M, N, K, num_experts, a_codes.data_ptr(), a_scales.data_ptr(), b_codes.data_ptr(),
        b_scales.data_ptr(), k_offs.data_ptr(), _ptr(alpha_a), _ptr(alpha_b), _dt(out.dtype), out.data_ptr(),
        out.stride(1), _stream()), "altob200_grouped_gemm_wgrad_blockscaled")


class MacroScale:
    """Macro-block factor codes of one two-level GEMM operand: the uint8 tensor ``macro_block_scaling``
    returned plus how (operand row, 128-chunk of the reduction axis) maps into it; see
    ``altob200_macro_scale`` in the header."""

    __slots__ = ("codes", "row_stride", "chunk_stride", "expert_stride", "row_shift")

    def __init__(self, codes: torch.Tensor, row_stride: int, chunk_stride: int, row_shift: int, expert_stride: int = 0):
        assert codes.dtype == torch.uint8 and codes.is_contiguous()
        self.codes, self.row_stride, self.chunk_stride = codes, int(row_stride), int(chunk_stride)
        self.row_shift, self.expert_stride = int(row_shift), int(expert_stride)

    def desc(self) -> MacroScaleDesc:
        d = MacroScaleDesc()
        d.codes = self.codes.data_ptr()
        d.row_stride, d.chunk_stride, d.expert_stride, d.row_shift = (self.row_stride, self.chunk_stride,
                                                                      self.expert_stride, self.row_shift)
        return d


def gemm_mxfp4_two_level(M, N, K, a_codes, a_scales, a_macro: MacroScale, b_codes, b_scales, b_macro: MacroScale,
                         out, out_scale: float = 1.0, group_expert=None, k_offs=None, num_experts: int = 0) -> None:
    """Two-level scaled MXFP4 GEMM; ``group_expert`` selects the row-grouped form ([M, N] output, B
    stacked per expert), ``k_offs`` the grouped weight gradient ([num_experts, M, N] output)."""
    _require_cuda(a_codes, a_scales, a_macro.codes, b_codes, b_scales, b_macro.codes, out, group_expert, k_offs)
    assert out.stride(-1) == 1
    da, db = a_macro.desc(), b_macro.desc()
    common = (a_codes.data_ptr(), a_scales.data_ptr(), C.byref(da), b_codes.data_ptr(), b_scales.data_ptr(),
              C.byref(db))
    if group_expert is not None:
        assert out.dim() == 2 and group_expert.dtype == torch.int32
        _check(lib().altob200_grouped_gemm_mxfp4_two_level(M, N, K, num_experts, *common, group_expert.data_ptr(),
                                                           float(out_scale), _dt(out.dtype), out.data_ptr(),
                                                           out.stride(0), _stream()),
               "altob200_grouped_gemm_mxfp4_two_level")
    elif k_offs is not None:
        assert out.dim() == 3 and out.stride(0) == M * out.stride(1)
        assert k_offs.dtype == torch.int32 and k_offs.numel() == num_experts
        _check(lib().altob200_grouped_gemm_wgrad_mxfp4_two_level(M, N, K, num_experts, *common, k_offs.data_ptr(),
                                                                 float(out_scale), _dt(out.dtype), out.data_ptr(),
                                                                 out.stride(1), _stream()),
               "altob200_grouped_gemm_wgrad_mxfp4_two_level")
    else:
        assert out.dim() == 2
        _check(lib().altob200_gemm_mxfp4_two_level(M, N, K, *common, float(out_scale), _dt(out.dtype),
                                                   out.data_ptr(), out.stride(0), _stream()),
               "altob200_gemm_mxfp4_two_level")


def set_wait_limit_ns(limit_ns: int) -> None:
    """Wall-clock limit of every bounded wait inside GEMM kernels launched from now on (default 4 s)."""
    _check(lib().altob200_set_wait_limit_ns(int(limit_ns)), "altob200_set_wait_limit_ns")


def selftest_wait_timeout(limit_ns: int = 1_000_000) -> None:
    """Launches the kernel whose only wait cannot be satisfied; ``status_read`` then reports the timeout."""
    _check(lib().altob200_selftest_wait_timeout(int(limit_ns), _stream()), "altob200_selftest_wait_timeout")
