"""Helpers shared by the tests: golden-vector access and seeded synthetic inputs."""
from __future__ import annotations

import ast
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_vectors.npz"
_DT = {"torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}


def load_golden():
    z = np.load(GOLDEN, allow_pickle=False)
    meta = ast.literal_eval(str(z["meta"]))
    return z, meta


def tensor_from_bits(arr: np.ndarray, dtype) -> torch.Tensor:
    if dtype == torch.bfloat16:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return torch.from_numpy(arr.copy()).view(dtype)
    return torch.from_numpy(arr.copy())


def golden_cases(prefix: str):
    z, meta = load_golden()
    for m in meta:
        if m[0].startswith(prefix + "_"):
            yield z, m


MACRO_GOLDEN = GOLDEN.with_name("macro_block_vectors.npz")


def macro_cases():
    """(npz, (tag, shape, dtype, axis, use_2d_block)) for every macro-block scaling vector."""
    z = np.load(MACRO_GOLDEN, allow_pickle=False)
    for m in ast.literal_eval(str(z["meta"])):
        yield z, m


def bits_equal(t: torch.Tensor, arr: np.ndarray) -> bool:
    """Bit-for-bit comparison of a (CPU or CUDA) tensor with a stored array (bf16 stored as uint16)."""
    t = t.detach().cpu().contiguous()
    if tuple(t.shape) != tuple(arr.shape):
        return False
    if t.dtype == torch.bfloat16:
        return np.array_equal(t.view(torch.int16).numpy().view(np.uint16), arr)
    if t.dtype == torch.float32:
        return np.array_equal(t.numpy().view(np.uint32), arr.view(np.uint32))
    return np.array_equal(t.numpy(), arr)


def case_input(z, m) -> torch.Tensor:
    return tensor_from_bits(z[m[0] + "_x"], _DT[m[2]])


def reference_data(shape, dtype, seed, device="cpu", outliers=True):
    """The reference tests' data recipe (N(0,1) plus 0.5 % outliers x100,
    tests/unittest/mxfp4/utils.py:16-22) drawn on CPU from an explicit seed."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    if outliers:
        mask = (torch.rand(shape, generator=g) < 0.005).float()
        x = x + 100 * torch.randn(shape, generator=g) * mask
    return x.to(dtype).to(device)


def rand_u32(shape, seed, device="cpu") -> torch.Tensor:
    """Uniform uint32 values held in an int64 tensor (CPU) — the explicit SR random bits."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 2 ** 32, shape, generator=g, dtype=torch.int64).to(device)


def to_u32_device(r: torch.Tensor, device) -> torch.Tensor:
    """int64 holding uint32 -> int32 bit pattern on `device` (what the kernels read)."""
    return (r & 0xFFFFFFFF).to(torch.uint32).view(torch.int32).to(device) if hasattr(torch, "uint32") else \
        torch.from_numpy(r.numpy().astype(np.uint32).view(np.int32)).to(device)
