"""Generates tests/golden/macro_block_vectors.npz by running the REFERENCE's macro-block scaling
kernels (alto/kernels/fp4/mxfp4/macro_block_scaling.py) under the Triton interpreter on CPU.

The interpreter is exact for the fp32 arithmetic of these kernels (loads, max, one IEEE division,
integer bit operations, an fp32 multiply or divide).  It is NOT exact for the final fp32 -> bf16
store: the interpreter truncates where the GPU rounds to nearest even, so bf16 cases are run with
fp32 storage and rounded afterwards (see the loop below).  The file is loaded by path (the `alto`
package itself needs a TorchTitan fork to import).

Usage: python tests/golden/make_golden_macro.py      (needs the reference checkout, its path in
$ALTO_REFERENCE; the output is committed)
"""
from __future__ import annotations

import importlib.util
import os
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

REF = Path(os.environ.get("ALTO_REFERENCE", "/root/reference"))
OUT = Path(__file__).resolve().parent

CASES = [  # shape, dtype, axis, use_2d_block, pattern
    ((64, 256), torch.bfloat16, -1, False, "random"),
    ((256, 32), torch.bfloat16, -2, False, "random"),
    ((128, 128), torch.bfloat16, -1, True, "random"),
    ((130, 136), torch.bfloat16, 0, True, "random"),
    ((70, 200), torch.bfloat16, -1, False, "random"),
    ((130, 36), torch.float32, -2, False, "random"),
    ((129, 132), torch.float32, -1, True, "random"),
    ((33, 133), torch.bfloat16, -1, False, "random"),   # rows not on a 4-element boundary
    ((129, 133), torch.bfloat16, -2, True, "random"),
    ((2, 40, 136), torch.bfloat16, -1, False, "lognormal"),
    ((2, 130, 36), torch.bfloat16, -2, False, "lognormal"),
    ((2, 36, 132), torch.float32, -1, True, "tiny"),
    ((16, 128), torch.bfloat16, -1, False, "zeros"),
    ((16, 256), torch.float32, -1, False, "huge"),
]


def _data(shape, dtype, seed, pattern):
    g = torch.Generator().manual_seed(seed)
    if pattern == "random":
        x = torch.randn(shape, generator=g)
        mask = (torch.rand(shape, generator=g) < 0.005).float()
        x = x + 100 * torch.randn(shape, generator=g) * mask
    elif pattern == "lognormal":
        x = torch.exp(torch.randn(shape, generator=g) * 1.5) * torch.sign(torch.randn(shape, generator=g))
    elif pattern == "tiny":
        x = torch.randn(shape, generator=g) * 1e-9
    elif pattern == "zeros":
        x = torch.zeros(shape)
    elif pattern == "huge":
        x = torch.randn(shape, generator=g) * 1e30
    else:
        raise ValueError(pattern)
    return x.to(dtype)


def _bits(t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()


def main():
    spec = importlib.util.spec_from_file_location("ref_macro", str(REF / "alto/kernels/fp4/mxfp4/macro_block_scaling.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out, meta = {}, []
    for k, (shape, dt, axis, is2d, pattern) in enumerate(CASES):
        x = _data(shape, dt, 900 + k, pattern)
        # bf16 cases go through the kernels as fp32 tensors holding the bf16 values (an exact
        # widening, the same one the kernel's load performs) and the fp32 result is rounded to
        # bf16 here, to nearest even as the GPU's conversion does
        y32, s = ref._macro_block_scaling_triton_impl(x.float(), axis=axis, use_2d_block=is2d)
        y = y32.to(dt)
        xr = ref._macro_block_descaling_triton_impl(y.float(), s, axis=axis, use_2d_block=is2d).to(dt)
        tag = f"macro_{k}"
        out[tag + "_x"] = _bits(x)
        out[tag + "_y"] = _bits(y)
        out[tag + "_s"] = s.contiguous().numpy()
        out[tag + "_xr"] = _bits(xr)
        meta.append((tag, list(shape), str(dt), axis, is2d))
    out["meta"] = np.array(repr(meta))
    np.savez_compressed(OUT / "macro_block_vectors.npz", **out)
    print("wrote", OUT / "macro_block_vectors.npz", "entries:", len(out))


if __name__ == "__main__":
    main()
