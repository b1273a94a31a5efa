"""Generates tests/golden/sr2d_vectors.npz: the reference's MXFP4 Triton kernel, run under the Triton
interpreter, on 2-D (32 x 32) blocks WITH stochastic rounding from (philox_seed, philox_offset).

This pins how the reference pairs its Philox words with the elements of a 2-D-block launch (the
gradient of a `use_2dblock_x` linear is quantised this way, alto/kernels/fp4/mxfp4/mxfp_linear.py:447-458).
Needs the reference checkout (its path in $ALTO_REFERENCE); the output is committed.

Usage: python tests/golden/make_golden_sr2d.py
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import make_golden as G  # noqa: E402  (stubs of the reference package, data recipe)


def main():
    G._stub_packages()
    from alto.kernels.fp4.mxfp4.mxfp_quantization import convert_to_mxfp4 as ref_to_mxfp4_triton
    seed, off = 2468, 1357
    out = {"philox_seed_offset": np.array([seed, off], dtype=np.int64)}
    meta = []
    for j, (shape, axis) in enumerate([((64, 64), -1), ((128, 192), -1), ((128, 64), 0), ((2, 64, 96), -2)]):
        x = (G.data(shape, torch.float32, 700 + j) * 1.5).to(torch.bfloat16)
        q, s = ref_to_mxfp4_triton(x, axis=axis, is_2d_block=True, use_asm=False, use_sr=True, philox_seed=seed,
                                   philox_offset=off)
        tag = f"sr2d_{j}"
        out[tag + "_x"] = G.bits_of(x)
        out[tag + "_q"] = q.contiguous().view(torch.uint8).numpy()   # logical shape (a transposed view for axis 0 / -2)
        out[tag + "_s"] = s.contiguous().numpy()
        meta.append((tag, list(shape), axis))
    out["meta"] = np.array(repr(meta))
    np.savez_compressed(G.OUT / "sr2d_vectors.npz", **out)
    print("wrote", G.OUT / "sr2d_vectors.npz", [m[0] for m in meta])


if __name__ == "__main__":
    main()
