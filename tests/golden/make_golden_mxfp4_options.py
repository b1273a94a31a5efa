"""Generates tests/golden/mxfp4_options_vectors.npz: the MXFP4 quantizer's `clip_mode` and `use_uos`
options, from the REFERENCE's PyTorch emulation (tests/unittest/mxfp4/utils.py:285-400), which the
reference's GPU tests assert equal to its Triton kernel for these options
(tests/unittest/mxfp4/test_mxfp_quantization.py:29-100; for clip_mode='dynamic' with bf16 inputs the
reference itself only checks a mean error, so those cases are fp32).

Usage: python tests/golden/make_golden_mxfp4_options.py   (needs the reference checkout)
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
from make_golden import REF, _load, _stub_packages, bits_of, data  # noqa: E402

OUT = Path(__file__).resolve().parent

CASES = [  # shape, dtype, axis, is_2d, clip_mode, use_uos, pattern
    ((64, 128), torch.bfloat16, -1, False, "static", False, "random"),
    ((64, 128), torch.bfloat16, 0, False, "static", False, "random"),
    ((64, 64), torch.bfloat16, -1, True, "static", False, "random"),
    ((64, 128), torch.float32, -1, False, "static", False, "random"),
    ((64, 128), torch.bfloat16, -1, False, "none", True, "random"),
    ((64, 128), torch.bfloat16, 0, False, "none", True, "lognormal"),
    ((64, 64), torch.bfloat16, -1, True, "none", True, "random"),
    ((64, 128), torch.float32, -1, False, "none", True, "lognormal"),
    ((32, 64), torch.bfloat16, -1, False, "none", True, "zeros"),
    ((64, 128), torch.bfloat16, -1, False, "static", True, "random"),
    ((64, 128), torch.float32, -1, False, "dynamic", False, "random"),
    ((64, 128), torch.float32, 0, False, "dynamic", False, "lognormal"),
    ((64, 128), torch.float32, -1, False, "dynamic", True, "random"),
    ((64, 128), torch.float32, -1, True, "dynamic", False, "random"),
    ((128, 64), torch.float32, 0, True, "dynamic", False, "lognormal"),
    ((64, 64), torch.float32, -1, True, "dynamic", True, "random"),
]


def main():
    _stub_packages()
    mx_u = _load(REF / "tests/unittest/mxfp4/utils.py", "ref_mx_utils")
    out, meta = {}, []
    for k, (shape, dt, axis, is2d, clip, uos, pattern) in enumerate(CASES):
        x = data(shape, dt, 700 + k, pattern)
        q, s = mx_u.convert_to_mxfp4_pytorch(x, axis=axis, is_2d_block=is2d, clip_mode=clip, use_uos=uos)
        tag = f"mxopt_{k}"
        out[tag + "_x"] = bits_of(x)
        out[tag + "_q"] = q.contiguous().numpy()
        out[tag + "_s"] = s.contiguous().numpy()
        for odt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            dq = mx_u.convert_from_mxfp4_pytorch(q, s, output_dtype=odt, axis=axis, is_2d_block=is2d, clip_mode=clip)
            out[tag + "_dq_" + name] = bits_of(dq)
        meta.append((tag, list(shape), str(dt), axis, is2d, clip, uos))
    out["meta"] = np.array(repr(meta))
    np.savez_compressed(OUT / "mxfp4_options_vectors.npz", **out)
    print("wrote", OUT / "mxfp4_options_vectors.npz", "entries:", len(out))


if __name__ == "__main__":
    main()
