"""Generates tests/golden/*.npz by running the REFERENCE's own code on CPU.

Needs the reference checkout (its path in $ALTO_REFERENCE); it is therefore
run only where that checkout exists, and its outputs are committed.  Two sources are used:

* the reference's PyTorch emulations (tests/unittest/{mxfp4,nvfp4,mxfp8}/utils.py), which its
  own GPU tests assert bit-equal to its kernels, and
* the reference's Triton kernels run under the Triton interpreter (MXFP4 RTN and SR, where the
  interpreter is exact).  Interpreter results that pass through an fp8 cast are not used: the
  interpreter's fp32->fp8 conversion differs from the hardware's.

The `alto` package itself cannot be imported (it needs a TorchTitan fork), so the package
names are stubbed as namespace modules and the needed files are loaded by path, which is the
trick the reference's own CPU test uses (tests/unittest/mxfp4/test_mxfp_pnq.py:38-60).

Usage: python tests/golden/make_golden.py
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch
import torch.library

REF = Path(os.environ.get("ALTO_REFERENCE", "/root/reference"))
OUT = Path(__file__).resolve().parent


def _stub_packages():
    root = REF / "alto"
    for name, sub in [("alto", ""), ("alto.kernels", "kernels"), ("alto.kernels.fp4", "kernels/fp4"),
                      ("alto.kernels.fp4.mxfp4", "kernels/fp4/mxfp4"), ("alto.kernels.fp4.nvfp4", "kernels/fp4/nvfp4")]:
        m = types.ModuleType(name)
        m.__path__ = [str(root / sub)]
        sys.modules[name] = m

    def _triton_op(name, mutates_args=None):
        def deco(fn):
            fn.register_fake = lambda f: f
            return fn
        return deco

    torch.library.triton_op = _triton_op
    torch.library.wrap_triton = lambda k: k


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits_of(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def data(shape, dtype, seed, pattern="random"):
    g = torch.Generator().manual_seed(seed)
    if pattern == "random":  # the reference's recipe: N(0,1) plus 0.5 % outliers x100
        x = torch.randn(shape, generator=g, dtype=torch.float32)
        mask = (torch.rand(shape, generator=g) < 0.005).float()
        x = x + 100 * torch.randn(shape, generator=g) * mask
    elif pattern == "zeros":
        x = torch.zeros(shape)
    elif pattern == "large":
        x = torch.full(shape, 5000.0)
    elif pattern == "nan":
        x = torch.randn(shape, generator=g)
        x.view(-1)[7] = float("nan")
    elif pattern == "lognormal":
        x = torch.exp(torch.randn(shape, generator=g) * 1.5)
    elif pattern == "tiny":
        x = torch.randn(shape, generator=g) * 1e-4
    else:
        raise ValueError(pattern)
    return x.to(dtype)


def main():
    _stub_packages()
    import triton
    import triton.language as tl
    mx_u = _load(REF / "tests/unittest/mxfp4/utils.py", "ref_mx_utils")
    nv_u = _load(REF / "tests/unittest/nvfp4/utils.py", "ref_nv_utils")
    m8_u = _load(REF / "tests/unittest/mxfp8/utils.py", "ref_m8_utils")
    from alto.kernels.fp4.mxfp4.mxfp_quantization import convert_to_mxfp4 as ref_to_mxfp4_triton
    from alto.kernels.fp4.nvfp4.nvfp_quantization import compute_dynamic_outer_scale as ref_outer

    out = {}
    meta = []

    # ---------------- MXFP4 (emulation) ----------------
    k = 0
    for shape, dt, axis, is2d in [((128, 64), torch.bfloat16, -1, False), ((64, 128), torch.float32, -1, False),
                                  ((128, 64), torch.bfloat16, 0, False), ((64, 64), torch.bfloat16, -1, True),
                                  ((64, 128), torch.bfloat16, 0, True), ((2, 64, 64), torch.bfloat16, -2, False)]:
        x = data(shape, dt, 100 + k)
        q, s = mx_u.convert_to_mxfp4_pytorch(x, axis=axis, is_2d_block=is2d)
        dq = mx_u.convert_from_mxfp4_pytorch(q, s, output_dtype=torch.float32, axis=axis, is_2d_block=is2d)
        tag = f"mxfp4_{k}"
        out[tag + "_x"] = bits_of(x)
        out[tag + "_q"] = q.contiguous().numpy()
        out[tag + "_s"] = s.contiguous().numpy()
        out[tag + "_dq"] = dq.contiguous().numpy()
        meta.append((tag, list(shape), str(dt), axis, is2d))
        k += 1

    # ---------------- MXFP4 stochastic rounding (reference Triton kernel, interpreted) ----------------
    @triton.jit
    def dump_philox(o0, o1, seed, offset, M: tl.constexpr, N: tl.constexpr):
        ms = tl.arange(0, M)
        ns = tl.arange(0, N)
        offs = offset + ms[:, None] * N + ns[None, :]
        r1, r2, _, _ = tl.randint4x(seed, offs)
        tl.store(o0 + ms[:, None] * N + ns[None, :], r1)
        tl.store(o1 + ms[:, None] * N + ns[None, :], r2)

    seed, off = 123, 456
    r0 = torch.empty(64, 32, dtype=torch.int32)
    r1 = torch.empty(64, 32, dtype=torch.int32)
    dump_philox[(1,)](r0, r1, seed, off, 64, 32)
    out["philox_seed_offset"] = np.array([seed, off], dtype=np.int64)
    out["philox_r0"] = r0.numpy().view(np.uint32)
    out["philox_r1"] = r1.numpy().view(np.uint32)
    for j, (shape, axis) in enumerate([((64, 64), -1), ((128, 128), -1), ((128, 64), 0)]):
        x = (data(shape, torch.float32, 200 + j) * 1.5).to(torch.bfloat16)
        q, s = ref_to_mxfp4_triton(x, axis=axis, use_asm=False, use_sr=True, philox_seed=seed, philox_offset=off)
        # the kernel restarts the Philox offsets in every 64x64 tile of the axis-last view:
        # the effective per-element planes are the 64x32 dump tiled over the view
        R, Cc = (shape[0], shape[1]) if axis == -1 else (shape[1], shape[0])
        p0 = r0.repeat(R // 64, Cc // 64)
        p1 = r1.repeat(R // 64, Cc // 64)
        tag = f"mxfp4sr_{j}"
        out[tag + "_x"] = bits_of(x)
        out[tag + "_q"] = q.contiguous().numpy()
        out[tag + "_s"] = s.contiguous().numpy()
        out[tag + "_rand"] = torch.stack([p0, p1]).numpy().view(np.uint32)
        meta.append((tag, list(shape), "torch.bfloat16", axis, False))

    # ---------------- NVFP4 (emulation) ----------------
    k = 0
    for shape, dt, axis, is2d, pattern, outer in [
        ((128, 64), torch.bfloat16, -1, False, "random", True),
        ((128, 64), torch.bfloat16, -1, False, "random", False),
        ((64, 128), torch.float32, -1, False, "random", True),
        ((128, 64), torch.bfloat16, 0, False, "random", True),
        ((64, 64), torch.bfloat16, -1, True, "random", True),
        ((64, 128), torch.bfloat16, 0, True, "lognormal", True),
        ((150, 64), torch.bfloat16, -1, False, "random", True),
        ((64, 64), torch.bfloat16, -1, False, "zeros", True),
        ((64, 64), torch.bfloat16, -1, False, "large", False),
        ((64, 64), torch.bfloat16, -1, False, "nan", False),
        ((64, 64), torch.bfloat16, -1, False, "tiny", True),
        ((4, 128, 64), torch.bfloat16, -1, False, "random", True),
    ]:
        x = data(shape, dt, 300 + k, pattern)
        os_ = ref_outer(x) if outer else None
        q, s = nv_u.convert_to_nvfp4_pytorch(x, axis=axis, is_2d_block=is2d, outer_scale=os_)
        dq = nv_u.convert_from_nvfp4_pytorch(q, s, output_dtype=torch.float32, axis=axis, is_2d_block=is2d,
                                             outer_scale=os_)
        tag = f"nvfp4_{k}"
        out[tag + "_x"] = bits_of(x)
        out[tag + "_q"] = q.contiguous().numpy()
        out[tag + "_s"] = s.contiguous().numpy()
        out[tag + "_dq"] = dq.contiguous().numpy()
        out[tag + "_outer"] = (os_.numpy() if os_ is not None else np.zeros(0, np.float32))
        meta.append((tag, list(shape), str(dt), axis, is2d))
        k += 1

    # ---------------- MXFP8 (emulation) ----------------
    k = 0
    for shape, dt, axis, is2d, fmt in [((128, 64), torch.bfloat16, -1, False, "e4m3"),
                                       ((128, 64), torch.bfloat16, -1, False, "e5m2"),
                                       ((64, 128), torch.float32, -1, False, "e4m3"),
                                       ((128, 64), torch.bfloat16, 0, False, "e4m3"),
                                       ((64, 64), torch.bfloat16, -1, True, "e4m3"),
                                       ((64, 128), torch.bfloat16, 0, True, "e5m2")]:
        x = data(shape, dt, 400 + k)
        q, s = m8_u.convert_to_mxfp8_pytorch(x, mxfp_format=fmt, axis=axis, is_2d_block=is2d)
        dq = m8_u.convert_from_mxfp8_pytorch(q, s, output_dtype=torch.float32, axis=axis, is_2d_block=is2d)
        tag = f"mxfp8_{k}"
        out[tag + "_x"] = bits_of(x)
        out[tag + "_q"] = bits_of(q)
        out[tag + "_s"] = s.contiguous().numpy()
        out[tag + "_dq"] = dq.contiguous().numpy()
        meta.append((tag, list(shape), str(dt), axis, is2d, fmt))
        k += 1

    # ---------------- randomised Hadamard transform ----------------
    import safetensors  # noqa: F401  (the reference opens its matrix file with safetensors)
    had_mod_path = REF / "alto/kernels/hadamard_transform"
    pkg = types.ModuleType("ref_had")
    pkg.__path__ = [str(had_mod_path)]
    sys.modules["ref_had"] = pkg
    hadamard = _load(had_mod_path / "hadamard.py", "ref_had.hadamard")
    sys.modules["ref_had.hadamard"] = hadamard
    # the checkout holds a git-LFS pointer; the identical file ships with compressed_tensors
    import compressed_tensors.transform.utils as ctu
    real_file = Path(ctu.__file__).parent / "hadamards.safetensors"
    hadamard.REPO_PATH = real_file
    d = list(hadamard._fetch_hadamard_divisor.__defaults__)
    d[-1] = real_file  # the default argument was bound to the pointer file at import
    hadamard._fetch_hadamard_divisor.__defaults__ = tuple(d)
    sys.modules["ref_had.matrix"] = _load(had_mod_path / "matrix.py", "ref_had.matrix")
    spec = importlib.util.spec_from_file_location("ref_had.transform", str(had_mod_path / "transform.py"))
    transform = importlib.util.module_from_spec(spec)
    transform.__package__ = "ref_had"
    spec.loader.exec_module(transform)
    for n in (16, 32):
        transform.HadamardFactory.configure(block_size=n, randomized=True, dtype=torch.float32, seed=0)
        t = transform.HadamardFactory.create_transform(device=torch.device("cpu"))
        W = t.weight[t.perm][:, t.perm]
        x = data((4 * n, 48), torch.bfloat16, 500 + n)
        y = t(x, left_mul=True)
        out[f"rht{n}_W"] = W.numpy()
        out[f"rht{n}_weight"] = t.weight.numpy()
        out[f"rht{n}_perm"] = t.perm.numpy()
        out[f"rht{n}_x"] = bits_of(x)
        out[f"rht{n}_y"] = bits_of(y)

    out["meta"] = np.array(repr(meta))
    np.savez_compressed(OUT / "reference_vectors.npz", **out)
    print("wrote", OUT / "reference_vectors.npz", "entries:", len(out))


if __name__ == "__main__":
    main()
