"""Pins the CPU oracle to outputs of the reference's own code (tests/golden/reference_vectors.npz,
made by tests/golden/make_golden.py).  Everything here is bit-exact."""
import numpy as np
import pytest
import torch

from oracle import alto_oracle as O
from tests.helpers import case_input, golden_cases, load_golden, tensor_from_bits


def _eq(a: torch.Tensor, b: np.ndarray):
    assert tuple(a.shape) == tuple(b.shape), (a.shape, b.shape)
    got = a.contiguous().numpy() if a.dtype != torch.bfloat16 else a.contiguous().view(torch.int16).numpy()
    assert np.array_equal(got.view(b.dtype) if got.dtype != b.dtype else got, b, equal_nan=True) \
        if b.dtype.kind == "f" else np.array_equal(got, b)


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp4")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_mxfp4_matches_reference(z, m):
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m)
    q, s = O.quantize_mxfp4(x, 32, axis, is2d)
    _eq(q, z[tag + "_q"])
    _eq(s, z[tag + "_s"])
    dq = O.dequantize_mxfp4(q, s, torch.float32, 32, axis, is2d)
    _eq(dq, z[tag + "_dq"])


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp4sr")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_mxfp4_stochastic_rounding_matches_reference_kernel(z, m):
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m)
    rand = torch.from_numpy(z[tag + "_rand"].astype(np.int64))
    q, s = O.quantize_mxfp4(x, 32, axis, False, rand)
    _eq(s, z[tag + "_s"])
    _eq(q, z[tag + "_q"])
    # sanity: stochastic rounding really differs from round-to-nearest on this input
    q_rtn, _ = O.quantize_mxfp4(x, 32, axis, False)
    assert (q_rtn != q).float().mean() > 0.05


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp4sr")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_reference_sr_word_layout(z, m):
    """(seed, offset) -> the per-element words the reference kernel consumed (dumped beside its codes)."""
    tag, shape, dt, axis, is2d = m
    seed, off = [int(v) for v in z["philox_seed_offset"]]
    R, Cc = (shape[0], shape[1]) if axis == -1 else (shape[1], shape[0])
    planes = O.reference_sr_planes(seed, off, R, Cc)
    assert np.array_equal(planes.numpy().astype(np.uint32), z[tag + "_rand"])
    q, s = O.quantize_mxfp4(case_input(z, m), 32, axis, False, planes)
    _eq(q, z[tag + "_q"])


def test_philox_matches_triton_randint4x():
    z, _ = load_golden()
    seed, off = [int(v) for v in z["philox_seed_offset"]]
    idx = torch.arange(64 * 32, dtype=torch.int64) + off
    zero = torch.zeros_like(idx)
    k0 = torch.full_like(idx, seed & 0xFFFFFFFF)
    k1 = torch.full_like(idx, (seed >> 32) & 0xFFFFFFFF)
    c0, c1, _, _ = O.philox4x32_10(idx & 0xFFFFFFFF, zero, zero, zero, k0, k1)
    assert np.array_equal(c0.reshape(64, 32).numpy().astype(np.uint32), z["philox_r0"])
    assert np.array_equal(c1.reshape(64, 32).numpy().astype(np.uint32), z["philox_r1"])


@pytest.mark.parametrize("z,m", list(golden_cases("nvfp4")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_nvfp4_matches_reference(z, m):
    tag, shape, dt, axis, is2d = m
    x = case_input(z, m)
    outer = z[tag + "_outer"]
    outer_t = torch.from_numpy(outer.copy()) if outer.size else None
    if outer_t is not None:
        assert torch.equal(O.compute_dynamic_outer_scale(x), outer_t)
    q, s = O.quantize_nvfp4(x, 16, axis, is2d, outer_t)
    _eq(s, z[tag + "_s"])
    _eq(q, z[tag + "_q"])
    dq = O.dequantize_nvfp4(q, s, torch.float32, 16, axis, is2d, outer_t)
    _eq(dq, z[tag + "_dq"])


@pytest.mark.parametrize("z,m", list(golden_cases("mxfp8")), ids=lambda v: v[0] if isinstance(v, tuple) else "")
def test_mxfp8_matches_reference(z, m):
    tag, shape, dt, axis, is2d, fmt = m
    x = case_input(z, m)
    q, s = O.quantize_mxfp8(x, 32, fmt, axis, is2d)
    _eq(s, z[tag + "_s"])
    assert np.array_equal(q.contiguous().view(torch.uint8).numpy(), z[tag + "_q"])
    dq = O.dequantize_mxfp8(q, s, torch.float32, 32, axis, is2d)
    _eq(dq, z[tag + "_dq"])


@pytest.mark.parametrize("n", [16, 32])
def test_hadamard_matches_reference(n):
    z, _ = load_golden()
    W = torch.from_numpy(z[f"rht{n}_W"])
    x = tensor_from_bits(z[f"rht{n}_x"], torch.bfloat16)
    # the vectors were made by the reference's code on CPU, where PyTorch divides by sqrt(n); on
    # CUDA it multiplies by the reciprocal (the oracle's default).  Both must hold for n = 16; for
    # n = 32 the two may differ by one bf16 ulp where the fp32 value sits on a rounding boundary.
    y = O.rht_apply(x, W, cuda_division=False)
    assert np.array_equal(y.view(torch.int16).numpy().view(np.uint16), z[f"rht{n}_y"])
    y_cuda = O.rht_apply(x, W)
    diff = (y_cuda.view(torch.int16).int() - y.view(torch.int16).int()).abs()
    assert diff.max().item() <= (0 if n == 16 else 1) and (diff != 0).float().mean().item() < 1e-3
    # the factory draws the sign vector first and the permutation second from one generator
    g = torch.Generator().manual_seed(0)
    base = None if n == 16 else _file_hadamard(32)
    W2, perm, sign = O.random_hadamard(n, g, base)
    assert torch.equal(W2, W)
    assert np.array_equal(perm.numpy(), z[f"rht{n}_perm"])


def _file_hadamard(n):
    """The reference's n = 32 base matrix is not the Sylvester one; it is read from the data file
    that ships (byte-identical) with the installed compressed_tensors package."""
    from pathlib import Path

    import compressed_tensors.transform.utils as ctu
    from safetensors import safe_open

    with safe_open(str(Path(ctu.__file__).parent / "hadamards.safetensors"), framework="pt") as fh:
        return fh.get_tensor(str(n)).float()


def test_reference_special_values():
    """Known answers asserted by the reference's own tests
    (tests/unittest/nvfp4/test_nvfp_quantization.py:167-263)."""
    zeros = torch.zeros(64, 64, dtype=torch.bfloat16)
    q, s = O.quantize_nvfp4(zeros)
    assert torch.all(s == 2.0 ** -6) and torch.all(q == 0)
    big = torch.full((64, 64), 5000.0, dtype=torch.bfloat16)
    q, s = O.quantize_nvfp4(big)
    assert torch.all(s == 448.0) and torch.all(q == 0x77)
    outer = O.compute_dynamic_outer_scale(zeros)
    assert outer.item() == pytest.approx(1e-30) and outer.dtype == torch.float32
    q, s = O.quantize_nvfp4(zeros, outer_scale=outer)
    assert torch.isfinite(s).all() and (s * outer).min() > 1.17e-38


def _sr2d_cases():
    import ast
    from pathlib import Path
    z = np.load(Path(__file__).resolve().parent / "golden" / "sr2d_vectors.npz")
    return z, ast.literal_eval(str(z["meta"]))


def test_2d_blocks_with_stochastic_rounding_match_the_reference_kernel():
    """The reference's MXFP4 kernel (interpreted) on 32 x 32 blocks with (philox_seed, philox_offset):
    pins how its Philox words pair with the elements of a 2-D-block launch."""
    z, meta = _sr2d_cases()
    seed, off = [int(v) for v in z["philox_seed_offset"]]
    for tag, shape, axis in meta:
        x = torch.from_numpy(z[tag + "_x"].view(np.int16)).view(torch.bfloat16).reshape(shape)
        # words are indexed in the view with the quantisation axis last, leading dimensions flattened into rows
        view = x.transpose(axis, -1).shape
        planes = O.reference_sr_planes(seed, off, int(np.prod(view[:-1])), view[-1])
        q, s = O.quantize_mxfp4(x, 32, axis, True, planes)
        assert np.array_equal(q.contiguous().view(torch.uint8).numpy(), z[tag + "_q"]), tag
        assert np.array_equal(s.contiguous().numpy(), z[tag + "_s"]), tag
