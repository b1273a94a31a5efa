"""CPU tests: the C-ABI library loads and exports what the header declares, host-side logic
(Hadamard factory draws, packed-scale repacking, argument contracts) and the absence of any CPU
compute path in the product."""
import re
from pathlib import Path

import pytest
import torch

from oracle import alto_oracle as O

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    from alto_b200 import _lib as L
    header = (ROOT / "include" / "altob200.h").read_text()
    declared = set(re.findall(r"\b(altob200_[a-z0-9_]+)\s*\(", header))
    declared.discard("altob200_quant_params")
    assert declared, "no declarations found in the header"
    lib = L.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/altob200.h but not exported"
    assert declared == set(L.EXPORTED_SYMBOLS)
    assert lib.altob200_version() >= 1
    assert L.status_string(0) == "ok" and "timed out" in L.status_string(L.E_TIMEOUT)
    assert L.packed_scale_bytes(8192, 256) == 64 * 64 * 512
    assert L.packed_scale_bytes(150, 6) == 2 * 2 * 512


def test_header_cites_the_reference_for_every_entry_point():
    header = (ROOT / "include" / "altob200.h").read_text()
    for fn in ("altob200_amax", "altob200_quantize_rowwise", "altob200_quantize_colwise", "altob200_quantize_2d",
               "altob200_dequantize", "altob200_rht", "altob200_gemm_blockscaled",
               "altob200_grouped_gemm_blockscaled"):
        pos = header.index(f"int {fn}(")
        comment = header[header.rindex("/*", 0, pos):pos]
        assert re.search(r"alto/kernels/[\w/]+\.py:\d+", comment), f"{fn}: no reference citation"


def test_product_has_no_cpu_path_and_never_imports_the_oracle():
    from alto_b200 import mxfp4, mxfp8, nvfp4
    x = torch.zeros(32, 64, dtype=torch.bfloat16)
    for call in (lambda: nvfp4.convert_to_nvfp4(x), lambda: mxfp4.convert_to_mxfp4(x),
                 lambda: mxfp8.convert_to_mxfp8(x), lambda: nvfp4._to_nvfp4_then_scaled_mm(x, x, False, True, False),
                 lambda: nvfp4.compute_dynamic_outer_scale(x)):
        with pytest.raises(RuntimeError):
            call()
    for py in (ROOT / "alto_b200").rglob("*.py"):
        src = py.read_text()
        assert "oracle" not in src.replace("the oracle", ""), f"{py} mentions the oracle package"
        assert "import triton" not in src


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from alto_b200 import _lib as L
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", tmp_path / "libaltob200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        L.lib()


def test_hadamard_factory_draws_like_the_reference():
    """Sign vector first, permutation second, from one seeded generator
    (alto/kernels/hadamard_transform/transform.py:63-96)."""
    from alto_b200.hadamard import HadamardFactory, HadamardTransform
    from tests.helpers import load_golden
    z, _ = load_golden()
    HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
    t = HadamardFactory.create_transform(device="cpu")
    assert torch.equal(t.matrix(), torch.from_numpy(z["rht16_W"]))
    assert torch.equal(t.perm, torch.from_numpy(z["rht16_perm"]))
    p = t.device_params()
    W, perm, sign = O.random_hadamard(16, torch.Generator().manual_seed(0))
    assert p.n == 16 and p.perm == perm.tolist() and p.sign == [int(v) for v in sign.tolist()]
    HadamardFactory.configure(block_size=32, seed=0)
    t32 = HadamardFactory.create_transform(device="cpu")
    assert torch.equal(t32.matrix(), torch.from_numpy(z["rht32_W"]))
    with pytest.raises(NotImplementedError):
        t32.device_params()
    HadamardFactory.configure(block_size=16, randomized=False)
    td = HadamardFactory.create_transform(device="cpu")
    assert td.perm is None and torch.equal(td.weight, O.sylvester(16))
    assert td.device_params().sign == [1] * 16
    with pytest.raises(NotImplementedError):
        HadamardTransform(torch.ones(16, 16), None).device_params()
    HadamardFactory.configure(block_size=16, randomized=True, seed=0)


def test_plain_scale_repacking_matches_the_packed_layout():
    from alto_b200 import _linear as E
    g = torch.Generator().manual_seed(0)
    sf = torch.randint(0, 255, (200, 6), generator=g, dtype=torch.uint8)
    assert torch.equal(E.pack_plain_scales(sf, 200, False, 32), O.pack_scale_bytes(sf))
    s2 = torch.randint(0, 255, (8, 5), generator=g, dtype=torch.uint8)
    assert torch.equal(E.pack_plain_scales(s2, 256, True, 32), O.pack_scale_bytes(s2.repeat_interleave(32, 0)))
    inner = torch.tensor([[2.0 ** -6, 1.0, 448.0, 1.75]])
    assert E.pack_plain_scales(inner, 1, False, 16)[:4].tolist() == [0x08, 0x38, 0x7E, 0x3E]


def test_oracle_gemm_definition_and_linear_consistency():
    """(Hx)^T (H dY) == x^T dY for the orthogonal transform, and the oracle's three products have
    the right shapes and a sane signal-to-noise ratio."""
    g = torch.Generator().manual_seed(0)
    W, _, _ = O.random_hadamard(16, g)
    assert torch.equal(W @ W.t(), 16 * torch.eye(16))
    x = torch.randn(64, 96, generator=g).bfloat16()
    w = (torch.randn(32, 96, generator=g) * 0.05).bfloat16()
    dy = torch.randn(64, 32, generator=g).bfloat16()
    y, dx, dw = O.nvfp4_linear(x, w, dy, W_had=W)
    assert y.shape == (64, 32) and dx.shape == (64, 96) and dw.shape == (32, 96)
    ref = dy.float().t() @ x.float()
    snr = 10 * torch.log10(ref.pow(2).sum() / (dw - ref).pow(2).sum())
    assert snr > 9.0


def test_boundary_signatures_match_the_reference():
    """Parameter names, order, kinds and defaults of every boundary callable equal the reference's, as
    read from its source by tests/golden/make_boundary_signatures.py.  Two quantizers carry one extra
    trailing parameter (``rand_bits``: explicit random words for stochastic rounding)."""
    import importlib
    import inspect
    import json
    from pathlib import Path
    table = json.loads((Path(__file__).resolve().parent / "golden" / "boundary_signatures.json").read_text())
    assert len(table) >= 25
    allowed_extra = {"convert_to_mxfp4": ["rand_bits"], "convert_to_nvfp4": ["rand_bits"]}
    for entry in table:
        fn = getattr(importlib.import_module(entry["module"]), entry["function"])
        mine = [[n, "keyword_only" if p.kind == p.KEYWORD_ONLY else "positional",
                 "<required>" if p.default is p.empty else repr(p.default)]
                for n, p in inspect.signature(fn).parameters.items()]
        ref = entry["params"]
        assert mine[:len(ref)] == ref, (entry["function"], ref, mine)
        assert [m[0] for m in mine[len(ref):]] == allowed_extra.get(entry["function"], []), entry["function"]


def test_nvtx_ranges_wrap_boundary_calls_only_when_asked(monkeypatch):
    """Tracing: with ALTO_B200_NVTX=1 a boundary call runs inside a named NVTX range (pushed and popped
    even when the call raises); without it the decorator returns the function untouched."""
    from alto_b200 import _lib as L

    def f(a, b=2):
        if a < 0:
            raise ValueError("neg")
        return a + b

    monkeypatch.setattr(L, "NVTX", False)
    assert L.traced("plain")(f) is f
    events = []
    monkeypatch.setattr(L, "NVTX", True)
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: events.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: events.append(("pop",)))
    g = L.traced("unit")(f)
    assert g(1, b=3) == 4 and g.__name__ == "f"
    with pytest.raises(ValueError):
        g(-1)
    assert events == [("push", "alto_b200::unit"), ("pop",), ("push", "alto_b200::unit"), ("pop",)]
