"""Writes tests/golden/boundary_signatures.json: parameter names, kinds and defaults of the reference's
boundary callables, read from the reference's source files with `ast` (nothing is imported or run).

    ALTO_REFERENCE=/path/to/reference python tests/golden/make_boundary_signatures.py

The test tests/test_cpu_host.py::test_boundary_signatures_match_the_reference compares this package's
callables of the same names with the table.
"""
import ast
import json
import os
from pathlib import Path

REF = Path(os.environ.get("ALTO_REFERENCE", "/root/reference"))
K = "alto/kernels/"
TARGETS = [
    # (reference file, function, module of this package that must offer the same signature)
    (K + "fp4/mxfp4/mxfp_quantization.py", "convert_to_mxfp4", "alto_b200.mxfp4"),
    (K + "fp4/mxfp4/mxfp_quantization.py", "convert_from_mxfp4", "alto_b200.mxfp4"),
    (K + "fp4/mxfp4/mxfp_linear.py", "blockwise_mxfp4_gemm", "alto_b200.mxfp4"),
    (K + "fp4/mxfp4/mxfp_linear.py", "_to_mxfp4_then_scaled_mm", "alto_b200.mxfp4"),
    (K + "fp4/mxfp4/macro_block_scaling.py", "macro_block_scaling", "alto_b200.macro_block_scaling"),
    (K + "fp4/mxfp4/macro_block_scaling.py", "macro_block_descaling", "alto_b200.macro_block_scaling"),
    (K + "fp4/nvfp4/nvfp_quantization.py", "compute_dynamic_outer_scale", "alto_b200.nvfp4"),
    (K + "fp4/nvfp4/nvfp_quantization.py", "convert_to_nvfp4", "alto_b200.nvfp4"),
    (K + "fp4/nvfp4/nvfp_quantization.py", "convert_from_nvfp4", "alto_b200.nvfp4"),
    (K + "fp4/nvfp4/nvfp_linear.py", "_to_nvfp4_then_scaled_mm", "alto_b200.nvfp4"),
    (K + "mxfp8/mxfp8_quantization.py", "convert_to_mxfp8", "alto_b200.mxfp8"),
    (K + "mxfp8/mxfp8_quantization.py", "convert_from_mxfp8", "alto_b200.mxfp8"),
    (K + "mxfp8/mxfp8_quantization.py", "calculate_mxfp8_scales", "alto_b200.mxfp8"),
    (K + "mxfp8/mxfp8_linear.py", "blockwise_mxfp8_gemm", "alto_b200.mxfp8"),
    (K + "mxfp8/mxfp8_linear.py", "_to_mxfp8_then_scaled_mm", "alto_b200.mxfp8"),
    (K + "fp4/mxfp4/mxfp_grouped_gemm/functional.py", "_quantize_then_mxfp_scaled_grouped_mm", "alto_b200.grouped"),
    (K + "fp4/nvfp4/nvfp_grouped_gemm/functional.py", "_quantize_then_nvfp4_scaled_grouped_mm", "alto_b200.grouped"),
    (K + "mxfp8/mxfp8_grouped_gemm/functional.py", "_quantize_then_mxfp8_scaled_grouped_mm", "alto_b200.grouped"),
    (K + "fp4/mxfp4/mxfp_grouped_gemm/cg_forward.py", "mxfp4_grouped_gemm_forward", "alto_b200.grouped"),
    (K + "fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py", "mxfp4_grouped_gemm_backward_inputs", "alto_b200.grouped"),
    (K + "fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py", "mxfp4_grouped_gemm_backward_weights", "alto_b200.grouped"),
    (K + "mxfp8/mxfp8_grouped_gemm/cg_forward.py", "mxfp8_grouped_gemm_forward", "alto_b200.grouped"),
    (K + "mxfp8/mxfp8_grouped_gemm/cg_backward.py", "mxfp8_grouped_gemm_backward_inputs", "alto_b200.grouped"),
    (K + "mxfp8/mxfp8_grouped_gemm/cg_backward.py", "mxfp8_grouped_gemm_backward_weights", "alto_b200.grouped"),
    (K + "dispatch/conversion.py", "swap_params", "alto_b200.dispatch"),
]


def _constant(path: Path, name: str):
    """Value of a module-level `NAME = literal` in `path` or in a sibling file of its directory."""
    for f in [path] + sorted(path.parent.glob("*.py")) + sorted(path.parent.parent.glob("*.py")):
        for node in ast.parse(f.read_text()).body:
            if isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id == name for t in node.targets):
                try:
                    return repr(ast.literal_eval(node.value))
                except Exception:
                    pass
    return name


def _default(node, path: Path):
    if node is None:
        return "<required>"
    try:
        return repr(ast.literal_eval(node))
    except Exception:
        if isinstance(node, ast.Name):
            return _constant(path, node.id)
        return ast.unparse(node)


def signature_of(path: Path, name: str):
    tree = ast.parse(path.read_text())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == name:
            a = node.args
            pos = a.posonlyargs + a.args
            defaults = [None] * (len(pos) - len(a.defaults)) + list(a.defaults)
            out = [[p.arg, "positional", _default(d, path)] for p, d in zip(pos, defaults)]
            out += [[p.arg, "keyword_only", _default(d, path)] for p, d in zip(a.kwonlyargs, a.kw_defaults)]
            return out
    raise KeyError(f"{name} not found in {path}")


def main():
    table = []
    for rel, fn, module in TARGETS:
        table.append({"reference": rel, "function": fn, "module": module, "params": signature_of(REF / rel, fn)})
    out = Path(__file__).resolve().parent / "boundary_signatures.json"
    out.write_text(json.dumps(table, indent=1) + "\n")
    print(f"wrote {out} ({len(table)} callables)")


if __name__ == "__main__":
    main()
