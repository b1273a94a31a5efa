"""The scheme surface of the low-precision path: ``TrainingOpConfig``, the weight-wrapper tensor
subclasses that intercept GEMM ops, and ``swap_params``.

Same names, fields and routing rules as the reference
(alto/kernels/dispatch/config.py:10-57, alto/kernels/dispatch/tensor.py:53-503,
alto/kernels/dispatch/conversion.py:20-124), re-based on a plain ``torch.Tensor`` wrapper
subclass (the reference derives from ``torchao.utils.TorchAOBaseTensor``; torchao is not needed
here).  A weight wrapped in one of the subclasses makes ``F.linear`` / ``mm`` / ``matmul`` /
``addmm`` / ``torch._grouped_mm`` run the B200 quantize + block-scaled GEMM path; model code
does not change.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Callable, Literal, Optional, Tuple, Type

import torch
import torch.utils._pytree as pytree
from torch import nn
from torch._prims_common import suggest_memory_format

from . import grouped as _grouped
from . import mxfp4 as _mxfp4
from . import mxfp8 as _mxfp8
from . import nvfp4 as _nvfp4

logger = logging.getLogger("alto_b200")

# Boundary functions are looked up on this module at call time so that tests (and users) can
# replace them, as the reference's dispatch-guard tests do with monkeypatch.
_to_mxfp4_then_scaled_mm = _mxfp4._to_mxfp4_then_scaled_mm
_to_nvfp4_then_scaled_mm = _nvfp4._to_nvfp4_then_scaled_mm
_to_mxfp8_then_scaled_mm = _mxfp8._to_mxfp8_then_scaled_mm
_quantize_then_mxfp_scaled_grouped_mm = _grouped._quantize_then_mxfp_scaled_grouped_mm
_quantize_then_nvfp4_scaled_grouped_mm = _grouped._quantize_then_nvfp4_scaled_grouped_mm
_quantize_then_mxfp8_scaled_grouped_mm = _grouped._quantize_then_mxfp8_scaled_grouped_mm


@dataclass(unsafe_hash=True, kw_only=True, slots=True)
class TrainingOpConfig:
    """Quantisation recipe of one group of modules (alto/kernels/dispatch/config.py:10-54).

    precision          "mxfp4" | "mxfp8_e4m3" | "mxfp8_e5m2" | "nvfp4" ("amdfp4" is AMD-only: it is
                       accepted as a value, and refused when a GEMM is dispatched)
    use_2dblock_x/_w   square blocks for activations / weights
    use_hadamard       randomised Hadamard rotation of the wgrad operands
    use_sr_grad        stochastic rounding of gradients
    use_dge            differentiable gradient estimator on dW
    clip_mode          "none" | "static" | "dynamic" (MXFP4)
    two_level_scaling  "none" | "tensorwise" (NVFP4 outer scale) | "blockwise" (MXFP4 macro blocks)
    use_uos            7.25 instead of 6 as the MXFP4 target maximum
    """

    precision: Literal["mxfp4", "mxfp8_e4m3", "mxfp8_e5m2", "nvfp4", "amdfp4"]
    use_2dblock_x: bool
    use_2dblock_w: bool
    use_hadamard: bool
    use_sr_grad: bool
    use_dge: bool
    clip_mode: Literal["none", "static", "dynamic"] = "none"
    two_level_scaling: Literal["none", "tensorwise", "blockwise"] = "none"
    use_uos: bool = False


torch.serialization.add_safe_globals([TrainingOpConfig])

_ops_to_preserve_subclass = {
    torch.ops.aten.empty_like.default,
    torch.ops.aten.new_zeros.default,
    torch.ops.aten.slice.Tensor,
    torch.ops.aten.copy_.default,
    torch.ops.aten.view.default,
    torch.ops.aten.as_strided.default,
    torch.ops.aten._to_copy.default,
    torch.ops.aten._pin_memory.default,
    torch.ops.aten.split.Tensor,
    torch.ops.aten.clone.default,
    torch.ops.aten.transpose.int,
    torch.ops.aten.t.default,
}
if hasattr(torch.ops, "c10d") and hasattr(torch.ops.c10d, "scatter_"):
    _ops_to_preserve_subclass.add(torch.ops.c10d.scatter_.default)  # tensor parallel weight distribution

gemm_ops = ("linear", "mm.default", "matmul.default", "addmm.default", "matmul")


class TrainingWeightWrapperBaseTensor(torch.Tensor):
    """Wrapper subclass holding the high-precision weight in ``_data`` and the recipe in ``config``."""

    config: Optional[TrainingOpConfig] = None

    @staticmethod
    def __new__(cls, tensor: torch.Tensor, config: TrainingOpConfig):
        self = torch.Tensor._make_wrapper_subclass(
            cls, tensor.size(), strides=tensor.stride(), storage_offset=tensor.storage_offset(),
            memory_format=suggest_memory_format(tensor), dtype=tensor.dtype, layout=tensor.layout,
            device=tensor.device, pin_memory=tensor.is_pinned(), requires_grad=tensor.requires_grad)
        self.config = config
        return self

    def __init__(self, tensor: torch.Tensor, config: TrainingOpConfig):
        self._data = tensor
        self.config = config

    @classmethod
    def __torch_function__(cls, func, types, args, kwargs={}):
        raise NotImplementedError(
            f"{cls.__name__} not intended to be used directly, please override this method in a tensor "
            "subclass for your intended derived dtype.")

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs={}):
        config = None

        def unwrap(t):
            nonlocal config
            if config is None:
                config = t.config
            else:
                assert t.config == config, (
                    "All TrainingWeightWrapperBaseTensor instances must have the same config, but found "
                    f"{t.config} and {config}")
            return t._data

        args_u, kwargs_u = pytree.tree_map_only(TrainingWeightWrapperBaseTensor, unwrap, (args, kwargs or {}))
        assert config is not None, (
            f"__torch_dispatch__ called on {func.__name__} without any TrainingWeightWrapperBaseTensor arguments")
        if func == torch.ops.aten.detach.default:
            return cls(args_u[0], config)
        if func.__name__ in gemm_ops or func.__name__ == "_grouped_mm":
            raise ValueError("You have reached the __torch_dispatch__ method of low-precision GEMMs, "
                             "which does not support Autograd Function."
                             "This is commonly caused by unsupported tensor parallel.")
        out = func(*args_u, **kwargs_u)
        if func not in _ops_to_preserve_subclass:
            return out
        return pytree.tree_map_only(torch.Tensor, lambda x: cls(x, config), out)

    def __repr__(self):
        return f"{type(self).__name__}(data={self._data}, config={self.config})"

    def __tensor_flatten__(self):
        return ["_data"], {"config": self.config}

    @classmethod
    def __tensor_unflatten__(cls, inner_tensors, flatten_spec, outer_size, outer_stride):
        return cls(inner_tensors["_data"], flatten_spec["config"])

    def untyped_storage(self):
        return self._data.untyped_storage()

    # FSDP2 extension hooks: the high-precision weight is all-gathered in the mixed-precision
    # parameter dtype; quantisation happens per step on the gathered weight
    # (alto/kernels/dispatch/tensor.py:159-211).
    def fsdp_pre_all_gather(self, mesh, outer_size, outer_stride, module, mp_policy):
        return (self._data.to(mp_policy.param_dtype),), ()

    def fsdp_post_all_gather(self, all_gather_outputs: Tuple[torch.Tensor, ...], metadata: Any,
                             param_dtype: torch.dtype, *, out: Optional[torch.Tensor] = None):
        (data,) = all_gather_outputs
        if out is not None:
            from torch.distributed._tensor import DTensor
            if isinstance(out, TrainingWeightWrapperBaseTensor):
                out_data = out._data
                out.config = self.config
            elif isinstance(out, DTensor) and isinstance(out._local_tensor, TrainingWeightWrapperBaseTensor):
                out_data = out._local_tensor._data
                out._local_tensor.config = self.config
            else:
                raise RuntimeError(
                    "expect out to be TrainingWeightWrapperBaseTensor or DTensor with "
                    f"local_tensor=TrainingWeightWrapperBaseTensor, but got {type(out)}")
            if data.dtype == param_dtype:
                assert data.untyped_storage().data_ptr() == out_data.untyped_storage().data_ptr()
            else:
                assert out_data.dtype == param_dtype, f"{out_data.dtype} {param_dtype}"
                out_data.copy_(data)
            return
        return type(self)(data, self.config), (data,)


def _split_gemm_args(func, args):
    if func.__name__ == "addmm.default":
        return args[1], args[2], args[0]
    return args[0], args[1], (args[2] if len(args) > 2 else None)


def _grouped_args(cls, args, kwargs):
    A, B = args[0], args[1]
    bias = kwargs.get("bias", None)
    offs = kwargs.get("offs", None)
    assert not isinstance(A, cls), f"A should not be a {cls.__name__}"
    assert isinstance(B, cls), f"B should be a {cls.__name__}"
    assert A.ndim == 2 and B.ndim == 3 and offs is not None, "Only 2d x 3d with offsets is supported for now"
    assert bias is None, "Bias is not supported for now"
    return A, B, offs


def _passthrough(func, args, kwargs):
    with torch._C.DisableTorchFunctionSubclass():
        return func(*args, **kwargs)


class MXFP4TrainingWeightWrapperTensor(TrainingWeightWrapperBaseTensor):
    """Routes GEMMs whose weight is wrapped to the MXFP4 path (alto/kernels/dispatch/tensor.py:214-303)."""

    @classmethod
    def __torch_function__(cls, func, types, args, kwargs={}):
        import alto_b200.dispatch as D
        if func.__name__ == "_grouped_mm":
            A, B, offs = _grouped_args(cls, args, kwargs)
            config = B.config
            assert config.precision == "mxfp4", "expected TrainingOpConfig with precision=mxfp4"
            return D._quantize_then_mxfp_scaled_grouped_mm(
                A, B, offs=offs, use_2dblock_x=config.use_2dblock_x, use_2dblock_w=config.use_2dblock_w,
                use_sr_grad=config.use_sr_grad, use_dge=config.use_dge, use_hadamard=config.use_hadamard,
                clip_mode=config.clip_mode, use_macro_block_scaling=config.two_level_scaling == "blockwise",
                use_uos=config.use_uos)
        if func.__name__ in gemm_ops:
            trans_b = func.__name__ == "linear"
            A, B, bias = _split_gemm_args(func, args)
            assert not isinstance(A, cls), f"A should not be a {cls.__name__} for func {func.__name__}"
            assert isinstance(B, cls), f"B should be a {cls.__name__} for func {func.__name__}"
            config = B.config
            assert config.precision == "mxfp4", "expected TrainingOpConfig with precision=mxfp4"
            Y = D._to_mxfp4_then_scaled_mm(
                A, B if trans_b else B.T, use_2dblock_x=config.use_2dblock_x, use_2dblock_w=config.use_2dblock_w,
                use_sr_grad=config.use_sr_grad, use_dge=config.use_dge, clip_mode=config.clip_mode,
                use_hadamard=config.use_hadamard, use_macro_block_scaling=config.two_level_scaling == "blockwise",
                use_uos=config.use_uos)
            return Y if bias is None else Y + bias
        return _passthrough(func, args, kwargs)


class NVFP4TrainingWeightWrapperTensor(TrainingWeightWrapperBaseTensor):
    """Routes GEMMs to the NVFP4 path; ``two_level_scaling == "tensorwise"`` turns the outer scale on
    (alto/kernels/dispatch/tensor.py:306-421)."""

    @classmethod
    def __torch_function__(cls, func, types, args, kwargs={}):
        import alto_b200.dispatch as D
        if func.__name__ == "_grouped_mm" or func.__name__ in gemm_ops:
            grouped = func.__name__ == "_grouped_mm"
            if grouped:
                A, B, offs = _grouped_args(cls, args, kwargs)
                bias = None
            else:
                A, B, bias = _split_gemm_args(func, args)
                assert not isinstance(A, cls), f"A should not be a {cls.__name__} for func {func.__name__}"
                assert isinstance(B, cls), f"B should be a {cls.__name__} for func {func.__name__}"
            config = B.config
            assert config.precision in ("nvfp4", "amdfp4"), (
                f"expected TrainingOpConfig with precision in {{'nvfp4','amdfp4'}}, got {config.precision}")
            if config.precision == "amdfp4":
                raise NotImplementedError("scheme 'amdfp4' (UE5M3 inner scales) is an AMD-only format and is not "
                                          "part of the B200 path; use 'nvfp4'")
            common = dict(use_2dblock_x=config.use_2dblock_x, use_2dblock_w=config.use_2dblock_w,
                          use_sr_grad=config.use_sr_grad, use_outer_scale=config.two_level_scaling == "tensorwise",
                          use_hadamard=config.use_hadamard, use_dge=config.use_dge)
            if grouped:
                return D._quantize_then_nvfp4_scaled_grouped_mm(A, B, offs=offs, **common)
            Y = D._to_nvfp4_then_scaled_mm(A, B if func.__name__ == "linear" else B.T, **common)
            return Y if bias is None else Y + bias
        return _passthrough(func, args, kwargs)


class MXFP8TrainingWeightWrapperTensor(TrainingWeightWrapperBaseTensor):
    """Routes GEMMs to the MXFP8 path (alto/kernels/dispatch/tensor.py:424-496)."""

    _PRECISION_TO_FP8_VARIANT = {"mxfp8_e4m3": "e4m3", "mxfp8_e5m2": "e5m2"}

    @classmethod
    def __torch_function__(cls, func, types, args, kwargs={}):
        import alto_b200.dispatch as D
        if func.__name__ == "_grouped_mm":
            A, B, offs = _grouped_args(cls, args, kwargs)
            config = B.config
            assert config.precision == "mxfp8_e4m3", (
                f"MXFP8 grouped_mm V1 supports only mxfp8_e4m3; got {config.precision} "
                "(e5m2 grouped path is not yet validated)")
            assert not config.use_hadamard and not config.use_dge, (
                "MXFP8 grouped_mm V1 does not support Hadamard or DGE options.")
            return D._quantize_then_mxfp8_scaled_grouped_mm(
                A, B, offs=offs, use_2dblock_x=config.use_2dblock_x, use_2dblock_w=config.use_2dblock_w,
                use_sr_grad=config.use_sr_grad)
        if func.__name__ in gemm_ops:
            trans_b = func.__name__ == "linear"
            A, B, bias = _split_gemm_args(func, args)
            assert not isinstance(A, cls), f"A should not be a {cls.__name__} for func {func.__name__}"
            assert isinstance(B, cls), f"B should be a {cls.__name__} for func {func.__name__}"
            config = B.config
            assert config.precision in cls._PRECISION_TO_FP8_VARIANT, (
                f"expected TrainingOpConfig with precision in {tuple(cls._PRECISION_TO_FP8_VARIANT)}, "
                f"got {config.precision}")
            assert not config.use_hadamard and not config.use_dge, (
                "MXFP8 dispatch does not support Hadamard or DGE options.")
            Y = D._to_mxfp8_then_scaled_mm(
                A, B if trans_b else B.T, fp8_variant=cls._PRECISION_TO_FP8_VARIANT[config.precision],
                use_sr_grad=config.use_sr_grad, use_2dblock_x=config.use_2dblock_x,
                use_2dblock_w=config.use_2dblock_w)
            return Y if bias is None else Y + bias
        return _passthrough(func, args, kwargs)


torch.serialization.add_safe_globals([
    MXFP4TrainingWeightWrapperTensor, NVFP4TrainingWeightWrapperTensor, MXFP8TrainingWeightWrapperTensor])


def _get_tensor_cls_for_config(config: TrainingOpConfig) -> Type[torch.Tensor]:
    if config.precision == "mxfp4":
        return MXFP4TrainingWeightWrapperTensor
    if config.precision in ("mxfp8_e4m3", "mxfp8_e5m2"):
        return MXFP8TrainingWeightWrapperTensor
    if config.precision in ("nvfp4", "amdfp4"):
        return NVFP4TrainingWeightWrapperTensor
    raise ValueError(f"Unsupported training op config: {config}")


def swap_params(module: nn.Module, *, module_filter_fn: Optional[Callable[[nn.Module, str], bool]] = None,
                config: Optional[TrainingOpConfig] = None, target_parameter_name: Optional[str] = None,
                module_name: Optional[str] = None) -> nn.Module:
    """Wraps the data of every non-bias parameter of ``module`` (post-order over its children) in
    the tensor subclass chosen by ``config`` (alto/kernels/dispatch/conversion.py:42-124)."""
    if config is None:
        raise ValueError("training op config is required")
    tensor_cls = _get_tensor_cls_for_config(config)

    if isinstance(module, nn.Parameter) and (module_filter_fn is None or module_filter_fn(module, "")):
        if not isinstance(module.data, TrainingWeightWrapperBaseTensor):
            return nn.Parameter(tensor_cls(module.data, config), requires_grad=module.requires_grad)
        return module

    def visit(mod: nn.Module, fqn: str):
        for child_name, child in mod.named_children():
            visit(child, child_name if fqn == "" else f"{fqn}.{child_name}")
        if module_filter_fn is not None and not module_filter_fn(mod, fqn):
            return
        for param_name, param in list(mod.named_parameters(recurse=False)):
            if target_parameter_name is not None and param_name != target_parameter_name:
                continue
            prefix = f"{module_name}." if module_name else ""
            full = f"{prefix}{fqn}{'.' if fqn else ''}{param_name}"
            if target_parameter_name is None and "bias" in param_name:
                logger.debug("Skipped %s because it is a bias parameter", full)
                continue
            if isinstance(param.data, TrainingWeightWrapperBaseTensor):
                continue
            setattr(mod, param_name, nn.Parameter(tensor_cls(param.data, config), requires_grad=param.requires_grad))
            logger.info("Swapped %s to %s", full, tensor_cls.__name__)
            original = mod.__class__.__name__
            mod._get_name = lambda original=original: f"{original}[{config}]"

    visit(module, "")
    return module
