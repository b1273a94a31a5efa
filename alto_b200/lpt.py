"""``LowPrecisionTrainingModifier``: the recipe-facing scheme surface.

Field for field the reference's pydantic model (alto/modifiers/lpt/base.py:29-258): ``scheme``
(one of mxfp4 / mxfp8_e4m3 / mxfp8_e5m2 / nvfp4 / amdfp4, or a dict scheme -> targets),
``targets``, ``ignore``, the recipe flags, ``lora_rank`` and the de-oscillation knobs, the same
validators, ``resolved_config`` and the modifier lifecycle (convert / convert_config / initialize /
pre_step / post_step / finalize, alto/modifiers/base.py:56-113).  ``on_convert`` wraps the
parameters of every matched ``nn.Linear`` and ``*GroupedExperts`` module with ``swap_params``.

Parts of the reference's modifier that belong to other subsystems are refused with a clear
error instead of being imitated: LoRA decomposition (``lora_rank > 0``), the low-precision
attention swap and the TorchTitan config rewriting
(``on_convert_config`` needs the TorchTitan fork; without it the call only records that routed
experts must be padded to ``ALIGN_SIZE_M`` = 128 tokens by the dispatcher).
"""
from __future__ import annotations

import logging
from typing import Literal, Optional

import torch
from pydantic import BaseModel, ConfigDict, Field, PrivateAttr, field_validator, model_validator
from torch.nn import Module

from .dispatch import TrainingOpConfig, swap_params
from .grouped import ALIGN_SIZE_M

logger = logging.getLogger("alto_b200")

__all__ = ["LowPrecisionTrainingModifier"]

_SCHEMES = ["mxfp4", "mxfp8_e4m3", "mxfp8_e5m2", "nvfp4", "amdfp4"]


def _match_named_modules(model: Module, targets, ignore):
    """compressed_tensors.utils.match_named_modules when available (the reference's matcher), else
    the subset of its rules the recipes use: class name, exact module name, or ``re:`` pattern."""
    try:
        from compressed_tensors.utils import match_named_modules
        yield from match_named_modules(model, targets, ignore)
        return
    except ImportError:
        pass
    import re

    def hit(name, module, pats):
        for p in pats:
            if p.startswith("re:"):
                if re.match(p[3:], name):
                    return True
            elif p == name or p == module.__class__.__name__:
                return True
        return False

    for name, module in model.named_modules():
        if hit(name, module, targets) and not hit(name, module, ignore or []):
            yield name, module


class LowPrecisionTrainingModifier(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True, extra="forbid")

    scheme: str | dict[str, list[str]]
    targets: str | list[str] = Field(default_factory=lambda: ["Linear"])
    ignore: list[str] = Field(default_factory=lambda: ["output"])

    use_2dblock_x: bool = False
    use_2dblock_w: bool = True
    use_hadamard: bool = False
    use_sr_grad: bool = False
    use_dge: bool = False
    two_level_scaling: Literal["none", "tensorwise", "blockwise"] = "none"
    clip_mode: Literal["none", "static", "dynamic"] = "none"
    use_uos: bool = False

    lora_rank: int = 0
    deosc_step: int = 0
    deosc_period: int = 200
    deosc_ratio: float = 4.0
    deosc_log_freq: int = 1

    initialized_: bool = False
    finalized_: bool = False
    started_: bool = False
    ended_: bool = False

    _resolved_config: Optional[dict] = PrivateAttr(default=None)
    _token_alignment: Optional[int] = PrivateAttr(default=None)

    @field_validator("targets", mode="before")
    def validate_targets(cls, value):
        return [value] if isinstance(value, str) else value

    @field_validator("scheme", mode="before")
    def validate_scheme(cls, value):
        if isinstance(value, str) and value not in _SCHEMES:
            raise ValueError(f"Unsupported training op scheme: {value}")
        if isinstance(value, dict):
            for scheme_name in value:
                cls.validate_scheme(scheme_name)
            for key, target in value.items():
                value[key] = cls.validate_targets(target)
        return value

    @model_validator(mode="after")
    def validate_lora_rank_alignment(self):
        schemes = self.scheme if isinstance(self.scheme, dict) else {self.scheme: None}
        if self.lora_rank > 0:
            for scheme_name in schemes:
                if scheme_name in ("nvfp4", "amdfp4") and self.lora_rank % 16 != 0:
                    raise ValueError(f"lora_rank must be divisible by 16 for {scheme_name}, got {self.lora_rank}")
                if scheme_name in ("mxfp4", "mxfp8_e4m3", "mxfp8_e5m2") and self.lora_rank % 32 != 0:
                    raise ValueError(f"lora_rank must be divisible by 32 for {scheme_name}, got {self.lora_rank}")
            if self.use_uos:
                assert all(s in ("mxfp4",) for s in schemes), "UOS is only supported for mxfp4"
                assert self.clip_mode == "none", "UOS is only supported with clip mode none"
        return self

    @field_validator("deosc_step", mode="after")
    def validate_deosc_step(cls, value: int) -> int:
        if value < 0:
            raise ValueError("deosc_step must be non-negative")
        return value

    @field_validator("deosc_period", mode="after")
    def validate_deosc_period(cls, value: int) -> int:
        if value <= 0:
            raise ValueError("deosc_period must be positive")
        return value

    @field_validator("deosc_ratio", mode="after")
    def validate_deosc_ratio(cls, value: float) -> float:
        if value <= 0:
            raise ValueError("deosc_ratio must be positive")
        return value

    @field_validator("deosc_log_freq", mode="after")
    def validate_deosc_log_freq(cls, value: int) -> int:
        if value < 0:
            raise ValueError("deosc_log_freq must be non-negative")
        return value

    @property
    def requires_training_mode(self) -> bool:
        return True

    @property
    def resolved_config(self) -> dict:
        """TrainingOpConfig -> target patterns (alto/modifiers/lpt/base.py:148-169)."""
        if self._resolved_config is None:
            if isinstance(self.scheme, str):
                self.scheme = {self.scheme: self.targets}
            self._resolved_config = {}
            for scheme_name, targets in self.scheme.items():
                cfg = TrainingOpConfig(
                    precision=scheme_name, use_2dblock_x=self.use_2dblock_x, use_2dblock_w=self.use_2dblock_w,
                    use_hadamard=self.use_hadamard, use_sr_grad=self.use_sr_grad, use_dge=self.use_dge,
                    two_level_scaling=self.two_level_scaling, clip_mode=self.clip_mode, use_uos=self.use_uos)
                self._resolved_config[cfg] = targets
        return self._resolved_config

    # ---- lifecycle (alto/modifiers/base.py:56-113) ----
    def convert(self, model: Module, **kwargs) -> bool:
        return self.on_convert(model, **kwargs)

    def convert_config(self, model_config) -> bool:
        return self.on_convert_config(model_config)

    def initialize(self, model_parts: list, **kwargs):
        if self.initialized_:
            raise RuntimeError("Cannot initialize a modifier that has already been initialized")
        if self.finalized_:
            raise RuntimeError("Cannot initialize a modifier that has already been finalized")
        assert isinstance(model_parts, list), "model_parts must be a list of nn.Module"
        self.initialized_ = self.on_initialize(model_parts, **kwargs)

    def finalize(self, model_parts: list, **kwargs):
        if self.finalized_:
            raise RuntimeError("cannot finalize a modifier twice")
        if not self.initialized_:
            raise RuntimeError("cannot finalize an uninitialized modifier")
        assert isinstance(model_parts, list), "model_parts must be a list of nn.Module"
        self.finalized_ = self.on_finalize(model_parts, **kwargs)

    def pre_step(self, model_parts: list, **kwargs):
        if not self.initialized_ or self.finalized_:
            raise RuntimeError("cannot call pre-step method on an uninitialized or finalized modifier")
        self.started_ = self.on_pre_step(model_parts, **kwargs)

    def post_step(self, model_parts: list, **kwargs):
        if not self.initialized_ or self.finalized_:
            raise RuntimeError("cannot call post-step method on an uninitialized or finalized modifier")
        self.ended_ = self.on_post_step(model_parts, **kwargs)

    # ---- hooks ----
    def on_convert(self, model: Module, **kwargs) -> bool:
        if self.lora_rank > 0:
            raise NotImplementedError("lora_rank > 0 (DecomposedLinear) is outside the low-precision linear path")
        for scheme_obj, targets in self.resolved_config.items():
            if scheme_obj.precision == "amdfp4":
                raise NotImplementedError("scheme 'amdfp4' is an AMD-only format and is not part of the B200 path")
            for name, module in _match_named_modules(model, targets, self.ignore):
                if isinstance(module, torch.nn.Linear):
                    swap_params(module, config=scheme_obj, module_name=name)
                elif module.__class__.__name__.endswith("GroupedExperts"):
                    swap_params(module, config=scheme_obj, module_name=name)
                elif module.__class__.__name__.endswith("Attention"):
                    raise NotImplementedError("the low-precision attention swap is out of scope: attention stays "
                                              "bf16 on this path; remove attention modules from `targets`")
                else:
                    raise ValueError(f"Unsupported module type: {type(module)}")
        logger.info("LowPrecisionTrainingModifier converted model: %s", model)
        return True

    def on_convert_config(self, model_config) -> bool:
        """With the TorchTitan fork: swap the token dispatcher of every GroupedExperts config so that
        routed tokens per expert are padded to ALIGN_SIZE_M (alto/modifiers/lpt/base.py:194-201).
        Without it, record the requirement for the caller's dispatcher."""
        self._token_alignment = ALIGN_SIZE_M
        try:
            from torchtitan.components.quantization.utils import swap_token_dispatcher
            from torchtitan.models.common.moe import GroupedExperts
        except ImportError:
            return True
        for _fqn, _config, parent, _attr in model_config.traverse(GroupedExperts.Config):
            swap_token_dispatcher(parent, ALIGN_SIZE_M)
        return True

    @property
    def token_alignment(self) -> Optional[int]:
        return self._token_alignment

    def on_initialize(self, model_parts: list, **kwargs) -> bool:
        return True

    def on_pre_step(self, model_parts: list, **kwargs) -> bool:
        """From step ``deosc_step`` on, install the de-oscillation hook on the trainer's optimizers
        (alto/modifiers/lpt/base.py:237-251)."""
        trainer = kwargs.get("trainer", None)
        if self.deosc_step > 0:
            if trainer is None:
                raise ValueError("Trainer must be passed to the pre_step method to enable weight de-oscillation.")
            if trainer.step >= self.deosc_step:
                from .deosc import DeOscillationConfig, enable_de_oscillation
                enable_de_oscillation(trainer.optimizers, DeOscillationConfig(
                    enable=True, period=self.deosc_period, ratio_threshold=self.deosc_ratio,
                    log_freq=self.deosc_log_freq))
        return True

    def on_post_step(self, model_parts: list, **kwargs) -> bool:
        return True

    def on_finalize(self, model_parts: list, **kwargs) -> bool:
        return True
