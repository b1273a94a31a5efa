"""Weight de-oscillation for FP4 training: the optimizer ``step_post_hook`` that is the other
per-step caller of the quantizers.

Same knobs, per-parameter state keys and decisions as the reference
(alto/components/optimizer.py:43-413): after every optimizer step each FP4-wrapped weight
accumulates how far it moved (``osci_dist_w += |w - prev|``) and how far its quantise-dequantise image
moved (``osci_dist_w_qdq += |Q(w) - Q(prev)|``); at the end of a period of ``period`` steps the
elements whose ratio ``dist_w_qdq / dist_w`` reaches ``ratio_threshold`` are snapped to their current
bin centre ``Q(w)`` and a new period starts.  ``Q`` is the forward pass's quantizer for that weight
(format, 1-D/2-D blocks, tensorwise outer scale, use_uos), along the weight's reduction axis.

The round trips run through this package's quantizer and dequantizer kernels and the three
accumulations of a step are one fused kernel (``altob200_deosc_accumulate``).
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Callable, Iterable

import torch
import torch.nn as nn

from . import _lib as L
from .dispatch import (MXFP4TrainingWeightWrapperTensor, NVFP4TrainingWeightWrapperTensor, TrainingOpConfig,
                       TrainingWeightWrapperBaseTensor)

logger = logging.getLogger("alto_b200")

__all__ = ["DeOscillationConfig", "enable_de_oscillation"]

_FP4_WRAPPER_TYPES = (MXFP4TrainingWeightWrapperTensor, NVFP4TrainingWeightWrapperTensor)


def _infer_reduction_axis(w: torch.Tensor) -> int:
    if w.dim() == 2:
        return -1
    if w.dim() == 3:
        return -2
    raise ValueError(f"Unexpected weight shape: {w.shape}")


def _peel_to_fp4_wrapper(p: torch.Tensor):
    """The FP4 wrapper tensor backing ``p`` (plain parameter, or a DTensor whose local tensor is one)."""
    t = p.data if isinstance(p, nn.Parameter) else p
    if hasattr(t, "_local_tensor"):
        t = t._local_tensor
    return t if isinstance(t, _FP4_WRAPPER_TYPES) else None


def _make_qdq_fn_for(cfg: TrainingOpConfig) -> Callable[[torch.Tensor, int], torch.Tensor]:
    """``dequant(quant(., axis))`` matching the wrapper's forward-path quantizer
    (alto/components/optimizer.py:123-220), including the row padding to a whole block."""
    from . import mxfp4, nvfp4
    is_2d = cfg.use_2dblock_w
    if cfg.precision == "mxfp4":
        block = 32

        def convert(w, axis):
            q, s = mxfp4.convert_to_mxfp4(w, axis=axis, is_2d_block=is_2d, use_uos=cfg.use_uos)
            return mxfp4.convert_from_mxfp4(q, s, output_dtype=w.dtype, axis=axis, is_2d_block=is_2d)
    elif cfg.precision == "nvfp4":
        block = 16
        use_outer = cfg.two_level_scaling == "tensorwise"

        def convert(w, axis):
            outer = torch.empty(1, dtype=torch.float32, device=w.device) if use_outer else None
            q, s = nvfp4.convert_to_nvfp4(w, axis=axis, is_2d_block=is_2d, outer_scale=outer,
                                          update_outer_scale=use_outer)
            return nvfp4.convert_from_nvfp4(q, s, output_dtype=w.dtype, axis=axis, is_2d_block=is_2d,
                                            outer_scale=outer)
    else:
        raise ValueError(f"de-oscillation only supports FP4 wrappers, got precision={cfg.precision!r}")

    def qdq(w: torch.Tensor, axis: int) -> torch.Tensor:
        rows = -1
        if w.dim() == 2 and w.shape[0] % block != 0:
            rows = w.shape[0]
            w = torch.nn.functional.pad(w, (0, 0, 0, block - rows % block))
        out = convert(w, axis)
        return out[:rows, :] if rows != -1 else out

    return qdq


@dataclass(kw_only=True, slots=True)
class DeOscillationConfig:
    """enable: master switch; period: optimizer steps per window; ratio_threshold: an element is reset
    when dist_w_qdq / dist_w >= ratio_threshold over the window; log_freq: log every that many
    triggered periods (0 = never).  (alto/components/optimizer.py:223-253)"""
    enable: bool = False
    period: int = 25
    ratio_threshold: float = 16.0
    log_freq: int = 0


class _DeOscillationHook:
    KEY_STEP = "osci_step_in_period"
    KEY_DIST_FP = "osci_dist_w"
    KEY_DIST_QDQ = "osci_dist_w_qdq"
    KEY_PREV = "osci_prev_weight"
    _EPS = 1.0e-30

    def __init__(self, cfg: DeOscillationConfig) -> None:
        self._cfg = cfg
        self._qdq_cache: dict = {}
        self._periods_completed = 0

    def _wrapper_if_eligible(self, p: nn.Parameter):
        if not p.requires_grad:
            return None
        wrapper = _peel_to_fp4_wrapper(p)
        if wrapper is None:
            return None
        cfg = wrapper.config
        if cfg is None or cfg.precision not in ("mxfp4", "nvfp4"):
            return None
        return wrapper

    def _qdq_for(self, wrapper) -> Callable:
        cfg = wrapper.config
        fn = self._qdq_cache.get(cfg)
        if fn is None:
            fn = _make_qdq_fn_for(cfg)
            self._qdq_cache[cfg] = fn
        return fn

    def __call__(self, optimizer, args, kwargs) -> None:  # noqa: ARG002
        triggered, n_reset, n_total = 0, 0, 0
        for group in optimizer.param_groups:
            for p in group["params"]:
                wrapper = self._wrapper_if_eligible(p)
                if wrapper is None:
                    continue
                r, t, did = self._step_param(wrapper, optimizer.state[p])
                if did:
                    triggered += 1
                    n_reset += r
                    n_total += t
        if triggered and self._cfg.log_freq:
            self._periods_completed += 1
            if self._periods_completed % self._cfg.log_freq == 0 and n_total > 0:
                logger.info("[de-osc] period#%d triggered_params=%d reset_ratio=%.4f%% (%d/%d)",
                            self._periods_completed, triggered, n_reset / n_total * 100.0, n_reset, n_total)

    def _step_param(self, wrapper: TrainingWeightWrapperBaseTensor, state: dict) -> tuple:
        cfg = self._cfg
        raw = wrapper._data
        w_now = raw.detach()
        if self.KEY_PREV not in state or self.KEY_STEP not in state:
            self._init_period_state(state, w_now)
            return 0, 0, False
        prev = state[self.KEY_PREV]
        dist_w = state[self.KEY_DIST_FP]
        dist_q = state[self.KEY_DIST_QDQ]
        qdq_fn = self._qdq_for(wrapper)
        axis = _infer_reduction_axis(w_now)
        w_c = w_now.contiguous()
        w_qdq = qdq_fn(w_c, axis).contiguous()
        prev_qdq = qdq_fn(prev, axis).contiguous()
        L.deosc_accumulate(w_c, prev, w_qdq, prev_qdq, dist_w, dist_q)   # also prev <- w
        state[self.KEY_STEP] += 1
        if state[self.KEY_STEP] < cfg.period:
            return 0, 0, False
        ratio = dist_q / dist_w.clamp(min=self._EPS)
        reset_mask = (dist_w > 0) & (ratio >= cfg.ratio_threshold)
        reset_count, total = 0, dist_w.numel()
        if reset_mask.any():
            reset_count = int(reset_mask.sum().item())
            raw[reset_mask] = w_qdq[reset_mask]
            prev.copy_(raw)
        dist_w.zero_()
        dist_q.zero_()
        state[self.KEY_STEP] = 0
        return reset_count, total, True

    def _init_period_state(self, state: dict, w: torch.Tensor) -> None:
        state[self.KEY_PREV] = w.detach().clone().contiguous()
        state[self.KEY_DIST_FP] = torch.zeros_like(state[self.KEY_PREV])
        state[self.KEY_DIST_QDQ] = torch.zeros_like(state[self.KEY_PREV])
        state[self.KEY_STEP] = 0


_HOOK_ATTR = "_alto_b200_deosc_hook"


def enable_de_oscillation(optimizers: Any, cfg: DeOscillationConfig) -> None:
    """Registers the hook on every optimizer once (a container with ``.optimizers``, an iterable of
    optimizers, or one optimizer)."""
    if not cfg.enable:
        return
    if hasattr(optimizers, "optimizers"):
        opts: Iterable = optimizers.optimizers
    elif isinstance(optimizers, torch.optim.Optimizer):
        opts = [optimizers]
    else:
        opts = list(optimizers)
    for opt in opts:
        if getattr(opt, _HOOK_ATTR, None) is not None:
            continue
        hook = _DeOscillationHook(cfg)
        opt.register_step_post_hook(hook)
        setattr(opt, _HOOK_ATTR, hook)
