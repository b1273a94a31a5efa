"""``torch.ops`` registration of the quantizer and GEMM ops, with shape functions.

The reference exposes these as ``torch.library.triton_op`` ops with ``register_fake`` shape functions
-- ``torch.ops.torchtitan.{convert_to_mxfp4, convert_from_mxfp4, blockwise_mxfp4_gemm}``
(alto/kernels/fp4/mxfp4/mxfp_quantization.py:410,548-585; mxfp_linear.py:143) and
``torch.ops.alto.{convert_to_nvfp4, convert_from_nvfp4, convert_to_mxfp8, convert_from_mxfp8,
calculate_mxfp8_scales, blockwise_mxfp8_gemm}`` -- so that traced callers keep working; likewise the
grouped GEMMs on quantised operands, ``torchtitan::mxfp4_grouped_gemm_{forward, backward_inputs,
backward_weights}`` (mxfp_grouped_gemm/cg_forward.py:200, cg_backward.py:398, 500) and
``alto::mxfp8_grouped_gemm_{forward, backward_inputs, backward_weights}`` (mxfp8_grouped_gemm/cg_forward.py:222,
cg_backward.py:313, 416).  The MXFP4 backward ops serve operands packed along the reduction axis
(``k_pack_* = True``); the reference's other packing cannot feed the FP4 tensor cores and raises.  The same
ops are registered here as ``torch.library.custom_op`` around this package's functions.  By default
they go under the namespace ``alto_b200``; a build that does not import the reference can claim the
reference's own names with ``register("torchtitan", "alto")``.

Arguments follow the reference ops; ``output_dtype`` is passed as a ``torch.dtype``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import grouped as _grp
from . import mxfp4 as _mx4
from . import mxfp8 as _mx8
from . import nvfp4 as _nv4

_registered = set()


def _axis_last_shape(t: torch.Tensor, axis: int):
    shp = list(t.shape)
    a = axis % len(shp)
    shp[a], shp[-1] = shp[-1], shp[a]
    return shp


def _quant_shapes(x, block, axis, is_2d, fp4):
    """(codes shape, scales shape) in the reference's logical (un-transposed) coordinates."""
    v = _axis_last_shape(x, axis)
    codes = list(v)
    codes[-1] = v[-1] // 2 if fp4 else v[-1]
    scales = list(v)
    scales[-1] = v[-1] // block
    if is_2d:
        scales[-2] = v[-2] // block
    a = axis % x.dim()

    def back(s):
        s = list(s)
        s[a], s[-1] = s[-1], s[a]
        return s

    return back(codes), back(scales)


def register(mxfp4_namespace: str = "alto_b200", namespace: str = "alto_b200") -> None:
    """Registers the ops (idempotent per namespace pair)."""
    key = (mxfp4_namespace, namespace)
    if key in _registered:
        return
    _registered.add(key)
    op = torch.library.custom_op

    # ---------------- MXFP4 ----------------
    @op(f"{mxfp4_namespace}::convert_to_mxfp4", mutates_args=())
    def convert_to_mxfp4(data_hp: torch.Tensor, block_size: int = 32, axis: int = -1, is_2d_block: bool = False,
                         use_sr: bool = False, use_asm: Optional[bool] = None, philox_seed: Optional[int] = None,
                         philox_offset: Optional[int] = None, clip_mode: str = "none",
                         use_uos: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        return _mx4.convert_to_mxfp4(data_hp, block_size, axis, is_2d_block, use_sr, use_asm, philox_seed,
                                     philox_offset, clip_mode, use_uos)

    @convert_to_mxfp4.register_fake
    def _(data_hp, block_size=32, axis=-1, is_2d_block=False, use_sr=False, use_asm=None, philox_seed=None,
          philox_offset=None, clip_mode="none", use_uos=False):
        c, s = _quant_shapes(data_hp, block_size, axis, is_2d_block, True)
        return data_hp.new_empty(c, dtype=torch.uint8), data_hp.new_empty(s, dtype=torch.uint8)

    @op(f"{mxfp4_namespace}::convert_from_mxfp4", mutates_args=())
    def convert_from_mxfp4(data_lp: torch.Tensor, scales: torch.Tensor, output_dtype: torch.dtype = torch.float32,
                           block_size: int = 32, axis: int = -1, is_2d_block: bool = False,
                           use_asm: Optional[bool] = None, clip_mode: str = "none") -> torch.Tensor:
        return _mx4.convert_from_mxfp4(data_lp, scales, output_dtype, block_size, axis, is_2d_block, use_asm,
                                       clip_mode).contiguous()

    @convert_from_mxfp4.register_fake
    def _(data_lp, scales, output_dtype=torch.float32, block_size=32, axis=-1, is_2d_block=False, use_asm=None,
          clip_mode="none"):
        shp = list(data_lp.shape)
        shp[axis % len(shp)] *= 2
        return data_lp.new_empty(shp, dtype=output_dtype)

    @op(f"{mxfp4_namespace}::blockwise_mxfp4_gemm", mutates_args=())
    def blockwise_mxfp4_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor,
                             use_2dblock_a: bool = False, use_2dblock_b: bool = False, k_pack_a: bool = True,
                             k_pack_b: bool = True, trans_a: bool = False, trans_b: bool = False,
                             block_size: int = 32, output_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return _mx4.blockwise_mxfp4_gemm(a, a_s, b, b_s, use_2dblock_a=use_2dblock_a, use_2dblock_b=use_2dblock_b,
                                         k_pack_a=k_pack_a, k_pack_b=k_pack_b, trans_a=trans_a, trans_b=trans_b,
                                         block_size=block_size, output_dtype=output_dtype)

    @blockwise_mxfp4_gemm.register_fake
    def _(a, a_s, b, b_s, use_2dblock_a=False, use_2dblock_b=False, k_pack_a=True, k_pack_b=True, trans_a=False,
          trans_b=False, block_size=32, output_dtype=torch.float32):
        M = a.shape[1] if trans_a else a.shape[0]
        N = b.shape[0] if trans_b else b.shape[1]
        return a.new_empty((M, N), dtype=output_dtype)

    # ---------------- NVFP4 ----------------
    # the reference declares no mutation for this op although `update_outer_scale` refreshes a
    # caller-supplied outer_scale buffer in place (nvfp_quantization.py:490, 572-575); same here
    @op(f"{namespace}::convert_to_nvfp4", mutates_args=())
    def convert_to_nvfp4(data_hp: torch.Tensor, block_size: int = 16, axis: int = -1, is_2d_block: bool = False,
                         outer_scale: Optional[torch.Tensor] = None, update_outer_scale: bool = True,
                         scale_format: str = "e4m3", use_sr: bool = False, philox_seed: Optional[int] = None,
                         philox_offset: Optional[int] = None,
                         use_asm: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        return _nv4.convert_to_nvfp4(data_hp, block_size, axis, is_2d_block, outer_scale, update_outer_scale,
                                     scale_format, use_sr, philox_seed, philox_offset, use_asm)

    @convert_to_nvfp4.register_fake
    def _(data_hp, block_size=16, axis=-1, is_2d_block=False, outer_scale=None, update_outer_scale=True,
          scale_format="e4m3", use_sr=False, philox_seed=None, philox_offset=None, use_asm=None):
        c, s = _quant_shapes(data_hp, block_size, axis, is_2d_block, True)
        return data_hp.new_empty(c, dtype=torch.uint8), data_hp.new_empty(s, dtype=torch.float32)

    @op(f"{namespace}::convert_from_nvfp4", mutates_args=())
    def convert_from_nvfp4(data_lp: torch.Tensor, scales: torch.Tensor, output_dtype: torch.dtype = torch.float32,
                           block_size: int = 16, axis: int = -1, is_2d_block: bool = False,
                           outer_scale: Optional[torch.Tensor] = None, scale_format: str = "e4m3",
                           use_asm: Optional[bool] = None) -> torch.Tensor:
        return _nv4.convert_from_nvfp4(data_lp, scales, output_dtype, block_size, axis, is_2d_block, outer_scale,
                                       scale_format, use_asm).contiguous()

    @convert_from_nvfp4.register_fake
    def _(data_lp, scales, output_dtype=torch.float32, block_size=16, axis=-1, is_2d_block=False, outer_scale=None,
          scale_format="e4m3", use_asm=None):
        shp = list(data_lp.shape)
        shp[axis % len(shp)] *= 2
        return data_lp.new_empty(shp, dtype=output_dtype)

    # ---------------- MXFP8 ----------------
    @op(f"{namespace}::convert_to_mxfp8", mutates_args=())
    def convert_to_mxfp8(data_hp: torch.Tensor, block_size: int = 32, mxfp_format: str = "e4m3", axis: int = -1,
                         is_2d_block: bool = False, use_sr: bool = False, use_asm: Optional[bool] = None,
                         philox_seed: Optional[int] = None,
                         philox_offset: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        return _mx8.convert_to_mxfp8(data_hp, block_size, mxfp_format, axis, is_2d_block, use_sr, use_asm,
                                     philox_seed, philox_offset)

    @convert_to_mxfp8.register_fake
    def _(data_hp, block_size=32, mxfp_format="e4m3", axis=-1, is_2d_block=False, use_sr=False, use_asm=None,
          philox_seed=None, philox_offset=None):
        c, s = _quant_shapes(data_hp, block_size, axis, is_2d_block, False)
        dt = torch.float8_e4m3fn if mxfp_format == "e4m3" else torch.float8_e5m2
        return data_hp.new_empty(c, dtype=dt), data_hp.new_empty(s, dtype=torch.uint8)

    @op(f"{namespace}::convert_from_mxfp8", mutates_args=())
    def convert_from_mxfp8(data_lp: torch.Tensor, scales: torch.Tensor, output_dtype: torch.dtype = torch.float32,
                           block_size: int = 32, axis: int = -1, is_2d_block: bool = False,
                           use_asm: Optional[bool] = None) -> torch.Tensor:
        return _mx8.convert_from_mxfp8(data_lp, scales, output_dtype, block_size, axis, is_2d_block,
                                       use_asm).contiguous()

    @convert_from_mxfp8.register_fake
    def _(data_lp, scales, output_dtype=torch.float32, block_size=32, axis=-1, is_2d_block=False, use_asm=None):
        return data_lp.new_empty(list(data_lp.shape), dtype=output_dtype)

    @op(f"{namespace}::calculate_mxfp8_scales", mutates_args=())
    def calculate_mxfp8_scales(data_hp: torch.Tensor, block_size: int = 32, mxfp_format: str = "e4m3",
                               axis: int = -1, is_2d_block: bool = False) -> torch.Tensor:
        return _mx8.calculate_mxfp8_scales(data_hp, block_size, mxfp_format, axis, is_2d_block).contiguous()

    @calculate_mxfp8_scales.register_fake
    def _(data_hp, block_size=32, mxfp_format="e4m3", axis=-1, is_2d_block=False):
        return data_hp.new_empty(_quant_shapes(data_hp, block_size, axis, is_2d_block, False)[1], dtype=torch.uint8)

    @op(f"{namespace}::blockwise_mxfp8_gemm", mutates_args=())
    def blockwise_mxfp8_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor,
                             trans_a: bool = False, trans_b: bool = False, use_2dblock_a: bool = False,
                             use_2dblock_b: bool = False, block_size: int = 32,
                             output_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return _mx8.blockwise_mxfp8_gemm(a, a_s, b, b_s, trans_a, trans_b, use_2dblock_a, use_2dblock_b, block_size,
                                         output_dtype)

    @blockwise_mxfp8_gemm.register_fake
    def _(a, a_s, b, b_s, trans_a=False, trans_b=False, use_2dblock_a=False, use_2dblock_b=False, block_size=32,
          output_dtype=torch.float32):
        M = a.shape[1] if trans_a else a.shape[0]
        N = b.shape[0] if trans_b else b.shape[1]
        return a.new_empty((M, N), dtype=output_dtype)

    # ---------------- grouped (MoE) forward GEMMs on quantised operands ----------------
    @op(f"{mxfp4_namespace}::mxfp4_grouped_gemm_forward", mutates_args=())
    def mxfp4_grouped_gemm_forward(inputs: torch.Tensor, expert_weights: torch.Tensor, expert_indices: torch.Tensor,
                                   input_scales: torch.Tensor, weight_scales: torch.Tensor,
                                   trans_weights: bool = True, use_2dblock_x: bool = False,
                                   use_2dblock_w: bool = True,
                                   output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return _grp.mxfp4_grouped_gemm_forward(inputs, expert_weights, expert_indices, input_scales, weight_scales,
                                               trans_weights, use_2dblock_x, use_2dblock_w, output_dtype)

    @mxfp4_grouped_gemm_forward.register_fake
    def _(inputs, expert_weights, expert_indices, input_scales, weight_scales, trans_weights=True,
          use_2dblock_x=False, use_2dblock_w=True, output_dtype=torch.bfloat16):
        N = expert_weights.shape[1] if trans_weights else expert_weights.shape[2]
        return inputs.new_empty((inputs.shape[0], N), dtype=output_dtype)

    @op(f"{namespace}::mxfp8_grouped_gemm_forward", mutates_args=())
    def mxfp8_grouped_gemm_forward(inputs: torch.Tensor, expert_weights: torch.Tensor, expert_indices: torch.Tensor,
                                   input_scales: torch.Tensor, weight_scales: torch.Tensor,
                                   trans_weights: bool = True, use_2dblock_x: bool = False,
                                   use_2dblock_w: bool = True, lhs_format_id: int = 0, rhs_format_id: int = 0,
                                   output_dtype: torch.dtype = torch.bfloat16,
                                   use_dot_scaled: Optional[bool] = None) -> torch.Tensor:
        return _grp.mxfp8_grouped_gemm_forward(inputs, expert_weights, expert_indices, input_scales, weight_scales,
                                               trans_weights, use_2dblock_x, use_2dblock_w, lhs_format_id,
                                               rhs_format_id, output_dtype, use_dot_scaled)

    @mxfp8_grouped_gemm_forward.register_fake
    def _(inputs, expert_weights, expert_indices, input_scales, weight_scales, trans_weights=True,
          use_2dblock_x=False, use_2dblock_w=True, lhs_format_id=0, rhs_format_id=0, output_dtype=torch.bfloat16,
          use_dot_scaled=None):
        N = expert_weights.shape[1] if trans_weights else expert_weights.shape[2]
        return inputs.new_empty((inputs.shape[0], N), dtype=output_dtype)

    # ---------------- grouped (MoE) backward GEMMs on quantised operands ----------------
    def _dx_shape(grad_output, expert_weights, trans_weights):
        K = expert_weights.shape[2] if trans_weights else expert_weights.shape[1]
        return (grad_output.shape[0], K)

    @op(f"{mxfp4_namespace}::mxfp4_grouped_gemm_backward_inputs", mutates_args=())
    def mxfp4_grouped_gemm_backward_inputs(grad_output: torch.Tensor, expert_weights: torch.Tensor,
                                           expert_indices: torch.Tensor, go_scales: torch.Tensor,
                                           expert_weight_scales: torch.Tensor, trans_weights: bool = True,
                                           use_2dblock_x: bool = False, use_2dblock_w: bool = True,
                                           k_pack_w: bool = True,
                                           output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return _grp.mxfp4_grouped_gemm_backward_inputs(grad_output, expert_weights, expert_indices, go_scales,
                                                       expert_weight_scales, trans_weights, use_2dblock_x,
                                                       use_2dblock_w, k_pack_w, output_dtype)

    @mxfp4_grouped_gemm_backward_inputs.register_fake
    def _(grad_output, expert_weights, expert_indices, go_scales, expert_weight_scales, trans_weights=True,
          use_2dblock_x=False, use_2dblock_w=True, k_pack_w=True, output_dtype=torch.bfloat16):
        return grad_output.new_empty(_dx_shape(grad_output, expert_weights, trans_weights), dtype=output_dtype)

    @op(f"{mxfp4_namespace}::mxfp4_grouped_gemm_backward_weights", mutates_args=())
    def mxfp4_grouped_gemm_backward_weights(grad_output: torch.Tensor, inputs: torch.Tensor,
                                            expert_indices: torch.Tensor, num_experts: int, go_scales: torch.Tensor,
                                            input_scales: torch.Tensor, trans_weights: bool = True,
                                            use_2dblock_go: bool = False, use_2dblock_x: bool = True,
                                            k_pack_go: bool = True, k_pack_x: bool = True,
                                            output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return _grp.mxfp4_grouped_gemm_backward_weights(grad_output, inputs, expert_indices, num_experts, go_scales,
                                                        input_scales, trans_weights, use_2dblock_go, use_2dblock_x,
                                                        k_pack_go, k_pack_x, output_dtype).contiguous()

    @mxfp4_grouped_gemm_backward_weights.register_fake
    def _(grad_output, inputs, expert_indices, num_experts, go_scales, input_scales, trans_weights=True,
          use_2dblock_go=False, use_2dblock_x=True, k_pack_go=True, k_pack_x=True, output_dtype=torch.bfloat16):
        N, K = grad_output.shape[1], inputs.shape[1]
        return grad_output.new_empty((num_experts, N, K) if trans_weights else (num_experts, K, N), dtype=output_dtype)

    @op(f"{namespace}::mxfp8_grouped_gemm_backward_inputs", mutates_args=())
    def mxfp8_grouped_gemm_backward_inputs(grad_output: torch.Tensor, expert_weights: torch.Tensor,
                                           expert_indices: torch.Tensor, go_scales: torch.Tensor,
                                           expert_weight_scales: torch.Tensor, trans_weights: bool = True,
                                           use_2dblock_x: bool = False, use_2dblock_w: bool = True,
                                           lhs_format_id: int = 0, rhs_format_id: int = 0,
                                           output_dtype: torch.dtype = torch.bfloat16,
                                           use_dot_scaled: Optional[bool] = None) -> torch.Tensor:
        return _grp.mxfp8_grouped_gemm_backward_inputs(grad_output, expert_weights, expert_indices, go_scales,
                                                       expert_weight_scales, trans_weights, use_2dblock_x,
                                                       use_2dblock_w, lhs_format_id, rhs_format_id, output_dtype,
                                                       use_dot_scaled)

    @mxfp8_grouped_gemm_backward_inputs.register_fake
    def _(grad_output, expert_weights, expert_indices, go_scales, expert_weight_scales, trans_weights=True,
          use_2dblock_x=False, use_2dblock_w=True, lhs_format_id=0, rhs_format_id=0, output_dtype=torch.bfloat16,
          use_dot_scaled=None):
        return grad_output.new_empty(_dx_shape(grad_output, expert_weights, trans_weights), dtype=output_dtype)

    @op(f"{namespace}::mxfp8_grouped_gemm_backward_weights", mutates_args=())
    def mxfp8_grouped_gemm_backward_weights(grad_output: torch.Tensor, inputs: torch.Tensor,
                                            expert_indices: torch.Tensor, num_experts: int, go_scales: torch.Tensor,
                                            input_scales: torch.Tensor, trans_weights: bool = True,
                                            use_2dblock_go: bool = False, use_2dblock_x: bool = False,
                                            lhs_format_id: int = 0, rhs_format_id: int = 0,
                                            output_dtype: torch.dtype = torch.bfloat16,
                                            use_dot_scaled: Optional[bool] = None) -> torch.Tensor:
        return _grp.mxfp8_grouped_gemm_backward_weights(grad_output, inputs, expert_indices, num_experts, go_scales,
                                                        input_scales, trans_weights, use_2dblock_go, use_2dblock_x,
                                                        lhs_format_id, rhs_format_id, output_dtype,
                                                        use_dot_scaled).contiguous()

    @mxfp8_grouped_gemm_backward_weights.register_fake
    def _(grad_output, inputs, expert_indices, num_experts, go_scales, input_scales, trans_weights=True,
          use_2dblock_go=False, use_2dblock_x=False, lhs_format_id=0, rhs_format_id=0, output_dtype=torch.bfloat16,
          use_dot_scaled=None):
        N, K = grad_output.shape[1], inputs.shape[1]
        return grad_output.new_empty((num_experts, N, K) if trans_weights else (num_experts, K, N), dtype=output_dtype)

