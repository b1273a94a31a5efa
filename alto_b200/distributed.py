"""Multi-GPU forms of the low-precision linear path (one process per GPU, ``torch.distributed``).

Four ways the path shards, each with exactly the exchange it needs and nothing more:

* data parallel replicas        -- every rank runs the full linear on its own batch; the only
  exchange is the all-reduce of the weight gradients (``allreduce_gradients``).
* column-sharded linear         -- W [N, K] split along N; forward and wgrad are local, dgrad is a
  sum over ranks (``column_sharded_linear``: all-reduce of dX in backward).  N / world must be a
  multiple of 32 so that 2-D weight blocks never straddle ranks.
* fully sharded weight          -- every rank owns rows of W, quantises them and all-gathers the 4.5-bit
  payload instead of bf16 (``gathered_weight_linear``); dW is reduce-scattered.
* expert parallel MoE           -- experts split across ranks, tokens exchanged by all-to-all with
  variable splits each way (``ExpertParallelDispatcher``), local rows sorted by expert and padded
  to runs of 128 for the grouped GEMMs.

The reference has no multi-GPU code of its own for this path: it relies on its TorchTitan fork
(alto/modifiers/lpt/base.py:194-201 swaps the token dispatcher so that per-expert row counts are
padded to ALIGN_SIZE_M = 128; alto/kernels/dispatch/tensor.py:159-211 are the FSDP hooks).  The
semantics here are those of stock TorchTitan's expert-parallel dispatch (tokens sorted by expert,
all-to-all by owner rank, local re-sort by expert, padding rows of zeros, weighted combine).

Quantisation placement: everything that depends on which rows sit next to each other (token-axis
blocks, the Hadamard rotation along tokens, the tensorwise amax) runs after the exchange on local
data, so a rank's results are bit-identical to a single-GPU run on the same local rows.

Data always sits in local HBM before a kernel reads it: the exchanges are NCCL collectives, no
kernel of this library reads a peer's memory.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib as L

__all__ = ["allreduce_gradients", "shard_rows", "column_sharded_linear", "gathered_weight_linear",
           "gather_packed_rows", "gather_columns", "interleave_gathered_columns", "outer_scale_from_amax_bits",
           "ExpertParallelDispatcher", "permute_pad_plan", "ALIGN_SIZE_M"]

ALIGN_SIZE_M = 128


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


# ------------------------------------------------------------------------------------------
# data parallel: all-reduce of weight gradients
# ------------------------------------------------------------------------------------------
def allreduce_gradients(params: Sequence[torch.Tensor], group=None, bucket_bytes: int = 64 << 20,
                        average: bool = True, max_in_flight: int = 2) -> int:
    """Sums (or averages) ``p.grad`` over the ranks of ``group`` in buckets of ``bucket_bytes``:
    each bucket is one flat all-reduce, issued asynchronously so that copy-in of the next bucket
    overlaps the reduction of the previous one.  Returns the number of collectives issued.

    The bucket plan is a function of the parameter list alone (shapes and dtypes), not of which
    gradients exist on this rank: a parameter without a gradient contributes zeros, so every rank
    issues the same collectives.  At most ``max_in_flight`` flat buffers are alive at a time (the
    oldest bucket is waited for and scattered back before another one is flattened), which bounds
    the extra memory at ``max_in_flight * bucket_bytes`` instead of a copy of all gradients.

    Buckets are sized for launch latency and overlap, not for link count: NVSwitch gives every
    peer full bandwidth, and NCCL reduces inside the switch when it can."""
    world = _world(group)
    params = [p for p in params if p.requires_grad]
    if world == 1 or not params:
        return 0
    buckets: List[List[torch.Tensor]] = [[]]
    size = 0
    for p in params:
        nbytes = p.numel() * p.element_size()
        if buckets[-1] and (size + nbytes > bucket_bytes or p.dtype != buckets[-1][0].dtype):
            buckets.append([])
            size = 0
        buckets[-1].append(p)
        size += nbytes

    def finish(work, flat, bucket):
        work.wait()
        if average:
            flat.div_(world)
        off = 0
        for p in bucket:
            piece = flat[off:off + p.numel()].view(p.shape)
            if p.grad is None:
                p.grad = piece.clone()
            else:
                p.grad.copy_(piece)
            off += p.numel()

    pending = []
    for b in buckets:
        if len(pending) >= max_in_flight:
            finish(*pending.pop(0))
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in b])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        pending.append((work, flat, b))
    for item in pending:
        finish(*item)
    return len(buckets)


# ------------------------------------------------------------------------------------------
# column-sharded linear
# ------------------------------------------------------------------------------------------
def shard_rows(w: torch.Tensor, group=None, multiple: int = 32) -> torch.Tensor:
    """This rank's rows [r * N / world, (r + 1) * N / world) of w [N, K] (a view)."""
    world, rank = _world(group), _rank(group)
    N = w.shape[0]
    torch._check(N % world == 0 and (N // world) % multiple == 0,
                 lambda: f"out_features {N} must split into {world} shards that are multiples of {multiple}")
    n = N // world
    return w[rank * n:(rank + 1) * n]


class _DxReduction:
    """The all-reduce of one backward pass's partial dX, started inside the linear's backward."""

    def __init__(self):
        self.work = None
        self.tensor = None


class _CopyToShards(torch.autograd.Function):
    """Identity in forward; in backward the partial input gradients of the shards are summed."""

    @staticmethod
    def forward(ctx, x, group, pending):
        ctx.group = group
        ctx.pending = pending
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        from . import _linear as E
        E.take_dx_ready_hook()          # a linear that did not take the hook must not leave it armed
        p = ctx.pending
        if p is not None and p.work is not None:
            # started right after the dgrad GEMM; it ran beside the wgrad quantizer and GEMM
            p.work.wait()
            grad = p.tensor.view(grad.shape)
            p.work = p.tensor = None
        elif _world(ctx.group) > 1:
            grad = grad.contiguous()
            dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=ctx.group)
        return grad, None, None


class _ArmDxAllReduce(torch.autograd.Function):
    """Identity on the linear's output; its backward runs right before the linear's and arms the hook
    through which that backward hands over dX as soon as the dgrad GEMM is in the stream."""

    @staticmethod
    def forward(ctx, y, group, pending):
        ctx.group = group
        ctx.pending = pending
        return y.view_as(y)

    @staticmethod
    def backward(ctx, grad):
        from . import _linear as E
        group, pending = ctx.group, ctx.pending

        def start(dx: torch.Tensor) -> None:
            pending.tensor = dx
            pending.work = dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group, async_op=True)

        E.set_dx_ready_hook(start)
        return grad, None, None


def column_sharded_linear(x: torch.Tensor, w_shard: torch.Tensor, linear_fn: Callable, group=None,
                          overlap_dx_reduction: bool = False) -> torch.Tensor:
    """Y_r = linear_fn(x, W_r) with W_r this rank's [N / world, K] shard; x is replicated.

    Forward has no exchange (the concatenation of the Y_r along N is implicit in the sharding of
    whatever consumes them), wgrad is local (dY_r, x), and dgrad dX = sum_r dY_r W_r is one
    all-reduce of the bf16 partials.  With ``overlap_dx_reduction`` the all-reduce is issued
    asynchronously right after the dgrad GEMM and waited for at the end of the backward, so that it
    runs beside the second quantizer of dY and the wgrad GEMM (a linear function that is not one of
    this package's simply ignores the request and the all-reduce happens after its backward).  Off
    by default: the persistent GEMM wants every SM, and a collective kernel beside it takes some.
    ``linear_fn(a, b)`` is one of the boundary functions with its recipe bound, e.g.
    ``lambda a, b: _to_mxfp8_then_scaled_mm(a, b, "e4m3", False, False, True)``."""
    if _world(group) == 1 or not overlap_dx_reduction or not x.is_cuda:
        return linear_fn(_CopyToShards.apply(x, group, None), w_shard)
    pending = _DxReduction()
    y = linear_fn(_CopyToShards.apply(x, group, pending), w_shard)
    return _ArmDxAllReduce.apply(y, group, pending)


# ------------------------------------------------------------------------------------------
# fully sharded weights: all-gather of the QUANTISED weight
# ------------------------------------------------------------------------------------------
def gather_packed_rows(local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenation over ranks of a per-rank buffer whose rank order is its memory order: codes of a
    row shard [n, K/2] -> [N, K/2], packed scales of a row shard with n % 128 == 0 (whole 128-row
    tiles, tiles row-block major)."""
    world = _world(group)
    if world == 1:
        return local
    out = torch.empty(world * local.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous().view(-1), group=group)
    return out.view(world * local.shape[0], *local.shape[1:]) if local.dim() > 1 else out


def interleave_gathered_columns(gathered: torch.Tensor, world: int, rows: int, inner: int) -> torch.Tensor:
    """``gathered`` = [world, rows, inner] (rank-major all-gather of per-rank [rows, inner] buffers whose
    columns are that rank's slice of a wider row) -> [rows, world * inner], rank slices side by side.

    Used for the weight packed along N ([K, n/2] codes per rank -> [K, N/2]) and for its packed scales
    viewed as [K/128 tile rows, tiles_per_rank * 512 bytes] (each rank owns whole tiles when its
    n / block is a multiple of 4)."""
    return gathered.view(world, rows, inner).permute(1, 0, 2).reshape(rows, world * inner)


def gather_columns(local: torch.Tensor, rows: int, group=None) -> torch.Tensor:
    world = _world(group)
    flat = local.contiguous().view(rows, -1)
    if world == 1:
        return flat
    out = torch.empty(world * flat.numel(), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, flat.view(-1), group=group)
    return interleave_gathered_columns(out, world, rows, flat.shape[1])


def outer_scale_from_amax_bits(bits: torch.Tensor) -> torch.Tensor:
    """NVFP4 tensorwise outer scale from the fp32 bit pattern of a tensor amax, as
    ``compute_dynamic_outer_scale`` defines it (alto/kernels/fp4/nvfp4/nvfp_quantization.py:460-487):
    nan_to_num(amax) / (448 * 6), at least 1e-30."""
    amax = torch.nan_to_num(bits.view(torch.float32))
    return (amax / (448.0 * 6.0)).clamp_min(1e-30)


class _GatheredWeightLinear(torch.autograd.Function):
    """y = x W^T where every rank holds the rows [r n, (r + 1) n) of W [N, K] (the layout of a fully
    sharded data-parallel weight).  The shard is quantised locally in 2-D blocks and the 4.5-bit
    payload (codes + scale bytes, both packings) is all-gathered instead of the bf16 weight: 3.5x
    fewer bytes on NVLink, and numerically nothing changes, because 2-D blocks never straddle a
    shard and the NVFP4 tensorwise scale is taken from the all-reduced (MAX) amax.

    The reference gathers ``param_dtype`` weights and quantises the full tensor on every rank
    (alto/kernels/dispatch/tensor.py:159-211); results here are bit-identical to that.

    backward: dX with the gathered weight packed along N; dW [N, K] is computed in full from the
    local batch and reduce-scattered (summed) so that every rank receives the gradient of its rows."""

    @staticmethod
    def forward(ctx, x, w_shard, group, fmt, use_outer_scale, use_sr_grad, hadamard_transform):
        from . import _linear as E
        world = _world(group)
        x2 = E.as_2d_rows(x.detach())
        w2 = E.as_2d_rows(w_shard.detach())
        if w2.dtype != x2.dtype:
            w2 = w2.to(x2.dtype)
        M, K = x2.shape
        n = w2.shape[0]
        N = n * world
        b = L.block_of(fmt)
        E.check_dims("gathered-weight linear", M, K, N)
        torch._check(n % 128 == 0 and (n // b) % 4 == 0, lambda: (
            f"a weight shard of {n} rows cannot be gathered in quantised form: rows per rank must be a multiple "
            f"of 128 (whole tiles of packed scales) and of {4 * b}"))
        rht, dense = E.split_transform(hadamard_transform, False)
        # tensorwise scale of the WHOLE weight: local amax, MAX over ranks
        ow = None
        if use_outer_scale:
            bits = torch.empty(2, dtype=torch.int32, device=w2.device)
            L.amax(w2, bits, None, E.amax_scratch(w2.device), None)
            if world > 1:
                dist.all_reduce(bits, op=dist.ReduceOp.MAX, group=group)  # non-negative floats order like ints
            ow = outer_scale_from_amax_bits(bits[0:1])
        wk_l, wt_l = E.quant_2d(w2, fmt, ow, True)
        w_k = E.Operand(gather_packed_rows(wk_l.codes, group), gather_packed_rows(wk_l.scales, group), ow, N, K, fmt)
        w_t = E.Operand(gather_columns(wt_l.codes, K, group),
                        gather_columns(wt_l.scales, (K + 127) // 128, group).reshape(-1), ow, K, N, fmt)
        ox = E.outer_scales(x2, use_outer_scale, rht)
        x_k = E.quant_rows(x2, fmt, None if ox is None else ox[0:1], E.RTN)
        x_m = E.cols_operand(x2, fmt, use_outer_scale, ox, rht, dense, E.RTN)
        y = E.gemm(x_k, w_k, x.dtype)
        extra_x = [x_m.outer] if x_m.outer is not None else []
        extra_w = [w_t.outer] if w_t.outer is not None else []
        ctx.save_for_backward(x_m.codes, x_m.scales, *extra_x, w_t.codes, w_t.scales, *extra_w)
        ctx.dims, ctx.fmt, ctx.group, ctx.n_local = (M, K, N), fmt, group, n
        ctx.use_outer_scale, ctx.use_sr_grad, ctx.rht, ctx.dense = use_outer_scale, use_sr_grad, rht, dense
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, grad_output):
        from . import _linear as E
        M, K, N = ctx.dims
        saved = ctx.saved_tensors
        if ctx.use_outer_scale:
            xc, xs, xo, wc, ws, wo = saved
        else:
            (xc, xs, wc, ws), xo, wo = saved, None, None
        x_m = E.Operand(xc, xs, xo, K, M, ctx.fmt)
        w_t = E.Operand(wc, ws, wo, K, N, ctx.fmt)
        g2 = E.as_2d_rows(grad_output)
        g_n, g_m = E.backward_operands(g2, ctx.fmt, use_2dblock_x=False, use_sr_grad=ctx.use_sr_grad,
                                       use_outer_scale=ctx.use_outer_scale, rht=ctx.rht, dense=ctx.dense)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = E.gemm(g_n, w_t, grad_output.dtype).view(*grad_output.shape[:-1], K)
        if ctx.needs_input_grad[1]:
            dw_full = E.gemm(g_m, x_m, grad_output.dtype)
            if _world(ctx.group) > 1:
                dw = torch.empty(ctx.n_local, K, dtype=dw_full.dtype, device=dw_full.device)
                dist.reduce_scatter_tensor(dw, dw_full, op=dist.ReduceOp.SUM, group=ctx.group)
            else:
                dw = dw_full
        return dx, dw, None, None, None, None, None


def gathered_weight_linear(x: torch.Tensor, w_shard: torch.Tensor, precision: str = "nvfp4", group=None, *,
                           use_outer_scale: bool = False, use_sr_grad: bool = False,
                           hadamard_transform=None) -> torch.Tensor:
    """Linear layer over a row-sharded weight whose quantised form is all-gathered (see
    ``_GatheredWeightLinear``).  ``precision``: "nvfp4", "mxfp4", "mxfp8_e4m3" or "mxfp8_e5m2"; weights are
    quantised in 2-D blocks, activations and gradients in 1-D blocks."""
    fmts = {"nvfp4": L.FMT_NVFP4, "mxfp4": L.FMT_MXFP4, "mxfp8_e4m3": L.FMT_MXFP8_E4M3, "mxfp8_e5m2": L.FMT_MXFP8_E5M2}
    if precision not in fmts:
        raise ValueError(f"unsupported precision {precision!r}")
    if use_outer_scale and precision != "nvfp4":
        raise ValueError("the tensorwise outer scale belongs to NVFP4")
    return _GatheredWeightLinear.apply(x, w_shard, group, fmts[precision], use_outer_scale, use_sr_grad,
                                       hadamard_transform)


# ------------------------------------------------------------------------------------------
# expert parallel: dispatch / combine
# ------------------------------------------------------------------------------------------
def permute_pad_plan(recv_counts: torch.Tensor, align: int = ALIGN_SIZE_M, total: Optional[int] = None,
                     m_pad: Optional[int] = None):
    """Row plan of the local re-sort after the dispatch all-to-all.

    ``recv_counts`` (int64 [sources, local_experts], on any device): rows received from each source
    rank for each local expert; the receive buffer holds them source-major, expert-minor.  Returns
    tensors on the same device ``(index, inverse, offs)``: ``index`` int32 [M_pad] gives for every row
    of the expert-major, padded layout its row in the receive buffer (-1 = padding row); ``inverse``
    int32 [rows_received] is the opposite map; ``offs`` int32 [local_experts] are the cumulative
    padded row counts the grouped GEMMs take (every count a multiple of ``align`` and at least ``align``).

    ``total`` (rows received) and ``m_pad`` (padded rows, ``offs[-1]``) are read back from the counts
    when not given; a caller that has the counts on the host passes both, so that a plan built on
    the GPU needs no synchronisation of its own."""
    c = recv_counts.to(torch.int64)
    dev = c.device
    S, E = c.shape
    per_expert = c.sum(0)
    # an expert without rows still gets one aligned run of padding, as TorchTitan's permute step gives it:
    # a rank whose experts received nothing then has a non-empty buffer and takes part in every exchange
    padded = ((per_expert + align - 1) // align * align).clamp(min=align)
    offs = torch.cumsum(padded, 0)
    pad_start = offs - padded                                   # [E]
    recv_start = (torch.cumsum(c.reshape(-1), 0) - c.reshape(-1)).reshape(S, E)
    within = torch.cumsum(c, 0) - c                             # rows of expert e from earlier sources
    dst_start = pad_start.unsqueeze(0) + within                 # [S, E]
    if total is None:
        total = int(c.sum())
    if m_pad is None:
        m_pad = int(offs[-1]) if E > 0 else 0
    index = torch.full((m_pad,), -1, dtype=torch.int32, device=dev)
    inverse = torch.empty(total, dtype=torch.int32, device=dev)
    if total > 0:
        counts = c.reshape(-1)
        block = torch.repeat_interleave(torch.arange(S * E, device=dev), counts,
                                        output_size=total)                    # block id of every received row
        pos = torch.arange(total, device=dev) - recv_start.reshape(-1)[block]  # position inside its block
        dst = dst_start.reshape(-1)[block] + pos
        inverse.copy_(dst.to(torch.int32))
        index[dst] = torch.arange(total, dtype=torch.int32, device=dev)
    return index, inverse, offs.to(torch.int32)


class _GatherRows(torch.autograd.Function):
    """out[i] = x[index[i]] (zeros where index < 0); ``index`` uses every row of x at most once, so
    the gradient is the gather by the opposite map ``inverse``."""

    @staticmethod
    def forward(ctx, x, index, inverse):
        ctx.save_for_backward(index, inverse)
        return L.gather_rows(x.contiguous(), index)

    @staticmethod
    def backward(ctx, grad):
        index, inverse = ctx.saved_tensors
        return L.gather_rows(grad.contiguous(), inverse), None, None


class _CombineRows(torch.autograd.Function):
    """out[t] = sum_j rows[index[t k + j]] * scores[t, j]: the last gather of the combine, the weighting
    by the routing scores and the sum over the k routed rows of a token in one pass.  ``position`` is
    the opposite map (row -> routed slot).  Gradients: rows by the spread kernel; scores (when they
    require one) as the dot products of the gathered rows with the token's output gradient."""

    @staticmethod
    def forward(ctx, rows, index, position, scores, tokens, k):
        rows = rows.contiguous()
        sc = None if scores is None else scores.to(rows.dtype).contiguous()
        ctx.save_for_backward(rows, index, position, sc)
        ctx.tokens, ctx.k = tokens, k
        ctx.scores_dtype = None if scores is None else scores.dtype
        return L.combine_rows(rows, index, sc, tokens, k)

    @staticmethod
    def backward(ctx, grad):
        rows, index, position, sc = ctx.saved_tensors
        grad = grad.contiguous()
        g_rows = L.spread_rows(grad, position, sc, ctx.k) if ctx.needs_input_grad[0] else None
        g_scores = None
        if sc is not None and ctx.needs_input_grad[3]:
            routed = L.gather_rows(rows, index).view(ctx.tokens, ctx.k, -1)
            g_scores = (routed.float() * grad.float().unsqueeze(1)).sum(-1).to(ctx.scores_dtype)
        return g_rows, None, None, g_scores, None, None


class _ReplicateSorted(torch.autograd.Function):
    """Routed rows sorted by expert: out[i] = x[order[i] // k].  A token feeds k routed rows, so the
    gradient gathers the routed rows back into token order and sums each token's k rows."""

    @staticmethod
    def forward(ctx, x, token_of_sorted, inv_order, k):
        ctx.save_for_backward(inv_order)
        ctx.k = k
        return L.gather_rows(x.contiguous(), token_of_sorted)

    @staticmethod
    def backward(ctx, grad):
        (inv_order,) = ctx.saved_tensors
        grad = grad.contiguous()
        if grad.dtype == torch.bfloat16 and (grad.shape[-1] * 2) % 16 == 0:
            # gather and sum over the k routed rows of a token in one pass
            return L.combine_rows(grad, inv_order, None, inv_order.numel() // ctx.k, ctx.k), None, None, None
        g = L.gather_rows(grad, inv_order)
        return g.view(-1, ctx.k, g.shape[-1]).sum(1).to(grad.dtype), None, None, None


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all of rows; the gradient is the same exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        out = grad.new_empty((sum(ctx.in_splits),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(out, grad.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


class _DispatchState:
    __slots__ = ("k", "tokens", "inv_order", "order", "in_splits", "out_splits", "index", "inverse", "offs")


class ExpertParallelDispatcher:
    """Token exchange of an expert-parallel MoE layer around the grouped GEMMs.

    ``num_experts`` experts are split evenly over the ranks of ``group`` (rank r owns experts
    [r * E / world, (r + 1) * E / world)); tokens are data parallel.

        x_local, offs, state = d.dispatch(x, expert_ids)       # x [T, D], expert_ids [T, k]
        h = experts(x_local, offs)                              # grouped GEMMs on [M_pad, D]
        out = d.combine(h, state, scores)                       # [T, D'] = sum_k scores * h(routed row)

    dispatch: routed rows sorted by expert -> per-expert counts exchanged -> row all-to-all ->
    local re-sort to expert-major order with every expert's run padded to ``align`` rows (zeros).
    combine is the inverse followed by the score-weighted sum over each token's k routed rows.
    Both are differentiable.  One host synchronisation per dispatch (the split sizes of the
    all-to-all live on the host); with a single rank the all-to-alls are skipped."""

    def __init__(self, num_experts: int, group=None, align: int = ALIGN_SIZE_M):
        self.group = group
        self.world = _world(group)
        self.rank = _rank(group)
        torch._check(num_experts % self.world == 0,
                     lambda: f"{num_experts} experts do not split over {self.world} ranks")
        self.num_experts = num_experts
        self.local_experts = num_experts // self.world
        self.align = align

    def dispatch(self, x: torch.Tensor, expert_ids: torch.Tensor):
        assert x.dim() == 2 and expert_ids.dim() == 2 and expert_ids.shape[0] == x.shape[0]
        T, k = expert_ids.shape
        dev = x.device
        flat = expert_ids.reshape(-1).to(torch.int64)
        order = torch.argsort(flat, stable=True)
        inv_order = torch.empty_like(order)
        inv_order[order] = torch.arange(order.numel(), device=dev)
        counts = torch.bincount(flat, minlength=self.num_experts)            # rows per global expert
        send = counts.view(self.world, self.local_experts)
        if self.world > 1:
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send.contiguous(), group=self.group)
        else:
            recv = send
        both = torch.stack((send, recv)).cpu()                               # the one host synchronisation
        send_h, recv_h = both[0], both[1]
        st = _DispatchState()
        st.k, st.tokens = k, T
        st.inv_order = inv_order.to(torch.int32)
        st.order = order.to(torch.int32)
        st.in_splits = [int(v) for v in send_h.sum(1)]
        st.out_splits = [int(v) for v in recv_h.sum(1)]
        # The row plan is built on the GPU from the device copy of the counts; the host copy only
        # sizes its buffers (and the all-to-all), so the host is free to run ahead again at once.
        per_expert = recv_h.sum(0)
        m_pad = int(((per_expert + self.align - 1) // self.align * self.align).clamp(min=self.align).sum())
        st.index, st.inverse, st.offs = permute_pad_plan(recv, self.align, total=sum(st.out_splits), m_pad=m_pad)
        token_of_sorted = torch.div(order, k, rounding_mode="floor").to(torch.int32)
        rows = _ReplicateSorted.apply(x, token_of_sorted, st.inv_order, k)
        if self.world > 1:
            rows = _AllToAllRows.apply(rows, st.out_splits, st.in_splits, self.group)
        x_local = _GatherRows.apply(rows, st.index, st.inverse)
        return x_local, st.offs, st

    def combine(self, y_local: torch.Tensor, state: _DispatchState, scores: Optional[torch.Tensor] = None):
        rows = _GatherRows.apply(y_local, state.inverse, state.index)
        if self.world > 1:
            rows = _AllToAllRows.apply(rows, state.in_splits, state.out_splits, self.group)
        # back to routed-row order (token-major, k minor: the inverse of the dispatch's sort), weighted by
        # the routing scores and summed over each token's k rows
        if rows.dtype == torch.bfloat16 and (rows.shape[-1] * 2) % 16 == 0:
            return _CombineRows.apply(rows, state.inv_order, state.order, scores, state.tokens, state.k)
        routed = _GatherRows.apply(rows, state.inv_order, state.order)
        routed = routed.view(state.tokens, state.k, routed.shape[-1])
        if scores is not None:
            routed = routed * scores.to(routed.dtype).unsqueeze(-1)
        return routed.sum(1)
