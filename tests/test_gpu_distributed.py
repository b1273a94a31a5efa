"""GPU tests of the multi-GPU forms of the path.

One GPU: the row-gather kernel, and the expert-parallel dispatcher with a single rank feeding the
grouped GEMMs.  Two, four and eight GPUs (each skipped when fewer are visible): that many NCCL
ranks as child processes -- the column-sharded MXFP8 linear (dgrad all-reduce), the expert-parallel
MoE (two all-to-alls each way) and the fully sharded NVFP4 weight (quantised all-gather, dW
reduce-scatter) against single-GPU runs of the same kernels.  NVLS is switched off in the children: a
rank that dies while bound to an NVLink multicast object can fault its peers."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


@pytest.mark.parametrize("dtype,cols", [(torch.bfloat16, 2880), (torch.float32, 20), (torch.uint8, 48)])
def test_gather_rows_matches_index_select(dtype, cols):
    from alto_b200 import _lib as L
    g = torch.Generator().manual_seed(0)
    src = (torch.randn(300, cols, generator=g) * 50).to(dtype).cuda()
    index = torch.randint(-1, 300, (1000,), generator=g, dtype=torch.int32)
    index[5] = 300      # out of range -> zero row
    out = L.gather_rows(src, index.cuda())
    idx = index.long()
    ok = (idx >= 0) & (idx < 300)
    want = torch.where(ok.unsqueeze(1).cuda(), src[idx.clamp(0, 299).cuda()], torch.zeros((), dtype=dtype, device="cuda"))
    assert torch.equal(out, want)
    assert L.gather_rows(src, index[:0].cuda()).shape == (0, cols)
    with pytest.raises(L.Altob200Error):
        L.gather_rows(src[:, :cols - 1].contiguous(), index.cuda())  # rows not a multiple of 16 bytes


def _moe(x, ids, scores, W13, W2, dispatcher):
    from alto_b200.grouped import _quantize_then_mxfp8_scaled_grouped_mm as gmm
    xl, offs, st = dispatcher.dispatch(x, ids)
    h = gmm(xl, W13.transpose(-2, -1), offs)
    h = torch.nn.functional.silu(h)
    y = gmm(h, W2.transpose(-2, -1), offs)
    return dispatcher.combine(y, st, scores)


def _moe_inputs(seed, T, D, H, E, k, dev):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).bfloat16().to(dev)
    logits = torch.randn(T, E, generator=g)
    scores, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    gw = torch.Generator().manual_seed(99)
    W13 = (torch.randn(E, H, D, generator=gw) * 0.05).bfloat16().to(dev)
    W2 = (torch.randn(E, D, H, generator=gw) * 0.05).bfloat16().to(dev)
    return x, ids.to(dev), scores.bfloat16().to(dev), W13, W2


def test_single_rank_dispatcher_feeds_grouped_gemms():
    """dispatch -> grouped MXFP8 GEMMs -> combine equals the same GEMMs on rows sorted and padded by
    hand with tensor ops, bit for bit, and gradients reach the tokens."""
    from alto_b200.distributed import ExpertParallelDispatcher
    from alto_b200.grouped import _quantize_then_mxfp8_scaled_grouped_mm as gmm
    d = _dev()
    T, D, H, E, k = 512, 256, 384, 4, 2
    x, ids, scores, W13, W2 = _moe_inputs(1, T, D, H, E, k, d)
    x.requires_grad_(True)
    out = _moe(x, ids, scores, W13, W2, ExpertParallelDispatcher(E))
    out.float().sum().backward()
    assert out.shape == (T, D) and torch.isfinite(out).all() and torch.isfinite(x.grad).all()
    # by hand
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    padded = (counts + 127) // 128 * 128
    offs = torch.cumsum(padded, 0).to(torch.int32)
    rows = x.detach()[order // k]
    xl = torch.zeros(int(offs[-1]), D, dtype=x.dtype, device=d)
    start_sorted = torch.cumsum(counts, 0) - counts
    start_pad = torch.cumsum(padded, 0) - padded
    e_of = flat[order]
    dst = start_pad[e_of] + (torch.arange(order.numel(), device=d) - start_sorted[e_of])
    xl[dst] = rows
    y = gmm(torch.nn.functional.silu(gmm(xl, W13.transpose(-2, -1), offs)), W2.transpose(-2, -1), offs)
    routed = torch.empty(T * k, D, dtype=y.dtype, device=d)
    routed[order] = y[dst]
    want = (routed.view(T, k, D) * scores.unsqueeze(-1)).sum(1)
    assert torch.equal(out.detach(), want)


# ---------------------------------------------------------------------------------------------
# two ranks over NCCL
# ---------------------------------------------------------------------------------------------
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_rank_worker(rank, world, port):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from alto_b200 import distributed as D
        from alto_b200 import mxfp8 as M8
        fn = lambda a, b: M8._to_mxfp8_then_scaled_mm(a, b, "e4m3", False, False, True)  # noqa: E731
        # ---- column-sharded MXFP8 linear ----
        g = torch.Generator().manual_seed(5)
        n = 128                       # output features per rank (whole 32 x 32 weight blocks)
        x = torch.randn(256, 512, generator=g).bfloat16().to(dev).requires_grad_(True)
        W = (torch.randn(n * world, 512, generator=g) * 0.05).bfloat16().to(dev)
        dy = torch.randn(256, n * world, generator=g).bfloat16().to(dev)
        w_r = D.shard_rows(W).clone().requires_grad_(True)
        y_r = D.column_sharded_linear(x, w_r, fn)
        y_r.backward(dy[:, rank * n:(rank + 1) * n])
        # single-GPU runs of every shard on this rank: forward identical, dgrad = sum of the partials
        partial = []
        for r in range(world):
            xs = x.detach().clone().requires_grad_(True)
            ws = W[r * n:(r + 1) * n].clone().requires_grad_(True)
            ys = fn(xs, ws)
            ys.backward(dy[:, r * n:(r + 1) * n])
            partial.append(xs.grad)
            if r == rank:
                assert torch.equal(ys, y_r) and torch.equal(ws.grad, w_r.grad)
        want = torch.stack([p_.float() for p_ in partial]).sum(0)
        assert torch.allclose(x.grad.float(), want, rtol=2e-2, atol=1e-2 * want.abs().max().item())
        # ---- expert-parallel MoE: every rank has its own tokens ----
        import tests.test_gpu_distributed as T_
        E = max(4, world)
        xt, ids, scores, W13, W2 = T_._moe_inputs(10 + rank, 384, 256, 384, E, 2, dev)
        xt.requires_grad_(True)
        E_local = E // world
        ep = D.ExpertParallelDispatcher(E)
        out = T_._moe(xt, ids, scores, W13[rank * E_local:(rank + 1) * E_local],
                      W2[rank * E_local:(rank + 1) * E_local], ep)
        out.float().sum().backward()
        # the same tokens through all the experts on this GPU alone: forward and the token gradient
        # are row-local (row-wise MXFP8 blocks), hence bit-identical
        x1 = xt.detach().clone().requires_grad_(True)
        one = D.ExpertParallelDispatcher.__new__(D.ExpertParallelDispatcher)
        one.group, one.world, one.rank, one.num_experts, one.local_experts, one.align = None, 1, 0, E, E, 128
        out1 = T_._moe(x1, ids, scores, W13, W2, one)
        out1.float().sum().backward()
        assert torch.equal(out, out1)
        assert torch.equal(xt.grad, x1.grad)
        # ---- fully sharded weight: the quantised shard is all-gathered, dW reduce-scattered ----
        from alto_b200 import nvfp4 as NV
        NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)
        had = NV.HadamardFactory.create_transform(device=dev)
        g = torch.Generator().manual_seed(9)
        xf = torch.randn(256, 512, generator=g).bfloat16().to(dev)
        nw = max(512 // world, 128)   # weight rows per rank (multiples of 128)
        Wf = (torch.randn(nw * world, 512, generator=g) * 0.05).bfloat16().to(dev)
        dyf = (torch.randn(256, nw * world, generator=g) * 1e-2).bfloat16().to(dev)
        xs, ws = xf.clone().requires_grad_(True), D.shard_rows(Wf, multiple=128).clone().requires_grad_(True)
        ys = D.gathered_weight_linear(xs, ws, "nvfp4", use_outer_scale=True, hadamard_transform=had)
        ys.backward(dyf)
        x1, w1 = xf.clone().requires_grad_(True), Wf.clone().requires_grad_(True)
        NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)  # same matrix
        y1 = NV._to_nvfp4_then_scaled_mm(x1, w1, False, True, False, use_outer_scale=True, use_hadamard=True)
        y1.backward(dyf)
        assert torch.equal(ys, y1) and torch.equal(xs.grad, x1.grad)
        # every rank ran the same batch: the reduce-scattered gradient is world x the single-GPU rows
        # (bit for bit on two ranks; with more, the bf16 partial sums 3g, 5g, ... of the reduction round)
        want_w = w1.grad[rank * nw:(rank + 1) * nw].float() * world
        if world == 2:
            assert torch.equal(ws.grad, want_w.bfloat16())
        else:
            assert torch.allclose(ws.grad.float(), want_w, rtol=2e-2, atol=0.0)
        # ---- bucketed gradient all-reduce ----
        p = torch.nn.Parameter(torch.zeros(1000, device=dev))
        p.grad = torch.full_like(p, float(rank))
        assert D.allreduce_gradients([p]) == 1
        assert torch.allclose(p.grad, torch.full_like(p, (world - 1) / 2.0))
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_nccl_ranks_column_sharded_expert_parallel_and_sharded_weight(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_nccl_rank_worker, args=(world, _free_port()), nprocs=world, join=True)


@pytest.mark.parametrize("precision,kw", [("nvfp4", dict(use_outer_scale=True)), ("nvfp4", dict()), ("mxfp4", dict()),
                                          ("mxfp8_e4m3", dict())])
def test_gathered_weight_linear_single_rank_equals_the_plain_linear(precision, kw):
    """World size 1: the gathers are identities, so the function must reproduce the boundary functions bit
    for bit (same quantizers, same GEMMs); the 2-rank NCCL test checks the exchanges."""
    from alto_b200 import distributed as D
    from alto_b200 import mxfp4 as MX, mxfp8 as M8, nvfp4 as NV
    d = torch.device("cuda")
    g = torch.Generator().manual_seed(3)
    x = torch.randn(128, 256, generator=g).bfloat16().to(d)
    W = (torch.randn(384, 256, generator=g) * 0.05).bfloat16().to(d)
    dy = (torch.randn(128, 384, generator=g) * 1e-2).bfloat16().to(d)
    xa, wa = x.clone().requires_grad_(True), W.clone().requires_grad_(True)
    ya = D.gathered_weight_linear(xa, wa, precision, **kw)
    ya.backward(dy)
    xb, wb = x.clone().requires_grad_(True), W.clone().requires_grad_(True)
    if precision == "nvfp4":
        yb = NV._to_nvfp4_then_scaled_mm(xb, wb, False, True, False, use_outer_scale=bool(kw))
    elif precision == "mxfp4":
        yb = MX._to_mxfp4_then_scaled_mm(xb, wb, False, True, False, False, "none", False)
    else:
        yb = M8._to_mxfp8_then_scaled_mm(xb, wb, "e4m3", False, False, True)
    yb.backward(dy)
    assert torch.equal(ya, yb) and torch.equal(xa.grad, xb.grad) and torch.equal(wa.grad, wb.grad)
    with pytest.raises(RuntimeError, match="multiple"):
        D.gathered_weight_linear(x, W[:96], precision, **kw)


# ---------------------------------------------------------------------------------------------
# The two sharded benchmark configurations at their full sizes on 1, 2, 4 and 8 ranks
# ---------------------------------------------------------------------------------------------
def _swiglu_moe(x, ids, scores, W13, W2, dispatcher, gmm):
    """Routed experts with the gate and up projections fused in W13 [E, 2H, D] and W2 [E, D, H]."""
    xl, offs, st = dispatcher.dispatch(x, ids)
    from alto_b200.swiglu import swiglu
    h = gmm(xl, W13.transpose(-2, -1), offs)
    y = gmm(swiglu(h), W2.transpose(-2, -1), offs)
    return dispatcher.combine(y, st, scores)


def _full_size_worker(rank, world, port):
    """MXFP4 MoE (32 experts, top-4, hidden = intermediate = 2880, 16384 tokens in total, experts and
    tokens split over the ranks) and the column-sharded MXFP8 linear (X [8192, 4096], W [4096, 4096]
    split by output features): forward of this rank's tokens against all experts on this GPU alone,
    finite gradients, and the step times (CUDA events, slowest rank)."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from alto_b200 import distributed as D
        from alto_b200 import mxfp8 as M8
        from alto_b200.grouped import _quantize_then_mxfp_scaled_grouped_mm as mx4
        from alto_b200.hadamard import HadamardFactory
        HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)

        def gmm(A, B, offs):  # 1-D activation blocks, 2-D weight blocks, RHT on wgrad operands, SR on gradients
            return mx4(A, B, offs, False, True, True, False, True, "none", False)

        def step_time(fn, reps=5):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        # ---- expert-parallel MoE ----
        T, Dm, E, k = 16384, 2880, 32, 4
        g = torch.Generator(device=dev).manual_seed(0)
        logits = torch.randn(T, E, generator=g, device=dev)
        x_all = torch.randn(T, Dm, generator=g, device=dev).bfloat16()
        W13 = (torch.randn(E, 2 * Dm, Dm, generator=g, device=dev) * 0.02).bfloat16()
        W2 = (torch.randn(E, Dm, Dm, generator=g, device=dev) * 0.02).bfloat16()
        scores_all, ids_all = torch.topk(torch.softmax(logits, -1), k, dim=-1)
        n, El = T // world, E // world
        x = x_all[rank * n:(rank + 1) * n].clone().requires_grad_(True)
        ids, scores = ids_all[rank * n:(rank + 1) * n], scores_all[rank * n:(rank + 1) * n].bfloat16()
        w13 = W13[rank * El:(rank + 1) * El].clone().requires_grad_(True)
        w2 = W2[rank * El:(rank + 1) * El].clone().requires_grad_(True)
        ep = D.ExpertParallelDispatcher(E)
        out = _swiglu_moe(x, ids, scores, w13, w2, ep, gmm)
        out.backward(torch.ones_like(out) * 1e-3)
        assert torch.isfinite(out).all() and torch.isfinite(x.grad).all()
        assert torch.isfinite(w13.grad).all() and torch.isfinite(w2.grad).all()
        if world > 1:
            # this rank's tokens through all 32 experts on this GPU alone: the forward is row-local
            one = D.ExpertParallelDispatcher.__new__(D.ExpertParallelDispatcher)
            one.group, one.world, one.rank, one.num_experts, one.local_experts, one.align = None, 1, 0, E, E, 128
            with torch.no_grad():
                assert torch.equal(out, _swiglu_moe(x.detach(), ids, scores, W13, W2, one, gmm))
        del W13, W2, x_all

        def moe_step():
            x.grad = w13.grad = w2.grad = None
            _swiglu_moe(x, ids, scores, w13, w2, ep, gmm).backward(torch.ones_like(out) * 1e-3)

        t_moe = step_time(moe_step)
        routed = T * k
        flop_moe = 3 * 2 * routed * (2 * Dm * Dm + Dm * Dm)
        # ---- column-sharded MXFP8 linear ----
        fn = lambda a, b: M8._to_mxfp8_then_scaled_mm(a, b, "e4m3", False, False, True)  # noqa: E731
        g = torch.Generator(device=dev).manual_seed(1)
        xs = torch.randn(8192, 4096, generator=g, device=dev).bfloat16().requires_grad_(True)
        W = (torch.randn(4096, 4096, generator=g, device=dev) * 0.02).bfloat16()
        dy = (torch.randn(8192, 4096, generator=g, device=dev) * 1e-3).bfloat16()
        nw = 4096 // world
        ws = D.shard_rows(W).clone().requires_grad_(True)
        dys = dy[:, rank * nw:(rank + 1) * nw].contiguous()
        ys = D.column_sharded_linear(xs, ws, fn)
        ys.backward(dys)
        with torch.no_grad():
            assert torch.equal(ys, fn(xs.detach(), W[rank * nw:(rank + 1) * nw]))
        assert torch.isfinite(xs.grad).all() and torch.isfinite(ws.grad).all()

        def lin_step():
            xs.grad = ws.grad = None
            D.column_sharded_linear(xs, ws, fn).backward(dys)

        t_lin = step_time(lin_step)
        if rank == 0:
            print(f"\n[{world} rank(s)] MXFP4 MoE 32 experts top-4, 16384 tokens, fwd+dgrad+wgrad incl. dispatch/combine: "
                  f"{t_moe:.2f} ms = {flop_moe / t_moe / 1e9:.0f} TFLOP/s whole job; "
                  f"column-sharded MXFP8 linear 8192 x 4096 x 4096 fwd+dgrad+wgrad incl. dX all-reduce: "
                  f"{t_lin:.3f} ms = {3 * 2 * 8192 * 4096 * 4096 / t_lin / 1e9:.0f} TFLOP/s whole job", flush=True)
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_full_size_expert_parallel_moe_and_column_sharded_linear(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_full_size_worker, args=(world, _free_port()), nprocs=world, join=True)


# ---------------------------------------------------------------------------------------------
# FSDP2 (`fully_shard`) over wrapped parameters: the all-gather carries the quantised weight
# ---------------------------------------------------------------------------------------------
def _fsdp_worker(rank, world, port, precision, two_level):
    """A Linear whose weight was wrapped by ``swap_params`` under ``fully_shard``: the pre / post all-gather
    hooks of the wrapper quantise the row shard and gather the operands.  Forward must equal the
    unsharded boundary function bit for bit (2-D blocks never straddle a shard), dX too, and the
    reduce-scattered weight gradient must be the mean over ranks of the single-GPU gradients."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from torch.distributed.fsdp import fully_shard
        from alto_b200 import dispatch as D
        from alto_b200 import mxfp8 as M8, nvfp4 as NV
        N, K, M = 512, 256, 128
        g = torch.Generator().manual_seed(7)
        W = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(dev)
        xs = [torch.randn(M, K, generator=g).bfloat16().to(dev) for _ in range(world)]
        dys = [(torch.randn(M, N, generator=g) * 1e-2).bfloat16().to(dev) for _ in range(world)]
        cfg = D.TrainingOpConfig(precision=precision, use_2dblock_x=False, use_2dblock_w=True, use_hadamard=False,
                                 use_sr_grad=False, use_dge=False, two_level_scaling=two_level)
        lin = torch.nn.Linear(K, N, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(W)
        calls = {"n": 0}
        real = D.quantize_shard_for_gather

        def counting(*a, **k):
            calls["n"] += 1
            return real(*a, **k)

        D.quantize_shard_for_gather = counting
        D.swap_params(lin, config=cfg)
        fully_shard(lin)

        def ref(a, w):
            if precision == "nvfp4":
                return NV._to_nvfp4_then_scaled_mm(a, w, False, True, False, use_outer_scale=two_level == "tensorwise")
            return M8._to_mxfp8_then_scaled_mm(a, w, "e4m3", False, False, True)

        for it in range(2):                      # second pass: the hooks refill the operands in place
            x = xs[rank].clone().requires_grad_(True)
            y = lin(x)
            y.backward(dys[rank])
            wr = W.clone().requires_grad_(True)
            xr = xs[rank].clone().requires_grad_(True)
            yr = ref(xr, wr)
            yr.backward(dys[rank])
            assert torch.equal(y, yr), f"forward differs on pass {it}"
            assert torch.equal(x.grad, xr.grad), f"dX differs on pass {it}"
            # mean over ranks of the full single-GPU weight gradients, this rank's rows
            dws = []
            for r in range(world):
                w_ = W.clone().requires_grad_(True)
                ref(xs[r].clone(), w_).backward(dys[r])
                dws.append(w_.grad.float())
            want = (sum(dws) / world)[rank * (N // world):(rank + 1) * (N // world)]
            got = lin.weight.grad
            got = got.to_local() if hasattr(got, "to_local") else got
            got = got._data if hasattr(got, "_data") else got
            assert got.shape == want.shape
            assert ((got.float() - want).norm() / want.norm()).item() <= 1e-2
            lin.weight.grad = None
        if world > 1:
            assert calls["n"] >= 2, "the quantised all-gather was not taken"
        else:
            assert calls["n"] == 0      # one rank: nothing to gather, the weight stays in high precision
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("precision,two_level", [("nvfp4", "tensorwise"), ("mxfp8_e4m3", "none")])
def test_fully_shard_gathers_the_quantised_weight(world, precision, two_level):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_fsdp_worker, args=(world, _free_port(), precision, two_level), nprocs=world, join=True)
