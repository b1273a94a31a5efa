"""Host logic of the multi-GPU forms of the path, run as 2 gloo ranks on CPU: the expert-parallel
dispatch / combine plan and exchanges, the column-sharded linear's dgrad all-reduce and the bucketed
gradient all-reduce.  The CUDA row gather is replaced by a tensor-op stand-in (the device kernel
itself is checked in the GPU tests); no other kernel is involved.  The reference pins none of this
(it lives in its TorchTitan fork); the checks are against a single-process dense computation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from alto_b200 import distributed as D


def _gather_rows_cpu(src, index, out_rows=None):
    idx = index.to(torch.int64)
    ok = (idx >= 0) & (idx < src.shape[0])
    out = src[idx.clamp(0, max(src.shape[0] - 1, 0))] if src.shape[0] > 0 else src.new_zeros(idx.numel(), src.shape[1])
    return torch.where(ok.unsqueeze(1), out, torch.zeros_like(out))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(rank, world, port, fn, args):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D.L.gather_rows = _gather_rows_cpu
        fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def _spawn(fn, *args, world=2):
    mp.spawn(_run, args=(world, _free_port(), fn, args), nprocs=world, join=True)


# ---------------------------------------------------------------------------------------------
def test_permute_pad_plan_layout():
    c = torch.tensor([[3, 0, 130], [2, 0, 1]])        # 2 sources x 3 local experts
    index, inverse, offs = D.permute_pad_plan(c, 128)
    # expert 1 received nothing and still gets one aligned run of padding (TorchTitan's permute step
    # clamps every expert to the alignment)
    assert offs.tolist() == [128, 256, 256 + 256]
    assert index.numel() == 512 and inverse.numel() == 136
    # expert 0: 3 rows of source 0 (receive rows 0..2) then 2 rows of source 1 (rows 133, 134)
    assert index[:5].tolist() == [0, 1, 2, 133, 134] and (index[5:256] == -1).all()
    # expert 2 starts at 256: 130 rows of source 0 (receive rows 3..132) then row 135 of source 1
    assert index[256:386].tolist() == list(range(3, 133)) and index[386].item() == 135
    assert (index[387:] == -1).all()
    ok = index >= 0
    assert torch.equal(inverse[index[ok].long()].long(), torch.nonzero(ok).squeeze(1))
    # no rows at all: every expert is one run of padding, so a rank that received nothing still has a
    # buffer the grouped GEMMs accept and stays in step with its peers
    index, inverse, offs = D.permute_pad_plan(torch.zeros(2, 3, dtype=torch.int64))
    assert index.numel() == 384 and (index == -1).all() and inverse.numel() == 0 and offs.tolist() == [128, 256, 384]


def _experts(x_local, offs, W):
    """Per-expert matmul over runs given by cumulative `offs` (padding rows are zeros in, zeros out)."""
    out = x_local.new_zeros(x_local.shape[0], W.shape[-1])
    start = 0
    for e in range(offs.numel()):
        end = int(offs[e])
        out[start:end] = x_local[start:end] @ W[e]
        start = end
    return out


def _ep_worker(rank, world, num_experts, T, k, Dm, Do):
    g = torch.Generator().manual_seed(100 + rank)
    gw = torch.Generator().manual_seed(7)
    W = torch.randn(num_experts, Dm, Do, generator=gw, dtype=torch.float64)
    x = torch.randn(T, Dm, generator=g, dtype=torch.float64, requires_grad=True)
    logits = torch.randn(T, num_experts, generator=g, dtype=torch.float64)
    scores, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    d = D.ExpertParallelDispatcher(num_experts)
    x_local, offs, st = d.dispatch(x, ids)
    E_local = num_experts // world
    assert offs.numel() == E_local and x_local.shape[0] == int(offs[-1])
    counts = torch.diff(offs, prepend=offs.new_zeros(1))
    assert (counts % 128 == 0).all()
    W_local = W[rank * E_local:(rank + 1) * E_local]
    h = _experts(x_local, offs.cpu(), W_local)
    out = d.combine(h, st, scores)
    # dense single-process reference on this rank's tokens
    xr = x.detach().clone().requires_grad_(True)
    ref = sum(scores[:, j:j + 1] * torch.einsum("td,tdo->to", xr, W[ids[:, j]]) for j in range(k))
    assert torch.allclose(out, ref, rtol=1e-12, atol=1e-12)
    wsum = torch.randn(T, Do, generator=g, dtype=torch.float64)
    (out * wsum).sum().backward()
    (ref * wsum).sum().backward()
    assert torch.allclose(x.grad, xr.grad, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("num_experts,k", [(4, 2), (8, 4)])
def test_expert_parallel_dispatch_combine_two_ranks(num_experts, k):
    _spawn(_ep_worker, num_experts, 96, k, 16, 24)


def test_expert_parallel_single_rank_matches_dense():
    D.L.gather_rows, keep = _gather_rows_cpu, D.L.gather_rows
    try:
        g = torch.Generator().manual_seed(3)
        W = torch.randn(4, 8, 8, generator=g, dtype=torch.float64)
        x = torch.randn(40, 8, generator=g, dtype=torch.float64)
        ids = torch.randint(0, 4, (40, 2), generator=g)
        d = D.ExpertParallelDispatcher(4)
        xl, offs, st = d.dispatch(x, ids)
        out = d.combine(_experts(xl, offs, W), st, None)
        ref = sum(torch.einsum("td,tdo->to", x, W[ids[:, j]]) for j in range(2))
        assert torch.allclose(out, ref, rtol=1e-12, atol=1e-12)
    finally:
        D.L.gather_rows = keep


def _column_worker(rank, world):
    g = torch.Generator().manual_seed(5)  # replicated inputs
    x = torch.randn(24, 32, generator=g, dtype=torch.float64, requires_grad=True)
    W = torch.randn(64, 32, generator=g, dtype=torch.float64)
    dy = torch.randn(24, 64, generator=g, dtype=torch.float64)
    w_r = D.shard_rows(W).clone().requires_grad_(True)
    n = 64 // world
    y_r = D.column_sharded_linear(x, w_r, torch.nn.functional.linear)
    assert torch.allclose(y_r, (x.detach() @ W.t())[:, rank * n:(rank + 1) * n])
    y_r.backward(dy[:, rank * n:(rank + 1) * n])
    assert torch.allclose(x.grad, dy @ W, rtol=1e-12, atol=1e-12)             # summed over the shards
    assert torch.allclose(w_r.grad, (dy.t() @ x.detach())[rank * n:(rank + 1) * n])
    with pytest.raises(RuntimeError):
        D.shard_rows(torch.zeros(48, 8))  # 24 rows per rank: not a multiple of 32


def test_column_sharded_linear_two_ranks():
    _spawn(_column_worker)


def _allreduce_worker(rank, world):
    ps = [torch.nn.Parameter(torch.zeros(n)) for n in (10, 1000, 7)]
    for i, p in enumerate(ps):
        p.grad = torch.full_like(p, float(rank + 1 + i))
    ps.append(torch.nn.Parameter(torch.zeros(3)))             # a gradient on rank 1 only: zeros elsewhere
    if rank == 1:
        ps[3].grad = torch.full((3,), 4.0)
    ps.append(torch.nn.Parameter(torch.zeros(2), requires_grad=False))   # frozen: not part of the plan
    n = D.allreduce_gradients(ps, bucket_bytes=4032, max_in_flight=1)
    assert n == 3  # 40 B | 4000 B + 28 B | 12 B: the same plan on both ranks whatever gradients exist
    for i, p in enumerate(ps[:3]):
        assert torch.allclose(p.grad, torch.full_like(p, (1 + i + 2 + i) / 2))
    assert torch.allclose(ps[3].grad, torch.full((3,), 2.0)) and ps[4].grad is None


def test_bucketed_gradient_allreduce_two_ranks():
    _spawn(_allreduce_worker)


# ---------------------------------------------------------------------------------------------
# all-gather of the quantised weight: assembly of the gathered buffers
# ---------------------------------------------------------------------------------------------
def _weight_payload(S, codes, rank, world, b):
    """What a rank holds after quantising its row shard of W [N, K]: codes along K, packed scales of
    both packings, codes along N.  S: plain 2-D scales [N/b, K/b]; codes: [N, K/2] stand-in bytes."""
    from alto_b200._linear import pack_plain_scales
    N, n = codes.shape[0], codes.shape[0] // world
    Ssh = S[rank * n // b:(rank + 1) * n // b]
    ck = codes[rank * n:(rank + 1) * n]
    ct = codes.t()[:, rank * n:(rank + 1) * n].contiguous()          # stand-in for the [K, n/2] packing
    sk = pack_plain_scales(Ssh, n, True, b)
    st = pack_plain_scales(Ssh.t().contiguous(), S.shape[1] * b, True, b)
    return ck, sk, ct, st


@pytest.mark.parametrize("b,N,K,world", [(16, 512, 192, 2), (32, 1024, 256, 4), (16, 256, 64, 2)])
def test_gathered_weight_buffers_assemble_to_the_full_tensor(b, N, K, world):
    from alto_b200._linear import pack_plain_scales
    g = torch.Generator().manual_seed(0)
    S = torch.randint(1, 255, (N // b, K // b), generator=g, dtype=torch.uint8)
    codes = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    parts = [_weight_payload(S, codes, r, world, b) for r in range(world)]
    # rows: plain concatenation in rank order
    assert torch.equal(torch.cat([p[0] for p in parts]), codes)
    assert torch.equal(torch.cat([p[1] for p in parts]), pack_plain_scales(S, N, True, b))
    # columns: rank slices side by side
    ct = D.interleave_gathered_columns(torch.stack([p[2] for p in parts]), world, K // 2, parts[0][2].shape[1])
    assert torch.equal(ct, codes.t().contiguous())
    kt = (K + 127) // 128
    st = D.interleave_gathered_columns(torch.stack([p[3].view(kt, -1) for p in parts]), world, kt,
                                       parts[0][3].numel() // kt).reshape(-1)
    assert torch.equal(st, pack_plain_scales(S.t().contiguous(), K, True, b))


def test_outer_scale_from_amax_bits():
    vals = torch.tensor([0.0, 1.0, 5000.0, float("inf"), float("nan"), 1e-38], dtype=torch.float32)
    got = D.outer_scale_from_amax_bits(vals.view(torch.int32))
    exp = (torch.nan_to_num(vals) / (448.0 * 6.0)).clamp_min(1e-30)
    assert torch.equal(got, exp) and got[0].item() == pytest.approx(1e-30) and torch.isfinite(got).all()


def _gather_worker(rank, world):
    full = torch.arange(4 * world * 6, dtype=torch.uint8).view(4 * world, 6)
    rows = D.gather_packed_rows(full[4 * rank:4 * rank + 4].clone())
    assert torch.equal(rows, full)
    wide = torch.arange(3 * 5 * world, dtype=torch.int32).view(3, 5 * world)
    cols = D.gather_columns(wide[:, 5 * rank:5 * rank + 5].clone(), 3)
    assert torch.equal(cols, wide)
    bits = torch.tensor([rank + 1, 7 - rank], dtype=torch.int32)
    dist.all_reduce(bits, op=dist.ReduceOp.MAX)
    assert bits.tolist() == [world, 7]


def test_quantised_weight_gathers_two_ranks():
    _spawn(_gather_worker)


# ---------------------------------------------------------------------------------------------
# The wrapper's FSDP hooks: pre-all-gather payload of a row shard -> gather -> assembled operands
# ---------------------------------------------------------------------------------------------
def _cpu_quantize_shard(data, config, plan):
    """CPU stand-in for ``dispatch.quantize_shard_for_gather`` built on the oracle: MXFP4 in 32 x 32 blocks,
    both packings, packed scales (tests may use the oracle; the product hook runs the CUDA quantizer)."""
    from oracle import alto_oracle as O
    from alto_b200._linear import pack_plain_scales
    n, K = data.shape
    q, s = O.quantize_mxfp4(data, 32, -1, True)                       # [n, K/2], [n/32, K/32]
    qt, _ = O.quantize_mxfp4(data.t().contiguous(), 32, -1, True)     # [K, n/2]
    payload = (q.reshape(-1), pack_plain_scales(s, n, True, 32), qt.reshape(-1),
               pack_plain_scales(s.t().contiguous(), K, True, 32))
    meta = dict(world=plan["world"], fmt=1, block=32, n=n, K=K, dtype=data.dtype, has_outer=False)
    return payload, meta


def _fsdp_hook_worker(rank, world):
    from types import SimpleNamespace
    from alto_b200 import dispatch as Dp
    from alto_b200._linear import pack_plain_scales
    from oracle import alto_oracle as O
    N, K = 256 * world, 256
    g = torch.Generator().manual_seed(3)
    W = torch.randn(N, K, generator=g).bfloat16()
    cfg = Dp.TrainingOpConfig(precision="mxfp4", use_2dblock_x=False, use_2dblock_w=True, use_hadamard=False,
                              use_sr_grad=False, use_dge=False)
    n = N // world
    shard = Dp.MXFP4TrainingWeightWrapperTensor(W[rank * n:(rank + 1) * n].clone(), cfg)
    # the product plan wants CUDA data; everything else of it is exercised as it is
    real_plan = Dp.quantized_gather_plan
    Dp.quantized_gather_plan = lambda data, config, mesh: dict(group=None, world=world, fmt=1, block=32,
                                                               n=data.shape[0], K=data.shape[1])
    Dp.quantize_shard_for_gather = _cpu_quantize_shard
    try:
        policy = SimpleNamespace(param_dtype=torch.bfloat16)
        payload, meta = shard.fsdp_pre_all_gather(None, torch.Size([N, K]), (K, 1), None, policy)
        assert len(payload) == 4 and all(p.dtype == torch.uint8 for p in payload)
        gathered = []
        for p in payload:                                            # what FSDP's all-gather does, per input
            out = torch.empty(world * p.numel(), dtype=p.dtype)
            dist.all_gather_into_tensor(out, p.contiguous().view(-1))
            gathered.append(out)
        full, inner = shard.fsdp_post_all_gather(tuple(gathered), meta, torch.bfloat16)
        assert isinstance(full, Dp.MXFP4TrainingWeightWrapperTensor) and full.shape == (N, K)
        assert full.dtype == torch.bfloat16 and len(inner) == 4
        pre = full._prequant
        q, s = O.quantize_mxfp4(W, 32, -1, True)
        qt, _ = O.quantize_mxfp4(W.t().contiguous(), 32, -1, True)
        assert torch.equal(pre.w_k.codes, q) and torch.equal(pre.w_t.codes, qt)
        assert torch.equal(pre.w_k.scales, pack_plain_scales(s, N, True, 32))
        assert torch.equal(pre.w_t.scales, pack_plain_scales(s.t().contiguous(), K, True, 32))
        assert (pre.w_k.rows, pre.w_k.k, pre.w_t.rows, pre.w_t.k) == (N, K, K, N)
        # second gather into the same unsharded parameter: operands are refilled in place
        W2 = (W.float() * 0.5 + 1.0).bfloat16()
        shard2 = Dp.MXFP4TrainingWeightWrapperTensor(W2[rank * n:(rank + 1) * n].clone(), cfg)
        payload2, meta2 = shard2.fsdp_pre_all_gather(None, torch.Size([N, K]), (K, 1), None, policy)
        for out, p in zip(gathered, payload2):
            dist.all_gather_into_tensor(out, p.contiguous().view(-1))
        t_codes = pre.w_t.codes
        assert shard2.fsdp_post_all_gather(tuple(gathered), meta2, torch.bfloat16, out=full) is None
        q2, _ = O.quantize_mxfp4(W2, 32, -1, True)
        qt2, _ = O.quantize_mxfp4(W2.t().contiguous(), 32, -1, True)
        assert full._prequant is pre and pre.w_t.codes is t_codes
        assert torch.equal(pre.w_k.codes, q2) and torch.equal(pre.w_t.codes, qt2)
        # only identity re-views and detach are allowed on a weight that exists in quantised form
        assert torch.as_strided(full, full.shape, full.stride())._prequant is pre
        with pytest.raises(RuntimeError, match="quantised form"):
            full.t()
        # shards that do not end on scale-tile boundaries keep the high-precision gather of the reference
        Dp.quantized_gather_plan = real_plan
        (hp,), none_meta = shard.fsdp_pre_all_gather(None, torch.Size([N, K]), (K, 1), None, policy)
        assert none_meta is None and hp.dtype == torch.bfloat16 and hp.shape == (n, K)
    finally:
        Dp.quantized_gather_plan = real_plan


def test_fsdp_hooks_gather_quantised_operands_two_ranks():
    _spawn(_fsdp_hook_worker)
