"""The allocation-free amax entry point (``altob200_amax_noalloc``).

Some callers of this library may not allocate device memory at all: code running inside a
memory plan that is already fixed, a plugin inside another runtime, a server whose allocator is
frozen after start-up.  For them the library offers one entry point whose working memory is a
fixed array inside the library itself.  This test calls it through the C ABI twice in a row
(the array keeps the previous call's contents, so the second call is the interesting one) and
checks both results against the regular ``altob200_amax`` entry point: the outputs are integer
bit patterns of maxima, so the comparison is exact.  The file name makes pytest collect it last.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(L, x):
    bits = torch.empty(2, dtype=torch.int32, device=x.device)
    outer = torch.empty(2, dtype=torch.float32, device=x.device)
    scratch = torch.zeros(L.AMAX_SCRATCH_BYTES // 4, dtype=torch.int32, device=x.device)
    L.amax(x, bits, outer, scratch)
    return bits[:1].clone(), outer[:1].clone()


def _noalloc(L, x):
    bits = torch.full((1,), -1, dtype=torch.int32, device=x.device)
    outer = torch.full((1,), -1.0, dtype=torch.float32, device=x.device)
    L.amax_noalloc(x, bits, outer)
    return bits, outer


def test_noalloc_amax_matches_regular_entry_point_twice_in_a_row():
    from alto_b200 import _lib as L
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(7)
    # first call: many blocks, bf16; second call: fewer blocks, a smaller maximum and fp32, so that
    # stale partial maxima or a stale counter from the first call would change the answer
    x1 = (torch.randn(4096, 4096, generator=g, device=dev) * 3.0).bfloat16()
    x1[1234, 567] = 977.0
    x2 = torch.randn(96, 2880, generator=g, device=dev) * 1e-3
    for x in (x1, x2):
        want_bits, want_outer = _regular(L, x)
        got_bits, got_outer = _noalloc(L, x)
        torch.cuda.synchronize()
        assert torch.equal(got_bits, want_bits), (got_bits, want_bits)
        assert torch.equal(got_outer, want_outer), (got_outer, want_outer)
        # and against plain tensor arithmetic, independent of this library: the fp32 bit pattern of
        # max |x| and the outer scale max(amax / (448 * 6), 1e-30) divided on the CPU (correctly rounded)
        amax = x.abs().amax().float().cpu()
        assert got_bits.cpu().item() == amax.view(torch.int32).item()
        want = torch.clamp(amax / (448.0 * 6.0), min=1e-30)
        assert got_outer.cpu().view(torch.int32).item() == want.view(torch.int32).item()
    # a strided view (leading dimension larger than the row) and a NaN, which must give amax 0 ->
    # the floor of the outer scale, exactly like the regular entry point
    x3 = x1[:, :2048]
    x3[5, 5] = float("nan")
    want_bits, want_outer = _regular(L, x3)
    got_bits, got_outer = _noalloc(L, x3)
    assert torch.equal(got_bits, want_bits) and torch.equal(got_outer, want_outer)
    assert got_outer.item() == pytest.approx(1e-30)


def test_noalloc_amax_rejects_inputs_beyond_its_fixed_array():
    from alto_b200 import _lib as L
    dev = torch.device("cuda")
    bits = torch.zeros(1, dtype=torch.int32, device=dev)
    # a fake shape over the limit: the size check refuses it before anything is launched or read
    rows, cols = (L.NOALLOC_MAX_BYTES // 2) // 4096 + 1, 4096
    small = torch.zeros(16, cols, dtype=torch.bfloat16, device=dev)
    with pytest.raises(L.Altob200Error) as e:
        L._check(L.lib().altob200_amax_noalloc(small.data_ptr(), L.DT_BF16, rows, cols, cols, bits.data_ptr(), None,
                                               torch.cuda.current_stream().cuda_stream), "altob200_amax_noalloc")
    assert e.value.status == L.E_LIMIT
