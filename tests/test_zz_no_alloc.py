"""The allocation-free prune entry point (hyc_softmax_prune_static) against the two-phase one.

Some callers cannot hand the library a workspace because they must not allocate device memory at
call time; for them the tile offsets live in an array inside the library.  This test drives the
entry point through the C ABI on buffers that exist before the call, twice in a row (the built-in
array keeps the previous call's contents, and the second call must not be disturbed by them), and
checks indices, values and the count bit for bit against hyc_softmax_prune_count/fill.
Collected last on purpose: a run that stops at the first failure has then run everything else."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _map(b, h, s, seed):
    g = torch.Generator().manual_seed(seed)
    logits = 3 * torch.randn(b, h, s, s, generator=g) + torch.triu(torch.full((s, s), float("-inf")), diagonal=1)
    return torch.softmax(logits, dim=-1).to(torch.bfloat16).to(DEV)


def test_static_prune_matches_two_phase_twice_in_a_row():
    from hyc_lora_release_b200._lib import check, lib, ptr, stream_of
    from hyc_lora_release_b200.operators import compress_function as cf
    cases = [(_map(2, 4, 256, 1), 0.05), (_map(1, 2, 100, 2), 0.3)]   # second call: smaller map, other threshold
    refs = []
    for a, ratio in cases:
        thr = float(cf.get_statistics_softmax(a, ratio))
        sp = cf.compression_softmax(a, thr)            # existing entry points (caller-provided workspace)
        refs.append((thr, sp.indices().reshape(-1).clone(), sp.values().clone()))
    # every buffer exists before the calls; the entry point itself allocates nothing
    outs = [(torch.full((r[1].numel() + 8,), -1, dtype=torch.int64, device=DEV),
             torch.zeros(r[1].numel() + 8, dtype=torch.bfloat16, device=DEV),
             torch.zeros(1, dtype=torch.int64, device=DEV)) for r in refs]
    for rep in range(2):                                # the pair of calls, repeated
        for (a, _), (thr, ridx, rval), (idx, val, nnz) in zip(cases, refs, outs):
            idx.fill_(-1)
            check(lib.hyc_softmax_prune_static(ptr(a), a.numel(), ctypes.c_float(thr), ptr(idx), ptr(val),
                                               idx.numel(), ptr(nnz), stream_of(a)), "hyc_softmax_prune_static")
            n = int(nnz.item())
            assert n == ridx.numel()
            assert torch.equal(idx[:n], ridx) and torch.equal(val[:n], rval)
            assert bool((idx[n:] == -1).all())          # nothing written past the end


def test_static_prune_limits():
    from hyc_lora_release_b200._lib import lib, ptr, stream_of
    a = _map(1, 1, 64, 3)
    nnz = torch.zeros(1, dtype=torch.int64, device=DEV)
    too_big = 65536 * 4096 + 1
    assert lib.hyc_softmax_prune_static(ptr(a), too_big, ctypes.c_float(0.1), None, None, 0, ptr(nnz), stream_of(a)) == -7
    # capacity 0: count only
    assert lib.hyc_softmax_prune_static(ptr(a), a.numel(), ctypes.c_float(0.0), None, None, 0, ptr(nnz), stream_of(a)) == 0
    assert int(nnz.item()) == int((a != 0).sum())


def test_static_prune_tail_negative_threshold_and_short_capacity():
    """The branches a regression would land in: a map whose size ends inside a 16-byte chunk, a negative threshold
    on a map with exact zeros (a zero is no entry), and buffers shorter than the list (the full count is still
    reported, the first `capacity` entries are the two-phase list's, nothing is written past the end)."""
    from hyc_lora_release_b200._lib import check, lib, ptr, stream_of
    from hyc_lora_release_b200.operators import compress_function as cf
    g = torch.Generator().manual_seed(11)
    for shape, thr in (((1, 1, 99, 99), 0.02), ((1, 1, 99, 99), -1.0)):
        x = torch.randn(*shape, generator=g)
        x[torch.rand(*shape, generator=g) < 0.25] = 0.0
        a = x.to(torch.bfloat16).to(DEV)
        sp = cf.compression_softmax(a, thr)
        ridx, rval = sp.indices().reshape(-1), sp.values()
        n = ridx.numel()
        assert n > 16
        for cap in (n + 8, n - 5):
            idx = torch.full((n + 8,), -1, dtype=torch.int64, device=DEV)
            val = torch.zeros(n + 8, dtype=torch.bfloat16, device=DEV)
            nnz = torch.zeros(1, dtype=torch.int64, device=DEV)
            check(lib.hyc_softmax_prune_static(ptr(a), a.numel(), ctypes.c_float(thr), ptr(idx), ptr(val), cap, ptr(nnz),
                                               stream_of(a)), "hyc_softmax_prune_static")
            kept = min(cap, n)
            assert int(nnz.item()) == n
            assert torch.equal(idx[:kept], ridx[:kept]) and torch.equal(val[:kept], rval[:kept])
            assert bool((idx[kept:] == -1).all())
