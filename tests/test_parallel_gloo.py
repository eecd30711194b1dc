"""The multi-rank host logic on CPU: two gloo ranks, token shards, the LoRA-gradient all-reduce and
the calibration sync.  (The device kernels need no collective.)"""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hyc_lora_release_b200 import parallel


def test_shard_bounds_cover_everything():
    for total in (0, 1, 7, 8192, 8193):
        for world in (1, 2, 3, 8):
            spans = [parallel.shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100)
        x = torch.randn(64, 32, generator=g)               # all tokens; each rank takes its shard
        gm = torch.randn(64, 16, generator=g)
        b, e = parallel.shard_bounds(64, rank, world)
        grads = {"grad_a": (gm[b:e].t() @ x[b:e]).to(torch.bfloat16), "grad_b": (x[b:e].t() @ gm[b:e])}
        red = parallel.allreduce_lora_grads(grads, average=False)
        full_a = (gm.t() @ x)
        ok = torch.allclose(red["grad_a"].float(), full_a, atol=0.25, rtol=2e-2) and \
            torch.allclose(red["grad_b"], x.t() @ gm, atol=1e-4) and red["grad_a"].dtype == torch.bfloat16
        # the asynchronous form gives the same sums (and the average when asked)
        pend = parallel.allreduce_lora_grads_async(grads, average=True)
        other = torch.randn(8, 8, generator=g) @ torch.randn(8, 8, generator=g)     # work enqueued meanwhile
        avg = pend.wait()
        ok = ok and torch.allclose(avg["grad_b"], (x.t() @ gm) / world, atol=1e-4) and other.shape == (8, 8)
        sv = {"x": {"outlier_channel_index": torch.tensor([rank, rank + 5]), "scale": torch.full((1, 4), float(rank + 1))}}
        sv = parallel.sync_calibration(sv)
        ok = ok and sv["x"]["outlier_channel_index"].tolist() == [0, 5] and \
            torch.allclose(sv["x"]["scale"], torch.full((1, 4), (1 + world) / 2.0))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_allreduce_and_calibration_sync():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, 29531, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world)), dict(ret)
