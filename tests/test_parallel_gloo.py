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
        checks = {}
        checks["allreduce"] = torch.allclose(red["grad_a"].float(), full_a, atol=0.25, rtol=2e-2) and \
            torch.allclose(red["grad_b"], x.t() @ gm, atol=1e-4) and red["grad_a"].dtype == torch.bfloat16
        # the asynchronous form gives the same sums (and the average when asked)
        pend = parallel.allreduce_lora_grads_async(grads, average=True)
        other = torch.randn(8, 8, generator=g) @ torch.randn(8, 8, generator=g)     # work enqueued meanwhile
        avg = pend.wait()
        checks["async"] = torch.allclose(avg["grad_b"], (x.t() @ gm) / world, atol=1e-4) and other.shape == (8, 8)
        # calibration sync: a plain scale is averaged; a channel-base entry takes rank 0's index and the LARGEST scale
        # (the ranks' outlier sets differ here: channel 1 is an outlier only on rank 1, whose own scale for it is the
        # guard value, while rank 0 measured it)
        sv = {"x": {"outlier_channel_index": torch.tensor([0, 5 + rank]),
                    "scale": torch.tensor([[1e-3, 2.0 if rank == 0 else 1e-3, 0.5 + rank, 0.25]])},
              "q": {"scale": torch.full((1, 4), float(rank + 1))}}
        sv = parallel.sync_calibration(sv)
        checks["calibration"] = sv["x"]["outlier_channel_index"].tolist() == [0, 5] and \
            torch.allclose(sv["x"]["scale"], torch.tensor([[1e-3, 2.0, 0.5 + world - 1, 0.25]])) and \
            torch.allclose(sv["q"]["scale"], torch.full((1, 4), (1 + world) / 2.0))
        # the bucketed reducer: three "layers" deliver their gradients in backward order on two steps; every rank ends
        # with the same averaged values in .grad, and the buckets cover the buffer
        red = parallel.LoraGradReducer(bucket_bytes=2 * 2 * 16 * 32 * 4)      # two layers per bucket
        params = {}
        for layer in range(3):
            for name in ("grad_a", "grad_b"):
                p_ = torch.nn.Parameter(torch.zeros(16, 32) if name == "grad_a" else torch.zeros(32, 16))
                params[(layer, name)] = p_
                red.bind(layer, name, p_)
        sums = []
        for step in range(2):
            want = {}
            for layer in (2, 1, 0):
                gg = torch.Generator().manual_seed(1000 * step + 10 * layer)
                per_rank = [{"grad_a": torch.randn(16, 32, generator=gg), "grad_b": torch.randn(32, 16, generator=gg)}
                            for _ in range(world)]
                red.add(layer, per_rank[rank])
                for name in ("grad_a", "grad_b"):
                    want[(layer, name)] = sum(pr[name] for pr in per_rank) / world
            red.finish()
            checks["reducer step %d" % step] = all(torch.allclose(params[k].grad, want[k], atol=1e-6) for k in want)
            sums.append(red.checksum())
        checks["buckets"] = len(red._bucket_range) == 2 and red._bucket_range[0][0] == 0 and \
            red._bucket_range[-1][1] == red.flat.numel()
        gathered = [None] * world
        dist.all_gather_object(gathered, sums)
        checks["identical on all ranks"] = all(g_ == gathered[0] for g_ in gathered)
        ret[rank] = [k for k, v in checks.items() if not v]
    finally:
        dist.destroy_process_group()


def test_two_rank_allreduce_and_calibration_sync():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, 29531, ret), nprocs=world, join=True)
        assert all(ret.get(r) == [] for r in range(world)), dict(ret)
