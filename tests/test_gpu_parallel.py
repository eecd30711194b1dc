"""Data-parallel step on two GPUs over NCCL (skipped where there is one): every rank runs the MLP half on its own
token shard, the LoRA gradients go through the bucketed reducer started from the backward's hook, and all ranks must
end the step with bit-identical averaged gradients that equal the mean of the ranks' local ones."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from hyc_lora_release_b200 import mlp, parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        BF16 = torch.bfloat16
        g = torch.Generator().manual_seed(5)                 # weights: shared
        gr = torch.Generator().manual_seed(50 + rank)        # tokens: this rank's shard
        B, M, H, I, R = 2, 128, 512, 1024, 16
        rn = lambda *sh, sc=1.0, gen=g: (torch.randn(*sh, generator=gen) * sc).to(BF16).to(dev)
        W = mlp.MLPWeights(norm_w=torch.ones(H, dtype=BF16, device=dev), wg=rn(I, H, sc=.02), wu=rn(I, H, sc=.02),
                           wd=rn(H, I, sc=.02), ag=rn(R, H, sc=.02), bg=rn(I, R, sc=.02), au=rn(R, H, sc=.02),
                           bu=rn(I, R, sc=.02), ad=rn(R, I, sc=.02), bd=rn(H, R, sc=.02))
        x, gout = rn(B, M, H, gen=gr), rn(B, M, H, gen=gr)
        state = mlp.MLPState(q_bit=4, layernorm_outlier_ratio=0.01)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        reducer = parallel.LoraGradReducer(bucket_bytes=64 << 10)
        params = {n: torch.nn.Parameter(torch.zeros_like(getattr(W, n[5:]))) for n in
                  ("grad_ag", "grad_bg", "grad_au", "grad_bu", "grad_ad", "grad_bd")}
        for n, p in params.items():
            reducer.bind("mlp", n, p)
        local = {}
        for it in range(7):
            out, saved = mlp.mlp_forward(x, W, state, status=st)
            mlp.mlp_backward(gout, saved, W, status=st,
                             on_lora_grads=lambda g_: (local.update({k: v.float().clone() for k, v in g_.items()}), reducer.add("mlp", g_)))
            reducer.finish()
            if it < state.iteration_threshold:
                parallel.sync_calibration(state.static_value)
        mlp.check_status(st, "mlp")
        problems = []
        sums = [None] * world
        dist.all_gather_object(sums, reducer.checksum())
        if any(v != sums[0] for v in sums):
            problems.append("ranks hold different averaged gradients")
        for n, p in params.items():
            mean = local[n].clone()
            dist.all_reduce(mean)
            mean /= world
            if not torch.allclose(p.grad.float(), mean, rtol=2e-2, atol=1e-3 * float(mean.abs().max())):
                problems.append("%s is not the mean of the local gradients" % n)
        # the calibrated statistics are the same everywhere
        sv = state.static_value["gate"]["scale"].float()
        lo, hi = sv.clone(), sv.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if not torch.equal(lo, hi):
            problems.append("calibrated scales differ between ranks")
        ret[rank] = problems
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_step_leaves_identical_averaged_lora_gradients():
    import torch.multiprocessing as mp
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, 29541, ret), nprocs=world, join=True)
        assert all(ret.get(r) == [] for r in range(world)), dict(ret)
