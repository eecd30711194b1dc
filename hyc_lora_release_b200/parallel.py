"""Token-shard data parallelism for the compression path.

Every operator on the path is independent per token row (or per attention-map row), so the
multi-GPU layout is: contiguous token shards per rank, frozen and LoRA weights replicated, and
ONE exchange per step: a sum all-reduce of the flattened LoRA gradients (then a division by the
world size).  During calibration the statistics are made identical on all ranks: scales and
thresholds are averaged, rank 0's outlier channel index is broadcast.  The reference has no
distributed code at all; this is the minimal scheme its data-parallel use would need.
"""
from typing import Dict, Iterable, List, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of `total` tokens for `rank`; the first total % world ranks get one more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def flatten_grads(grads: Iterable[torch.Tensor], dtype=torch.float32) -> Tuple[torch.Tensor, List[Tuple[torch.Size, int]]]:
    grads = list(grads)
    meta = [(g.shape, g.numel()) for g in grads]
    flat = torch.cat([g.reshape(-1).to(dtype) for g in grads]) if grads else torch.empty(0, dtype=dtype)
    return flat, meta


def unflatten_grads(flat: torch.Tensor, meta, like: Iterable[torch.Tensor]) -> List[torch.Tensor]:
    out, off = [], 0
    for (shape, n), ref in zip(meta, like):
        out.append(flat[off:off + n].reshape(shape).to(ref.dtype))
        off += n
    return out


def allreduce_lora_grads(grads: Dict[str, torch.Tensor], group=None, average=True) -> Dict[str, torch.Tensor]:
    """One all-reduce over a single flattened fp32 buffer holding every LoRA gradient."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return grads
    names = sorted(grads)
    flat, meta = flatten_grads([grads[n] for n in names])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat /= dist.get_world_size(group)
    return dict(zip(names, unflatten_grads(flat, meta, [grads[n] for n in names])))


class PendingLoraGrads:
    """Handle of an all-reduce that is in flight; ``wait()`` returns the averaged gradients."""

    def __init__(self, names, flat, meta, like, work, world, average):
        self._names, self._flat, self._meta, self._like = names, flat, meta, like
        self._work, self._world, self._average = work, world, average

    def wait(self) -> Dict[str, torch.Tensor]:
        if self._flat is None:
            return dict(zip(self._names, self._like))
        if self._work is not None:
            self._work.wait()          # the current stream waits for the collective
        flat = self._flat
        if self._average and self._world > 1:
            flat = flat / self._world
        return dict(zip(self._names, unflatten_grads(flat, self._meta, self._like)))


def allreduce_lora_grads_async(grads: Dict[str, torch.Tensor], group=None, average=True) -> PendingLoraGrads:
    """Start the all-reduce of the flattened LoRA gradients and return at once: the collective runs beside
    whatever the caller enqueues next (``mlp_backward`` calls this through its ``on_lora_grads`` hook before the
    grad_x GEMM and the RMSNorm backward, which do not need the reduced values)."""
    names = sorted(grads)
    like = [grads[n] for n in names]
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return PendingLoraGrads(names, None, None, like, None, 1, average)      # nothing to exchange
    flat, meta = flatten_grads(like)
    work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
    return PendingLoraGrads(names, flat, meta, like, work, dist.get_world_size(group), average)


def sync_calibration(static_value: dict, group=None) -> dict:
    """Make calibration statistics identical on all ranks: floating-point entries are averaged,
    the outlier channel index of rank 0 wins."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return static_value
    world = dist.get_world_size(group)
    for entry in static_value.values():
        for name, t in entry.items():
            if t is None:
                continue
            if name == 'outlier_channel_index':
                dist.broadcast(t, src=0, group=group)
            else:
                buf = t.float()
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
                entry[name] = (buf / world).to(t.dtype)
    return static_value
