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
    """Make calibration statistics identical on all ranks.  Entries without an outlier index (plain per-channel
    scales, the map threshold) are averaged.  A channel-base entry (outlier index + scale) takes rank 0's index and
    the MAXIMUM of the ranks' scales: every rank computed its scale with its OWN outlier channels zeroed (guard
    value 1e-3 there), so a channel that is an outlier on some rank but not in the agreed list still gets the scale
    of a rank that measured it, instead of a mean dragged down by guard values (which would clip it everywhere)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return static_value
    world = dist.get_world_size(group)
    for entry in static_value.values():
        channel_base = entry.get('outlier_channel_index') is not None
        for name, t in entry.items():
            if t is None:
                continue
            if name == 'outlier_channel_index':
                dist.broadcast(t, src=0, group=group)
            elif channel_base:
                buf = t.float()
                dist.all_reduce(buf, op=dist.ReduceOp.MAX, group=group)
                entry[name] = buf.to(t.dtype)
            else:
                buf = t.float()
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
                entry[name] = (buf / world).to(t.dtype)
    return static_value


_MLP_GRAD_NAMES = frozenset(("grad_ag", "grad_bg", "grad_au", "grad_bu", "grad_ad", "grad_bd"))


class LoraGradReducer:
    """The data-parallel exchange of a model's LoRA gradients: ONE persistent flat fp32 buffer, a few bucketed
    asynchronous all-reduces per step, averaged values left in ``.grad``.

    Use: ``reducer.add(key, grads)`` from the layers' ``on_lora_grads`` hooks (``key`` identifies the caller, e.g.
    ``(layer_index, "mlp")``; ``grads`` is the hook's dictionary); ``reducer.finish()`` once the backward pass is
    over.  The first step records the order in which the gradients arrive and gives every tensor a slice of the
    buffer in that order; from then on each ``add`` is one multi-tensor copy into the slices, and a bucket's
    all-reduce starts as soon as its last slice is filled (``bucket_bytes`` of consecutive arrivals), so the
    exchange overlaps the rest of the backward pass.  ``bind(key, name, param)`` attaches the parameter whose
    ``.grad`` receives the averaged gradient in ``finish()``.  Without an initialised process group (or with one
    rank) nothing is exchanged and ``finish()`` only fills ``.grad``."""

    def __init__(self, group=None, bucket_bytes=16 << 20, dtype=torch.float32):
        self.group, self.bucket_bytes, self.dtype = group, int(bucket_bytes), dtype
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._slots = {}            # (key, name) -> (offset, numel, shape)
        self._order = []            # keys in arrival order
        self._names = {}            # key -> sorted names
        self._params = {}           # (key, name) -> parameter
        self._frozen = False
        self._first = {}            # first step: key -> dict of gradients (kept until the layout is frozen)
        self.flat = None
        self._views = {}            # key -> list of fp32 views (order of self._names[key])
        self._bucket_of = {}        # key -> bucket index
        self._bucket_range = []     # bucket -> (begin, end) in elements
        self._bucket_left = []      # bucket -> keys still missing in this step
        self._bucket_size = []
        self._works = []
        self._layers = []
        self._local = {}

    def bind(self, key, name, param):
        self._params[(key, name)] = param

    def attach_layer(self, index, layer):
        """Wire a fused decoder layer module: its ``on_lora_grads`` hook feeds this reducer (the attention half and the
        MLP half arrive separately, keys ``(index, "attn")`` and ``(index, "mlp")``), and the 14 adapter weights it is
        driven with get the averaged gradients in ``.grad`` (bound after the first step, when the layer has seen them)."""
        self._layers.append((index, layer))
        layer.on_lora_grads = lambda grads, _i=index: self.add((_i, "mlp" if "grad_ag" in grads else "attn"), grads)

    def _bind_layers(self):
        for index, layer in self._layers:
            names = layer.named_lora_weights()
            for name, p in names.items():
                self.bind((index, "mlp" if name in _MLP_GRAD_NAMES else "attn"), name, p)

    # ---- layout (end of the first step)
    def _freeze(self, device):
        off = 0
        for key in self._order:
            for name in self._names[key]:
                g = self._first[key][name]
                self._slots[(key, name)] = (off, g.numel(), g.shape)
                off += g.numel()
        self.flat = torch.zeros(off, dtype=self.dtype, device=device)
        esize = self.flat.element_size()
        begin, cur = 0, 0
        for key in self._order:
            views = []
            for name in self._names[key]:
                o, n, shape = self._slots[(key, name)]
                views.append(self.flat[o:o + n].view(shape))
                cur = o + n
            self._views[key] = views
            self._bucket_of[key] = len(self._bucket_range)
            if (cur - begin) * esize >= self.bucket_bytes:
                self._bucket_range.append((begin, cur))
                begin = cur
        if cur > begin or not self._bucket_range:
            self._bucket_range.append((begin, cur))
        self._bucket_size = [0] * len(self._bucket_range)
        for key in self._order:
            self._bucket_size[self._bucket_of[key]] += 1
        self._frozen = True

    def _launch(self, b):
        lo, hi = self._bucket_range[b]
        if self.world > 1 and hi > lo:
            op = dist.ReduceOp.AVG if dist.get_backend(self.group) == "nccl" else dist.ReduceOp.SUM
            self._works.append((dist.all_reduce(self.flat[lo:hi], op=op, group=self.group, async_op=True), op, lo, hi))

    def add(self, key, grads):
        if self.world == 1:
            # nothing to exchange: the local gradients ARE the result; finish() hands them to .grad without a copy
            self._local[key] = grads
            return
        if not self._frozen:
            if key in self._first:
                raise RuntimeError("LoraGradReducer: %r delivered twice in one step" % (key,))
            self._order.append(key)
            self._names[key] = sorted(grads)
            self._first[key] = dict(grads)
            return
        if key not in self._views:
            raise RuntimeError("LoraGradReducer: %r was not part of the first step" % (key,))
        torch._foreach_copy_(self._views[key], [grads[n] for n in self._names[key]])
        b = self._bucket_of[key]
        self._bucket_left[b] -= 1
        if self._bucket_left[b] == 0:
            self._launch(b)

    def finish(self):
        """Wait for the exchange, write the averaged gradients into the bound parameters' ``.grad`` and return the
        flat buffer (fp32, averaged; None on a single rank, where ``.grad`` simply becomes the local gradient)."""
        if self.world == 1:
            if self._layers and not self._params:
                self._bind_layers()
            for (key, name), p in self._params.items():
                g = self._local.get(key, {}).get(name)
                if g is not None:
                    p.grad = g if (g.dtype == p.dtype and g.shape == p.shape) else g.to(p.dtype).reshape(p.shape)
            self._local = {}
            return None
        if not self._frozen:
            if not self._first:
                return None
            dev = next(iter(next(iter(self._first.values())).values())).device
            self._freeze(dev)
            self._bind_layers()
            self._bucket_left = list(self._bucket_size)
            first, self._first = self._first, {}
            for key in self._order:            # replay the first step through the frozen layout
                self.add(key, first[key])
        for work, op, lo, hi in self._works:
            work.wait()
            if op == dist.ReduceOp.SUM:
                self.flat[lo:hi].div_(self.world)
        self._works = []
        dst, src = [], []
        for (key, name), p in self._params.items():
            o, n, shape = self._slots[(key, name)]
            if p.grad is None:
                p.grad = torch.empty_like(p)
            dst.append(p.grad)
            src.append(self.flat[o:o + n].view(shape))
        if dst:
            torch._foreach_copy_(dst, src)
        self._bucket_left = list(self._bucket_size)
        return self.flat

    def checksum(self):
        """A 64-bit fingerprint of the averaged buffer (for checking that all ranks hold identical gradients)."""
        if self.flat is None:
            return 0
        bits = self.flat.view(torch.int32).to(torch.int64)
        w = torch.arange(1, bits.numel() + 1, device=bits.device, dtype=torch.int64) % 1000003
        return int((bits * w).sum().item())
