"""Host-side mirror of the reference's ``operators/compress_function.py``.

Same function names, argument meaning and return tuples as the reference module, so the
fused decoder layers of the reference can import this module in its place.  Every
function forwards to a kernel of libhyc.so; nothing here computes on the CPU.

Differences that a caller can observe, all deliberate:
  * ``outlier_subtraction_fuse_compression_quantization`` does not zero the outlier columns
    of its argument in place (reference: compress_function.py:130); the kernel never needs
    the zeroed copy, so callers may stop cloning.
  * only ``q_method='per-channel'`` can be quantized (the reference's 'per-tensor' scale is
    a 0-dim tensor that its own launch wrappers cannot take, compress_function.py:195-203).
  * the order of equal-norm outlier channels is fixed: norm descending, index ascending.
"""
import ctypes

import torch

from .. import _lib
from .._lib import check, lib, ptr, require_cuda, stream_of

BF16 = torch.bfloat16


# ******************** utils ********************

def hidden_to_head_shape(x: torch.Tensor, num_heads: int):
    """compress_function.py:6-9."""
    bsz, seq_len, hidden_dim = x.shape
    return x.reshape(bsz, seq_len, num_heads, hidden_dim // num_heads).transpose(1, 2)


def head_to_hidden_shape(x: torch.Tensor):
    """compress_function.py:11-13."""
    bsz, _, seq_len, _ = x.shape
    return x.transpose(1, 2).reshape(bsz, seq_len, -1)


def update_dict(old_dict, new_dict, iteration):
    """Running mean of the calibration statistics; the outlier index is replaced
    (compress_function.py:15-27)."""
    for name in old_dict.keys():
        if name == 'outlier_channel_index' or old_dict[name] is None:
            old_dict[name] = new_dict[name]
        else:
            old_dict[name] = (iteration * old_dict[name] + new_dict[name]) / (iteration + 1)
    return old_dict


def _as_hidden(x):
    if x.dim() == 4:
        x = head_to_hidden_shape(x)
    if x.dim() != 3:
        raise ValueError("expected a [B, M, N] or [B, heads, M, d] tensor, got shape %s" % (tuple(x.shape),))
    return x


def _rows_view(x):
    """[B, M, N] bf16 -> (tensor whose memory is [B*M rows, N] with one row stride, rows, ld)."""
    x = x.to(BF16)
    B, M, N = x.shape
    if x.stride(2) != 1 or (B > 1 and x.stride(0) != M * x.stride(1)) or x.stride(1) < N \
            or x.stride(1) % 8 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    return x, B * M, x.stride(1)


def _scale_vec(s, N):
    s = s.to(BF16).reshape(-1)
    if s.numel() != N:
        raise ValueError("per-channel scale with %d entries for %d channels (per-tensor scales cannot be quantized with)" % (s.numel(), N))
    return s.contiguous()


def _check_q(q_bit):
    if q_bit not in (2, 4, 8):
        raise ValueError("quantize_bit must be 2, 4 or 8")


# ******************** statistics ********************

def get_statistics_softmax(x: torch.Tensor, outlier_ratio: float):
    """compress_function.py:30-32.  Calibration only; the k-th value comes from the
    framework's selection routine."""
    require_cuda(x)
    return torch.kthvalue(x.float().flatten(), int(x.numel() * (1 - outlier_ratio))).values


def _colstats(x, q_bit, idx=None, want_zp=False):
    require_cuda(x)
    _check_q(q_bit)
    x = _as_hidden(x)
    x0 = x[0].to(BF16)
    if x0.stride(1) != 1 or x0.stride(0) % 8 != 0 or x0.data_ptr() % 16 != 0:
        x0 = x0.contiguous()
    M, N = x0.shape
    scale = torch.empty((1, N), dtype=BF16, device=x.device)
    zp = torch.empty((1, N), dtype=torch.int8, device=x.device) if want_zp else None
    k = 0
    if idx is not None:
        idx = idx.to(torch.int64).contiguous()
        k = idx.numel()
        if k == 0:   # a non-null pointer selects the zero-guarded (channel-base) variant
            idx = torch.zeros(1, dtype=torch.int64, device=x.device)
    check(lib.hyc_colstats_scale(ptr(x0), M, N, x0.stride(0), q_bit, ptr(idx), k, ptr(scale), ptr(zp),
                                 stream_of(x)), "hyc_colstats_scale")
    return scale, zp


def get_statistics_only_quant(x: torch.Tensor, q_bit: int = 8, q_method: str = 'per-tensor'):
    """compress_function.py:45-59."""
    if q_method == 'per-channel':
        return _colstats(x, q_bit)[0]
    if q_method == 'per-tensor':
        require_cuda(x)
        x0 = _as_hidden(x)[0]
        return ((x0.max() - x0.min()) / (2 ** q_bit - 1)).to(BF16)
    raise ValueError("Unsupport Quantize Method")


def get_statistics_only_quant_zero_point(x: torch.Tensor, q_bit: int = 8, q_method: str = 'per-tensor'):
    """compress_function.py:62-77 (only the per-channel branch defines a zero point there)."""
    if q_method != 'per-channel':
        raise ValueError("Unsupport Quantize Method")
    return _colstats(x, q_bit, want_zp=True)


def get_statistics_channel_base(x: torch.Tensor, outlier_ratio: float, q_bit: int = 8, q_method: str = 'per-tensor'):
    """compress_function.py:80-105 -> (outlier_channel_index int64 [k], scale bf16 [1, N])."""
    if q_method != 'per-channel':
        raise ValueError("Unsupport Quantize Method")
    require_cuda(x)
    x = _as_hidden(x)
    x0 = x[0].to(BF16)
    if x0.stride(1) != 1 or x0.stride(0) % 8 != 0 or x0.data_ptr() % 16 != 0:
        x0 = x0.contiguous()
    M, N = x0.shape
    k = int(N * outlier_ratio)
    norm = torch.empty(N, dtype=BF16, device=x.device)
    idx = torch.empty(k, dtype=torch.int64, device=x.device)
    check(lib.hyc_channel_norm_topk(ptr(x0), M, N, x0.stride(0), k, ptr(norm), ptr(idx) if k else None,
                                    stream_of(x)), "hyc_channel_norm_topk")
    scale, _ = _colstats(x, q_bit, idx=idx)
    return idx, scale


# ******************** compress / decompress interface ********************

def _quant(x, s, q_bit, z=None, channel=None, out=None):
    require_cuda(x, s)
    _check_q(q_bit)
    x = _as_hidden(x)
    xr, rows, ld = _rows_view(x)
    B, M, N = x.shape
    if N % 32 != 0:
        raise ValueError("the hidden size must be a multiple of 32")
    s = _scale_vec(s, N)
    zt = None
    if z is not None:
        zt = z.reshape(-1).to(torch.int8).contiguous()
    epp = 8 // q_bit
    k, idx, xo = 0, None, None
    if channel is not None:
        idx = channel.to(device=x.device, dtype=torch.int64).contiguous()
        k = idx.numel()
    if out is not None:      # caller-provided (q, x_outlier) buffers, e.g. reused across steps
        q, xo = out
    else:
        q = torch.empty((B, M, N // epp), dtype=torch.uint8, device=x.device)
        if channel is not None:
            xo = torch.empty((B, M, k), dtype=BF16, device=x.device)
    if rows == 0:
        return q, xo
    check(lib.hyc_quant_pack(ptr(xr), rows, N, ld, ptr(s), ptr(zt), ptr(idx) if k else None, k, ptr(q),
                             ptr(xo) if k else None, q_bit, stream_of(x)), "hyc_quant_pack")
    return q, xo


def _dequant(q, s, q_bit, z=None, channel=None, x_outlier=None, out=None):
    require_cuda(q, s)
    _check_q(q_bit)
    B, M, _ = q.shape
    N = s.shape[-1]
    q = q.contiguous()
    s = _scale_vec(s, N)
    zt = None
    if z is not None:
        zt = z.reshape(-1).to(torch.int8).contiguous()
    x = out if out is not None else torch.empty((B, M, N), dtype=BF16, device=q.device)
    if B * M == 0:
        return x
    k, idx, xo = 0, None, None
    if channel is not None:
        idx = channel.to(device=q.device, dtype=torch.int64).contiguous()
        k = idx.numel()
        xo = x_outlier.to(BF16).contiguous()
    check(lib.hyc_unpack_dequant(ptr(q), B * M, N, ptr(s), ptr(zt), ptr(idx) if k else None, k,
                                 ptr(xo) if k else None, ptr(x), N, q_bit, stream_of(q)), "hyc_unpack_dequant")
    return x


def outlier_subtraction_fuse_compression_quantization(x, s, channel, quantize_bit=8, dtype=torch.bfloat16, out=None):
    """compress_function.py:111-143 -> (x_outlier [B,M,k] bf16, q uint8).  One kernel: the
    outlier columns are gathered and encoded as zero; ``x`` is left untouched.
    ``out=(q, x_outlier)`` (not in the reference) writes into existing buffers."""
    q, xo = _quant(x, s, quantize_bit, channel=channel, out=out)
    return xo, q


def outlier_addition_fuse_decompression_dequantization(q, s, x_outlier, channel, quantize_bit=8, is_head=False,
                                                       num_heads=1, dtype=torch.bfloat16, out=None):
    """compress_function.py:147-174.  ``out`` (not in the reference): an existing [B,M,N] bf16 buffer."""
    x = _dequant(q, s, quantize_bit, channel=channel, x_outlier=x_outlier, out=out)
    return hidden_to_head_shape(x, num_heads=num_heads) if is_head else x


def compression_quantization(x, s, quantize_bit=8, dtype=torch.bfloat16):
    """compress_function.py:178-210."""
    return _quant(x, s, quantize_bit)[0]


def decompression_dequantization(q, s, quantize_bit=8, is_head=False, num_heads=1, dtype=torch.bfloat16):
    """compress_function.py:214-241 (the result is bf16 whatever ``dtype`` says, as there)."""
    x = _dequant(q, s, quantize_bit)
    return hidden_to_head_shape(x, num_heads=num_heads) if is_head else x


def decompression_dequantization_lora_add(q, s, x_lora_a, w_lora_b, quantize_bit=8):
    """``decompression_dequantization(q, s, quantize_bit) + x_lora_a @ w_lora_b`` in one kernel (no counterpart
    in the reference, which runs the two steps: fused_llama_layer_intra_inter_full_fuse.py:416-452).
    q [B, M, N*bit/8], s [.., N], x_lora_a [B, M, 16], w_lora_b [16, N] (``lora_B.weight.T``) -> [B, M, N] bf16."""
    from ._fused_common import lora_b_transposed
    require_cuda(q, s, x_lora_a, w_lora_b)
    _check_q(quantize_bit)
    B, M, _ = q.shape
    N = s.shape[-1]
    sc = _scale_vec(s, N)
    xa = x_lora_a.to(BF16).contiguous()
    bt = lora_b_transposed(w_lora_b)
    y = torch.empty((B, M, N), dtype=BF16, device=q.device)
    if B * M:
        check(lib.hyc_dequant_lora_add(ptr(q.contiguous()), ptr(sc), ptr(xa), ptr(bt), ptr(y), B * M, N, xa.shape[-1],
                                       quantize_bit, stream_of(q)), "hyc_dequant_lora_add")
    return y


def compression_quantization_with_zero_point(x, s, z, quantize_bit=8, dtype=torch.bfloat16):
    """compress_function.py:245-275."""
    return _quant(x, s, quantize_bit, z=z)[0]


def decompression_dequantization_with_zero_point(q, s, z, quantize_bit=8, is_head=False, num_heads=1,
                                                 dtype=torch.bfloat16):
    """compress_function.py:278-306."""
    x = _dequant(q, s, quantize_bit, z=z)
    return hidden_to_head_shape(x, num_heads=num_heads) if is_head else x


# ---- attention map, threshold prune (reference behaviour) ----

def compression_softmax(x: torch.Tensor, outlier):
    """compress_function.py:309-313: entries above the threshold as a 1-D sparse COO tensor
    of the flattened map (int64 indices, values in x's dtype), built by a two-phase stream
    compaction.  One device-to-host copy of the count sizes the result, as in ``to_sparse``."""
    require_cuda(x)
    xf = x.to(BF16).contiguous()
    numel = xf.numel()
    thr = float(outlier)
    ws_bytes = lib.hyc_softmax_prune_workspace_bytes(numel)
    ws = torch.empty((ws_bytes + 7) // 8, dtype=torch.int64, device=x.device)
    st = stream_of(x)
    check(lib.hyc_softmax_prune_count(ptr(xf), numel, thr, ptr(ws), ws_bytes, st), "hyc_softmax_prune_count")
    nnz = int(ws[0].item())
    idx = torch.empty((1, nnz), dtype=torch.int64, device=x.device)
    val = torch.empty(nnz, dtype=BF16, device=x.device)
    check(lib.hyc_softmax_prune_fill(ptr(xf), numel, thr, ptr(ws), ptr(idx) if nnz else None,
                                     ptr(val) if nnz else None, nnz, st), "hyc_softmax_prune_fill")
    return torch.sparse_coo_tensor(idx, val, (numel,), is_coalesced=True)


def decompression_softmax(x_sparse: torch.Tensor):
    """compress_function.py:316-317 (flattened dense map; callers reshape)."""
    require_cuda(x_sparse)
    idx = x_sparse.indices().reshape(-1).contiguous()
    val = x_sparse.values().to(BF16).contiguous()
    numel = x_sparse.shape[0]
    out = torch.empty(numel, dtype=BF16, device=val.device)
    check(lib.hyc_softmax_prune_restore(ptr(idx) if idx.numel() else None, ptr(val) if idx.numel() else None,
                                        idx.numel(), ptr(out), numel, stream_of(val)), "hyc_softmax_prune_restore")
    return out


class PrunedMap:
    """The threshold-pruned map with its length left on the device: index and value buffers of a fixed
    capacity plus a device-side count.  ``to_dense()`` is what the layers call on their sparse handle; nothing
    here synchronises with the host, so a training step that uses it is a fixed launch sequence."""

    def __init__(self, idx, val, nnz, shape):
        self.idx, self.val, self.nnz, self.shape = idx, val, nnz, tuple(shape)

    @property
    def capacity(self):
        return self.idx.numel()

    def nbytes(self):
        return self.idx.numel() * 8 + self.val.numel() * 2 + 8

    def overflowed(self):
        """True if more entries passed the threshold than the buffers hold (synchronises)."""
        return int(self.nnz.item()) > self.capacity

    def to_dense(self, out=None):
        numel = 1
        for d in self.shape:
            numel *= d
        if out is None:
            out = torch.empty(self.shape, dtype=BF16, device=self.val.device)
        elif out.numel() != numel or out.dtype != BF16 or not out.is_contiguous():
            raise ValueError("`out` must be a contiguous bf16 tensor with the map's number of elements")
        check(lib.hyc_softmax_prune_restore_counted(ptr(self.idx), ptr(self.val), ptr(self.nnz), self.capacity, ptr(out),
                                                    numel, stream_of(self.val)), "hyc_softmax_prune_restore_counted")
        return out


class TiledPrunedMap:
    """The threshold-pruned map in the tiled form of ``hyc_softmax_prune_tiled``: 4-byte words (offset inside a
    2048-element batch << 16 | bf16 bits) in per-batch spans, a directory of {span start, entries} per batch and the
    device-side count.  ``to_dense()`` rebuilds the map in one pass; nothing synchronises with the host.
    ``nnz`` holds the number of kept entries when everything fit, else capacity + the number of dropped entries
    (the word list is used as 64 equal sub-lists that fill evenly but not identically, so keep ``capacity`` a good
    margin above the expected count: the default is 1.5 x)."""

    BATCH = 2048

    def __init__(self, words, directory, nnz, shape):
        self.words, self.directory, self.nnz, self.shape = words, directory, nnz, tuple(shape)

    @property
    def capacity(self):
        return self.words.numel()

    def nbytes(self):
        return self.words.numel() * 4 + self.directory.numel() * 4 + 8

    def overflowed(self):
        """True if more entries passed the threshold than the buffers hold (synchronises)."""
        return int(self.nnz.item()) > self.capacity

    def to_dense(self, out=None):
        numel = 1
        for d in self.shape:
            numel *= d
        if out is None:
            out = torch.empty(self.shape, dtype=BF16, device=self.words.device)
        elif out.numel() != numel or out.dtype != BF16 or not out.is_contiguous():
            raise ValueError("`out` must be a contiguous bf16 tensor with the map's number of elements")
        check(lib.hyc_softmax_prune_tiled_restore(ptr(self.words), self.capacity, ptr(self.directory), ptr(out), numel,
                                                  stream_of(self.words)), "hyc_softmax_prune_tiled_restore")
        return out

    def entries(self):
        """(flattened index int64, value bf16) of the stored entries in ascending index order, decoded with torch
        operations (for inspection and tests; synchronises)."""
        numel = 1
        for n in self.shape:
            numel *= n
        n_batches = (numel + self.BATCH - 1) // self.BATCH          # the buffer also holds the call's counters behind these
        d = self.directory[:2 * n_batches].view(-1, 2).to(torch.int64)
        start, cnt = d[:, 0], d[:, 1]
        batch = torch.repeat_interleave(torch.arange(d.shape[0], device=d.device), cnt)
        first = torch.repeat_interleave(start, cnt)
        ofs = torch.arange(batch.numel(), device=d.device) - torch.repeat_interleave(torch.cumsum(cnt, 0) - cnt, cnt)
        w = self.words[first + ofs].to(torch.int64)
        idx = batch * self.BATCH + (w >> 16)
        val = (w & 0xffff).to(torch.int16).view(BF16) if w.numel() else torch.empty(0, dtype=BF16, device=d.device)
        order = torch.argsort(idx)
        return idx[order], val[order]


def compression_softmax_static(x: torch.Tensor, outlier, capacity=None, margin=1.5, ratio=None, ordered=False):
    """``compression_softmax`` (compress_function.py:309-313) without the device-to-host read of the count: the
    kept entries go into buffers of a fixed ``capacity`` (default: ``margin`` x ``ratio`` x numel + 1024, for a
    threshold calibrated to keep ``ratio`` of the entries) and the count stays on the device.  Entries beyond the
    capacity are dropped; ``PrunedMap.overflowed()`` tells.  ``outlier``: a Python float or a tensor (one
    synchronisation if it lives on the device: pass the calibrated threshold as a float in steady state).

    ``ordered=False`` (default) -> ``TiledPrunedMap``: one pass over the map, the same (index, value) pairs as the
    reference's sparse tensor kept as 4-byte words in per-batch spans (their order depends on the run --
    ``to_dense()`` does not care), restored in one pass.  -> ``PrunedMap`` otherwise:
    ``ordered=True``: ascending flattened index like ``to_sparse``, through the count + scan + fill kernels with the
    library's built-in scratch: maps of up to 268,435,456 elements, calls on one GPU must not overlap (they share
    that scratch), and the first call on a device must be made outside of stream capture."""
    require_cuda(x)
    xf = x.to(BF16).contiguous()
    numel = xf.numel()
    if capacity is None:
        if ratio is None:
            raise ValueError("give `capacity` or the calibrated `ratio`")
        capacity = int(numel * ratio * margin) + 1024
    capacity = min(int(capacity), numel)
    nnz = torch.empty(1, dtype=torch.int64, device=x.device)
    if not ordered:
        words = torch.empty(capacity, dtype=torch.int32, device=x.device)
        directory = torch.empty(lib.hyc_softmax_prune_tiled_directory_bytes(numel) // 4, dtype=torch.int32, device=x.device)
        check(lib.hyc_softmax_prune_tiled(ptr(xf), numel, float(outlier), ptr(words), capacity, ptr(directory), ptr(nnz),
                                          stream_of(x)), "hyc_softmax_prune_tiled")
        return TiledPrunedMap(words, directory, nnz, x.shape)
    idx = torch.empty(capacity, dtype=torch.int64, device=x.device)
    val = torch.empty(capacity, dtype=BF16, device=x.device)
    check(lib.hyc_softmax_prune_static(ptr(xf), numel, float(outlier), ptr(idx), ptr(val), capacity, ptr(nnz),
                                       stream_of(x)), "hyc_softmax_prune_static")
    return PrunedMap(idx, val, nnz, x.shape)


# ---- modes without a counterpart in the reference ----

def compression_group(x, quantize_bit=4):
    """64-wide groups along the last dimension, scale and zero point from each group.
    -> (q uint8 [..., N/epp], scale bf16 [..., N/64], zero_point int8 [..., N/64])."""
    require_cuda(x)
    _check_q(quantize_bit)
    xb = x.to(BF16).contiguous()
    N = xb.shape[-1]
    if N % 64 != 0:
        raise ValueError("the last dimension must be a multiple of 64")
    rows = xb.numel() // N
    lead = xb.shape[:-1]
    q = torch.empty(lead + (N * quantize_bit // 8,), dtype=torch.uint8, device=x.device)
    s = torch.empty(lead + (N // 64,), dtype=BF16, device=x.device)
    z = torch.empty(lead + (N // 64,), dtype=torch.int8, device=x.device)
    check(lib.hyc_group_quant_pack(ptr(xb), rows, N, N, ptr(q), ptr(s), ptr(z), quantize_bit, stream_of(x)),
          "hyc_group_quant_pack")
    return q, s, z


def decompression_group(q, s, z, quantize_bit=4):
    require_cuda(q, s, z)
    _check_q(quantize_bit)
    N = s.shape[-1] * 64
    lead = q.shape[:-1]
    rows = q.numel() // q.shape[-1]
    x = torch.empty(lead + (N,), dtype=BF16, device=q.device)
    check(lib.hyc_group_unpack_dequant(ptr(q.contiguous()), rows, N, ptr(s.contiguous()), ptr(z.contiguous()),
                                       ptr(x), N, quantize_bit, stream_of(q)), "hyc_group_unpack_dequant")
    return x


class TopkMap:
    """Per-row top-k compressed attention map; ``to_dense()`` restores it (same call the
    reference's layers make on their sparse handle)."""

    def __init__(self, val, col, q, scale, zp, shape, q_bit):
        self.val, self.col, self.q, self.scale, self.zp = val, col, q, scale, zp
        self.shape, self.q_bit = tuple(shape), q_bit

    def tensors(self):
        return self.val, self.col, self.q, self.scale, self.zp

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in self.tensors())

    def to_dense(self, out=None):
        return decompression_softmax_topk(self, out=out)

    def softmax_backward(self, grad, out=None, scale=1.0):
        """``softmax_backward(self.to_dense(), grad)`` (operators/softmax_kernels.py:41) without writing the
        restored map: one kernel where the shapes allow it, restore + softmax backward otherwise.  ``scale``: the
        bf16 result times ``scale`` as a second bf16 operation (the layer's ``grad_s / sqrt(head_dim)``)."""
        require_cuda(grad, self.q)
        g = grad.to(BF16).contiguous()
        if tuple(g.shape) != self.shape:
            raise ValueError("the gradient must have the map's shape %s" % (self.shape,))
        S, rows, k = self.shape[-1], self.q.shape[0], self.val.shape[1]
        if out is None:
            out = torch.empty(self.shape, dtype=BF16, device=self.q.device)
        rc = lib.hyc_softmax_topk_restore_bwd(ptr(self.val) if k else None, ptr(self.col) if k else None, k, ptr(self.q),
                                              ptr(self.scale), ptr(self.zp), rows, S, ptr(g), ptr(out), self.q_bit,
                                              float(scale), stream_of(self.q))
        if rc == -8:      # HYC_ERR_UNSUPPORTED: shape outside the fused kernel
            from .softmax_kernels import softmax_backward as _sb
            res = _sb(self.to_dense(), g, scale)
            out.copy_(res.reshape(self.shape))
            return out
        check(rc, "hyc_softmax_topk_restore_bwd")
        return out


def compression_softmax_topk(x, outlier_ratio, quantize_bit=4, out=None):
    """Top-k per row (k = int(S * ratio)) as bf16 value + uint16 column, the remainder
    group-quantized.  x [..., S] with S % 64 == 0, S <= 4096.  ``out``: a TopkMap of an earlier call
    on the same shape, ratio and bit width whose buffers are overwritten (a ring of saved maps)."""
    require_cuda(x)
    _check_q(quantize_bit)
    xb = x.to(BF16).contiguous()
    S = xb.shape[-1]
    rows = xb.numel() // S
    k = int(S * outlier_ratio)
    dev = x.device
    if out is not None:
        if (out.shape != tuple(x.shape) or out.q_bit != quantize_bit or out.val.shape != (rows, k)
                or out.q.device != dev):
            raise ValueError("`out` was made for another shape, ratio, bit width or device")
        val, col, q, s, z = out.tensors()
    else:
        val = torch.empty((rows, k), dtype=BF16, device=dev)
        col = torch.empty((rows, k), dtype=torch.int16, device=dev)   # holds uint16 column numbers
        q = torch.empty((rows, S * quantize_bit // 8), dtype=torch.uint8, device=dev)
        s = torch.empty((rows, S // 64), dtype=BF16, device=dev)
        z = torch.empty((rows, S // 64), dtype=torch.int8, device=dev)
    check(lib.hyc_softmax_topk_compress(ptr(xb), rows, S, k, ptr(val) if k else None, ptr(col) if k else None,
                                        ptr(q), ptr(s), ptr(z), quantize_bit, stream_of(x)),
          "hyc_softmax_topk_compress")
    return out if out is not None else TopkMap(val, col, q, s, z, x.shape, quantize_bit)


def decompression_softmax_topk(m: TopkMap, out=None):
    """``out``: an existing contiguous bf16 tensor of the map's shape."""
    S = m.shape[-1]
    rows = m.q.shape[0]
    k = m.val.shape[1]
    if out is None:
        out = torch.empty(m.shape, dtype=BF16, device=m.q.device)
    elif tuple(out.shape) != m.shape or out.dtype != BF16 or not out.is_contiguous() or out.device != m.q.device:
        raise ValueError("`out` must be a contiguous bf16 tensor of shape %s on the map's device" % (m.shape,))
    check(lib.hyc_softmax_topk_restore(ptr(m.val) if k else None, ptr(m.col) if k else None, k, ptr(m.q),
                                       ptr(m.scale), ptr(m.zp), rows, S, ptr(out), m.q_bit, stream_of(m.q)),
          "hyc_softmax_topk_restore")
    return out


# ******************** pack "get statistics" and "compress" ********************

def compression_pack_channel_base(x, o_ratio, q_bit, q_method, it_num, it_num_thd, static_value):
    """compress_function.py:346-352 -> (x_outlier, q, outlier_channel_index, scale)."""
    if it_num < it_num_thd:
        o_channel_idx, scale = get_statistics_channel_base(x, o_ratio, q_bit, q_method)
    else:
        o_channel_idx, scale = static_value['outlier_channel_index'], static_value['scale']
    o, q = outlier_subtraction_fuse_compression_quantization(x, scale, o_channel_idx, q_bit)
    return o, q, o_channel_idx, scale


def compression_pack_quant_base(x, q_bit, q_method, it_num, it_num_thd, static_value):
    """compress_function.py:355-361 -> (q, scale)."""
    if it_num < it_num_thd:
        scale = get_statistics_only_quant(x, q_bit, q_method)
    else:
        scale = static_value['scale']
    return compression_quantization(x, scale, q_bit), scale


def compression_pack_quant_zp_base(x, q_bit, q_method, it_num, it_num_thd, static_value):
    """compress_function.py:364-370 -> (q, scale, zero_point)."""
    if it_num < it_num_thd:
        scale, zero_point = get_statistics_only_quant_zero_point(x, q_bit, q_method)
    else:
        scale, zero_point = static_value['scale'], static_value['zero_point']
    return compression_quantization_with_zero_point(x, scale, zero_point, q_bit), scale, zero_point


def compression_pack_softmax_base(x, o_ratio, it_num, it_num_thd, static_value):
    """compress_function.py:373-379 -> (sparse handle, threshold)."""
    if it_num < it_num_thd:
        outlier = get_statistics_softmax(x, o_ratio)
    else:
        outlier = static_value['outlier']
    return compression_softmax(x, outlier), outlier
