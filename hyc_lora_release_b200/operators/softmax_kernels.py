"""Drop-in for the reference's ``operators/softmax_kernels.py`` wrapper (:41-56)."""
import torch

from .._lib import check, lib, ptr, require_cuda, stream_of

BF16 = torch.bfloat16


def softmax_backward(y, grad_y, scale=1.0):
    """o = (grad_y - sum(y * grad_y, -1)) * y for a [b, h, n, n] map.  ``scale`` (extension): the bf16 result
    times ``scale`` as a second bf16 operation, for the layer's ``grad_s / sqrt(head_dim)``."""
    require_cuda(y, grad_y)
    assert grad_y.shape == y.shape
    yc, gc = y.to(BF16).contiguous(), grad_y.to(BF16).contiguous()
    S = yc.shape[-1]
    o = torch.empty_like(yc)
    check(lib.hyc_softmax_bwd(ptr(yc), ptr(gc), ptr(o), yc.numel() // S, S, float(scale), stream_of(y)), "hyc_softmax_bwd")
    return o


def _mask_args(attention_mask, b, h, n, S):
    """-> (mask tensor or None, batch stride, head stride, row stride) for the C entry points."""
    if attention_mask is None:
        return None, 0, 0, 0
    mk = attention_mask.to(BF16)
    if mk.dim() != 4 or mk.shape[-1] != S or mk.shape[-2] != n or mk.shape[0] not in (1, b) or mk.shape[1] not in (1, h):
        raise ValueError("attention_mask must be [b or 1, h or 1, n, S]")
    if mk.stride(-1) != 1:
        mk = mk.contiguous()

    def strides(t):
        return (0 if t.shape[0] == 1 else t.stride(0)), (0 if t.shape[1] == 1 else t.stride(1)), t.stride(2)
    mb, mh, mr = strides(mk)
    if (mb | mh | mr) & 7 or mk.data_ptr() & 15:
        mk = mk.contiguous()
        mb, mh, mr = strides(mk)
    return mk, mb, mh, mr


def softmax_forward_topk_save(scores, scale, attention_mask, outlier_ratio, quantize_bit=4, inplace=False):
    """``a = softmax(scores * scale + attention_mask)`` and the save of ``a`` as a top-k map in ONE pass over the
    scores: -> (a, TopkMap).  The same results as ``softmax_forward_scale_mask`` followed by
    ``compression_softmax_topk(a, ...)`` (the probabilities may differ from the two-kernel path in the last bf16 bit
    where the fp32 row sums, taken in another order, round differently; the saved map is exactly the compression of
    the probabilities this call returns).  Shapes outside the fused kernel take the two kernels.
    Measured on a B200 the fused kernel is the SLOWER choice today (the save is bound by instruction issue, so the
    softmax arithmetic does not hide behind memory traffic: [1,32,2048,2048] 281 us against 118 + 145 us); it saves
    one 268 MB read of the map and is kept for GPUs or shapes where that read is what counts."""
    from .compress_function import TopkMap, compression_softmax_topk
    require_cuda(scores, attention_mask)
    if scores.dim() != 4:
        raise ValueError("scores must be [batch, heads, n, S]")
    if quantize_bit not in (2, 4, 8):
        raise ValueError("quantize_bit must be 2, 4 or 8")
    if inplace and (scores.dtype != BF16 or not scores.is_contiguous()):
        raise ValueError("inplace needs contiguous bf16 scores")
    sc = scores.to(BF16).contiguous()
    b, h, n, S = sc.shape
    rows, k, dev = b * h * n, int(S * outlier_ratio), sc.device
    mk, mb, mh, mr = _mask_args(attention_mask, b, h, n, S)
    out = sc if inplace else torch.empty_like(sc)
    if S % 64 == 0:
        val = torch.empty((rows, k), dtype=BF16, device=dev)
        col = torch.empty((rows, k), dtype=torch.int16, device=dev)
        q = torch.empty((rows, S * quantize_bit // 8), dtype=torch.uint8, device=dev)
        s = torch.empty((rows, S // 64), dtype=BF16, device=dev)
        z = torch.empty((rows, S // 64), dtype=torch.int8, device=dev)
        rc = lib.hyc_softmax_fwd_topk_save(ptr(sc), float(scale), ptr(mk), mb, mh, mr, h, n, rows, S, k, ptr(out),
                                           ptr(val) if k else None, ptr(col) if k else None, ptr(q), ptr(s), ptr(z),
                                           quantize_bit, stream_of(sc))
        if rc != -8:          # HYC_ERR_UNSUPPORTED: shape outside the fused kernel, nothing was launched
            check(rc, "hyc_softmax_fwd_topk_save")
            return out, TopkMap(val, col, q, s, z, sc.shape, quantize_bit)
    a = softmax_forward_scale_mask(sc, scale, attention_mask, inplace=inplace)
    return a, compression_softmax_topk(a, outlier_ratio, quantize_bit)


def softmax_forward_scale_mask(scores, scale, attention_mask=None, inplace=False):
    """a = softmax(scores * scale + attention_mask, dim=-1) for raw scores [b, h, n, S] in one pass, with the
    rounding points of the layer's three tensor operations (the scaling and the mask addition are bf16
    operations, the softmax is fp32 inside with a bf16 result;
    models/llama/fused_llama_layer_intra_inter_full_fuse.py:150-160).  ``attention_mask``: additive, broadcastable
    as [b, 1 or h, n, S].  ``inplace`` overwrites ``scores`` (which must then be contiguous bf16)."""
    require_cuda(scores, attention_mask)
    if scores.dim() != 4:
        raise ValueError("scores must be [batch, heads, n, S]")
    if inplace and (scores.dtype != BF16 or not scores.is_contiguous()):
        raise ValueError("inplace needs contiguous bf16 scores")
    sc = scores.to(BF16).contiguous()
    b, h, n, S = sc.shape
    out = sc if inplace else torch.empty_like(sc)
    mb = mh = mr = 0
    mk = None
    if attention_mask is not None:
        mk = attention_mask.to(BF16)
        if mk.dim() != 4 or mk.shape[-1] != S or mk.shape[-2] != n or mk.shape[0] not in (1, b) or mk.shape[1] not in (1, h):
            raise ValueError("attention_mask must be [b or 1, h or 1, n, S]")
        if mk.stride(-1) != 1:
            mk = mk.contiguous()
        mb = 0 if mk.shape[0] == 1 else mk.stride(0)
        mh = 0 if mk.shape[1] == 1 else mk.stride(1)
        mr = mk.stride(2)
        if (mb | mh | mr) & 7 or mk.data_ptr() & 15:
            mk = mk.contiguous()
            mb = 0 if mk.shape[0] == 1 else mk.stride(0)
            mh = 0 if mk.shape[1] == 1 else mk.stride(1)
            mr = mk.stride(2)
    check(lib.hyc_softmax_fwd_scale_mask(ptr(sc), float(scale), ptr(mk), mb, mh, mr, h, n, ptr(out), b * h * n, S,
                                         stream_of(scores)), "hyc_softmax_fwd_scale_mask")
    return out
