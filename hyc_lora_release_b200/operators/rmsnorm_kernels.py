"""Drop-in for the reference's ``operators/rmsnorm_kernels.py`` wrappers (:116-185)."""
import torch

from .._lib import check, lib, ptr, require_cuda, stream_of

BF16 = torch.bfloat16


def rmsnorm_forward(x, weight, eps):
    """-> (y, mean, rstd, BLOCK_SIZE, num_warps).  ``mean`` is unused by RMSNorm (the reference
    returns an uninitialised buffer); the last two values are launch hints of the reference that
    its backward takes back and this implementation ignores."""
    require_cuda(x, weight)
    xc = x.to(BF16).contiguous()
    N = xc.shape[-1]
    rows = xc.numel() // N
    if N > 65536 // xc.element_size():
        raise RuntimeError("This layer norm doesn't support feature dim >= 64KB.")
    y = torch.empty_like(xc)
    rstd = torch.empty((rows,), dtype=torch.float32, device=x.device)
    mean = torch.zeros((rows,), dtype=torch.float32, device=x.device)
    w = weight.to(BF16).contiguous()
    check(lib.hyc_rmsnorm_fwd(ptr(xc), ptr(w), float(eps), ptr(y), ptr(rstd), rows, N, stream_of(x)), "hyc_rmsnorm_fwd")
    return y, mean, rstd, 0, 0


def rmsnorm_backward(dy, x, w, m, v, needs_inputs_grad, eps, num_warps, BLOCK_SIZE):
    """-> (dx, None).  ``v`` is the rstd of the forward."""
    if not needs_inputs_grad:
        return None, None
    require_cuda(dy, x, w, v)
    dyc, xc = dy.to(BF16).contiguous(), x.to(BF16).contiguous()
    N = xc.shape[-1]
    rows = xc.numel() // N
    dx = torch.empty_like(dyc)
    check(lib.hyc_rmsnorm_bwd(ptr(dyc), ptr(xc), ptr(w.to(BF16).contiguous()), ptr(v.contiguous()), ptr(dx), rows, N,
                              stream_of(dy)), "hyc_rmsnorm_bwd")
    return dx, None


# ---- RMSNorm fused with the saves of the fused layer (no counterpart in the reference: there the norm, the
# ---- channel-base pack of its input and the pack of its output are three separate passes)

def rmsnorm_forward_save(x, weight, eps, quantize_bit, x_scale, x_outlier_index, y_scale=None):
    """One pass over ``x`` [B, M, N]: -> (y, rstd, x_outlier [B, M, k], x_q, y_q or None).
    ``x_scale`` [.., N] and ``x_outlier_index`` int64 [k] are the calibrated statistics that
    ``compression_pack_channel_base`` would use in steady state, ``y_scale`` those of
    ``compression_pack_quant_base`` on the normalised tensor.  The five results are bit-identical to
    ``rmsnorm_forward`` + ``outlier_subtraction_fuse_compression_quantization(x, ...)`` +
    ``compression_quantization(y, ...)``."""
    require_cuda(x, weight, x_scale)
    if quantize_bit not in (2, 4, 8):
        raise ValueError("quantize_bit must be 2, 4 or 8")
    xc = x.to(BF16).contiguous()
    N = xc.shape[-1]
    rows = xc.numel() // N
    lead = xc.shape[:-1]
    dev = x.device
    w = weight.to(BF16).contiguous()
    sx = x_scale.to(BF16).reshape(-1).contiguous()
    if sx.numel() != N:
        raise ValueError("per-channel scale with %d entries for %d channels" % (sx.numel(), N))
    idx = x_outlier_index.to(device=dev, dtype=torch.int64).contiguous() if x_outlier_index is not None else None
    k = 0 if idx is None else idx.numel()
    sy = None if y_scale is None else y_scale.to(BF16).reshape(-1).contiguous()
    y = torch.empty_like(xc)
    rstd = torch.empty((rows,), dtype=torch.float32, device=dev)
    qx = torch.empty(lead + (N * quantize_bit // 8,), dtype=torch.uint8, device=dev)
    xo = torch.empty(lead + (k,), dtype=BF16, device=dev)
    qy = None if sy is None else torch.empty(lead + (N * quantize_bit // 8,), dtype=torch.uint8, device=dev)
    if rows:
        check(lib.hyc_rmsnorm_fwd_save(ptr(xc), ptr(w), float(eps), rows, N, ptr(sx), ptr(idx) if k else None, k,
                                       ptr(sy), ptr(y), ptr(rstd), ptr(qx), ptr(xo) if k else None, ptr(qy),
                                       quantize_bit, stream_of(x)), "hyc_rmsnorm_fwd_save")
    return y, rstd, xo, qx, qy


def rmsnorm_backward_packed(dy, x_q, x_scale, x_outlier, x_outlier_index, w, rstd, quantize_bit, residual_grad=None):
    """``rmsnorm_backward`` on the saved form of x (codes + outlier slab), with the residual gradient added:
    -> dx.  Bit-identical to ``outlier_addition_fuse_decompression_dequantization`` + ``rmsnorm_backward``
    (+ a bf16 tensor add of ``residual_grad``)."""
    require_cuda(dy, x_q, x_scale, w, rstd)
    dyc = dy.to(BF16).contiguous()
    N = dyc.shape[-1]
    rows = dyc.numel() // N
    sx = x_scale.to(BF16).reshape(-1).contiguous()
    idx = x_outlier_index.to(device=dy.device, dtype=torch.int64).contiguous() if x_outlier_index is not None else None
    k = 0 if idx is None else idx.numel()
    xo = x_outlier.to(BF16).contiguous() if k else None
    res = None if residual_grad is None else residual_grad.to(BF16).contiguous()
    dx = torch.empty_like(dyc)
    if rows:
        check(lib.hyc_rmsnorm_bwd_packed(ptr(dyc), ptr(x_q.contiguous()), ptr(sx), ptr(idx) if k else None, k, ptr(xo),
                                         ptr(w.to(BF16).contiguous()), ptr(rstd.contiguous()), ptr(res), ptr(dx), rows, N,
                                         quantize_bit, stream_of(dy)), "hyc_rmsnorm_bwd_packed")
    return dx
