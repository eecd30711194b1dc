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
