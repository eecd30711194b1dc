"""Drop-in for the wrappers of the reference's ``operators/rope_kernels.py`` (:81-131): rotary embedding in
the rotate-half form on ``[batch, seq_len, n_heads, head_dim]`` tensors, own sm_100a kernel."""
import torch

from .._lib import check, lib, ptr, require_cuda, stream_of

BF16 = torch.bfloat16
ROPE_GROUP_SIZE = 4


def calculate_settings(n):
    """Launch hints of the reference (block size = next power of two, warps by size).  Returned so that callers
    that pass them back to ``rope_backward`` keep working; this implementation ignores them."""
    block = 1 << max(0, int(n) - 1).bit_length()
    if block > 65536:
        raise RuntimeError("Cannot launch with a feature dim of %d: the maximum block size is 65536." % n)
    warps = 4
    if block >= 32768:
        warps = 32
    elif block >= 8192:
        warps = 16
    elif block >= 2048:
        warps = 8
    return block, warps


def _tables(cos, sin, seq_len, head_dim):
    cos, sin = cos.squeeze(), sin.squeeze()
    if cos.dim() != 2 or sin.shape != cos.shape:
        raise ValueError("cos / sin must squeeze to [seq_len, head_dim] tables")
    assert seq_len <= cos.shape[0]
    if cos.shape[1] < head_dim // 2:
        raise ValueError("cos / sin tables are narrower than head_dim / 2")
    if cos.dtype not in (BF16, torch.float32):
        cos, sin = cos.float(), sin.float()
    sin = sin.to(cos.dtype)
    if cos.stride(1) != 1 or sin.stride(1) != 1 or sin.stride(0) != cos.stride(0):
        cos, sin = cos.contiguous(), sin.contiguous()
    return cos, sin


def _rope(x, cos, sin, backward, out=None):
    require_cuda(x, cos, sin)
    batch, seq_len, n_heads, head_dim = x.shape
    cos, sin = _tables(cos, sin, seq_len, head_dim)
    xc = x.to(BF16).contiguous()
    if out is None:
        out = xc if xc.data_ptr() != x.data_ptr() else torch.empty_like(xc)
    check(lib.hyc_rope(ptr(xc), n_heads * head_dim, ptr(out), n_heads * head_dim, ptr(cos), ptr(sin), cos.stride(0),
                       1 if cos.dtype == torch.float32 else 0, batch * seq_len, seq_len, n_heads, head_dim,
                       1 if backward else 0, stream_of(x)), "hyc_rope")
    return out.view(batch, seq_len, n_heads, head_dim)


def rope_forward(x, cos, sin):
    """x [batch, seq_len, n_heads, head_dim] -> rotated tensor of the same shape (a new tensor; the input is
    left as it is, where the reference rotates a contiguous copy in place)."""
    return _rope(x, cos, sin, False)


def rope_backward(dy, cos, sin, n_groups=None, BLOCK_SIZE=None, num_warps=None):
    """Gradient of ``rope_forward``: the same rotation with the sine negated."""
    return _rope(dy, cos, sin, True)


def rope_inplace(x, cos, sin, backward=False):
    """Rotates a contiguous bf16 ``[batch, seq_len, n_heads, head_dim]`` tensor in place (no allocation)."""
    if x.dtype != BF16 or not x.is_contiguous():
        raise ValueError("rope_inplace needs a contiguous bf16 tensor")
    return _rope(x, cos, sin, backward, out=x)
