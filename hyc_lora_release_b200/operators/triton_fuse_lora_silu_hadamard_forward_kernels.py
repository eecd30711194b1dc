"""Drop-in for the reference module of the same name (its ``triton_fuse_silu_forward``,
operators/triton_fuse_lora_silu_hadamard_forward_kernels.py:152-181).  The name is kept so
the reference's layers can import it unchanged; the kernel behind it is CUDA (libhyc.so)."""
import torch

from .._lib import check, lib, ptr, stream_of
from ._fused_common import BF16, check_fused_args, lora_b_transposed, rows_nld, scale_vec


def triton_fuse_silu_forward(xa1, b1, x1, s1, xa2, b2, x2, s2, quantize_bit=8):
    """q1 = quant(x1, s1), q2 = quant(x2, s2), o = silu(x1 + xa1 @ b1) * (x2 + xa2 @ b2).
    xa*: [B, M, R] ; b*: [R, N] ; x*: [B, M, N] ; s*: [1, N].  -> (q1, q2, o)."""
    B, M, N = x1.shape
    R = b1.shape[0]
    check_fused_args(quantize_bit, N, R, xa1, b1, x1, s1, xa2, b2, x2, s2)
    x1c, rows, _ = rows_nld(x1)
    x2c, _, _ = rows_nld(x2)
    xa1c, xa2c = xa1.to(BF16).contiguous(), xa2.to(BF16).contiguous()
    bt1, bt2 = lora_b_transposed(b1), lora_b_transposed(b2)
    s1c, s2c = scale_vec(s1, N), scale_vec(s2, N)
    epp = 8 // quantize_bit
    q1 = torch.empty((B, M, N // epp), device=x1.device, dtype=torch.uint8)
    q2 = torch.empty((B, M, N // epp), device=x1.device, dtype=torch.uint8)
    o = torch.empty((B, M, N), device=x1.device, dtype=BF16)
    check(lib.hyc_fused_lora_silu_hadamard_fwd(ptr(xa1c), ptr(bt1), ptr(x1c), ptr(s1c), ptr(xa2c), ptr(bt2),
                                               ptr(x2c), ptr(s2c), ptr(q1), ptr(q2), ptr(o), rows, N, R,
                                               quantize_bit, stream_of(x1)), "hyc_fused_lora_silu_hadamard_fwd")
    return q1, q2, o
