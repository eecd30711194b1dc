"""Drop-in for the reference module of the same name (its ``triton_fuse_silu_backward``,
operators/triton_fuse_lora_silu_hadamard_backward_kernels.py:152-178)."""
import torch

from .._lib import check, lib, ptr, stream_of
from ._fused_common import BF16, check_fused_args, lora_b_transposed, scale_vec


def triton_fuse_silu_backward(xa1, b1, q1, s1, xa2, b2, q2, s2, grad_o, quantize_bit=8):
    """De-quantizes the saved gate/up main branches, recomputes the forward and returns
    (o, grad_gate, grad_up), each [B, M, N] bf16."""
    B, M, N = grad_o.shape
    R = b1.shape[0]
    check_fused_args(quantize_bit, N, R, xa1, b1, q1, s1, xa2, b2, q2, s2, grad_o)
    g = grad_o.to(BF16).contiguous()
    xa1c, xa2c = xa1.to(BF16).contiguous(), xa2.to(BF16).contiguous()
    bt1, bt2 = lora_b_transposed(b1), lora_b_transposed(b2)
    s1c, s2c = scale_vec(s1, N), scale_vec(s2, N)
    q1c, q2c = q1.contiguous(), q2.contiguous()
    o = torch.empty((B, M, N), device=g.device, dtype=BF16)
    gg = torch.empty((B, M, N), device=g.device, dtype=BF16)
    gu = torch.empty((B, M, N), device=g.device, dtype=BF16)
    check(lib.hyc_fused_lora_silu_hadamard_bwd(ptr(xa1c), ptr(bt1), ptr(q1c), ptr(s1c), ptr(xa2c), ptr(bt2),
                                               ptr(q2c), ptr(s2c), ptr(g), ptr(o), ptr(gg), ptr(gu), B * M, N, R,
                                               quantize_bit, stream_of(g)), "hyc_fused_lora_silu_hadamard_bwd")
    return o, gg, gu
