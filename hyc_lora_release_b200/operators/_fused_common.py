import torch

from .._lib import require_cuda

BF16 = torch.bfloat16


def lora_b_transposed(b):
    """[R, N] LoRA-B operand -> the [N, R] row-major matrix the kernels read.  The layers pass
    ``lora_B.weight.T``, a view of exactly that storage, so usually nothing is copied."""
    if b.dim() != 2:
        raise ValueError("LoRA B must be [R, N]")
    bt = b.t()
    if bt.dtype != BF16 or not bt.is_contiguous():
        bt = bt.to(BF16).contiguous()
    return bt


def rows_nld(x):
    """[B, M, N] -> contiguous bf16 tensor and (rows, N)."""
    x = x.to(BF16).contiguous()
    return x, x.numel() // x.shape[-1], x.shape[-1]


def scale_vec(s, n):
    s = s.to(BF16).reshape(-1).contiguous()
    if s.numel() != n:
        raise ValueError("per-channel scale with %d entries for %d channels" % (s.numel(), n))
    return s


def check_fused_args(q_bit, n, r, *tensors):
    require_cuda(*tensors)
    if q_bit not in (2, 4, 8):
        raise ValueError("quantize_bit must be 2, 4 or 8")
    if n % 32 != 0:
        raise ValueError("N must be a multiple of 32")
    if r != 16:
        raise ValueError("LoRA rank must be 16")
