"""GROUP-mode quantizer oracle (test infrastructure; see package docstring).

GROUP mode has no counterpart in the reference: the reference computes one
scale per hidden column from batch sample 0 (compress_function.py:45-59).
This mode applies the same min/max scale + zero-point arithmetic
(compress_function.py:62-77; compress_function_kernel.py:279-299, 376-387) to
every 64-wide group along the last dimension, with the statistics taken from
the group itself.  This file is the specification; **parity unpinned**.

Definition, per group g of 64 consecutive values of one row (bf16 in):
  mn, mx   = min, max of the group
  s        = bf16( f32( bf16(mx - mn) ) / (2^q - 1) );   s = bf16(1e-3) if s == 0
  z        = clamp( -roundf( f32(mn) / f32(s) ) - 2^(q-1), -128, 127 )   (int8)
  code     = clamp( roundf( f32(x) / f32(s) + z ), -2^(q-1), 2^(q-1)-1 ) + 2^(q-1)
  x_hat    = bf16( bf16( bf16(code - 2^(q-1)) - z ) * s )
with fp32 IEEE division, roundf = halves away from zero, and the reference's
interleaved 32-column byte layout for the codes.
"""
import torch
from .quant import roundf_half_away, ref_pack, ref_unpack

__all__ = ["GROUP", "group_stats", "group_quant_codes", "group_compress",
           "group_decompress"]

GROUP = 64
BF16 = torch.bfloat16


def group_stats(x: torch.Tensor, q_bit: int):
    """Per-group scale (bf16) and zero point (int8) of x[..., N]."""
    *lead, n = x.shape
    assert n % GROUP == 0
    xg = x.to(BF16).reshape(*lead, n // GROUP, GROUP)
    mx = xg.max(dim=-1).values
    mn = xg.min(dim=-1).values
    s = ((mx - mn).to(BF16).float() / float(2 ** q_bit - 1)).to(BF16)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=BF16), s)
    half = 2 ** (q_bit - 1)
    z = (-roundf_half_away(mn.float() / s.float()) - half).clamp(-128, 127)
    return s, z.to(torch.int8)


def group_quant_codes(x, s, z, q_bit: int) -> torch.Tensor:
    *lead, n = x.shape
    xg = x.to(BF16).float().reshape(*lead, n // GROUP, GROUP)
    r = xg / s.float().unsqueeze(-1) + z.float().unsqueeze(-1)
    half = 2 ** (q_bit - 1)
    c = roundf_half_away(r).clamp(-half, half - 1) + half
    return c.to(torch.uint8).reshape(*lead, n)


def group_compress(x, q_bit: int):
    """-> (packed uint8 [..., N/epp], scale bf16 [..., N/64], zp int8 [..., N/64])."""
    s, z = group_stats(x, q_bit)
    return ref_pack(group_quant_codes(x, s, z, q_bit), q_bit), s, z


def group_decompress(packed, s, z, q_bit: int) -> torch.Tensor:
    codes = ref_unpack(packed, q_bit)
    *lead, n = codes.shape
    half = 2 ** (q_bit - 1)
    v = (codes.float().to(BF16) - half).to(BF16).reshape(*lead, n // GROUP, GROUP)
    v = (v - z.to(BF16).unsqueeze(-1)).to(BF16)
    return (v * s.to(BF16).unsqueeze(-1)).to(BF16).reshape(*lead, n)
