"""GROUP-mode quantizer oracle (test infrastructure; see package docstring).

GROUP mode has no counterpart in the reference: the reference computes one scale per
hidden column from batch sample 0 (compress_function.py:45-59).  This mode takes scale
and zero point from every 64-wide group of a row, in the spirit of the reference's
zero-point variant (compress_function.py:62-77; compress_function_kernel.py:279-299,
376-387) but with arithmetic chosen so that a GPU can do it in one pass at memory speed:
a reciprocal multiply instead of a divide and round-half-to-even (``torch.round``)
instead of ``roundf``.  This file is the specification; **parity unpinned**.

Definition, per group of 64 consecutive values of one row (bf16 in, all arithmetic fp32
with one rounding per operation unless a bf16 rounding is written out):
  mn, mx  = min, max of the group
  d       = bf16(mx - mn)
  s       = bf16(d * (1 / levels)),  levels = 2^q - 1;   s = bf16(1e-3) if s == 0
  rc      = 1 / s
  z       = clamp( rint(clamp(-mn * rc, -300, 300)) - 2^(q-1), -128, 127 )      (int8)
  code    = rint( clamp( x * rc + (z + 2^(q-1)), 0, levels ) )                   (unsigned)
  x_hat   = bf16( (code - 2^(q-1) - z) * s )
rint = round half to even.  The codes use the reference's interleaved 32-column bytes.
"""
import torch
from .quant import ref_pack, ref_unpack

__all__ = ["GROUP", "group_stats", "group_quant_codes", "group_compress",
           "group_decompress"]

GROUP = 64
BF16 = torch.bfloat16
F32 = torch.float32


def group_stats(x: torch.Tensor, q_bit: int):
    """Per-group scale (bf16) and zero point (int8) of x[..., N]."""
    *lead, n = x.shape
    assert n % GROUP == 0
    xg = x.to(BF16).reshape(*lead, n // GROUP, GROUP)
    mx = xg.max(dim=-1).values.float()
    mn = xg.min(dim=-1).values.float()
    inv_levels = torch.tensor(1.0, dtype=F32) / float(2 ** q_bit - 1)
    d = (mx - mn).to(BF16).float()
    s = (d * inv_levels).to(BF16)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=BF16), s)
    rc = 1.0 / s.float()
    half = 2 ** (q_bit - 1)
    z = (torch.round((-mn * rc).clamp(-300, 300)) - half).clamp(-128, 127)
    return s, z.to(torch.int8)


def group_quant_codes(x, s, z, q_bit: int) -> torch.Tensor:
    *lead, n = x.shape
    xg = x.to(BF16).float().reshape(*lead, n // GROUP, GROUP)
    rc = (1.0 / s.float()).unsqueeze(-1)
    half = 2 ** (q_bit - 1)
    u = xg * rc + (z.float() + half).unsqueeze(-1)
    c = torch.round(torch.nan_to_num(u, nan=0.0).clamp(0, 2 ** q_bit - 1))
    return c.to(torch.uint8).reshape(*lead, n)


def group_compress(x, q_bit: int):
    """-> (packed uint8 [..., N/epp], scale bf16 [..., N/64], zp int8 [..., N/64])."""
    s, z = group_stats(x, q_bit)
    return ref_pack(group_quant_codes(x, s, z, q_bit), q_bit), s, z


def group_decompress(packed, s, z, q_bit: int) -> torch.Tensor:
    codes = ref_unpack(packed, q_bit)
    *lead, n = codes.shape
    half = 2 ** (q_bit - 1)
    v = (codes.float() - half).reshape(*lead, n // GROUP, GROUP) - z.float().unsqueeze(-1)
    return (v * s.float().unsqueeze(-1)).to(BF16).reshape(*lead, n)
