"""GROUP-mode quantizer oracle (test infrastructure; see package docstring).

GROUP mode has no counterpart in the reference: the reference computes one scale per
hidden column from batch sample 0 (compress_function.py:45-59).  This mode takes scale
and zero point from every 64-wide group of a row, in the spirit of the reference's
zero-point variant (compress_function.py:62-77; compress_function_kernel.py:279-299,
376-387) but with arithmetic chosen so that a GPU can do it in one pass at memory speed:
a reciprocal multiply instead of a divide and round-half-to-even (``torch.round``)
instead of ``roundf``.  This file is the specification; **parity unpinned**.

Definition, per group of 64 consecutive values of one row (bf16 in; fp32 arithmetic, one
rounding per operation; fma = fused multiply-add with a single rounding):
  mn, mx  = min, max of the group
  d       = bf16(mx - mn)
  il      = 1 / levels,  levels = 2^q - 1
  s       = bf16(d * il);   s = bf16(1e-3) if s == 0
  rc      = 1 / s
  z       = clamp( rint(clamp(-mn * rc, -300, 300)) - 2^(q-1), -128, 127 )      (int8)
  u       = min(max( fma(x, rc * il, (z + 2^(q-1)) * il), 0), 1)                 (NaN -> 0)
  code    = rint( u * levels )            (exact product, then half to even; unsigned code)
  x_hat   = bf16( (code - 2^(q-1) - z) * s )
rint = round half to even.  The codes use the reference's interleaved 32-column bytes.
On the GPU the two per-element steps are one saturating fma and one fma that adds 2^23.
"""
import fractions

import torch
from .quant import ref_pack, ref_unpack

__all__ = ["GROUP", "group_stats", "group_quant_codes", "group_compress",
           "group_decompress", "fma32", "group_compress_divide_roundf", "group_decompress_divide_roundf"]

GROUP = 64
BF16 = torch.bfloat16
F32 = torch.float32


def fma32(a, b, c):
    """fp32 fused multiply-add of float32 tensors whose product a*b is exact in fp64 (one
    factor has at most 29 significant bits).  The fp64 sum is checked for exactness with
    the TwoSum error term; the rare inexact elements are redone in rational arithmetic."""
    a, b, c = torch.broadcast_tensors(a.to(F32), b.to(F32), c.to(F32))
    p = a.double() * b.double()
    cd = c.double()
    s = p + cd
    bb = s - p
    err = (p - (s - bb)) + (cd - bb)
    r = s.float()
    bad = (err != 0) & torch.isfinite(s)
    if bad.any():
        r = r.clone()
        idx = bad.nonzero()
        for i in idx:
            i = tuple(i.tolist())
            exact = fractions.Fraction(float(a[i])) * fractions.Fraction(float(b[i])) + fractions.Fraction(float(c[i]))
            lo = torch.tensor(float(s[i]), dtype=torch.float64).float()
            # candidates: the fp32 neighbours of the fp64 sum; pick the nearest to the exact value, ties to even
            cands = {float(lo), float(torch.nextafter(lo, torch.tensor(float("inf")))),
                     float(torch.nextafter(lo, torch.tensor(float("-inf"))))}
            best = sorted(cands, key=lambda v: (abs(fractions.Fraction(v) - exact),
                                                torch.tensor(v, dtype=F32).view(torch.int32).item() & 1))[0]
            r[i] = best
    return r


def _il(q_bit):
    return torch.tensor(1.0, dtype=F32) / float(2 ** q_bit - 1)


def group_stats(x: torch.Tensor, q_bit: int):
    """Per-group scale (bf16) and zero point (int8) of x[..., N]."""
    *lead, n = x.shape
    assert n % GROUP == 0
    xg = x.to(BF16).reshape(*lead, n // GROUP, GROUP)
    mx = xg.max(dim=-1).values.float()
    mn = xg.min(dim=-1).values.float()
    d = (mx - mn).to(BF16).float()
    s = (d * _il(q_bit)).to(BF16)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=BF16), s)
    rc = 1.0 / s.float()
    half = 2 ** (q_bit - 1)
    z = (torch.round((-mn * rc).clamp(-300, 300)) - half).clamp(-128, 127)
    return s, z.to(torch.int8)


def group_quant_codes(x, s, z, q_bit: int) -> torch.Tensor:
    *lead, n = x.shape
    xg = x.to(BF16).float().reshape(*lead, n // GROUP, GROUP)
    half = 2 ** (q_bit - 1)
    levels = float(2 ** q_bit - 1)
    il = _il(q_bit)
    rcl = ((1.0 / s.float()) * il).unsqueeze(-1)
    zcl = ((z.float() + half) * il).unsqueeze(-1)
    u = torch.nan_to_num(fma32(xg, rcl, zcl), nan=0.0).clamp(0, 1)
    c = torch.round(u.double() * levels)
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


# ---- the same mode stated with the reference's zero-point arithmetic (comparison only) ----
# Applying compress_function.py:62-77 and compress_function_kernel.py:279-299, 376-387 literally to a 64-wide
# group gives: an fp32 IEEE divide, C roundf (halves away from zero), bf16 rounding after every step of the
# de-quantizer.  The specification above replaced the divide by a reciprocal multiply, roundf by round-half-
# to-even and the clamp by a saturating fma (two FMA-pipe instructions per element on the GPU instead of a
# division, two min/max and a conversion).  These two functions keep the literal form so that the difference
# between the two definitions can be measured (tests/test_oracle_golden.py).

def group_compress_divide_roundf(x, q_bit: int):
    from .quant import roundf_half_away
    *lead, n = x.shape
    xg = x.to(BF16).reshape(*lead, n // GROUP, GROUP)
    mx = xg.max(dim=-1).values
    mn = xg.min(dim=-1).values
    s = ((mx - mn).to(BF16).float() / float(2 ** q_bit - 1)).to(BF16)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=BF16), s)
    half = 2 ** (q_bit - 1)
    z = (-roundf_half_away(mn.float() / s.float()) - half).clamp(-128, 127)
    r = xg.float() / s.float().unsqueeze(-1) + z.unsqueeze(-1)
    c = (roundf_half_away(r).clamp(-half, half - 1) + half).to(torch.uint8).reshape(*lead, n)
    return ref_pack(c, q_bit), s, z.to(torch.int8)


def group_decompress_divide_roundf(packed, s, z, q_bit: int):
    codes = ref_unpack(packed, q_bit)
    *lead, n = codes.shape
    half = 2 ** (q_bit - 1)
    v = (codes.float().to(BF16) - half).to(BF16).reshape(*lead, n // GROUP, GROUP)
    v = (v - z.to(BF16).unsqueeze(-1)).to(BF16)
    return (v * s.to(BF16).unsqueeze(-1)).to(BF16).reshape(*lead, n)
