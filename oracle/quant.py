"""REF-mode quantizer oracle (test infrastructure; see package docstring).

Restates, on CPU tensors, the per-channel quantize / pack / unpack / dequantize
arithmetic of ``operators/compress_function.py`` and
``operators/compress_function_kernel.py`` with the same rounding points.
"""
import torch

__all__ = [
    "roundf_half_away", "ref_scale_per_channel", "ref_scale_zero_point",
    "ref_channel_norm", "ref_channel_topk", "ref_statistics_channel_base",
    "ref_quant_codes", "ref_pack", "ref_unpack", "ref_dequant",
    "ref_compress", "ref_decompress",
    "ref_compress_channel_base", "ref_decompress_channel_base",
]

BF16 = torch.bfloat16


def _hidden(x):
    """4-D head layout [B,h,M,d] -> [B,M,h*d] (compress_function.py:46-48)."""
    if x.dim() == 4:
        b, h, m, d = x.shape
        x = x.permute(0, 2, 1, 3).reshape(b, m, h * d)
    return x


def roundf_half_away(r: torch.Tensor) -> torch.Tensor:
    """C ``roundf`` on an fp32 tensor: nearest integer, halves away from zero.

    The reference kernel rounds with libdevice ``round``
    (compress_function_kernel.py:103), which is ``roundf``; ``torch.round`` is
    half-to-even and is NOT what runs.  ``r - trunc(r)`` is exact in fp32, so
    this is correct even where ``floor(r + 0.5)`` would double-round.
    """
    r = r.float()
    t = torch.trunc(r)
    frac = r - t
    step = torch.where(frac.abs() >= 0.5, torch.sign(r), torch.zeros_like(r))
    return torch.where(torch.isfinite(r), t + step, r)


def ref_scale_per_channel(x: torch.Tensor, q_bit: int) -> torch.Tensor:
    """``get_statistics_only_quant(x, q_bit, 'per-channel')``
    (compress_function.py:45-59): column max - min of batch sample 0 over the
    sequence axis, divided by 2^q - 1; every step is a bf16 tensor op."""
    x0 = _hidden(x)[0]
    mx = x0.max(dim=-2, keepdim=True).values
    mn = x0.min(dim=-2, keepdim=True).values
    return ((mx - mn) / (2 ** q_bit - 1)).to(BF16)


def ref_scale_zero_point(x: torch.Tensor, q_bit: int):
    """``get_statistics_only_quant_zero_point(..., 'per-channel')``
    (compress_function.py:62-77).  The zero point uses ``torch.round``
    (half-to-even) on a bf16 quotient and is stored as int8."""
    x0 = _hidden(x)[0]
    mx = x0.max(dim=-2, keepdim=True).values
    mn = x0.min(dim=-2, keepdim=True).values
    scale = (mx - mn) / (2 ** q_bit - 1)
    zp = -torch.round(mn / scale) - (2 ** (q_bit - 1))
    return scale.to(BF16), zp.to(torch.int8)


def ref_channel_norm(x0: torch.Tensor) -> torch.Tensor:
    """Column L2 norm of sample 0, result in bf16
    (``x_[0].abs().norm(dim=-2)``, compress_function.py:86).

    Specification used by both sides: the sum of squares is taken exactly
    (fp64 holds it exactly for bf16 inputs of these lengths), square-rooted in
    fp64, rounded to fp32 and then to bf16.  ``torch.norm`` accumulates in fp32
    in an unspecified order; after the bf16 rounding the two agree (the tests
    check this on the fixtures)."""
    s = (x0.double() ** 2).sum(dim=-2)
    return s.sqrt().float().to(BF16)


def ref_channel_topk(norm: torch.Tensor, k: int) -> torch.Tensor:
    """Top-k channels by norm (compress_function.py:87).  ``torch.topk`` leaves
    the order of equal norms unspecified; the contract here is (norm
    descending, index ascending)."""
    # a stable descending sort keeps equal norms in ascending index order
    order = torch.sort(norm.float(), descending=True, stable=True).indices
    return order[:k].to(torch.int64)


def ref_statistics_channel_base(x: torch.Tensor, outlier_ratio: float, q_bit: int):
    """``get_statistics_channel_base(x, ratio, q_bit, 'per-channel')``
    (compress_function.py:80-105): outlier channel index, and the per-channel
    scale of sample 0 with those channels zeroed; zero scales become 1e-3."""
    x = _hidden(x)
    x0 = x[0].clone()
    k = int(x0.shape[-1] * outlier_ratio)
    idx = ref_channel_topk(ref_channel_norm(x0), k)
    x0[:, idx] = 0
    mx = x0.max(dim=-2, keepdim=True).values
    mn = x0.min(dim=-2, keepdim=True).values
    scale = (mx - mn) / (2 ** q_bit - 1)
    scale += (scale == 0) * 1e-3
    return idx, scale.to(BF16)


def ref_quant_codes(x, s, q_bit: int, z=None) -> torch.Tensor:
    """Codes of ``compression_quantization_kernel``
    (compress_function_kernel.py:96-110) and of its zero-point twin
    (``:279-299``): fp32 IEEE quotient of the bf16 operands (plus the zero point
    in fp32), ``roundf``, clamp to the signed range, offset to unsigned."""
    x = _hidden(x)
    r = x.to(BF16).float() / s.to(BF16).float()
    if z is not None:
        r = r + z.to(BF16).float()
    half = 2 ** (q_bit - 1)
    c = roundf_half_away(r).clamp(-half, half - 1) + half
    return c.to(torch.uint8)


def ref_pack(codes: torch.Tensor, q_bit: int) -> torch.Tensor:
    """Interleaved byte layout of the reference kernels
    (compress_function_kernel.py:78-83, 96-110): inside every 32-column block,
    byte j holds the codes of columns j, j+32/epp, j+2*32/epp, ... in ascending
    bit position (epp = 8 // q_bit codes per byte)."""
    epp = 8 // q_bit
    *lead, n = codes.shape
    assert n % 32 == 0
    cb = codes.reshape(*lead, n // 32, epp, 32 // epp).to(torch.int32)
    out = torch.zeros(*lead, n // 32, 32 // epp, dtype=torch.int32, device=codes.device)
    for i in range(epp):
        out |= cb[..., i, :] << (q_bit * i)
    return out.to(torch.uint8).reshape(*lead, n // epp)


def ref_unpack(packed: torch.Tensor, q_bit: int) -> torch.Tensor:
    """Inverse of :func:`ref_pack` (compress_function_kernel.py:193-206)."""
    epp = 8 // q_bit
    *lead, nb = packed.shape
    n = nb * epp
    pb = packed.reshape(*lead, n // 32, 32 // epp).to(torch.int32)
    mask = (1 << q_bit) - 1
    parts = [((pb >> (q_bit * i)) & mask) for i in range(epp)]
    return torch.stack(parts, dim=-2).to(torch.uint8).reshape(*lead, n)


def ref_dequant(codes, s, q_bit: int, z=None) -> torch.Tensor:
    """``decompression_dequantization_kernel``
    (compress_function_kernel.py:196-205; zero-point twin ``:376-387``):
    code -> bf16, minus 2^(q-1) in bf16, (minus zero point in bf16,) times the
    bf16 scale, bf16 result."""
    half = 2 ** (q_bit - 1)
    v = (codes.float().to(BF16) - half).to(BF16)
    if z is not None:
        v = (v - z.to(BF16)).to(BF16)
    return (v * s.to(BF16)).to(BF16)


def ref_compress(x, s, q_bit: int, z=None) -> torch.Tensor:
    """``compression_quantization`` (compress_function.py:178-210) /
    ``compression_quantization_with_zero_point`` (``:245-275``)."""
    return ref_pack(ref_quant_codes(x, s, q_bit, z), q_bit)


def ref_decompress(packed, s, q_bit: int, z=None) -> torch.Tensor:
    """``decompression_dequantization`` (compress_function.py:214-241) /
    ``..._with_zero_point`` (``:278-306``), hidden layout."""
    return ref_dequant(ref_unpack(packed, q_bit), s, q_bit, z)


def ref_compress_channel_base(x, s, idx, q_bit: int):
    """``outlier_subtraction_fuse_compression_quantization``
    (compress_function.py:111-143) without the in-place side effect: gathers
    the outlier columns, quantizes the tensor with those columns zeroed."""
    x = _hidden(x).to(BF16)
    x_outlier = x[:, :, idx].clone()
    xz = x.clone()
    xz[:, :, idx] = 0
    return x_outlier, ref_compress(xz, s, q_bit)


def ref_decompress_channel_base(packed, s, x_outlier, idx, q_bit: int):
    """``outlier_addition_fuse_decompression_dequantization``
    (compress_function.py:147-174)."""
    x = ref_decompress(packed, s, q_bit)
    x[:, :, idx] = x_outlier
    return x
