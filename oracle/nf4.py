"""CPU restatement of 4-bit block-wise weight storage (test infrastructure only).

The format is the one bitsandbytes 0.43.2 (requirements.txt:3 of the reference) publishes for its 4-bit weights and
that the reference reads through ``BF.dequantize_nf4(w, quant_state)`` (models/utils/compute_utils.py:19, 29):
two codes per byte with the high nibble first, a 16-entry code table, one fp32 absolute maximum per block of
``blocksize`` consecutive elements, optionally stored as 8-bit codes themselves ("double quantization":
``absmax = table256[code] * absmax2[block // blocksize2] + offset``).  The library is absent from this build, so
parity with it is UNPINNED; the functions below pin the CUDA de-quantizer to this statement of the format and
produce test weights.  The quantizer here (nearest table entry) exists only to make such weights.
"""
import types

import torch


def normal_float_table(levels=16):
    """A 16-level table in the manner of the "normal float" type of the QLoRA paper: quantiles of a standard normal,
    eight levels for the negative half, a zero and seven for the positive half, scaled to [-1, 1]."""
    from scipy.stats import norm
    offset = 0.9677083
    pos = norm.ppf(torch.linspace(offset, 0.5, levels // 2 + 1)[:-1].double().numpy()).tolist()
    neg = (-norm.ppf(torch.linspace(offset, 0.5, levels // 2)[:-1].double().numpy())).tolist()
    vals = torch.tensor(sorted(pos + [0.0] + neg), dtype=torch.float64)
    return (vals / vals.abs().max()).float()


def byte_table():
    """A monotone 256-entry table on [-1, 1] for the 8-bit codes of the block maxima (denser near zero)."""
    t = torch.linspace(-1, 1, 256, dtype=torch.float64)
    return (t.sign() * t.abs() ** 2).float()


def _nearest(table, v):
    return (v.reshape(-1, 1) - table.reshape(1, -1)).abs().argmin(dim=1)


def quantize_4bit(w, table, blocksize=64, nested=False, blocksize2=256):
    """-> (packed uint8 [numel/2, 1], quant state with the attribute names of the library's ``QuantState``)."""
    flat = w.detach().float().reshape(-1)
    n = flat.numel()
    assert n % 2 == 0
    nb = (n + blocksize - 1) // blocksize
    padded = torch.zeros(nb * blocksize)
    padded[:n] = flat
    blocks = padded.view(nb, blocksize)
    absmax = blocks.abs().amax(dim=1).clamp(min=1e-12)
    codes = _nearest(table, (blocks / absmax[:, None]).reshape(-1))[:n].to(torch.uint8)
    packed = ((codes[0::2] << 4) | codes[1::2]).reshape(-1, 1)
    qs = types.SimpleNamespace(shape=torch.Size(w.shape), code=table.clone(), blocksize=blocksize, dtype=torch.bfloat16,
                               quant_type="nf4", nested=False, absmax=absmax, state2=None, offset=None)
    if nested:
        offset = absmax.mean()
        a = absmax - offset
        nb2 = (nb + blocksize2 - 1) // blocksize2
        pa = torch.zeros(nb2 * blocksize2)
        pa[:nb] = a
        absmax2 = pa.view(nb2, blocksize2).abs().amax(dim=1).clamp(min=1e-12)
        t256 = byte_table()
        acodes = _nearest(t256, (pa.view(nb2, blocksize2) / absmax2[:, None]).reshape(-1))[:nb].to(torch.uint8)
        qs.nested = True
        qs.absmax = acodes
        qs.offset = offset
        qs.state2 = types.SimpleNamespace(code=t256, absmax=absmax2, blocksize=blocksize2)
    return packed, qs


def block_maxima(qs):
    """fp32 absolute maxima of the blocks (two fp32 operations in the nested case: product, then the offset)."""
    if not qs.nested:
        return qs.absmax.float()
    s2 = qs.state2
    idx = torch.arange(qs.absmax.numel()) // s2.blocksize
    return s2.code.float()[qs.absmax.long()] * s2.absmax.float()[idx] + float(qs.offset)


def ref_dequantize_4bit(packed, qs):
    """-> bf16 tensor of shape ``qs.shape``: table[code] * absmax[element // blocksize] in fp32, one rounding."""
    n = 1
    for d in qs.shape:
        n *= int(d)
    b = packed.reshape(-1).long()
    codes = torch.stack((b >> 4, b & 15), dim=1).reshape(-1)[:n]
    scale = block_maxima(qs)[torch.arange(n) // qs.blocksize]
    return (qs.code.float()[codes] * scale).to(torch.bfloat16).reshape(tuple(qs.shape))
