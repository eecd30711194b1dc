"""Attention-map save/restore oracle (test infrastructure; see package docstring).

REF mode restates the reference's global-threshold prune
(compress_function.py:30-32, 309-317, 373-379).  TOPK mode (per-row top-k plus
a 64-wide grouped remainder) has no reference counterpart; its definition
lives here: **parity unpinned** for TOPK.
"""
import torch
from .group import group_compress, group_decompress

__all__ = ["ref_softmax_threshold", "ref_softmax_prune", "ref_softmax_restore",
           "topk_select", "topk_compress", "topk_decompress"]

BF16 = torch.bfloat16


def ref_softmax_threshold(x: torch.Tensor, outlier_ratio: float) -> torch.Tensor:
    """``get_statistics_softmax`` (compress_function.py:30-32): the
    int(numel*(1-ratio))-th smallest value of the flattened map, fp32 scalar."""
    return torch.kthvalue(x.float().flatten(), int(x.numel() * (1 - outlier_ratio))).values


def ref_softmax_prune(x: torch.Tensor, thr):
    """``compression_softmax`` (compress_function.py:309-313): keep x > thr,
    COO of the flattened tensor.  The comparison of a bf16 tensor with a 0-dim
    fp32 tensor is carried out in bf16, i.e. against bf16(thr); ``to_sparse``
    drops exact zeros.  -> (indices int64 [nnz] ascending, values bf16 [nnz])."""
    xf = x.to(BF16).flatten()
    t = torch.as_tensor(thr, dtype=torch.float32).to(BF16)
    keep = (xf > t) & (xf != 0)
    idx = torch.nonzero(keep).flatten().to(torch.int64)
    return idx, xf[idx]


def ref_softmax_restore(idx, val, shape) -> torch.Tensor:
    """``to_dense().reshape(shape)``
    (fused_llama_layer_intra_inter_full_fuse.py:414-415)."""
    out = torch.zeros(int(torch.tensor(shape).prod()), dtype=BF16, device=val.device)
    out[idx] = val
    return out.reshape(shape)


def topk_select(x2: torch.Tensor, k: int) -> torch.Tensor:
    """Per row of x2 [R, S]: the columns of the k largest magnitudes, equal
    magnitudes resolved towards the lower column, returned in ascending column
    order.  int64 [R, k]."""
    mag = x2.to(BF16).abs().float()
    order = torch.sort(mag, dim=-1, descending=True, stable=True).indices[:, :k]
    return torch.sort(order, dim=-1).values


def topk_compress(x: torch.Tensor, outlier_ratio: float, q_bit: int):
    """TOPK mode.  x [..., S] -> (vals bf16 [R,k], cols int64 [R,k],
    packed uint8 [R, S/epp], scale bf16 [R, S/64], zp int8 [R, S/64]) with
    R = prod(leading dims), k = int(S*ratio).  The selected positions are
    replaced by zero before the grouped statistics and quantization."""
    s_len = x.shape[-1]
    x2 = x.to(BF16).reshape(-1, s_len)
    k = int(s_len * outlier_ratio)
    cols = topk_select(x2, k)
    vals = torch.gather(x2, 1, cols)
    rest = x2.clone()
    rest.scatter_(1, cols, torch.zeros_like(vals))
    packed, s, z = group_compress(rest, q_bit)
    return vals, cols, packed, s, z


def topk_decompress(vals, cols, packed, s, z, q_bit: int, shape) -> torch.Tensor:
    x2 = group_decompress(packed, s, z, q_bit)
    x2.scatter_(1, cols.to(torch.int64), vals)
    return x2.reshape(shape)
