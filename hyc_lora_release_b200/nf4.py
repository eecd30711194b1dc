"""Frozen weights kept as 4-bit block-wise codes (the storage format of bitsandbytes 0.43.2).

The reference keeps its frozen projection weights as ``bitsandbytes`` ``Params4bit`` tensors and calls
``BF.dequantize_nf4(w, w.quant_state)`` before every frozen matmul, forward and backward
(models/utils/compute_utils.py:19, 29; models/llama/fused_llama_layer_intra_inter_full_fuse.py:218-219, 359, 367,
379).  That library is not part of this build.  This module reads the same objects by their attribute names and
de-quantizes them with a kernel of this package (``csrc/nf4.cu``):

  weight            uint8 tensor with two codes per byte, the high nibble first (``Params4bit.data``, [numel/2, 1])
  quant_state.shape       shape of the de-quantized weight ([out, in])
  quant_state.code        the 16-entry table of the 4-bit type (NF4 or FP4), fp32
  quant_state.blocksize   elements per absmax block
  quant_state.absmax      fp32 block maxima, or their 8-bit codes when ``quant_state.nested``
  quant_state.state2      (nested only) ``.code`` 256-entry table, ``.absmax`` fp32, ``.blocksize``
  quant_state.offset      (nested only) the fp32 scalar added back to the de-quantized maxima

Anything else about the library (its quantizer, its serialisation) is out of scope.  Parity is unpinned: there is
no copy of the library here to compare with; the tests pin the kernel to ``oracle/nf4.py``, a restatement of the
format above.
"""
import torch

from ._lib import check, lib, ptr, require_cuda, stream_of

BF16 = torch.bfloat16


def is_quantized(weight):
    """True for a weight that carries a 4-bit quant state (``Params4bit`` or anything shaped like it)."""
    return getattr(weight, "quant_state", None) is not None


def dequantize_nf4(weight, quant_state=None):
    """-> bf16 tensor of shape ``quant_state.shape`` (the reference's ``BF.dequantize_nf4(w, quant_state)``)."""
    return QuantizedWeight(weight, quant_state).dequantize()


class QuantizedWeight:
    """A frozen 4-bit weight as the fused layer holds it between steps: the packed codes and the tables of their quant
    state, moved to the weight's device once.  ``dequantize()`` builds the bf16 matrix for the duration of one pass,
    as the reference does."""

    def __init__(self, weight, quant_state=None):
        qs = quant_state if quant_state is not None else weight.quant_state
        missing = [a for a in ("shape", "code", "blocksize", "absmax") if not hasattr(qs, a)]
        if missing:
            raise NotImplementedError("unrecognised quant state (no %s): 4-bit block-wise weights in the storage format "
                                      "of bitsandbytes are what this layer reads" % ", ".join(missing))
        packed = weight.data if isinstance(weight, torch.nn.Parameter) else weight
        require_cuda(packed)
        if packed.dtype != torch.uint8:
            raise TypeError("a 4-bit weight is a uint8 tensor of packed codes (got %s)" % packed.dtype)
        self.quant_state = qs
        self.packed = packed.contiguous()
        self.shape = tuple(int(d) for d in qs.shape)
        self.device = dev = packed.device
        self.numel = 1
        for d in self.shape:
            self.numel *= d
        if self.packed.numel() * 2 < self.numel:
            raise ValueError("%d packed bytes cannot hold %d 4-bit codes" % (self.packed.numel(), self.numel))
        if getattr(qs, "dtype", BF16) != BF16:
            raise NotImplementedError("4-bit weights de-quantize to bf16 here (quant state says %s)" % qs.dtype)
        self.code = qs.code.to(device=dev, dtype=torch.float32).contiguous()
        if self.code.numel() != 16:
            raise NotImplementedError("the code table of a 4-bit weight has 16 entries (got %d)" % self.code.numel())
        self.blocksize = int(qs.blocksize)
        self.nested = bool(getattr(qs, "nested", False))
        if self.nested:
            s2 = qs.state2
            self.absmax = qs.absmax.to(dev).contiguous()
            if self.absmax.dtype != torch.uint8:
                raise TypeError("a nested quant state keeps its block maxima as uint8 codes")
            self.code2 = s2.code.to(device=dev, dtype=torch.float32).contiguous()
            self.absmax2 = s2.absmax.to(device=dev, dtype=torch.float32).contiguous()
            self.blocksize2 = int(s2.blocksize)
            self.offset = float(qs.offset)
        else:
            self.absmax = qs.absmax.to(device=dev, dtype=torch.float32).contiguous()

    def dequantize(self):
        out = torch.empty(self.shape, dtype=BF16, device=self.device)
        if self.nested:
            check(lib.hyc_dequant_nf4(ptr(self.packed), ptr(self.code), None, ptr(self.absmax), ptr(self.code2),
                                      ptr(self.absmax2), self.blocksize2, self.offset, self.numel, self.blocksize,
                                      ptr(out), stream_of(self.packed)), "hyc_dequant_nf4")
        else:
            check(lib.hyc_dequant_nf4(ptr(self.packed), ptr(self.code), ptr(self.absmax), None, None, None, 1, 0.0,
                                      self.numel, self.blocksize, ptr(out), stream_of(self.packed)), "hyc_dequant_nf4")
        return out


_CACHE_ATTRS = ("_pad", "_pad_key", "_gm64", "_gmq")      # what AttnWeights / MLPWeights keep between steps


def materialize(record):
    """A weights record (``AttnWeights`` / ``MLPWeights``) whose 4-bit entries are de-quantized to bf16 for one pass;
    the record itself when it holds none.  The copy shares the record's LoRA factors and cached scratch."""
    import copy
    import dataclasses
    names = [f.name for f in dataclasses.fields(record) if isinstance(getattr(record, f.name), QuantizedWeight)]
    if not names:
        return record
    new = copy.copy(record)
    for n in names:
        setattr(new, n, getattr(record, n).dequantize())
    return new


def release(record, used):
    """After the pass: keep the scratch the pass created on the copy (padded factors, zero blocks), drop the bf16
    weights."""
    if used is record:
        return
    for a in _CACHE_ATTRS:
        if hasattr(used, a):
            setattr(record, a, getattr(used, a))
