"""The C-ABI library loads on a machine without a GPU and exports everything the header
declares; argument validation answers without touching a device."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(hyc_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    from hyc_lora_release_b200 import _lib
    declared = _declared()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(_lib.lib, name), name
    # every declared entry point has a ctypes signature on the Python side
    assert declared <= set(_lib.SIGNATURES), declared - set(_lib.SIGNATURES)


def test_argument_validation_without_device():
    from hyc_lora_release_b200._lib import lib
    assert lib.hyc_quant_pack(None, 4, 64, 64, None, None, None, 0, None, None, 4, None) == -1
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 15) & ~15)
    assert lib.hyc_quant_pack(p, 4, 64, 64, p, None, None, 0, p, None, 3, None) == -2      # q_bit
    assert lib.hyc_quant_pack(p, 4, 48, 48, p, None, None, 0, p, None, 4, None) == -3      # N % 32
    assert lib.hyc_quant_pack(p, 4, 64, 68, p, None, None, 0, p, None, 4, None) == -4      # row stride
    assert lib.hyc_quant_pack(p, 0, 64, 64, p, None, None, 0, p, None, 4, None) == 0       # empty input
    assert lib.hyc_softmax_topk_compress(p, 1, 8192, 10, p, p, p, p, p, 4, None) == -3     # S too large
    assert lib.hyc_fused_lora_silu_hadamard_fwd(p, p, p, p, p, p, p, p, p, p, p, 16, 64, 8, 4, None) == -8
    assert lib.hyc_softmax_prune_workspace_bytes(4096 * 3 + 1) == 8 * 5
    # rotary embedding and scale + mask + softmax: geometry and alignment are checked before any launch
    assert lib.hyc_rope(None, 128, p, 128, p, p, 64, 0, 4, 4, 1, 128, 0, None) == -1
    assert lib.hyc_rope(p, 128, p, 128, p, p, 64, 0, 4, 4, 1, 24, 0, None) == -3           # head_dim % 16
    assert lib.hyc_rope(p, 64, p, 128, p, p, 64, 0, 4, 4, 1, 128, 0, None) == -3           # row stride < heads * head_dim
    assert lib.hyc_rope(p, 132, p, 132, p, p, 64, 0, 4, 4, 1, 128, 0, None) == -4          # stride not a multiple of 8
    assert lib.hyc_rope(p, 128, p, 128, p, p, 64, 0, 0, 4, 1, 128, 0, None) == 0           # no rows
    assert lib.hyc_softmax_fwd_scale_mask(p, 1.0, None, 0, 0, 0, 1, 4, p, 4, 60, None) == -3       # S % 8
    assert lib.hyc_softmax_fwd_scale_mask(p, 1.0, p, 0, 0, 68, 1, 4, p, 4, 64, None) == -4         # mask row stride
    assert lib.hyc_softmax_fwd_scale_mask(p, 1.0, None, 0, 0, 0, 1, 4, p, 0, 64, None) == 0        # no rows
    assert lib.hyc_softmax_bwd(p, p, None, 4, 64, 1.0, None) == -1
    assert b"q_bit" in lib.hyc_strerror(-2)


def test_operators_refuse_cpu_tensors():
    import pytest
    import torch
    from hyc_lora_release_b200.operators import compress_function as cf
    with pytest.raises(RuntimeError):
        cf.compression_quantization(torch.zeros(1, 32, 32), torch.ones(1, 32), 4)
    with pytest.raises(RuntimeError):
        cf.get_statistics_only_quant(torch.zeros(1, 32, 32), 4, "per-channel")
