"""4-bit block-wise frozen weights: the CPU statement of the storage format (oracle/nf4.py), the CUDA de-quantizer
against it bit for bit, and the fused layer driven with such weights against the same layer driven with the
de-quantized matrices.  (The library whose format this is, bitsandbytes 0.43.2, is not present: parity with it is
unpinned, see oracle/nf4.py.)"""
import types

import pytest
import torch

from oracle import nf4 as onf4

BF16 = torch.bfloat16


def test_format_statement_round_trip():
    """Nibble order, block maxima and the nested form, on the CPU."""
    table = onf4.normal_float_table()
    assert table.numel() == 16 and float(table[0]) == -1.0 and float(table[-1]) == 1.0 and float(table[7]) == 0.0
    assert bool((table[1:] > table[:-1]).all())
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(48, 64, generator=g) * 0.02).to(BF16)
    packed, qs = onf4.quantize_4bit(w, table, blocksize=64)
    assert packed.shape == (48 * 64 // 2, 1) and packed.dtype == torch.uint8 and qs.absmax.numel() == 48
    # element 0 sits in the HIGH nibble of byte 0
    first = int(packed[0, 0])
    blk0 = float(qs.absmax[0])
    assert abs(float(table[first >> 4]) * blk0 - float(w.reshape(-1)[0])) <= 0.2 * blk0
    back = onf4.ref_dequantize_4bit(packed, qs)
    assert back.shape == w.shape and back.dtype == BF16
    err = (back.float() - w.float()).abs().max() / w.float().abs().max()
    assert float(err) < 0.2                      # half the widest gap of the table, relative to a block maximum
    # exact at the block maxima and at zero
    z = torch.zeros(2, 64); z[0, 5] = 1.5; z[1, 9] = -0.25
    pz, qz = onf4.quantize_4bit(z.to(BF16), table, blocksize=64)
    bz = onf4.ref_dequantize_4bit(pz, qz).float()
    assert float(bz[0, 5]) == 1.5 and float(bz[1, 9]) == -0.25 and float(bz.abs().sum()) == 1.75
    # nested: the maxima come back within the resolution of the 8-bit table
    pn, qn = onf4.quantize_4bit(w, table, blocksize=64, nested=True, blocksize2=16)
    assert qn.absmax.dtype == torch.uint8 and qn.state2.absmax.numel() == 3
    m = onf4.block_maxima(qn)
    assert float((m - qs.absmax).abs().max()) < 0.05 * float(qs.absmax.max())


@pytest.mark.gpu
@pytest.mark.parametrize("shape,blocksize,nested", [((64, 64), 64, False), ((256, 1024), 64, False), ((300, 130), 64, False),
                                                   ((128, 512), 128, True), ((96, 4096), 64, True), ((7, 6), 2, False)])
def test_dequantizer_matches_the_format_statement(shape, blocksize, nested):
    from hyc_lora_release_b200 import nf4
    table = onf4.normal_float_table()
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    w = (torch.randn(*shape, generator=g) * 0.03).to(BF16)
    packed, qs = onf4.quantize_4bit(w, table, blocksize=blocksize, nested=nested, blocksize2=32)
    want = onf4.ref_dequantize_4bit(packed, qs)
    got = nf4.dequantize_nf4(packed.cuda(), qs)
    assert got.shape == tuple(shape) and got.dtype == BF16
    assert torch.equal(got.cpu(), want)
    # a parameter that carries its quant state, as the reference's modules hold it
    p = torch.nn.Parameter(packed.cuda(), requires_grad=False)
    p.quant_state = qs
    assert nf4.is_quantized(p) and torch.equal(nf4.dequantize_nf4(p).cpu(), want)


@pytest.mark.gpu
def test_layer_with_4bit_frozen_weights():
    """The layer module with 4-bit frozen weights gives bit for bit what it gives with the de-quantized matrices
    (the same kernels run on the same values), and it does not keep the bf16 matrices between the passes."""
    from hyc_lora_release_b200 import nf4
    from hyc_lora_release_b200.layer import FusedLlamaLayerIntraInterFullFuse
    from test_gpu_layer import layer_problem, _Holder, _base
    DEV = "cuda"
    g = torch.Generator().manual_seed(77)
    B, M, heads, d, kv, I, q = 2, 128, 4, 128, 2, 1024, 4
    H = heads * d
    x, p, cos, sin, mask = layer_problem(g, B, M, H, heads, d, kv, I)
    table = onf4.normal_float_table()
    cfg = types.SimpleNamespace(use_hyclora=True, iteration_threshold=5, softmax_outlier_ratio=0.05,
                                layernorm_outlier_ratio=0.01, q_bit=q, softmax_map_mode="prune")
    n1 = torch.nn.Parameter(p["norm_w1"].to(DEV), requires_grad=False)
    n2 = torch.nn.Parameter(p["norm_w2"].to(DEV), requires_grad=False)
    gy = torch.randn(B, M, H, generator=g).to(BF16).to(DEV)
    names = ("q", "k", "v", "o", "gate", "up", "down")
    quant = {}
    for i, n in enumerate(names):
        w = p["w" + n].t().contiguous()                       # [out, in]
        quant[n] = onf4.quantize_4bit(w, table, blocksize=64, nested=(i % 2 == 1), blocksize2=64)

    def run(four_bit):
        mods = {}
        for n in names:
            packed, qs = quant[n]
            if four_bit:
                base = torch.nn.Module()
                base.weight = torch.nn.Parameter(packed.to(DEV), requires_grad=False)
                base.weight.quant_state = qs
                base.bias = None
            else:
                base = _base(onf4.ref_dequantize_4bit(packed, qs).to(DEV))
            mods[n] = (base, _Holder(p["a" + n].t().to(DEV)), _Holder(p["b" + n].t().to(DEV)))
        layer = FusedLlamaLayerIntraInterFullFuse()
        layer.set_hyclora_config(cfg)
        layer.check_kernel_status = True
        outs = []
        for it in range(7):
            xin = x.to(DEV).requires_grad_(True)
            args = [xin, n1, None, cos.to(DEV), sin.to(DEV)]
            for n in ("q", "k", "v", "o"):
                args += list(mods[n])
            args += [n2, None]
            for n in ("gate", "up", "down"):
                args += list(mods[n])
            y = layer(*args, mask.to(DEV), heads, d, kv)
            for m3 in mods.values():
                m3[1].default.weight.grad = None
                m3[2].default.weight.grad = None
            y.backward(gy)
            outs.append((y.detach().clone(), xin.grad.clone(), [m3[k].default.weight.grad.clone() for m3 in mods.values() for k in (1, 2)]))
        return layer, outs

    layer4, o4 = run(True)
    layer16, o16 = run(False)
    for (y4, gx4, gl4), (y16, gx16, gl16) in zip(o4, o16):
        assert torch.equal(y4, y16) and torch.equal(gx4, gx16)
        assert all(torch.equal(a, b) for a, b in zip(gl4, gl16))
    aw, mw, _ = layer4._weights[1:]
    assert isinstance(aw.wq, nf4.QuantizedWeight) and isinstance(mw.wd, nf4.QuantizedWeight)
    assert "_pad" in vars(aw) and "_pad" in vars(mw)          # the scratch of the passes came back to the records
