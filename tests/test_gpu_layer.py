"""Attention half and whole fused decoder layer on the GPU against the CPU oracle: rotary embedding and
scale + mask + softmax kernels, the attention block forward/backward (calibration iterations and steady state,
both forms of the saved probability map, grouped key/value heads), and the layer module through autograd.
Tolerances as for the MLP path: max |err| <= 1e-2 * max|ref| and cosine > 0.999 for activations."""
import math
import types

import pytest
import torch

import oracle
from oracle.attention import (ref_attention_block_backward, ref_attention_block_forward, ref_layer_backward,
                              ref_layer_forward, ref_rope)
from test_oracle_layer import layer_problem

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16 = torch.bfloat16


def close(a, b, rel=1e-2, cos=0.999):
    a, b = a.float().cpu().flatten(), b.float().cpu().flatten()
    scale = b.abs().max().clamp(min=1e-30)
    c = torch.nn.functional.cosine_similarity(a, b, dim=0)
    ok = bool((a - b).abs().max() <= rel * scale) and bool(c > cos)
    if not ok:
        print("max rel err %.4g (bound %g), cosine %.5f (bound %g)" % (float((a - b).abs().max() / scale), rel, float(c), cos))
    return ok


@pytest.mark.parametrize("table_dtype", [BF16, torch.float32])
@pytest.mark.parametrize("B,M,heads,d", [(2, 64, 4, 32), (1, 100, 3, 128), (3, 17, 8, 64)])
def test_rope_forward_backward(B, M, heads, d, table_dtype, golden):
    from hyc_lora_release_b200.operators import rope_kernels as rk
    g = torch.Generator().manual_seed(B * M + d)
    pos = torch.arange(M + 5, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb = torch.cat([torch.outer(pos, inv)] * 2, dim=-1)
    cos, sin = emb.cos().to(table_dtype), emb.sin().to(table_dtype)
    x = torch.randn(B, M, heads, d, generator=g).to(BF16)
    for backward in (False, True):
        ref = ref_rope(x, cos, sin, backward=backward)
        fn = rk.rope_backward if backward else rk.rope_forward
        out = fn(x.to(DEV), cos.to(DEV).unsqueeze(0), sin.to(DEV).unsqueeze(0))
        assert out.shape == x.shape
        # the kernel follows the reference's arithmetic (the dtype of the sine table, no contraction): equal bits
        assert torch.equal(out.cpu(), ref)
    # the reference's own kernel (fixture made through the Triton interpreter)
    r = golden["rope"]
    nm = "bf16" if table_dtype == BF16 else "f32"
    assert torch.equal(rk.rope_forward(r["x"].to(DEV), r["cos_" + nm].to(DEV), r["sin_" + nm].to(DEV)).cpu(), r["fwd_" + nm])
    assert torch.equal(rk.rope_backward(r["x"].to(DEV), r["cos_" + nm].to(DEV), r["sin_" + nm].to(DEV)).cpu(), r["bwd_" + nm])
    xin = x.to(DEV).clone()
    rk.rope_inplace(xin, cos.to(DEV), sin.to(DEV))
    assert torch.equal(xin, rk.rope_forward(x.to(DEV), cos.to(DEV), sin.to(DEV)))
    # head geometry and tables are checked before any launch
    with pytest.raises(Exception):
        rk.rope_forward(torch.zeros(1, 4, 2, 24, dtype=BF16, device=DEV), cos.to(DEV), sin.to(DEV))


@pytest.mark.parametrize("B,h,M,S,mask_kind", [(2, 4, 64, 64, "causal"), (1, 3, 40, 520, None), (2, 2, 33, 1024, "batch"),
                                               (1, 2, 16, 4096, "head")])
def test_softmax_forward_scale_mask(B, h, M, S, mask_kind):
    from hyc_lora_release_b200.operators.softmax_kernels import softmax_forward_scale_mask
    g = torch.Generator().manual_seed(S + M)
    sc = (torch.randn(B, h, M, S, generator=g) * 8).to(BF16)
    mask = None
    if mask_kind == "causal":
        mask = torch.full((M, S), torch.finfo(BF16).min).triu(1).to(BF16).reshape(1, 1, M, S)
    elif mask_kind == "batch":
        mask = (torch.randn(B, 1, M, S, generator=g) * 3).to(BF16)
    elif mask_kind == "head":
        mask = (torch.randn(1, h, M, S, generator=g) * 3).to(BF16)
    scale = 1.0 / math.sqrt(128)
    t = (sc.float() * scale).to(BF16)
    if mask is not None:
        t = (t + mask).to(BF16)
    ref = torch.softmax(t.float(), dim=-1)
    out = softmax_forward_scale_mask(sc.to(DEV), scale, None if mask is None else mask.to(DEV))
    assert out.dtype == BF16 and out.shape == sc.shape
    assert close(out, ref, rel=5e-3)
    assert float((out.float().sum(-1).cpu() - 1).abs().max()) < 2e-2
    sc_d = sc.to(DEV).clone()
    out2 = softmax_forward_scale_mask(sc_d, scale, None if mask is None else mask.to(DEV), inplace=True)
    assert out2.data_ptr() == sc_d.data_ptr() and torch.equal(out2, out)


def _attn_weights(p):
    from hyc_lora_release_b200.attention import AttnWeights
    t = lambda k: p[k].t().contiguous().to(DEV)
    return AttnWeights(norm_w=p["norm_w1"].to(DEV), wq=t("wq"), wk=t("wk"), wv=t("wv"), wo=t("wo"), aq=t("aq"), bq=t("bq"),
                       ak=t("ak"), bk=t("bk"), av=t("av"), bv=t("bv"), ao=t("ao"), bo=t("bo"))


def _attn_static(sv):
    c = lambda v: v.cpu().to(BF16)
    st = dict(x_idx=sv["x"]["outlier_channel_index"].cpu(), x_scale=c(sv["x"]["scale"]),
              x_norm_1_scale=c(sv["x_norm_1"]["scale"]), q_scale=c(sv["q"]["scale"]), k_scale=c(sv["k"]["scale"]),
              v_scale=c(sv["v"]["scale"]), o_scale=c(sv["o"]["scale"]))
    if sv["a"]["outlier"] is not None:
        st["a_threshold"] = sv["a"]["outlier"].cpu().float()
    return st


ATTN_ARGS = ("wq", "wk", "wv", "wo", "aq", "bq", "ak", "bk", "av", "bv", "ao", "bo")


def _flipped_codes(a, b, q):
    """Fraction of q-bit codes that differ between two packed tensors."""
    x = (a.cpu() ^ b.cpu()).to(torch.int32)
    n = 0
    for i in range(8 // q):
        n += int((((x >> (q * i)) & ((1 << q) - 1)) != 0).sum())
    return n / (a.numel() * (8 // q))


def _attn_saved_for_oracle(saved):
    """The device's saved tensors of the attention half in the form the oracle's backward reads (CPU)."""
    from hyc_lora_release_b200.operators import compress_function as cf
    B, M, H = saved["shape"]
    out = dict(a_shape=saved["a_shape"], map_q_bit=4)
    for k in ("rstd", "x_o", "x_scale", "x_idx", "xn_scale", "q_scale", "k_scale", "v_scale", "o_scale"):
        out[k] = saved[k].cpu()
    for k in ("x_q", "xn_q", "q_q", "k_q", "v_q", "o_q", "q_xa", "k_xa", "v_xa", "o_xa"):
        out[k] = saved[k].cpu().reshape(B, M, -1)
    m = saved["a_saved"]
    if isinstance(m, cf.TopkMap):
        out["map_q_bit"] = m.q_bit
        out["a_saved"] = ("topk", m.val.cpu(), m.col.cpu().to(torch.int64), m.q.cpu(), m.scale.cpu(), m.zp.cpu())
    elif isinstance(m, cf.TiledPrunedMap):
        idx, val = m.entries()
        out["a_saved"] = ("prune", idx.cpu(), val.cpu(), None)
    elif isinstance(m, cf.PrunedMap):
        n = int(m.nnz.item())
        out["a_saved"] = ("prune", m.idx[:n].cpu(), m.val[:n].cpu(), None)
    else:
        mc = m.coalesce()
        out["a_saved"] = ("prune", mc.indices().reshape(-1).cpu(), mc.values().cpu(), None)
    return out


@pytest.mark.parametrize("q,heads,kv,map_mode", [(4, 4, 4, "topk"), (8, 4, 2, "topk"), (4, 4, 4, "prune"), (2, 4, 2, "prune")])
def test_attention_block_forward_backward(q, heads, kv, map_mode):
    from hyc_lora_release_b200 import attention as at
    from hyc_lora_release_b200.mlp import check_status
    g = torch.Generator().manual_seed(3 * q + kv)
    B, M, d, I = 2, 128, 128, 256
    H = heads * d
    x, p, cos, sin, mask = layer_problem(g, B, M, H, heads, d, kv, I)
    W = _attn_weights(p)
    state = at.AttnState(q_bit=q, layernorm_outlier_ratio=0.01, softmax_outlier_ratio=0.05, map_mode=map_mode)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    ow = [p[k] for k in ATTN_ARGS]
    gout = (torch.randn(B, M, H, generator=g)).to(BF16)
    xd, cosd, sind, maskd, goutd = x.to(DEV), cos.to(DEV), sin.to(DEV), mask.to(DEV), gout.to(DEV)
    static = None
    for it in range(7):      # 5 calibration iterations, then the steady-state branch
        if it >= 5:
            static = _attn_static(state.static_value)
        ref_out, ref_saved = ref_attention_block_forward(x, p["norm_w1"], cos, sin, *ow, mask, heads, d, kv, q, 0.01, 0.05,
                                                         map_mode=map_mode, static=static)
        out, saved = at.attention_forward(xd, W, state, cosd, sind, maskd, heads, d, kv, status=st)
        grads = at.attention_backward(goutd, saved, W, status=st)
        check_status(st, "attention")
        assert close(out, ref_out), it
        assert torch.equal(saved["x_q"].cpu(), ref_saved["x_q"]) and torch.equal(saved["x_o"].cpu(), ref_saved["x_o"])
        # codes of COMPUTED tensors (x_norm, the q/k/v main branches, o) are pinned by the operator tests (bit-exact
        # against the oracle quantizer on the emitted tensor); against the oracle's own forward a code flips where the
        # tensor-core sum and the CPU sum round differently: counted and bounded
        for name in ("xn_q", "q_q", "k_q", "v_q", "o_q"):
            flips = _flipped_codes(saved[name].reshape(B, M, -1), ref_saved[name], q)
            assert flips < 0.02, (it, name, flips)
        # the backward is checked on the DEVICE's saved tensors, so every gradient is held to the path's tolerance
        ref_g = ref_attention_block_backward(gout, _attn_saved_for_oracle(saved), p["norm_w1"], cos, sin, *ow, heads, d, kv, q)
        assert close(grads["grad_x"], ref_g["grad_x"]), it
        for name in ("q", "k", "v"):
            assert close(grads["grad_" + name], ref_g["grad_" + name]), (it, name)
        for name in ("aq", "bq", "ak", "bk", "av", "bv", "ao", "bo"):   # oracle [in, r] / [r, out] -> weight layout
            assert close(grads["grad_" + name], ref_g["grad_" + name].t()), (it, name)
    assert state.iteration == 7


class _Holder(torch.nn.Module):
    """Stand-in for a PEFT module dictionary: ``.default`` is the adapter's nn.Linear."""
    def __init__(self, w):
        super().__init__()
        self.default = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, device=DEV, dtype=BF16)
        with torch.no_grad():
            self.default.weight.copy_(w)


def _base(w, bias=None):
    lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=bias is not None, device=DEV, dtype=BF16)
    with torch.no_grad():
        lin.weight.copy_(w)
        if bias is not None:
            lin.bias.copy_(bias)
            lin.bias.requires_grad_(False)
    lin.weight.requires_grad_(False)
    return lin


@pytest.mark.parametrize("heads,kv,map_mode,with_bias", [(4, 4, "topk", False), (4, 2, "prune", False), (4, 2, "prune", True)])
def test_layer_module_through_autograd(heads, kv, map_mode, with_bias):
    from hyc_lora_release_b200.layer import FusedLlamaLayerIntraInterFullFuse, FusedMistralLayerIntraInterFullFuse
    assert FusedMistralLayerIntraInterFullFuse is FusedLlamaLayerIntraInterFullFuse
    g = torch.Generator().manual_seed(21 + kv)
    B, M, d, I, q = 2, 128, 128, 1024, 4
    H = heads * d
    x, p, cos, sin, mask = layer_problem(g, B, M, H, heads, d, kv, I)
    mods = {}
    for n in ("q", "k", "v", "o", "gate", "up", "down"):
        bias = None
        if with_bias and n not in ("gate", "up"):
            # the bias of a projection is part of its main branch (models/utils/compute_utils.py:21)
            bias = (0.3 * torch.randn(p["w" + n].shape[1], generator=g)).to(BF16)
            p["bias_" + n] = bias
        mods[n] = (_base(p["w" + n].t().to(DEV), bias), _Holder(p["a" + n].t().to(DEV)), _Holder(p["b" + n].t().to(DEV)))
    layer = FusedLlamaLayerIntraInterFullFuse()
    cfg = types.SimpleNamespace(use_hyclora=True, iteration_threshold=5, softmax_outlier_ratio=0.05,
                                layernorm_outlier_ratio=0.01, q_bit=q, softmax_map_mode=map_mode)
    layer.set_hyclora_config(cfg)
    layer.check_kernel_status = True
    layer.keep_saved = True
    n1 = torch.nn.Parameter(p["norm_w1"].to(DEV), requires_grad=False)
    n2 = torch.nn.Parameter(p["norm_w2"].to(DEV), requires_grad=False)
    gy = torch.randn(B, M, H, generator=g).to(BF16)

    def run():
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
        y.backward(gy.to(DEV))
        return xin, y

    for it in range(6):
        xin, y = run()
    assert layer.iteration == 6
    sv = layer.static_value
    assert set(sv) == {"x", "x_norm_1", "q", "k", "v", "a", "o", "x_medium", "x_norm_2", "gate", "up"}
    static = dict(attention=_attn_static(sv),
                  mlp=dict(x_medium_idx=sv["x_medium"]["outlier_channel_index"].cpu(),
                           x_medium_scale=sv["x_medium"]["scale"].cpu().to(BF16),
                           gate_scale=sv["gate"]["scale"].cpu().to(BF16), up_scale=sv["up"]["scale"].cpu().to(BF16),
                           x_norm_2_scale=sv["x_norm_2"]["scale"].cpu().to(BF16)))
    ref_y, ref_saved = ref_layer_forward(x, p, cos, sin, mask, heads, d, kv, q, 0.01, 0.05, map_mode=map_mode, static=static)
    assert close(y, ref_y)
    # backward: the oracle's backward on the tensors the DEVICE saved in this iteration (codes of computed tensors
    # may differ from the oracle's own forward in a few places, which the block tests count), path tolerance
    from test_gpu_mlp import _saved_for_oracle
    sa, sm = layer.last_saved
    ref_g = ref_layer_backward(gy, (_attn_saved_for_oracle(sa), _saved_for_oracle(sm)), p, cos, sin, heads, d, kv, q)
    # grad_x is the end of the longest chain of bf16 roundings (MLP backward, then attention backward): a large
    # element may land two bf16 steps (2 x 2^-7 of its value) from the oracle's; the LoRA gradients are held to 1e-2
    assert close(xin.grad, ref_g["grad_x"], rel=2 ** -6)
    for n in ("q", "k", "v", "o", "gate", "up", "down"):
        ga, gb = mods[n][1].default.weight.grad, mods[n][2].default.weight.grad
        assert ga is not None and gb is not None, n
        assert close(ga, ref_g["grad_a" + n].t()), n
        assert close(gb, ref_g["grad_b" + n].t()), n
    # a bias on the gate projection (which the reference's fused layer would drop) is refused, not silently ignored
    with pytest.raises(NotImplementedError):
        layer._bind(n1, n2, {**mods, "gate": (_base(p["wgate"].t().to(DEV), torch.zeros(I, dtype=BF16)), mods["gate"][1],
                                              mods["gate"][2])})
    # so is a quant state that is not a 4-bit block-wise one (those are covered in test_nf4.py)
    bad = _base(p["wq"].t().to(DEV))
    bad.weight.quant_state = object()
    with pytest.raises(NotImplementedError):
        layer._bind(n1, n2, {**mods, "q": (bad, mods["q"][1], mods["q"][2])})
    # so are adapters of another rank or dtype
    with pytest.raises(NotImplementedError):
        layer._bind(n1, n2, {**mods, "q": (mods["q"][0], _Holder(torch.zeros(8, H, dtype=BF16)), mods["q"][2])})
    f32 = _Holder(p["aq"].t().to(DEV))
    f32.default = f32.default.float()
    with pytest.raises(NotImplementedError):
        layer._bind(n1, n2, {**mods, "q": (mods["q"][0], f32, mods["q"][2])})


def test_layer_reports_dropped_map_entries_and_recalibrates():
    """Failures must not stay silent: a pruned map that does not fit its fixed-capacity buffers raises at the next
    periodic check (the flag is kept on the device in between, no synchronisation per step), and setting `iteration`
    back re-calibrates the threshold the steady state uses."""
    from hyc_lora_release_b200.layer import FusedLlamaLayerIntraInterFullFuse
    g = torch.Generator().manual_seed(77)
    B, M, heads, d, kv, I, q = 1, 128, 4, 128, 4, 512, 4
    H = heads * d
    x, p, cos, sin, mask = layer_problem(g, B, M, H, heads, d, kv, I)
    mods = {n: (_base(p["w" + n].t().to(DEV)), _Holder(p["a" + n].t().to(DEV)), _Holder(p["b" + n].t().to(DEV)))
            for n in ("q", "k", "v", "o", "gate", "up", "down")}
    layer = FusedLlamaLayerIntraInterFullFuse()
    layer.set_hyclora_config(types.SimpleNamespace(use_hyclora=True, iteration_threshold=2, softmax_outlier_ratio=0.05,
                                                   layernorm_outlier_ratio=0.01, q_bit=q, softmax_map_mode="prune"))
    layer.check_every = 3
    n1, n2 = p["norm_w1"].to(DEV), p["norm_w2"].to(DEV)
    gy = torch.randn(B, M, H, generator=g).to(BF16).to(DEV)

    def run():
        xin = x.to(DEV).requires_grad_(True)
        args = [xin, n1, None, cos.to(DEV), sin.to(DEV)]
        for n in ("q", "k", "v", "o"):
            args += list(mods[n])
        args += [n2, None]
        for n in ("gate", "up", "down"):
            args += list(mods[n])
        layer(*args, mask.to(DEV), heads, d, kv).backward(gy)
    for _ in range(4):
        run()                                    # 2 calibration steps, 2 steady ones: nothing to report
    layer.raise_on_device_errors()
    assert layer.attn_state.threshold_host is not None
    layer.attn_state.prune_capacity_margin = 0.01      # buffers far too small for the calibrated threshold
    with pytest.raises(RuntimeError, match="overflowed"):
        for _ in range(3):
            run()
    layer.attn_state.prune_capacity_margin = 1.5
    layer.iteration = 0                          # re-calibrate: the cached host threshold must go
    assert layer.attn_state.threshold_host is None
    for _ in range(3):
        run()
    layer.raise_on_device_errors()
    assert layer.attn_state.threshold_host is not None
