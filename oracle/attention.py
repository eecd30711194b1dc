"""Attention half of the fused decoder layer and the whole layer (test infrastructure; see the package
docstring).  CPU restatement, with the reference's bf16 rounding points, of
``FusedLlamaLayerIntraInterFullFuseFunc.forward`` (models/llama/fused_llama_layer_intra_inter_full_fuse.py:
99-201) and ``.backward`` (:400-493) with plain bf16 frozen weights (NF4 de-quantization = identity).

The rotary embedding follows the rotate-half formula the reference's kernel implements
(operators/rope_kernels.py:38-78), in the dtype of the sine table like the reference (pinned by the golden
vectors of that kernel).  Two map modes: ``prune`` is the
reference's global-threshold prune, ``topk`` the per-row top-k + grouped remainder defined in
``oracle/softmax_map.py``.
"""
import math

import torch

from .quant import (ref_scale_per_channel, ref_statistics_channel_base, ref_compress_channel_base,
                    ref_decompress_channel_base, ref_compress, ref_decompress)
from .softmax_map import (ref_softmax_threshold, ref_softmax_prune, ref_softmax_restore, topk_compress,
                          topk_decompress)
from .fused_mlp import (ref_lora_forward, ref_lora_backward, ref_rmsnorm_forward, ref_rmsnorm_backward,
                        ref_softmax_backward, ref_mlp_block_forward, ref_mlp_block_backward)

__all__ = ["ref_rope", "ref_attention_block_forward", "ref_attention_block_backward",
           "ref_layer_forward", "ref_layer_backward"]

BF16 = torch.bfloat16


def ref_rope(x, cos, sin, backward=False):
    """``rope_forward`` / ``rope_backward`` (operators/rope_kernels.py:81-131) on x [B, M, heads, d]; cos, sin
    [>= M, d] tables whose first d/2 columns are used (:55-58).  out1 = x1*cos - x2*sin, out2 = x2*cos + x1*sin
    (:77-78), sine negated in the backward pass (:62-63).  The kernel computes in the dtype of the sine table
    (:73-74): with bf16 tables the two products and the sum are three bf16 operations, with fp32 tables three
    fp32 operations and the store rounds."""
    b, m, h, d = x.shape
    half = d // 2
    dt = torch.float32 if sin.dtype == torch.float32 else BF16
    c = cos.squeeze()[:m, :half].to(dt).reshape(1, m, 1, half)
    s = sin.squeeze()[:m, :half].to(dt).reshape(1, m, 1, half)
    if backward:
        s = -s
    x1, x2 = x[..., :half].to(dt), x[..., half:].to(dt)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(BF16)


def _to_heads(x, n):
    """``hidden_to_head_shape`` (compress_function.py): [B, M, n*d] -> [B, n, M, d]."""
    b, m, hd = x.shape
    return x.reshape(b, m, n, hd // n).transpose(1, 2)


def _to_hidden(x):
    """``head_to_hidden_shape``: [B, n, M, d] -> [B, M, n*d]."""
    b, n, m, d = x.shape
    return x.transpose(1, 2).reshape(b, m, n * d)


def _repeat_kv(x, n_rep):
    b, n, m, d = x.shape
    if n_rep == 1:
        return x
    return x[:, :, None].expand(b, n, n_rep, m, d).reshape(b, n * n_rep, m, d)


def _repeat_kv_backward(g, n_rep):
    b, n, m, d = g.shape
    if n_rep == 1:
        return g
    return g.reshape(b, n // n_rep, n_rep, m, d).sum(dim=2)


def ref_attention_block_forward(x, norm_w, cos, sin, wq, wk, wv, wo, aq, bq, ak, bk, av, bv, ao, bo, mask,
                                num_heads, head_dim, num_kv_heads, q_bit, layernorm_ratio, softmax_ratio,
                                map_mode="prune", map_q_bit=4, static=None, biases=None):
    """:99-201.  w*: [in, out] bf16; a*: [in, r]; b*: [r, out]; ``biases``: optional dict with any of "q", "k", "v",
    "o" -> [out] bias of that projection.  -> (x_medium, saved)."""
    biases = biases or {}
    x = x.to(BF16)
    x_norm_1, rstd = ref_rmsnorm_forward(x, norm_w, 1e-5)
    if static is None:
        x_idx, x_scale = ref_statistics_channel_base(x, layernorm_ratio, q_bit)
    else:
        x_idx, x_scale = static["x_idx"], static["x_scale"]
    x_o, x_q = ref_compress_channel_base(x, x_scale, x_idx, q_bit)

    q, q_main, q_xa = ref_lora_forward(wq, aq, bq, x_norm_1, biases.get("q"))
    k, k_main, k_xa = ref_lora_forward(wk, ak, bk, x_norm_1, biases.get("k"))
    v, v_main, v_xa = ref_lora_forward(wv, av, bv, x_norm_1, biases.get("v"))
    if static is None:
        xn_scale = ref_scale_per_channel(x_norm_1, q_bit)
        q_scale = ref_scale_per_channel(q_main, q_bit)
        k_scale = ref_scale_per_channel(k_main, q_bit)
        v_scale = ref_scale_per_channel(v_main, q_bit)
    else:
        xn_scale, q_scale, k_scale, v_scale = (static["x_norm_1_scale"], static["q_scale"], static["k_scale"],
                                               static["v_scale"])
    xn_q = ref_compress(x_norm_1, xn_scale, q_bit)
    q_q = ref_compress(q_main, q_scale, q_bit)
    k_q = ref_compress(k_main, k_scale, q_bit)
    v_q = ref_compress(v_main, v_scale, q_bit)

    n_rep = num_heads // num_kv_heads
    qh = _to_heads(q, num_heads)
    kh = _to_heads(k, num_kv_heads)
    vh = _to_heads(v, num_kv_heads)
    qh = ref_rope(qh.transpose(1, 2), cos, sin).transpose(1, 2)
    kh = ref_rope(kh.transpose(1, 2), cos, sin).transpose(1, 2)
    kh = _repeat_kv(kh, n_rep)
    s = (qh @ kh.transpose(-2, -1)) / math.sqrt(head_dim)
    if mask is not None:
        s = s + mask
    a = torch.softmax(s, dim=-1, dtype=BF16)
    if map_mode == "prune":
        thr = ref_softmax_threshold(a, softmax_ratio) if static is None else static["a_threshold"]
        a_idx, a_val = ref_softmax_prune(a, thr)
        a_saved = ("prune", a_idx, a_val, thr)
    else:
        thr = None
        a_saved = ("topk",) + tuple(topk_compress(a, softmax_ratio, map_q_bit))
    o = a @ _repeat_kv(vh, n_rep)
    o = _to_hidden(o)
    o_final, _, o_xa = ref_lora_forward(wo, ao, bo, o, biases.get("o"))
    o_scale = ref_scale_per_channel(o, q_bit) if static is None else static["o_scale"]
    o_q = ref_compress(o, o_scale, q_bit)
    x_medium = x + o_final
    saved = dict(rstd=rstd, x_o=x_o, x_q=x_q, x_scale=x_scale, x_idx=x_idx, xn_q=xn_q, xn_scale=xn_scale,
                 q_q=q_q, q_scale=q_scale, k_q=k_q, k_scale=k_scale, v_q=v_q, v_scale=v_scale,
                 q_xa=q_xa, k_xa=k_xa, v_xa=v_xa, a_saved=a_saved, a_shape=tuple(a.shape), a_threshold=thr,
                 o_q=o_q, o_scale=o_scale, o_xa=o_xa, map_q_bit=map_q_bit,
                 a=a, q_main=q_main, k_main=k_main, v_main=v_main, o=o)
    return x_medium, saved


def ref_attention_block_backward(grad_medium, saved, norm_w, cos, sin, wq, wk, wv, wo, aq, bq, ak, bk, av, bv,
                                 ao, bo, num_heads, head_dim, num_kv_heads, q_bit):
    """:400-493.  -> dict(grad_x, grad_aq, grad_bq, ..., grad_ao, grad_bo) with the LoRA gradients in the
    [in, r] / [r, out] orientation of the arguments."""
    g = grad_medium.to(BF16)
    n_rep = num_heads // num_kv_heads
    o = ref_decompress(saved["o_q"], saved["o_scale"], q_bit)
    grad_ao, grad_bo, grad_o = ref_lora_backward(wo, ao, bo, o, saved["o_xa"], g)
    grad_o = _to_heads(grad_o, num_heads)

    mode = saved["a_saved"][0]
    if mode == "prune":
        _, a_idx, a_val, _ = saved["a_saved"]
        a = ref_softmax_restore(a_idx, a_val, saved["a_shape"])
    else:
        a = topk_decompress(*saved["a_saved"][1:], saved["map_q_bit"], saved["a_shape"])
    v_main = ref_decompress(saved["v_q"], saved["v_scale"], q_bit)
    v = v_main + saved["v_xa"].to(BF16) @ bv.to(BF16)
    v = _repeat_kv(_to_heads(v, num_kv_heads), n_rep)
    grad_v = a.transpose(-2, -1) @ grad_o
    grad_a = grad_o @ v.transpose(-2, -1)
    grad_v = _repeat_kv_backward(grad_v, n_rep)
    grad_s = ref_softmax_backward(a, grad_a)
    grad_s = grad_s / math.sqrt(head_dim)

    q_main = ref_decompress(saved["q_q"], saved["q_scale"], q_bit)
    q = q_main + saved["q_xa"].to(BF16) @ bq.to(BF16)
    q = _to_heads(q, num_heads)
    q = ref_rope(q.transpose(1, 2), cos, sin).transpose(1, 2)
    grad_k = grad_s.transpose(-2, -1) @ q
    k_main = ref_decompress(saved["k_q"], saved["k_scale"], q_bit)
    k = k_main + saved["k_xa"].to(BF16) @ bk.to(BF16)
    k = _to_heads(k, num_kv_heads)
    k = ref_rope(k.transpose(1, 2), cos, sin).transpose(1, 2)
    k = _repeat_kv(k, n_rep)
    grad_k = _repeat_kv_backward(grad_k, n_rep)
    grad_q = grad_s @ k
    grad_q = ref_rope(grad_q.transpose(1, 2), cos, sin, backward=True).transpose(1, 2)
    grad_k = ref_rope(grad_k.transpose(1, 2), cos, sin, backward=True).transpose(1, 2)
    grad_q, grad_k, grad_v = _to_hidden(grad_q), _to_hidden(grad_k), _to_hidden(grad_v)

    x_norm_1 = ref_decompress(saved["xn_q"], saved["xn_scale"], q_bit)
    grad_aq, grad_bq, grad_x = ref_lora_backward(wq, aq, bq, x_norm_1, saved["q_xa"], grad_q)
    grad_ak, grad_bk, t = ref_lora_backward(wk, ak, bk, x_norm_1, saved["k_xa"], grad_k)
    grad_x = grad_x + t
    grad_av, grad_bv, t = ref_lora_backward(wv, av, bv, x_norm_1, saved["v_xa"], grad_v)
    grad_x = grad_x + t
    x = ref_decompress_channel_base(saved["x_q"], saved["x_scale"], saved["x_o"], saved["x_idx"], q_bit)
    grad_norm_1 = ref_rmsnorm_backward(grad_x, x, norm_w, saved["rstd"])
    grad_input = grad_norm_1 + g
    return dict(grad_x=grad_input, grad_aq=grad_aq, grad_bq=grad_bq, grad_ak=grad_ak, grad_bk=grad_bk,
                grad_av=grad_av, grad_bv=grad_bv, grad_ao=grad_ao, grad_bo=grad_bo,
                grad_q=grad_q, grad_k=grad_k, grad_v=grad_v, grad_s=grad_s)


def ref_layer_forward(x, p, cos, sin, mask, num_heads, head_dim, num_kv_heads, q_bit, layernorm_ratio,
                      softmax_ratio, map_mode="prune", map_q_bit=4, static=None):
    """The whole decoder layer (:99-252): attention half then MLP half.  ``p`` is a dict with norm_w1, norm_w2,
    w{q,k,v,o,gate,up,down} [in, out], a* [in, r], b* [r, out] and optionally bias_{q,k,v,o,down} [out].
    -> (y, (saved_attention, saved_mlp))."""
    xm, sa = ref_attention_block_forward(
        x, p["norm_w1"], cos, sin, p["wq"], p["wk"], p["wv"], p["wo"], p["aq"], p["bq"], p["ak"], p["bk"],
        p["av"], p["bv"], p["ao"], p["bo"], mask, num_heads, head_dim, num_kv_heads, q_bit, layernorm_ratio,
        softmax_ratio, map_mode, map_q_bit, None if static is None else static["attention"],
        biases={n: p["bias_" + n] for n in ("q", "k", "v", "o") if p.get("bias_" + n) is not None})
    y, sm = ref_mlp_block_forward(xm, p["norm_w2"], p["wgate"], p["wup"], p["wdown"], p["agate"], p["bgate"],
                                  p["aup"], p["bup"], p["adown"], p["bdown"], q_bit, layernorm_ratio,
                                  None if static is None else static["mlp"], bias_d=p.get("bias_down"))
    return y, (sa, sm)


def ref_layer_backward(grad_y, saved, p, cos, sin, num_heads, head_dim, num_kv_heads, q_bit):
    """:255-493.  -> dict of grad_x and the 14 LoRA gradients."""
    sa, sm = saved
    gm = ref_mlp_block_backward(grad_y, sm, p["norm_w2"], p["wgate"], p["wup"], p["wdown"], p["agate"],
                                p["bgate"], p["aup"], p["bup"], p["adown"], p["bdown"], q_bit)
    ga = ref_attention_block_backward(gm["grad_x"], sa, p["norm_w1"], cos, sin, p["wq"], p["wk"], p["wv"],
                                      p["wo"], p["aq"], p["bq"], p["ak"], p["bk"], p["av"], p["bv"], p["ao"],
                                      p["bo"], num_heads, head_dim, num_kv_heads, q_bit)
    out = dict(grad_x=ga["grad_x"])
    for k in ("aq", "bq", "ak", "bk", "av", "bv", "ao", "bo"):
        out["grad_" + k] = ga["grad_" + k]
    out.update(grad_agate=gm["grad_ag"], grad_bgate=gm["grad_bg"], grad_aup=gm["grad_au"], grad_bup=gm["grad_bu"],
               grad_adown=gm["grad_ad"], grad_bdown=gm["grad_bd"])
    return out
