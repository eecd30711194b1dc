"""Fused LoRA-SiLU-Hadamard and MLP-block oracle (test infrastructure; see the
package docstring).  CPU restatement with the reference's bf16 rounding points.
"""
import torch
from .quant import (ref_quant_codes, ref_pack, ref_unpack, ref_dequant,
                    ref_scale_per_channel, ref_statistics_channel_base,
                    ref_compress_channel_base, ref_decompress_channel_base,
                    ref_compress, ref_decompress)

__all__ = ["ref_fused_silu_forward", "ref_fused_silu_backward",
           "ref_lora_forward", "ref_lora_backward",
           "ref_rmsnorm_forward", "ref_rmsnorm_backward", "ref_softmax_backward",
           "ref_mlp_block_forward", "ref_mlp_block_backward"]

BF16 = torch.bfloat16


def _lora_term(xa, b):
    """``tl.dot(xa, b).to(tl.bfloat16)``: fp32 accumulate, bf16 result
    (triton_fuse_lora_silu_hadamard_forward_kernels.py:120)."""
    return (xa.float() @ b.float()).to(BF16)


def ref_fused_silu_forward(xa1, b1, x1, s1, xa2, b2, x2, s2, q_bit: int):
    """``triton_fuse_silu_forward``
    (triton_fuse_lora_silu_hadamard_forward_kernels.py:96-149, wrapper :152-181).
    The *main* branches x1, x2 are quantized (not main + LoRA)."""
    q1 = ref_pack(ref_quant_codes(x1, s1, q_bit), q_bit)
    q2 = ref_pack(ref_quant_codes(x2, s2, q_bit), q_bit)
    y1 = (x1 + _lora_term(xa1, b1)).to(BF16)
    y1 = (y1 * torch.sigmoid(y1.float()).to(BF16)).to(BF16)
    y2 = (x2 + _lora_term(xa2, b2)).to(BF16)
    return q1, q2, (y1 * y2).to(BF16)


def ref_fused_silu_backward(xa1, b1, q1, s1, xa2, b2, q2, s2, grad_o, q_bit: int):
    """``triton_fuse_silu_backward``
    (triton_fuse_lora_silu_hadamard_backward_kernels.py:93-149, wrapper
    :152-178) -> (o, grad_gate, grad_up)."""
    x1 = ref_dequant(ref_unpack(q1, q_bit), s1, q_bit)
    x2 = ref_dequant(ref_unpack(q2, q_bit), s2, q_bit)
    y1 = (x1 + _lora_term(xa1, b1)).to(BF16)
    y2 = (x2 + _lora_term(xa2, b2)).to(BF16)
    sig = torch.sigmoid(y1.float()).to(BF16)
    y1s = (y1 * sig).to(BF16)
    o = (y1s * y2).to(BF16)
    g = grad_o.to(BF16)
    gh1 = (g * y2).to(BF16)
    g_up = (g * y1s).to(BF16)
    # sigma * (1 + y1 * bf16(1 - sigma)), each step a bf16 op (:139)
    one_m = (1.0 - sig).to(BF16)
    inner = (1.0 + (y1 * one_m).to(BF16)).to(BF16)
    g_gate = (gh1 * (sig * inner).to(BF16)).to(BF16)
    return o, g_gate, g_up


def ref_lora_forward(w, a, b, x, bias=None):
    """``lora_forward`` with plain bf16 weights (models/utils/compute_utils.py:
    18-25; NF4 de-quantization is the identity here).  w [in,out] bf16 (already
    transposed), a [in,r], b [r,out], bias [out] or None (part of the main
    branch, :21).  -> (y, x_main, x_lora_a)."""
    x = x.to(BF16)
    x_main = x @ w
    if bias is not None:
        x_main = x_main + bias.to(BF16)
    xa = x @ a
    return x_main + xa @ b, x_main, xa


def ref_lora_backward(w, a, b, x, xa, g):
    """``lora_backward`` (models/utils/compute_utils.py:28-36) on flattened
    tokens: -> (grad_a [in,r], grad_b [r,out], grad_x)."""
    g = g.to(BF16)
    gm = g @ b.mT
    x2 = x.reshape(-1, x.shape[-1])
    grad_a = x2.mT @ gm.reshape(-1, gm.shape[-1])
    grad_b = xa.reshape(-1, xa.shape[-1]).mT @ g.reshape(-1, g.shape[-1])
    grad_x = g @ w.T
    grad_x = grad_x + gm @ a.T
    return grad_a, grad_b, grad_x


def ref_rmsnorm_forward(x, w, eps):
    """``_rms_norm_fwd_fused`` (operators/rmsnorm_kernels.py:10-54):
    fp32 mean of squares, rstd = 1/sqrt(var+eps), y = x*rstd*w stored in the
    input dtype.  -> (y, rstd fp32 [T])."""
    xf = x.float()
    var = (xf * xf).sum(-1) / x.shape[-1]
    rstd = 1.0 / torch.sqrt(var + eps)
    y = (xf * rstd.unsqueeze(-1)) * w.float()
    return y.to(x.dtype), rstd.reshape(-1)


def ref_rmsnorm_backward(dy, x, w, rstd):
    """``_rms_norm_bwd_dx_fused`` (operators/rmsnorm_kernels.py:58-113); keeps
    the LayerNorm-style ``c2`` mean term of the reference (:96-98)."""
    n = x.shape[-1]
    xhat = x.float() * rstd.reshape(*x.shape[:-1], 1)
    wdy = w.float() * dy.float()
    c1 = (xhat * wdy).sum(-1, keepdim=True) / n
    c2 = wdy.sum(-1, keepdim=True) / n
    dx = (wdy - (xhat * c1 + c2)) * rstd.reshape(*x.shape[:-1], 1)
    return dx.to(dy.dtype)


def ref_softmax_backward(y, g):
    """``softmax_backward_kernel`` (operators/softmax_kernels.py:7-38):
    o = (g - sum(y*g)) * y per row; the product y*g is a bf16 op, the row sum
    and the rest are fp32, the store rounds to bf16."""
    yg = (y.to(BF16) * g.to(BF16)).float().sum(-1, keepdim=True)
    return ((g.float() - yg) * y.float()).to(BF16)


def ref_mlp_block_forward(x_medium, norm_w, wg, wu, wd, ag, bg, au, bu, ad, bd,
                          q_bit: int, outlier_ratio: float, static=None, bias_d=None):
    """MLP half of the fused decoder layer, forward
    (models/llama/fused_llama_layer_intra_inter_full_fuse.py:203-252), with
    plain bf16 weights.  wg, wu: [H,I]; wd: [I,H] (already transposed as the
    layer passes them); a*: [in,r]; b*: [r,out].
    Returns (x_out, saved) where ``saved`` holds exactly what the layer keeps
    for backward (packed codes, scales, outlier slab, LoRA-A activations, rstd).
    ``static`` (dict of calibrated statistics) switches to the steady-state
    branch (compress_function.py:347-350)."""
    x_norm_2, rstd = ref_rmsnorm_forward(x_medium, norm_w, 1e-5)
    if static is None:
        xm_idx, xm_scale = ref_statistics_channel_base(x_medium, outlier_ratio, q_bit)
    else:
        xm_idx, xm_scale = static["x_medium_idx"], static["x_medium_scale"]
    xm_o, xm_q = ref_compress_channel_base(x_medium, xm_scale, xm_idx, q_bit)

    gate_main = x_norm_2 @ wg
    gate_xa = x_norm_2 @ ag
    up_main = x_norm_2 @ wu
    up_xa = x_norm_2 @ au
    if static is None:
        gate_scale = ref_scale_per_channel(gate_main, q_bit)
        up_scale = ref_scale_per_channel(up_main, q_bit)
        xn_scale = ref_scale_per_channel(x_norm_2, q_bit)
    else:
        gate_scale, up_scale, xn_scale = static["gate_scale"], static["up_scale"], static["x_norm_2_scale"]
    gate_q, up_q, had = ref_fused_silu_forward(gate_xa, bg, gate_main, gate_scale,
                                               up_xa, bu, up_main, up_scale, q_bit)
    xn_q = ref_compress(x_norm_2, xn_scale, q_bit)
    down, _, down_xa = ref_lora_forward(wd, ad, bd, had, bias_d)
    x_out = x_medium + down
    saved = dict(rstd=rstd, xm_o=xm_o, xm_q=xm_q, xm_scale=xm_scale, xm_idx=xm_idx,
                 xn_q=xn_q, xn_scale=xn_scale, gate_q=gate_q, gate_scale=gate_scale,
                 up_q=up_q, up_scale=up_scale, gate_xa=gate_xa, up_xa=up_xa,
                 down_xa=down_xa, gate_main=gate_main, up_main=up_main, hadamard=had)
    return x_out, saved


def ref_mlp_block_backward(grad_out, saved, norm_w, wg, wu, wd, ag, bg, au, bu, ad, bd,
                           q_bit: int):
    """MLP half of the fused decoder layer, backward
    (models/llama/fused_llama_layer_intra_inter_full_fuse.py:359-396).
    -> dict(grad_x, grad_ag, grad_bg, grad_au, grad_bu, grad_ad, grad_bd)."""
    g = grad_out.to(BF16)
    g2 = g.reshape(-1, g.shape[-1])
    grad_bd = saved["down_xa"].reshape(-1, ad.shape[1]).mT @ g2
    grad_down = g @ wd.T
    gdm = g @ bd.T
    grad_down = grad_down + gdm @ ad.T
    had, g_gate, g_up = ref_fused_silu_backward(
        saved["gate_xa"], bg, saved["gate_q"], saved["gate_scale"],
        saved["up_xa"], bu, saved["up_q"], saved["up_scale"], grad_down, q_bit)
    grad_ad = had.reshape(-1, had.shape[-1]).mT @ gdm.reshape(-1, gdm.shape[-1])
    x_norm_2 = ref_decompress(saved["xn_q"], saved["xn_scale"], q_bit)
    grad_ag, grad_bg, gx_gate = ref_lora_backward(wg, ag, bg, x_norm_2, saved["gate_xa"], g_gate)
    grad_au, grad_bu, gx_up = ref_lora_backward(wu, au, bu, x_norm_2, saved["up_xa"], g_up)
    grad_gate_up = gx_up + gx_gate
    x_medium = ref_decompress_channel_base(saved["xm_q"], saved["xm_scale"], saved["xm_o"],
                                           saved["xm_idx"], q_bit)
    grad_norm = ref_rmsnorm_backward(grad_gate_up, x_medium, norm_w, saved["rstd"])
    grad_x = grad_norm + g
    return dict(grad_x=grad_x, grad_ag=grad_ag, grad_bg=grad_bg, grad_au=grad_au,
                grad_bu=grad_bu, grad_ad=grad_ad, grad_bd=grad_bd,
                hadamard=had, g_gate=g_gate, g_up=g_up, grad_down=grad_down)
