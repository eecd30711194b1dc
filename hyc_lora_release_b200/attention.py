"""Attention half of the HyC-LoRA fused decoder layer.

Mirrors the attention part of ``FusedLlamaLayerIntraInterFullFuseFunc.forward/backward``
(models/llama/fused_llama_layer_intra_inter_full_fuse.py:99-201 and :400-493; the Mistral twin differs only
in its grouped key/value heads, which are covered) with plain bf16 frozen weights:

  forward : RMSNorm fused with the saves of x (outlier channels + codes) and x_norm (codes) -> q/k/v
            projections on the tcgen05 GEMM whose epilogue also packs the codes of the main branch ->
            rotary embedding in place -> scores (library batched GEMM) -> scale + mask + softmax in one pass
            -> save of the probability map (per-row top-k + 4-bit groups, or the reference's threshold
            prune) -> P.V (library batched GEMM) -> save of o -> o projection with the LoRA product as one
            more K block and the residual in the GEMM epilogue;
  backward: o projection backward (LoRA-A gradient straight from the packed o) -> restored map -> grad_v,
            grad_a -> restore fused with the softmax backward -> q, k rebuilt by de-quantize + LoRA re-add +
            rotary -> grad_q, grad_k -> inverse rotary -> LoRA gradients of q/k/v (A side from the packed
            x_norm in one pass for the three adapters) -> grad_x as ONE GEMM over the three K segments ->
            RMSNorm backward from the packed x with the residual gradient added in the same pass.

Weights use the nn.Linear layout ([out, in]); LoRA factors are ``lora_A.weight`` [r, in] and
``lora_B.weight`` [out, r].  The two batched attention products are plain library GEMMs (torch.matmul).
"""
import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ._lib import require_cuda
from .mlp import _status_tensor, gemm, linear_lora_save, lora_a_products, lora_grad_a, padded_block
from .operators import compress_function as cf
from .operators.rmsnorm_kernels import rmsnorm_backward_packed, rmsnorm_forward, rmsnorm_forward_save
from .operators.rope_kernels import rope_inplace
from .operators.softmax_kernels import softmax_backward, softmax_forward_scale_mask, softmax_forward_topk_save

BF16 = torch.bfloat16


@dataclass
class AttnWeights:
    """Frozen bf16 weights ([out, in]) and LoRA factors of one attention block."""
    norm_w: torch.Tensor   # [H]
    wq: torch.Tensor       # [heads*d, H]
    wk: torch.Tensor       # [kv_heads*d, H]
    wv: torch.Tensor       # [kv_heads*d, H]
    wo: torch.Tensor       # [H, heads*d]
    aq: torch.Tensor       # q lora_A.weight [r, H]
    bq: torch.Tensor       # q lora_B.weight [heads*d, r]
    ak: torch.Tensor
    bk: torch.Tensor
    av: torch.Tensor
    bv: torch.Tensor
    ao: torch.Tensor       # o lora_A.weight [r, heads*d]
    bo: torch.Tensor       # o lora_B.weight [H, r]
    # projection biases ([out] bf16) or None.  A bias belongs to the MAIN branch (x W^T + b is what the reference
    # saves, models/utils/compute_utils.py:21); a projection that has one runs as separate launches (GEMM, bias add,
    # quantized save, LoRA add) instead of the one GEMM with the save in its epilogue.  Biases get no gradient.
    bias_q: Optional[torch.Tensor] = None
    bias_k: Optional[torch.Tensor] = None
    bias_v: Optional[torch.Tensor] = None
    bias_o: Optional[torch.Tensor] = None

    def padded(self):
        """LoRA factors zero-padded to a K of 64 so that a rank-16 product rides along a GEMM as one more K block
        (rebuilt when a factor changes):
          ao_cols  [heads*d, 64]  columns 0..15 = Ao^T   (o -> padded LoRA activation of the o projection)
          bo_cols  [H, 64]        columns 0..15 = Bo     ([N, K] operand of the o projection's LoRA block)
          ao_rows  [64, heads*d]  rows 0..15 = Ao        ([K, N] operand of grad_o's LoRA block)
          aqkv_rows [64, H]       rows 0..15 = Aq, 16..31 = Ak, 32..47 = Av ([K, N] operand of grad_x's LoRA block)
        and the stacked factors of the batched rank-16 products:
          aqkv_t   [3, H, r]        Aq^T, Ak^T, Av^T (x_norm @ all three in one call)
          bqkv     [3, heads*d, r]  Bq, Bk, Bv (None with grouped key/value heads, whose shapes differ)"""
        ts = (self.aq, self.ak, self.av, self.ao, self.bo, self.bq, self.bk, self.bv)
        key = tuple((t.data_ptr(), t._version) for t in ts)
        if getattr(self, "_pad_key", None) != key:
            r, D = self.ao.shape
            H = self.bo.shape[0]
            dev, dt = self.ao.device, self.ao.dtype
            ao_rows = torch.zeros(64, D, dtype=dt, device=dev); ao_rows[:r] = self.ao
            bo_cols = torch.zeros(H, 64, dtype=dt, device=dev); bo_cols[:, :r] = self.bo
            aqkv = torch.zeros(64, self.aq.shape[1], dtype=dt, device=dev)
            aqkv[:r] = self.aq; aqkv[r:2 * r] = self.ak; aqkv[2 * r:3 * r] = self.av
            aqkv_t = torch.stack((self.aq.t(), self.ak.t(), self.av.t())).contiguous()      # [3, H, r]
            same = self.bq.shape == self.bk.shape == self.bv.shape
            bqkv = torch.stack((self.bq, self.bk, self.bv)).contiguous() if same else None   # [3, heads*d, r]
            self._pad = dict(ao_rows=ao_rows, ao_cols=ao_rows.t().contiguous(), bo_cols=bo_cols, aqkv_rows=aqkv,
                             aqkv_t=aqkv_t, bqkv=bqkv)
            self._pad_key = key
        return self._pad


@dataclass
class AttnState:
    """Calibration state of the attention part of a layer (the reference keeps the same entries in
    ``static_value``, fused_llama_layer_intra_inter_full_fuse.py:557-565).  ``map_mode``: "prune" = the
    reference's global-threshold prune of the probability map, "topk" = per-row top-k + ``map_q_bit`` groups."""
    iteration: int = 0
    iteration_threshold: int = 5
    q_bit: int = 4
    layernorm_outlier_ratio: float = 0.005
    softmax_outlier_ratio: float = 0.05
    map_mode: str = "topk"
    map_q_bit: int = 4
    prune_capacity_margin: float = 1.5     # "prune" steady state: buffers hold margin x ratio x numel entries
    # "topk": softmax and the save as ONE kernel.  Off by default: the save is bound by instruction issue, not by
    # memory, so the softmax arithmetic added to it costs more than the saved pass over the map
    # ([1,32,2048,2048]: 281 us fused against 118 + 145 us)
    fuse_softmax_with_save: bool = False
    threshold_host: float = None           # the calibrated threshold as a host number (set after calibration)
    static_value: dict = field(default_factory=lambda: {
        'x': {'outlier_channel_index': None, 'scale': None}, 'x_norm_1': {'scale': None},
        'q': {'scale': None}, 'k': {'scale': None}, 'v': {'scale': None}, 'a': {'outlier': None},
        'o': {'scale': None}})


def _repeat_kv(x, n_rep):
    """[B, kv, M, d] -> [B, kv * n_rep, M, d] (each key/value head serves n_rep query heads)."""
    if n_rep == 1:
        return x
    b, n, m, d = x.shape
    return x[:, :, None].expand(b, n, n_rep, m, d).reshape(b, n * n_rep, m, d)


def _repeat_kv_backward(g, n_rep):
    if n_rep == 1:
        return g
    b, n, m, d = g.shape
    return g.reshape(b, n // n_rep, n_rep, m, d).sum(dim=2)


def _heads(x2, B, M, n):
    """[B*M, n*d] (contiguous) -> [B, n, M, d] view."""
    return x2.view(B, M, n, -1).transpose(1, 2)


def _hidden(xh):
    """[B, n, M, d] -> contiguous [B*M, n*d]."""
    b, n, m, d = xh.shape
    return xh.transpose(1, 2).reshape(b * m, n * d)


def _matmul_to_hidden(a4, b4, out=None):
    """[B, n, M, K] @ [B, n, K, d] -> contiguous [B*M, n*d]: every batch's product is written by the library GEMM
    straight into the hidden layout (an [n, M, d] view with strides (d, n*d, 1)), no transposing copy.  ``out``: a
    contiguous [B*M, n*d] tensor to write into."""
    B, n, M, _ = a4.shape
    d = b4.shape[-1]
    out = torch.empty((B, M, n, d), dtype=a4.dtype, device=a4.device) if out is None else out.view(B, M, n, d)
    for b in range(B):
        torch.bmm(a4[b], b4[b], out=out[b].transpose(0, 1))
    return out.view(B * M, n * d)


def _project(xn2, w, a, b, q_bit, calib, sv, it, thd, status, B, bias=None, xa=None):
    """One LoRA projection and the save of its main branch -> (y [T,N], q_main, scale, xa [T,r]).  ``xa`` = x A^T when
    the caller has it already."""
    if not calib and bias is None:
        scale = sv['scale']
        y, qm, xa = linear_lora_save(xn2, w, a, b, scale, q_bit, status=status, xa=xa)
        return y, qm, scale, xa
    # calibration iterations (the scale depends on the finished main branch) and projections with a bias
    main = gemm(xn2, w, status=status)
    if bias is not None:
        main = main + bias.to(main.dtype)
    qm, scale = cf.compression_pack_quant_base(main.view(B, main.shape[0] // B, -1), q_bit, 'per-channel', it, thd, sv)
    if xa is None:
        xa = (xn2 @ a.t()).contiguous()
    y = main + xa @ b.t()
    return y, qm.reshape(main.shape[0], -1), scale, xa


def attention_forward(x, w: AttnWeights, state: AttnState, cos, sin, attention_mask, num_heads, head_dim,
                      num_key_value_heads, eps=1e-5, status=None):
    """-> (x_medium [B,M,H], saved dict).  Advances the calibration state like the layer does."""
    require_cuda(x)
    B, M, H = x.shape
    T, q = B * M, state.q_bit
    st = status if status is not None else _status_tensor(x.device)
    it, thd = state.iteration, state.iteration_threshold
    calib = it < thd
    sv = state.static_value
    n_rep = num_heads // num_key_value_heads

    if calib:
        x_norm, _, rstd, _, _ = rmsnorm_forward(x, w.norm_w, eps)
        x_o, x_q, x_idx, x_scale = cf.compression_pack_channel_base(x, state.layernorm_outlier_ratio, q, 'per-channel',
                                                                    it, thd, sv['x'])
        xn_q, xn_scale = cf.compression_pack_quant_base(x_norm, q, 'per-channel', it, thd, sv['x_norm_1'])
    else:
        x_idx, x_scale, xn_scale = sv['x']['outlier_channel_index'], sv['x']['scale'], sv['x_norm_1']['scale']
        x_norm, rstd, x_o, x_q, xn_q = rmsnorm_forward_save(x, w.norm_w, eps, q, x_scale, x_idx, xn_scale)
    xn2 = x_norm.reshape(T, H)

    xa3 = lora_a_products(xn2, w.padded()["aqkv_t"])         # x_norm @ Aq^T, Ak^T, Av^T in one call
    qy, q_q, q_scale, q_xa = _project(xn2, w.wq, w.aq, w.bq, q, calib, sv['q'], it, thd, st, B, w.bias_q, xa3[0])
    ky, k_q, k_scale, k_xa = _project(xn2, w.wk, w.ak, w.bk, q, calib, sv['k'], it, thd, st, B, w.bias_k, xa3[1])
    vy, v_q, v_scale, v_xa = _project(xn2, w.wv, w.av, w.bv, q, calib, sv['v'], it, thd, st, B, w.bias_v, xa3[2])
    del x_norm, xn2

    rope_inplace(qy.view(B, M, num_heads, head_dim), cos, sin)
    rope_inplace(ky.view(B, M, num_key_value_heads, head_dim), cos, sin)
    qh = _heads(qy, B, M, num_heads)
    kh = _repeat_kv(_heads(ky, B, M, num_key_value_heads), n_rep)
    vh = _repeat_kv(_heads(vy, B, M, num_key_value_heads), n_rep)
    scores = torch.matmul(qh, kh.transpose(-2, -1))
    if state.map_mode == "topk" and state.fuse_softmax_with_save:
        # scale + mask + softmax and the save of the map in one pass over the scores
        a, a_saved = softmax_forward_topk_save(scores, 1.0 / math.sqrt(head_dim), attention_mask,
                                               state.softmax_outlier_ratio, state.map_q_bit, inplace=True)
    else:
        a = softmax_forward_scale_mask(scores, 1.0 / math.sqrt(head_dim), attention_mask, inplace=True)
        a_saved = None
    del scores

    if state.map_mode == "topk":
        if a_saved is None:
            a_saved = cf.compression_softmax_topk(a, state.softmax_outlier_ratio, state.map_q_bit)
        a_thr = None
    elif state.map_mode == "prune":
        if calib:
            a_saved, a_thr = cf.compression_pack_softmax_base(a, state.softmax_outlier_ratio, it, thd, sv['a'])
        else:
            # steady state: the calibrated threshold as a host number (read once), fixed-capacity buffers and the
            # count left on the device -> no host synchronisation in the step
            if state.threshold_host is None:
                state.threshold_host = float(sv['a']['outlier'])
            a_thr = None
            a_saved = cf.compression_softmax_static(a, state.threshold_host, ratio=state.softmax_outlier_ratio,
                                                    margin=state.prune_capacity_margin)
    else:
        raise ValueError("map_mode must be 'topk' or 'prune'")
    o2 = _matmul_to_hidden(a, vh)
    a_shape = tuple(a.shape)
    del a

    pad = w.padded()
    o_xa64 = o2 @ pad["ao_cols"]
    x_medium = gemm(o2, w.wo, a2=o_xa64, b2=pad["bo_cols"], residual=x.reshape(T, H).to(BF16).contiguous(), status=st)
    if w.bias_o is not None:
        x_medium += w.bias_o.to(BF16)
    o_q, o_scale = cf.compression_pack_quant_base(o2.view(B, M, -1), q, 'per-channel', it, thd, sv['o'])

    if calib:
        sv['x'] = cf.update_dict(sv['x'], {'outlier_channel_index': x_idx, 'scale': x_scale}, it)
        sv['x_norm_1'] = cf.update_dict(sv['x_norm_1'], {'scale': xn_scale}, it)
        sv['q'] = cf.update_dict(sv['q'], {'scale': q_scale}, it)
        sv['k'] = cf.update_dict(sv['k'], {'scale': k_scale}, it)
        sv['v'] = cf.update_dict(sv['v'], {'scale': v_scale}, it)
        if a_thr is not None:
            sv['a'] = cf.update_dict(sv['a'], {'outlier': a_thr}, it)
        sv['o'] = cf.update_dict(sv['o'], {'scale': o_scale}, it)
    state.iteration += 1

    saved = dict(rstd=rstd, x_o=x_o, x_q=x_q, x_scale=x_scale, x_idx=x_idx, xn_q=xn_q, xn_scale=xn_scale,
                 q_q=q_q, q_scale=q_scale, k_q=k_q, k_scale=k_scale, v_q=v_q, v_scale=v_scale,
                 q_xa=q_xa, k_xa=k_xa, v_xa=v_xa, qkv_xa=xa3, a_saved=a_saved, a_shape=a_shape, map_mode=state.map_mode,
                 o_q=o_q.reshape(T, -1), o_scale=o_scale, o_xa=o_xa64[:, :w.ao.shape[0]], q_bit=q, shape=(B, M, H),
                 cos=cos, sin=sin, num_heads=num_heads, head_dim=head_dim, num_key_value_heads=num_key_value_heads)
    return x_medium.reshape(B, M, H), saved


def _rebuild(codes, scale, xa, b, q_bit):
    """De-quantized main branch + LoRA product of a projection, [T, N] (b = lora_B.weight [N, r])."""
    T = codes.shape[0]
    return cf.decompression_dequantization_lora_add(codes.view(1, T, -1), scale, xa.view(1, T, -1), b.t(), q_bit).view(T, -1)


def _vec(s):
    return s.to(BF16).reshape(-1).contiguous()


def attention_backward(grad_medium, saved, w: AttnWeights, status=None, on_lora_grads=None):
    """-> dict(grad_x, grad_aq, grad_bq, grad_ak, grad_bk, grad_av, grad_bv, grad_ao, grad_bo), the LoRA
    gradients in the layout of the weights they belong to ([r, in] / [out, r]).  ``on_lora_grads(dict)`` is
    called once the eight LoRA gradients are enqueued (before the grad_x GEMM and the RMSNorm backward)."""
    B, M, H = saved['shape']
    T, q = B * M, saved['q_bit']
    nh, d, nkv = saved['num_heads'], saved['head_dim'], saved['num_key_value_heads']
    n_rep = nh // nkv
    cos, sin = saved['cos'], saved['sin']
    dev = grad_medium.device
    st = status if status is not None else _status_tensor(dev)
    g = grad_medium.to(BF16).reshape(T, H).contiguous()
    pad = w.padded()
    r = w.ao.shape[0]

    # ---- o projection
    gm64 = g @ pad["bo_cols"]                                # [T, 64]; first r columns = g @ Bo
    grad_bo = g.t() @ saved['o_xa']                          # [H, r]
    grad_ao = lora_grad_a(saved['o_q'], _vec(saved['o_scale']), gm64, 16, q)[:r]     # [r, heads*d], o de-quantized in the kernel
    grad_o2 = gemm(g, w.wo, b_is_kn=True, a2=gm64, b2=pad["ao_rows"], status=st)      # [T, heads*d]
    grad_oh = _heads(grad_o2, B, M, nh)

    # ---- P.V backward on the restored map
    m = saved['a_saved']
    if saved['map_mode'] == "topk":
        a = m.to_dense()
    else:
        a = m.to_dense().reshape(saved['a_shape']) if isinstance(m, (cf.PrunedMap, cf.TiledPrunedMap)) else \
            cf.decompression_softmax(m).reshape(saved['a_shape'])
    v2 = _rebuild(saved['v_q'], saved['v_scale'], saved['v_xa'], w.bv, q)
    vh = _repeat_kv(_heads(v2, B, M, nkv), n_rep)
    # without grouped key/value heads grad_q, grad_k and grad_v have one shape: kept in one buffer, their rank-16
    # products below run as one batched library call each
    gqkv = torch.empty((3, T, nh * d), dtype=BF16, device=dev) if n_rep == 1 else None
    if n_rep == 1:
        grad_v = _matmul_to_hidden(a.transpose(-2, -1), grad_oh, out=gqkv[2])
    else:
        grad_v = _hidden(_repeat_kv_backward(torch.matmul(a.transpose(-2, -1), grad_oh), n_rep))
    grad_a = torch.matmul(grad_oh, vh.transpose(-2, -1))
    del vh, v2
    # ---- softmax backward (for the top-k form fused with a second restore: the map is not re-read)
    if saved['map_mode'] == "topk":
        del a
        grad_s = m.softmax_backward(grad_a, scale=1.0 / math.sqrt(d))
        del grad_a
    else:
        grad_s = softmax_backward(a, grad_a, scale=1.0 / math.sqrt(d))
        del a

    # ---- q, k rebuilt from their codes, rotary re-applied
    q2 = _rebuild(saved['q_q'], saved['q_scale'], saved['q_xa'], w.bq, q)
    rope_inplace(q2.view(B, M, nh, d), cos, sin)
    if n_rep == 1:
        grad_k = _matmul_to_hidden(grad_s.transpose(-2, -1), _heads(q2, B, M, nh), out=gqkv[1])
    else:
        grad_k = _hidden(_repeat_kv_backward(torch.matmul(grad_s.transpose(-2, -1), _heads(q2, B, M, nh)), n_rep))
    del q2
    k2 = _rebuild(saved['k_q'], saved['k_scale'], saved['k_xa'], w.bk, q)
    rope_inplace(k2.view(B, M, nkv, d), cos, sin)
    grad_q = _matmul_to_hidden(grad_s, _repeat_kv(_heads(k2, B, M, nkv), n_rep), out=None if gqkv is None else gqkv[0])
    del k2, grad_s
    rope_inplace(grad_q.view(B, M, nh, d), cos, sin, backward=True)
    rope_inplace(grad_k.view(B, M, nkv, d), cos, sin, backward=True)

    # ---- q/k/v projections: LoRA gradients, then grad_x_norm as one GEMM over the three K segments
    gmq = padded_block(w, "_gmq", T, dev)                    # g_q @ Bq | g_k @ Bk | g_v @ Bv side by side
    qkv_xa = saved.get('qkv_xa')
    if gqkv is not None and r == 16:
        # (B200, 2048 tokens: 11.5 us against 25.6 us as three products, 9.9 us against 19.7 us for the B gradients)
        gmq.view(T, 4, 16)[:, :3].copy_(torch.bmm(gqkv, pad["bqkv"]).transpose(0, 1))
        if qkv_xa is None:
            qkv_xa = torch.stack((saved['q_xa'], saved['k_xa'], saved['v_xa']))
        grad_b3 = torch.bmm(gqkv.transpose(1, 2), qkv_xa)     # [3, heads*d, r]
    else:
        torch.mm(grad_q, w.bq, out=gmq[:, :r])
        torch.mm(grad_k, w.bk, out=gmq[:, r:2 * r])
        torch.mm(grad_v, w.bv, out=gmq[:, 2 * r:3 * r])
        grad_b3 = None
    ga = lora_grad_a(saved['xn_q'].reshape(T, -1), _vec(saved['xn_scale']), gmq, 48, q)
    grad_aq, grad_ak, grad_av = ga[:r], ga[r:2 * r], ga[2 * r:3 * r]
    if grad_b3 is not None:
        grad_bq, grad_bk, grad_bv = grad_b3[0], grad_b3[1], grad_b3[2]
    else:
        grad_bq = grad_q.t() @ saved['q_xa']
        grad_bk = grad_k.t() @ saved['k_xa']
        grad_bv = grad_v.t() @ saved['v_xa']
    if on_lora_grads is not None:
        on_lora_grads(dict(grad_aq=grad_aq, grad_bq=grad_bq, grad_ak=grad_ak, grad_bk=grad_bk, grad_av=grad_av,
                           grad_bv=grad_bv, grad_ao=grad_ao, grad_bo=grad_bo))
    lora_x = gmq @ pad["aqkv_rows"]                          # [T, H]: the three LoRA-A back-projections
    grad_xn = gemm(grad_q, w.wq, b_is_kn=True, a2=grad_k, b2=w.wk, a3=grad_v, b3=w.wv, residual=lora_x, status=st)
    grad_x = rmsnorm_backward_packed(grad_xn.reshape(B, M, H), saved['x_q'], saved['x_scale'], saved['x_o'],
                                     saved['x_idx'], w.norm_w, saved['rstd'], q, residual_grad=g.reshape(B, M, H))
    return dict(grad_x=grad_x, grad_aq=grad_aq, grad_bq=grad_bq, grad_ak=grad_ak, grad_bk=grad_bk,
                grad_av=grad_av, grad_bv=grad_bv, grad_ao=grad_ao, grad_bo=grad_bo,
                grad_q=grad_q, grad_k=grad_k, grad_v=grad_v)
