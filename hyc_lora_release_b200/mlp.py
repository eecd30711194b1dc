"""MLP half of the HyC-LoRA fused decoder layer on the tcgen05 kernels.

Mirrors the MLP part of ``FusedLlamaLayerIntraInterFullFuseFunc.forward/backward``
(models/llama/fused_llama_layer_intra_inter_full_fuse.py:203-252 and :359-396; the Mistral
twin is identical for this part) with plain bf16 frozen weights:

  forward : RMSNorm -> save x (outlier channels + per-channel codes) -> gate/up GEMMs with the
            quantizer, LoRA add, SiLU and Hadamard in the GEMM epilogue -> save x_norm codes ->
            down GEMM with LoRA add and residual in the epilogue;
  backward: grad_down GEMM with the de-quantize / recompute / SiLU-Hadamard backward in the
            epilogue -> LoRA gradients -> grad_x GEMM (gate and up accumulated in one tile) ->
            RMSNorm backward on the restored x.

Only packed codes, scales, the outlier slab, the rank-16 LoRA activations and rstd are kept
between the two passes.  Weights use the nn.Linear layout ([out, in]); the LoRA factors are
``lora_A.weight`` [r, in] and ``lora_B.weight`` [out, r].
"""
import ctypes
from dataclasses import dataclass, field
from typing import Optional

import torch

from ._lib import HycError, check, lib, ptr, require_cuda, stream_of
from .operators import compress_function as cf
from .operators.rmsnorm_kernels import rmsnorm_backward_packed, rmsnorm_forward, rmsnorm_forward_save

BF16 = torch.bfloat16
_KERNEL_STATUS = {1: "TMA producer wait timed out", 2: "MMA issuer wait timed out", 3: "epilogue wait timed out"}


def _status_tensor(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status, what):
    """Raise if a bounded wait inside a tcgen05 kernel gave up (synchronises)."""
    v = int(status.item())
    if v != 0:
        raise HycError("%s: %s" % (what, _KERNEL_STATUS.get(v, "status %d" % v)))


def padded_block(owner, name, T, dev):
    """A [T, 64] bf16 block of zeros kept on ``owner`` between steps (the rank-16 products of a backward pass are
    written side by side into its first columns and ride a GEMM as one K block of 64; the other columns are never
    written and stay zero, so the block is filled once, not once per step)."""
    buf = getattr(owner, name, None)
    if buf is None or buf.shape[0] != T or buf.device != dev:
        buf = torch.zeros((T, 64), dtype=BF16, device=dev)
        setattr(owner, name, buf)
    return buf


def _lora(xa, bt, ld_col, ld_r):
    if xa is None:
        return [None, None, 0, 0]
    return [ptr(xa), ptr(bt), ld_col, ld_r]


def gemm(a, b, *, b_is_kn=False, a2=None, b2=None, a3=None, b3=None, lora0=None, lora1=None, residual=None,
         status=None):
    """D = a @ op(b) (+ a2 @ op(b2)) (+ a3 @ op(b3)) (+ LoRA terms) (+ residual) on the tcgen05 kernel.

    a [M,K] bf16; b [N,K] (b_is_kn=False) or [K,N] (b_is_kn=True), both row-major.
    lora = (xa [M,16], bt, ld_col, ld_r): adds xa @ Bt^T with Bt(col, r) = bt[col*ld_col + r*ld_r]."""
    require_cuda(a, b)
    M, K = a.shape
    N = b.shape[1] if b_is_kn else b.shape[0]
    K2 = 0 if a2 is None else a2.shape[1]
    K3 = 0 if a3 is None else a3.shape[1]
    d = torch.empty((M, N), dtype=BF16, device=a.device)
    st = status if status is not None else _status_tensor(a.device)
    l0 = _lora(*lora0) if lora0 else [None, None, 0, 0]
    l1 = _lora(*lora1) if lora1 else [None, None, 0, 0]
    check(lib.hyc_gemm_bf16_tcgen05(ptr(a), ptr(b), M, N, K, 1 if b_is_kn else 0, ptr(a2), ptr(b2), K2,
                                    ptr(a3), ptr(b3), K3, *l0, *l1, ptr(residual), ptr(d), ptr(st), stream_of(a)),
          "hyc_gemm_bf16_tcgen05")
    return d


def lora_a_products(x2, stacked):
    """x2 [T, K] times several LoRA-A factors at once: ``stacked`` [n, K, r] holds their transposes; one batched library
    call whose left operand is the same x2 for every batch (stride 0), -> [n, T, r], each [T, r] contiguous.  Measured
    on a B200, x2 [2048, 4096]: 9.5 us for three factors against 20.5 us as three products."""
    return torch.bmm(x2.unsqueeze(0).expand(stacked.shape[0], -1, -1), stacked)


def linear_lora_save(x, w, a, b, scale, q_bit, *, want_main=False, status=None, xa=None):
    """A LoRA projection with the save of its main branch in the GEMM epilogue (steady state of the q/k/v/o
    projections): x [T,K], w [N,K], a = lora_A.weight [r,K], b = lora_B.weight [N,r], scale [N] ->
    (y [T,N], q_main [T, N*q_bit/8], xa [T,r][, main])."""
    require_cuda(x, w, a, b, scale)
    T, K = x.shape
    N = w.shape[0]
    if xa is None:
        xa = (x @ a.t()).contiguous()
    dev = x.device
    y = torch.empty((T, N), dtype=BF16, device=dev)
    qm = torch.empty((T, N * q_bit // 8), dtype=torch.uint8, device=dev)
    main = torch.empty((T, N), dtype=BF16, device=dev) if want_main else None
    st = status if status is not None else _status_tensor(dev)
    sc = scale.to(BF16).reshape(-1).contiguous()
    check(lib.hyc_linear_lora_save_fwd_tcgen05(ptr(x), ptr(w), T, K, N, ptr(xa), ptr(b.contiguous()), b.shape[1], 1,
                                               ptr(sc), ptr(qm), ptr(y), ptr(main), q_bit, ptr(st), stream_of(x)),
          "hyc_linear_lora_save_fwd_tcgen05")
    return (y, qm, xa, main) if want_main else (y, qm, xa)


def lora_grad_a(q, scale, gm, r2, q_bit):
    """out [r2, H] = gm[:, :r2]^T @ dequant(q, scale), the packed activation de-quantized inside the kernel.
    q [T, H*q_bit/8] uint8, scale [H] bf16, gm [T, >= r2] bf16 (row stride a multiple of 8)."""
    require_cuda(q, scale, gm)
    T = q.shape[0]
    H = scale.numel()
    out = torch.empty((r2, H), dtype=BF16, device=q.device)
    nbytes = lib.hyc_lora_grad_a_workspace_bytes(T, H, r2)
    ws = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
    check(lib.hyc_lora_grad_a_dequant(ptr(q), ptr(scale), ptr(gm), gm.stride(0), r2, T, H, q_bit, ptr(out), ptr(ws),
                                      nbytes, stream_of(q)), "hyc_lora_grad_a_dequant")
    return out


@dataclass
class MLPWeights:
    """Frozen bf16 weights ([out, in]) and LoRA factors of one MLP."""
    norm_w: torch.Tensor   # [H]
    wg: torch.Tensor       # [I, H]
    wu: torch.Tensor       # [I, H]
    wd: torch.Tensor       # [H, I]
    ag: torch.Tensor       # gate lora_A.weight [r, H]
    bg: torch.Tensor       # gate lora_B.weight [I, r]
    au: torch.Tensor
    bu: torch.Tensor
    ad: torch.Tensor       # down lora_A.weight [r, I]
    bd: torch.Tensor       # down lora_B.weight [H, r]
    bias_d: Optional[torch.Tensor] = None    # bias of the down projection ([H] bf16) or None; no gradient

    def padded(self):
        """LoRA factors zero-padded to a K of 64 so that a rank-16 product can ride along a GEMM as one more
        K block (built once per optimizer step; a few hundred KB):
          ad_rows  [64, I]  rows 0..15 = Ad            (second operand of grad_down's LoRA part, [K, N])
          ad_cols  [I, 64]  columns 0..15 = Ad^T       (projects hadamard to the padded down LoRA activation)
          bd_cols  [H, 64]  columns 0..15 = Bd         (second operand of the down projection's LoRA part, [N, K])
          agu_rows [64, H]  rows 0..15 = Ag, 16..31 = Au (second operand of grad_x's LoRA part, [K, N])
        and the stacked factors of the batched rank-16 products:
          agu_t    [2, H, r]  Ag^T, Au^T  (x_norm @ both in one call)
          bgu      [2, I, r]  Bg, Bu      (grad_gate @ Bg and grad_up @ Bu in one call)"""
        key = tuple(t._version for t in (self.ag, self.au, self.ad, self.bd, self.bg, self.bu))
        if getattr(self, "_pad_key", None) != key:
            r, I = self.ad.shape
            H = self.bd.shape[0]
            dev, dt = self.ad.device, self.ad.dtype
            ad_rows = torch.zeros(64, I, dtype=dt, device=dev); ad_rows[:r] = self.ad
            bd_cols = torch.zeros(H, 64, dtype=dt, device=dev); bd_cols[:, :r] = self.bd
            agu_rows = torch.zeros(64, H, dtype=dt, device=dev); agu_rows[:r] = self.ag; agu_rows[r:2 * r] = self.au
            agu_t = torch.stack((self.ag.t(), self.au.t())).contiguous()      # [2, H, r]
            bgu = torch.stack((self.bg, self.bu)).contiguous()                # [2, I, r]
            self._pad = dict(ad_rows=ad_rows, ad_cols=ad_rows.t().contiguous(), bd_cols=bd_cols, agu_rows=agu_rows,
                             agu_t=agu_t, bgu=bgu)
            self._pad_key = key
        return self._pad


@dataclass
class MLPState:
    """Calibration state of the MLP part of a layer (the reference keeps the same entries in
    ``static_value``, fused_llama_layer_intra_inter_full_fuse.py:557-570)."""
    iteration: int = 0
    iteration_threshold: int = 5
    q_bit: int = 4
    layernorm_outlier_ratio: float = 0.005
    static_value: dict = field(default_factory=lambda: {
        'x_medium': {'outlier_channel_index': None, 'scale': None},
        'x_norm_2': {'scale': None}, 'gate': {'scale': None}, 'up': {'scale': None}})


def mlp_forward(x_medium, w: MLPWeights, state: MLPState, eps=1e-5, status=None):
    """-> (x_out [B,M,H], saved tuple).  Advances the calibration state like the layer does."""
    require_cuda(x_medium)
    B, M, H = x_medium.shape
    T, I, q = B * M, w.wg.shape[0], state.q_bit
    st = status if status is not None else _status_tensor(x_medium.device)
    calib = state.iteration < state.iteration_threshold
    sv = state.static_value

    if calib:
        x_norm, _, rstd, _, _ = rmsnorm_forward(x_medium, w.norm_w, eps)
        xm_o, xm_q, xm_idx, xm_scale = cf.compression_pack_channel_base(
            x_medium, state.layernorm_outlier_ratio, q, 'per-channel', state.iteration, state.iteration_threshold,
            sv['x_medium'])
        xn_q = None
    else:
        # steady state: the norm, the save of its input (codes + outlier channels) and the save of its output
        # are one pass over x_medium
        xm_idx, xm_scale, xn_scale = sv['x_medium']['outlier_channel_index'], sv['x_medium']['scale'], sv['x_norm_2']['scale']
        x_norm, rstd, xm_o, xm_q, xn_q = rmsnorm_forward_save(x_medium, w.norm_w, eps, q, xm_scale, xm_idx, xn_scale)
    xn2 = x_norm.reshape(T, H)
    gu_xa = lora_a_products(xn2, w.padded()["agu_t"])                # x_norm @ Ag^T and x_norm @ Au^T in one call
    gate_xa, up_xa = gu_xa[0], gu_xa[1]
    dev = x_medium.device
    epp = 8 // q
    q1 = torch.empty((B, M, I // epp), dtype=torch.uint8, device=dev)
    q2 = torch.empty((B, M, I // epp), dtype=torch.uint8, device=dev)
    had = torch.empty((B, M, I), dtype=BF16, device=dev)

    def gateup(s1, s2, m1=None, m2=None):
        check(lib.hyc_mlp_gateup_fwd_tcgen05(
            ptr(xn2), ptr(w.wg), ptr(w.wu), T, H, I,
            ptr(gate_xa), ptr(w.bg), 16, 1, ptr(up_xa), ptr(w.bu), 16, 1,
            ptr(s1), ptr(s2), ptr(q1), ptr(q2), ptr(had), ptr(m1), ptr(m2), q, ptr(st), stream_of(x_medium)),
            "hyc_mlp_gateup_fwd_tcgen05")

    if calib:
        # calibration iterations: the scales depend on the finished main branches, so the GEMM runs
        # twice (first pass only materialises gate_main / up_main); steady state is single-pass
        ones = torch.ones(I, dtype=BF16, device=dev)
        m1 = torch.empty((B, M, I), dtype=BF16, device=dev)
        m2 = torch.empty((B, M, I), dtype=BF16, device=dev)
        gateup(ones, ones, m1, m2)
        gate_scale = cf.get_statistics_only_quant(m1, q, 'per-channel')
        up_scale = cf.get_statistics_only_quant(m2, q, 'per-channel')
        del m1, m2
    else:
        gate_scale, up_scale = sv['gate']['scale'], sv['up']['scale']
    gs = gate_scale.to(BF16).reshape(-1).contiguous()
    us = up_scale.to(BF16).reshape(-1).contiguous()
    gateup(gs, us)

    if xn_q is None:
        xn_q, xn_scale = cf.compression_pack_quant_base(x_norm, q, 'per-channel', state.iteration,
                                                        state.iteration_threshold, sv['x_norm_2'])
    had2 = had.reshape(T, I)
    pad = w.padded()
    down_xa64 = had2 @ pad["ad_cols"]              # [T, 64]: the LoRA-A activation of the down projection, zero-padded
    down_xa = down_xa64[:, :16]
    # down = hadamard @ Wd^T + down_xa @ Bd^T (one more K block) + residual
    x_out = gemm(had2, w.wd, a2=down_xa64, b2=pad["bd_cols"], residual=x_medium.reshape(T, H).contiguous(), status=st)
    if w.bias_d is not None:
        x_out += w.bias_d.to(BF16)

    if calib:
        it = state.iteration
        sv['x_medium'] = cf.update_dict(sv['x_medium'], {'outlier_channel_index': xm_idx, 'scale': xm_scale}, it)
        sv['x_norm_2'] = cf.update_dict(sv['x_norm_2'], {'scale': xn_scale}, it)
        sv['gate'] = cf.update_dict(sv['gate'], {'scale': gate_scale}, it)
        sv['up'] = cf.update_dict(sv['up'], {'scale': up_scale}, it)
    state.iteration += 1

    saved = dict(rstd=rstd, xm_o=xm_o, xm_q=xm_q, xm_scale=xm_scale, xm_idx=xm_idx, xn_q=xn_q, xn_scale=xn_scale,
                 gate_q=q1, gate_scale=gs, up_q=q2, up_scale=us, gate_xa=gate_xa, up_xa=up_xa, gu_xa=gu_xa, down_xa=down_xa,
                 q_bit=q, shape=(B, M, H))
    return x_out.reshape(B, M, H), saved


def mlp_backward(grad_out, saved, w: MLPWeights, status=None, on_lora_grads=None):
    """-> dict(grad_x, grad_ag, grad_bg, grad_au, grad_bu, grad_ad, grad_bd); LoRA gradients in the
    layout of the weights they belong to ([r, in] / [out, r]).  ``on_lora_grads(dict)`` (optional) is called
    as soon as the six LoRA gradients are enqueued, before the grad_x GEMM and the RMSNorm backward: the
    place to start their all-reduce so that it overlaps the rest of the pass."""
    B, M, H = saved['shape']
    T, I, q = B * M, w.wg.shape[0], saved['q_bit']
    dev = grad_out.device
    st = status if status is not None else _status_tensor(dev)
    g = grad_out.to(BF16).reshape(T, H).contiguous()
    down_xa, gate_xa, up_xa = saved['down_xa'], saved['gate_xa'], saved['up_xa']

    pad = w.padded()
    grad_bd = g.t() @ down_xa                      # [H, r]
    gdm64 = g @ pad["bd_cols"]                     # [T, 64], first 16 columns = g @ Bd
    gdm = gdm64[:, :16]
    had = torch.empty((T, I), dtype=BF16, device=dev)
    ggu = torch.empty((2, T, I), dtype=BF16, device=dev)       # grad_gate and grad_up in one buffer: their rank-16
    gg, gu = ggu[0], ggu[1]                                    # products below run as one batched call each
    check(lib.hyc_mlp_graddown_bwd_tcgen05(
        ptr(g), ptr(w.wd), T, H, I, ptr(gdm64), ptr(pad["ad_rows"]), 64,
        ptr(gate_xa), ptr(w.bg), 16, 1, ptr(up_xa), ptr(w.bu), 16, 1,
        ptr(saved['gate_q']), ptr(saved['gate_scale']), ptr(saved['up_q']), ptr(saved['up_scale']),
        None, None, 0,
        ptr(had), ptr(gg), ptr(gu), q, ptr(st), stream_of(grad_out)), "hyc_mlp_graddown_bwd_tcgen05")
    grad_ad = gdm.t() @ had                        # [r, I]

    gm64 = padded_block(w, "_gm64", T, dev)
    # g_gate @ Bg and g_up @ Bu ([T, r] each) as one batched product, then side by side into the zero-padded K block
    # (B200, 2048 tokens: 19.8 us against 34.1 us as two products)
    gm64.view(T, 4, 16)[:, :2].copy_(torch.bmm(ggu, pad["bgu"]).transpose(0, 1))
    # LoRA-A gradients of gate and up in one pass over the packed x_norm (de-quantized in shared memory)
    ga = lora_grad_a(saved['xn_q'].reshape(T, -1), saved['xn_scale'].to(BF16).reshape(-1).contiguous(), gm64, 32, q)
    grad_ag, grad_au = ga[:16], ga[16:32]          # [r, H] each
    gu_xa = saved.get('gu_xa')
    if gu_xa is None:
        gu_xa = torch.stack((gate_xa, up_xa))
    grad_bgu = torch.bmm(ggu.transpose(1, 2), gu_xa)           # [2, I, r]
    grad_bg, grad_bu = grad_bgu[0], grad_bgu[1]
    if on_lora_grads is not None:
        on_lora_grads(dict(grad_ag=grad_ag, grad_bg=grad_bg, grad_au=grad_au, grad_bu=grad_bu, grad_ad=grad_ad,
                           grad_bd=grad_bd))
    # grad wrt x_norm: gate and up products accumulate in one tensor-memory tile
    grad_xn = gemm(gg, w.wg, b_is_kn=True, a2=gu, b2=w.wu, a3=gm64, b3=pad["agu_rows"], status=st)
    # RMSNorm backward straight from the saved form of x_medium, residual gradient added in the same pass
    grad_x = rmsnorm_backward_packed(grad_xn.reshape(B, M, H), saved['xm_q'], saved['xm_scale'], saved['xm_o'],
                                     saved['xm_idx'], w.norm_w, saved['rstd'], q, residual_grad=g.reshape(B, M, H))
    return dict(grad_x=grad_x, grad_ag=grad_ag, grad_bg=grad_bg, grad_au=grad_au, grad_bu=grad_bu,
                grad_ad=grad_ad, grad_bd=grad_bd, hadamard=had, g_gate=gg, g_up=gu)
