"""The fused decoder layer: drop-in for ``FusedLlamaLayerIntraInterFullFuse`` / ``...Func``
(models/llama/fused_llama_layer_intra_inter_full_fuse.py:29-708) and its Mistral twin
(models/mistral/fused_mistral_layer_intra_inter_full_fuse.py), on the sm_100a kernels.

The module keeps the reference's interface: ``set_hyclora_config(cfg)``, the ``iteration`` counter and the
``static_value`` dictionary of calibrated statistics, and a ``forward`` that takes the norm weights, the rotary
tables, the frozen ``*_proj_base`` modules and their ``*_proj_lora_a/b`` adapter dictionaries, the additive
attention mask and the head geometry.  Differences, all deliberate:

  * frozen weights are plain bf16 ``[out, in]`` matrices, or 4-bit block-wise weights in the storage format of
    bitsandbytes (packed codes with a ``quant_state``), de-quantized to bf16 for each pass by a kernel of this
    package (``nf4.py``; the library itself is not part of this build, parity with it is unpinned);
  * projection biases of q/k/v/o/down are added to the main branch (separate launches for such a projection);
    gate/up biases are refused (the reference's fused layer drops them);
  * ``hyclora_config.softmax_map_mode`` (optional, default ``"prune"`` = the reference's threshold prune) may
    be ``"topk"`` for the per-row top-k + 4-bit-group form of the saved probability map.

After the calibration iterations a step launches a fixed sequence of kernels with no host synchronisation in
either mode: the ``"prune"`` mode then keeps its list in buffers of a fixed capacity (1.5 x ratio x numel entries,
``AttnState.prune_capacity_margin``) with the count left on the device, instead of a sparse tensor whose size the
host has to read back.
"""
import torch

from .attention import AttnState, AttnWeights, attention_backward, attention_forward
from . import nf4
from .mlp import MLPState, MLPWeights, _status_tensor, check_status, mlp_backward, mlp_forward

BF16 = torch.bfloat16

def saved_nbytes(saved):
    """Bytes of device memory a ``saved`` dictionary of ``attention_forward`` / ``mlp_forward`` keeps alive between
    the two passes (tensors, the top-k map handle, a sparse COO map); the shared rotary tables are not counted."""
    total = 0
    for key, v in saved.items():
        if key in ("cos", "sin", "gu_xa", "qkv_xa"):      # shared tables; stacked views of tensors counted under their own keys
            continue
        if isinstance(v, torch.Tensor):
            if v.is_sparse:
                total += v.indices().numel() * 8 + v.values().numel() * v.values().element_size()
            else:
                total += v.numel() * v.element_size()
        elif hasattr(v, "nbytes") and callable(v.nbytes):
            total += v.nbytes()
    return total


class FusedLayerFunction(torch.autograd.Function):
    """forward(x, module, aw, mw, cos, sin, mask, heads, head_dim, kv_heads, *fourteen LoRA weights).
    The LoRA weights are listed as inputs only so that autograd routes their gradients; the computation reads
    them from ``aw`` / ``mw``.  Gradients come back in the layout of the weights ([r, in] and [out, r])."""

    @staticmethod
    def forward(ctx, x, module, aw, mw, cos, sin, attention_mask, num_heads, head_dim, num_key_value_heads, *lora):
        st = module._status_for(x.device)
        # 4-bit frozen weights become bf16 for the duration of the half that uses them, as in the reference
        # (BF.dequantize_nf4 before every frozen matmul); records without such weights pass through unchanged
        aw_now = nf4.materialize(aw)
        x_medium, sa = attention_forward(x, aw_now, module.attn_state, cos, sin, attention_mask, num_heads, head_dim,
                                         num_key_value_heads, status=st)
        nf4.release(aw, aw_now)
        del aw_now
        mw_now = nf4.materialize(mw)
        y, sm = mlp_forward(x_medium, mw_now, module.mlp_state, status=st)
        nf4.release(mw, mw_now)
        del mw_now
        if module.track_saved_bytes:
            module.last_saved_bytes = saved_nbytes(sa) + saved_nbytes(sm)
        if module.keep_saved:
            module.last_saved = (sa, sm)
        ctx.hyc = (sa, sm, aw, mw, st, module, x.dtype)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, grad_y):
        sa, sm, aw, mw, st, module, x_dtype = ctx.hyc
        ctx.hyc = None
        hook = module.on_lora_grads
        mw_now = nf4.materialize(mw)
        gm = mlp_backward(grad_y, sm, mw_now, status=st, on_lora_grads=hook)
        nf4.release(mw, mw_now)
        del mw_now
        saved_map = sa.get('a_saved')
        aw_now = nf4.materialize(aw)
        ga = attention_backward(gm['grad_x'], sa, aw_now, status=st, on_lora_grads=hook)
        nf4.release(aw, aw_now)
        del aw_now
        # fixed-capacity prune buffers: entries beyond the capacity were dropped; the flag stays on the device
        if hasattr(saved_map, "nnz") and hasattr(saved_map, "capacity"):
            module._overflow.add_((saved_map.nnz > saved_map.capacity).to(torch.int32))
        module._steps_since_check += 1
        every = 1 if module.check_kernel_status else module.check_every
        if every and module._steps_since_check >= every and not torch.cuda.is_current_stream_capturing():
            module.raise_on_device_errors()
        grads = [ga['grad_aq'], ga['grad_bq'], ga['grad_ak'], ga['grad_bk'], ga['grad_av'], ga['grad_bv'],
                 ga['grad_ao'], ga['grad_bo'], gm['grad_ag'], gm['grad_bg'], gm['grad_au'], gm['grad_bu'],
                 gm['grad_ad'], gm['grad_bd']]
        return (ga['grad_x'].to(x_dtype),) + (None,) * 9 + tuple(grads)


def _frozen(base, name):
    """The frozen weight of a projection: a plain bf16 [out, in] matrix, or a 4-bit block-wise weight (packed codes
    with a ``quant_state``, bitsandbytes' storage format) wrapped for de-quantization pass by pass."""
    w = base.weight
    if nf4.is_quantized(w):
        qw = getattr(w, "_hyc_quantized", None)        # wrapped once per parameter (the tables move to the device once)
        if qw is None or qw.quant_state is not w.quant_state:
            qw = nf4.QuantizedWeight(w)
            w._hyc_quantized = qw
        if len(qw.shape) != 2:
            raise NotImplementedError("%s: the quant state of a projection weight must describe a matrix" % name)
        return qw
    if w.dtype != BF16:
        raise NotImplementedError("%s: frozen weights must be bf16 [out, in] matrices or 4-bit block-wise weights with "
                                  "a quant_state (got %s)" % (name, w.dtype))
    return w


def _bias(base, name):
    """Bias of a frozen projection or None.  The reference's fused layer never adds the gate and up biases it is
    handed (models/llama/fused_llama_layer_intra_inter_full_fuse.py:218-226 inlines those two projections without
    them), so a model that has them would silently compute something else there; refused here instead."""
    b = getattr(base, "bias", None)
    if b is None:
        return None
    if name in ("gate_proj", "up_proj"):
        raise NotImplementedError("%s: a bias on the gate / up projection is not supported (the reference's fused "
                                  "layer drops it)" % name)
    if b.dtype != BF16:
        raise NotImplementedError("%s: the projection bias must be bf16 (got %s)" % (name, b.dtype))
    return b


def _adapter(mod, name, rank_dim):
    """``lora_A`` / ``lora_B`` module dictionary of a PEFT layer (``.default``) or a bare ``nn.Linear``.
    The kernels are built for bf16 adapters of rank 16."""
    inner = getattr(mod, "default", mod)
    w = inner.weight
    if w.dtype != BF16:
        raise NotImplementedError("%s: LoRA adapters must be bf16 (got %s)" % (name, w.dtype))
    if w.dim() != 2 or w.shape[rank_dim] != 16:
        raise NotImplementedError("%s: LoRA rank must be 16 (weight shape %s)" % (name, tuple(w.shape)))
    return w


class FusedLlamaLayerIntraInterFullFuse(torch.nn.Module):
    """One decoder layer (attention + MLP) with compressed saved activations."""

    def __init__(self):
        super().__init__()
        self.attn_state = AttnState()
        self.mlp_state = MLPState()
        self.use_hyclora = True
        self.on_lora_grads = None          # optional callable(dict of LoRA gradients): start their all-reduce early
        self.check_kernel_status = False   # True: read the bounded-wait status word back after every backward pass
        self.track_saved_bytes = False     # True: forward records the bytes kept for backward in last_saved_bytes
        self.last_saved_bytes = None
        self.keep_saved = False            # True: forward also leaves its two saved dictionaries in last_saved (inspection)
        self.last_saved = None
        # Failures stay visible without a host synchronisation per step: the bounded-wait status word of the tensor-core
        # kernels and the overflow flag of the fixed-capacity prune buffers live in two persistent device words that
        # are read back (one synchronisation) every `check_every` backward passes; 0 = never, check_kernel_status = every pass
        self.check_every = 100
        self._status = None
        self._overflow = None
        self._steps_since_check = 0
        self._weights = None

    def _status_for(self, device):
        if self._status is None or self._status.device != device:
            self._status = torch.zeros(1, dtype=torch.int32, device=device)
            self._overflow = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status

    def raise_on_device_errors(self):
        """Read the two persistent device words (synchronises) and raise if a tensor-core kernel gave up on a bounded
        wait or the pruned probability map did not fit its buffers since the last check."""
        self._steps_since_check = 0
        if self._status is None:
            return
        st, ov = int(self._status.item()), int(self._overflow.item())
        self._status.zero_()
        self._overflow.zero_()
        if st != 0:
            check_status(torch.tensor([st]), "fused layer")
        if ov != 0:
            raise RuntimeError("fused layer: the pruned probability map overflowed its buffers in %d step(s) since the last "
                               "check (entries were dropped); raise AttnState.prune_capacity_margin" % ov)

    # ---- the reference's attributes
    @property
    def iteration(self):
        return self.attn_state.iteration

    @iteration.setter
    def iteration(self, v):
        self.attn_state.iteration = v
        self.mlp_state.iteration = v
        self.attn_state.threshold_host = None      # a re-calibration ends with another threshold

    @property
    def static_value(self):
        d = dict(self.attn_state.static_value)
        d.update(self.mlp_state.static_value)
        return d

    def set_hyclora_config(self, hyclora_config):
        self.hyclora_config = hyclora_config
        self.use_hyclora = hyclora_config.use_hyclora
        self.iteration_threshold = hyclora_config.iteration_threshold
        self.softmax_outlier_ratio = hyclora_config.softmax_outlier_ratio
        self.layernorm_outlier_ratio = hyclora_config.layernorm_outlier_ratio
        self.q_bit = hyclora_config.q_bit
        a, m = self.attn_state, self.mlp_state
        a.iteration_threshold = m.iteration_threshold = self.iteration_threshold
        a.q_bit = m.q_bit = self.q_bit
        a.layernorm_outlier_ratio = m.layernorm_outlier_ratio = self.layernorm_outlier_ratio
        a.softmax_outlier_ratio = self.softmax_outlier_ratio
        a.map_mode = getattr(hyclora_config, "softmax_map_mode", "prune")
        a.map_q_bit = getattr(hyclora_config, "softmax_map_q_bit", 4)

    def _bind(self, norm_w1, norm_w2, mods):
        """Weight records for the two halves, rebuilt only when a tensor was replaced."""
        tensors = [norm_w1, norm_w2]
        idents = [id(norm_w1), id(norm_w2)]
        biases = {}
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            base, la, lb = mods[name]
            tensors += [_frozen(base, name + "_proj"), _adapter(la, name + "_proj lora_A", 0),
                        _adapter(lb, name + "_proj lora_B", 1)]
            # (a 4-bit weight is wrapped anew on every call: the parameter it wraps is what identifies it)
            idents += [id(base.weight), id(tensors[-2]), id(tensors[-1])]
            biases[name] = _bias(base, name + "_proj")
        key = tuple(idents) + tuple(id(b) for b in biases.values())
        if self._weights is None or self._weights[0] != key:
            (n1, n2, wq, aq, bq, wk, ak, bk, wv, av, bv, wo, ao, bo, wg, ag, bg, wu, au, bu, wd, ad, bd) = tensors
            aw = AttnWeights(norm_w=n1, wq=wq, wk=wk, wv=wv, wo=wo, aq=aq, bq=bq, ak=ak, bk=bk, av=av, bv=bv, ao=ao, bo=bo,
                             bias_q=biases["q"], bias_k=biases["k"], bias_v=biases["v"], bias_o=biases["o"])
            mw = MLPWeights(norm_w=n2, wg=wg, wu=wu, wd=wd, ag=ag, bg=bg, au=au, bu=bu, ad=ad, bd=bd, bias_d=biases["down"])
            lora = (aq, bq, ak, bk, av, bv, ao, bo, ag, bg, au, bu, ad, bd)
            self._weights = (key, aw, mw, lora)
        return self._weights[1:]

    def named_lora_weights(self):
        """{"grad_aq": q lora_A weight, "grad_bq": q lora_B weight, ...}: the 14 adapter weights of the last forward
        call under the names their gradients carry in the ``on_lora_grads`` dictionaries."""
        if self._weights is None:
            return {}
        names = ("aq", "bq", "ak", "bk", "av", "bv", "ao", "bo", "ag", "bg", "au", "bu", "ad", "bd")
        return {"grad_" + n: w for n, w in zip(names, self._weights[3])}

    def forward(self, input, norm_weight_1, norm_bias_1, cos, sin,
                q_proj_base, q_proj_lora_a, q_proj_lora_b, k_proj_base, k_proj_lora_a, k_proj_lora_b,
                v_proj_base, v_proj_lora_a, v_proj_lora_b, o_proj_base, o_proj_lora_a, o_proj_lora_b,
                norm_weight_2, norm_bias_2,
                gate_proj_base, gate_proj_lora_a, gate_proj_lora_b, up_proj_base, up_proj_lora_a, up_proj_lora_b,
                down_proj_base, down_proj_lora_a, down_proj_lora_b,
                attention_mask, num_heads, head_dim, num_key_value_heads):
        if norm_bias_1 is not None or norm_bias_2 is not None:
            raise NotImplementedError("RMSNorm has no bias")
        mods = dict(q=(q_proj_base, q_proj_lora_a, q_proj_lora_b), k=(k_proj_base, k_proj_lora_a, k_proj_lora_b),
                    v=(v_proj_base, v_proj_lora_a, v_proj_lora_b), o=(o_proj_base, o_proj_lora_a, o_proj_lora_b),
                    gate=(gate_proj_base, gate_proj_lora_a, gate_proj_lora_b),
                    up=(up_proj_base, up_proj_lora_a, up_proj_lora_b),
                    down=(down_proj_base, down_proj_lora_a, down_proj_lora_b))
        aw, mw, lora = self._bind(norm_weight_1, norm_weight_2, mods)
        return FusedLayerFunction.apply(input, self, aw, mw, cos, sin, attention_mask, num_heads, head_dim,
                                        num_key_value_heads, *lora)


# The Mistral layer of the reference differs from the Llama one only in its head geometry (grouped key/value
# heads), which is an argument of forward here.
FusedMistralLayerIntraInterFullFuse = FusedLlamaLayerIntraInterFullFuse
