"""The oracle's restatement of the whole fused decoder layer (forward and the hand-written backward of the
reference, with 8-bit saved activations) against a plain fp32 autograd model of the same layer: pins the
backward formulas of ``oracle/attention.py`` and ``oracle/fused_mlp.py`` to the mathematics, on CPU."""
import math

import pytest
import torch

import oracle
from oracle.attention import ref_layer_backward, ref_layer_forward, ref_rope

BF16 = torch.bfloat16


def layer_problem(g, B, M, H, heads, d, kv, I, R=16, outliers=True):
    def rn(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g) * scale).to(BF16)
    x = rn(B, M, H)
    if outliers:
        x[:, :, torch.randperm(H, generator=g)[: max(1, H // 200)]] *= 20
    D, Dkv = heads * d, kv * d
    sw = 1.0 / math.sqrt(H)
    p = dict(norm_w1=(1 + 0.1 * torch.randn(H, generator=g)).to(BF16), norm_w2=(1 + 0.1 * torch.randn(H, generator=g)).to(BF16),
             wq=rn(H, D, scale=sw), wk=rn(H, Dkv, scale=sw), wv=rn(H, Dkv, scale=sw), wo=rn(D, H, scale=sw),
             wgate=rn(H, I, scale=sw), wup=rn(H, I, scale=sw), wdown=rn(I, H, scale=1.0 / math.sqrt(I)),
             aq=rn(H, R, scale=sw), bq=rn(R, D, scale=0.05), ak=rn(H, R, scale=sw), bk=rn(R, Dkv, scale=0.05),
             av=rn(H, R, scale=sw), bv=rn(R, Dkv, scale=0.05), ao=rn(D, R, scale=sw), bo=rn(R, H, scale=0.05),
             agate=rn(H, R, scale=sw), bgate=rn(R, I, scale=0.05), aup=rn(H, R, scale=sw), bup=rn(R, I, scale=0.05),
             adown=rn(I, R, scale=1.0 / math.sqrt(I)), bdown=rn(R, H, scale=0.05))
    pos = torch.arange(M, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    fr = torch.outer(pos, inv)
    emb = torch.cat([fr, fr], dim=-1)
    cos, sin = emb.cos().to(BF16), emb.sin().to(BF16)
    mask = torch.full((M, M), torch.finfo(BF16).min).triu(1).to(BF16).reshape(1, 1, M, M)
    return x, p, cos, sin, mask


def autograd_layer(x, p, cos, sin, mask, heads, d, kv):
    """fp32 model of the layer: RMSNorm, LoRA projections, rotate-half rotary, softmax attention, SiLU MLP."""
    f = {k: v.float().requires_grad_(k[0] in "ab") for k, v in p.items()}
    x = x.float().requires_grad_(True)
    B, M, H = x.shape
    half = d // 2
    c, s = cos[:, :half].float().reshape(1, 1, M, half), sin[:, :half].float().reshape(1, 1, M, half)

    def norm(t, w):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + 1e-5) * w

    def lin(t, n):
        return t @ f["w" + n] + (t @ f["a" + n]) @ f["b" + n]

    def rope(t):
        t1, t2 = t[..., :half], t[..., half:]
        return torch.cat([t1 * c - t2 * s, t2 * c + t1 * s], dim=-1)

    xn = norm(x, f["norm_w1"])
    q = lin(xn, "q").reshape(B, M, heads, d).transpose(1, 2)
    k = lin(xn, "k").reshape(B, M, kv, d).transpose(1, 2)
    v = lin(xn, "v").reshape(B, M, kv, d).transpose(1, 2)
    q, k = rope(q), rope(k)
    rep = heads // kv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    a = torch.softmax(q @ k.transpose(-2, -1) / math.sqrt(d) + mask.float(), dim=-1)
    o = (a @ v).transpose(1, 2).reshape(B, M, heads * d)
    xm = x + lin(o, "o")
    xn2 = norm(xm, f["norm_w2"])
    y = xm + lin(torch.nn.functional.silu(lin(xn2, "gate")) * lin(xn2, "up"), "down")
    return x, f, y


def cosine(a, b):
    return float(torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0))


def test_rope_backward_is_the_transpose():
    g = torch.Generator().manual_seed(1)
    _, _, cos, sin, _ = layer_problem(g, 1, 16, 64, 2, 32, 2, 64)
    x = torch.randn(1, 16, 2, 32, generator=g).to(BF16)
    y = torch.randn(1, 16, 2, 32, generator=g).to(BF16)
    lhs = (ref_rope(x, cos, sin).float() * y.float()).sum()
    rhs = (x.float() * ref_rope(y, cos, sin, backward=True).float()).sum()
    assert abs(float(lhs - rhs)) < 2e-2 * float(lhs.abs() + rhs.abs() + 1)


@pytest.mark.parametrize("heads,kv,map_mode", [(4, 4, "prune"), (4, 2, "topk")])
def test_layer_oracle_against_autograd(heads, kv, map_mode):
    g = torch.Generator().manual_seed(11 + kv)
    B, M, H, d, I = 2, 64, 128, 32, 256
    x, p, cos, sin, mask = layer_problem(g, B, M, H, heads, d, kv, I)
    # all of the map is kept (ratio 1 -> k = S; the threshold form keeps everything above the smallest entry)
    ratio = 1.0 if map_mode == "topk" else 0.999
    y, saved = ref_layer_forward(x, p, cos, sin, mask, heads, d, kv, 8, 0.01, ratio, map_mode=map_mode, map_q_bit=8)
    gy = (torch.randn(B, M, H, generator=g)).to(BF16)
    grads = ref_layer_backward(gy, saved, p, cos, sin, heads, d, kv, 8)
    xa, f, ya = autograd_layer(x, p, cos, sin, mask, heads, d, kv)
    ya.backward(gy.float())
    assert cosine(y, ya.detach()) > 0.999
    assert cosine(grads["grad_x"], xa.grad) > 0.995
    names = {"aq": "aq", "bq": "bq", "ak": "ak", "bk": "bk", "av": "av", "bv": "bv", "ao": "ao", "bo": "bo",
             "agate": "agate", "bgate": "bgate", "aup": "aup", "bup": "bup", "adown": "adown", "bdown": "bdown"}
    for k, n in names.items():
        # bf16 intermediates and 8-bit saved activations cost a few 1e-3 of cosine; a wrong formula costs tenths
        assert cosine(grads["grad_" + k], f[n].grad) > 0.97, k
