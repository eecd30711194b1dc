"""The CPU oracle against fixtures produced by executing the reference's own source
(tests/golden/make_golden.py).  Everything here is bit-exact."""
import pytest
import torch

import oracle

QS = (2, 4, 8)


@pytest.mark.parametrize("q", QS)
def test_scale_pack_dequant(golden, q):
    d = golden[f"q{q}"]
    assert torch.equal(oracle.ref_scale_per_channel(d["x"], q), d["scale"])
    assert torch.equal(oracle.ref_compress(d["x"], d["scale_safe"], q), d["packed"])
    assert torch.equal(oracle.ref_decompress(d["packed"], d["scale_safe"], q), d["dequant"])
    # pack/unpack are inverse
    codes = oracle.ref_quant_codes(d["x"], d["scale_safe"], q)
    assert torch.equal(oracle.ref_unpack(oracle.ref_pack(codes, q), q), codes)


@pytest.mark.parametrize("q", QS)
def test_zero_point_variant(golden, q):
    d = golden[f"q{q}"]
    s, z = oracle.ref_scale_zero_point(d["xz"], q)
    assert torch.equal(s, d["zp_scale"]) and torch.equal(z, d["zp"])
    assert torch.equal(oracle.ref_compress(d["xz"], s, q, z), d["zp_packed"])
    assert torch.equal(oracle.ref_decompress(d["zp_packed"], s, q, z), d["zp_dequant"])


@pytest.mark.parametrize("q", QS)
def test_channel_base(golden, q):
    d = golden[f"q{q}"]
    idx, s = oracle.ref_statistics_channel_base(d["x"], d["cb_ratio"], q)
    # torch.topk leaves the order of equal norms open: compare as a set, and the gathered
    # slab column by column
    assert sorted(idx.tolist()) == sorted(d["cb_idx"].tolist())
    assert torch.equal(s, d["cb_scale"])
    xo, pk = oracle.ref_compress_channel_base(d["x"], d["cb_scale"], d["cb_idx"], q)
    assert torch.equal(xo, d["cb_outlier"]) and torch.equal(pk, d["cb_packed"])
    xr = oracle.ref_decompress_channel_base(pk, d["cb_scale"], xo, d["cb_idx"], q)
    assert torch.equal(xr, d["cb_restored"])
    assert torch.equal(oracle.ref_scale_per_channel(d["xh"], q), d["xh_scale"])


@pytest.mark.parametrize("q", QS)
def test_fused_forward_backward(golden, q):
    d = golden[f"q{q}"]
    q1, q2, o = oracle.ref_fused_silu_forward(d["f_xa1"], d["f_b1"], d["f_x1"], d["f_s1"],
                                              d["f_xa2"], d["f_b2"], d["f_x2"], d["f_s2"], q)
    assert torch.equal(q1, d["f_q1"]) and torch.equal(q2, d["f_q2"]) and torch.equal(o, d["f_o"])
    bo, gg, gu = oracle.ref_fused_silu_backward(d["f_xa1"], d["f_b1"], q1, d["f_s1"],
                                                d["f_xa2"], d["f_b2"], q2, d["f_s2"], d["f_go"], q)
    assert torch.equal(bo, d["f_bo"]) and torch.equal(gg, d["f_ggate"]) and torch.equal(gu, d["f_gup"])


def test_softmax_prune(golden):
    d = golden["softmax"]
    thr = oracle.ref_softmax_threshold(d["a"], d["ratio"])
    assert torch.equal(thr, d["thr"])
    for t, i, v in ((d["thr"], d["idx"], d["val"]), (d["thr2"], d["idx2"], d["val2"])):
        idx, val = oracle.ref_softmax_prune(d["a"], t)
        assert torch.equal(idx, i.flatten()) and torch.equal(val, v)
    idx, val = oracle.ref_softmax_prune(d["a"], d["thr"])
    assert torch.equal(oracle.ref_softmax_restore(idx, val, d["a"].shape), d["dense"])


def test_rmsnorm_golden(golden):
    """operators/rmsnorm_kernels.py:10-54, 58-113 run through the interpreter.  The mean of squares is an fp32
    sum whose order differs (the kernel reduces a block, torch sums pairwise): rstd within two fp32 ulps, the
    bf16 outputs equal."""
    d = golden["rmsnorm"]
    y, rstd = oracle.ref_rmsnorm_forward(d["x"], d["w"], d["eps"])
    assert torch.equal(y, d["y"])
    assert ((rstd - d["rstd"]).abs() <= d["rstd"].abs() * 2 ** -22).all()
    assert torch.equal(oracle.ref_rmsnorm_backward(d["dy"], d["x"], d["w"], d["rstd"]), d["dx"])
    # the LayerNorm-style mean term of the reference's backward (:96-98) is part of the pinned result
    n = d["x"].shape[-1]
    xhat = d["x"].float() * d["rstd"].reshape(3, 40, 1)
    wdy = d["w"].float() * d["dy"].float()
    no_c2 = ((wdy - xhat * (xhat * wdy).sum(-1, keepdim=True) / n) * d["rstd"].reshape(3, 40, 1)).bfloat16()
    assert not torch.equal(no_c2, d["dx"])


def test_softmax_backward_golden(golden):
    """operators/softmax_kernels.py:7-38 through the interpreter (bf16 product, fp32 row sum as in the pinned
    Triton release)."""
    d = golden["softmax_bwd"]
    assert torch.equal(oracle.ref_softmax_backward(d["y"], d["g"]), d["o"])


def test_rope_golden(golden):
    """operators/rope_kernels.py:38-131 through the interpreter, bf16 and fp32 tables, both directions."""
    from oracle.attention import ref_rope
    d = golden["rope"]
    for nm in ("bf16", "f32"):
        assert torch.equal(ref_rope(d["x"], d["cos_" + nm], d["sin_" + nm]), d["fwd_" + nm])
        assert torch.equal(ref_rope(d["x"], d["cos_" + nm], d["sin_" + nm], backward=True), d["bwd_" + nm])


def test_roundf_half_away():
    r = torch.tensor([0.5, -0.5, 1.5, -1.5, 2.5, 0.49999997, -0.49999997, 7.5, -8.5, 0.0, 1e9, float("inf")])
    want = torch.tensor([1.0, -1.0, 2.0, -2.0, 3.0, 0.0, -0.0, 8.0, -9.0, 0.0, 1e9, float("inf")])
    assert torch.equal(oracle.roundf_half_away(r), want)


def test_group_and_topk_roundtrip_properties():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(3, 5, 256, generator=g).bfloat16()
    for q in QS:
        pk, s, z = oracle.group_compress(x, q)
        xr = oracle.group_decompress(pk, s, z, q)
        # error bounded by one step per group (plus bf16 rounding of the result)
        err = (xr.float() - x.float()).abs().reshape(3, 5, 4, 64).amax(-1)
        assert (err <= 1.01 * s.float() + 0.02).all()
    logits = 3 * torch.randn(2, 2, 128, 128, generator=g)
    logits = logits + torch.triu(torch.full((128, 128), float("-inf")), diagonal=1)
    a = torch.softmax(logits, -1).bfloat16()
    vals, cols, pk, s, z = oracle.topk_compress(a, 0.05, 4)
    assert vals.shape == (2 * 2 * 128, 6) and (cols[:, 1:] > cols[:, :-1]).all()
    ar = oracle.topk_decompress(vals, cols, pk, s, z, 4, a.shape)
    assert torch.equal(torch.gather(ar.reshape(-1, 128), 1, cols), vals)
    assert (ar.float() - a.float()).abs().max() < 0.05


def test_group_definition_against_the_literal_zero_point_arithmetic():
    """GROUP mode has no reference code; its definition departs from a literal application of the reference's
    zero-point arithmetic to a 64-wide group (fp32 divide, roundf, bf16 de-quantizer steps) in favour of a
    reciprocal multiply, round-half-to-even and a saturating fma.  What that costs: a fraction of a percent of the
    codes move by ONE step (ties and quotients within an fp32 ulp of a tie), the reconstruction error is the same."""
    from oracle.group import (group_compress, group_compress_divide_roundf, group_decompress,
                              group_decompress_divide_roundf)
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(1, 256, 4096, generator=g)
    x[:, :, torch.randperm(4096, generator=g)[:20]] *= 30
    logits = 3 * torch.randn(1, 4, 256, 256, generator=g) + torch.triu(torch.full((256, 256), float("-inf")), 1)
    for t in (x.bfloat16(), torch.softmax(logits, -1).bfloat16()):
        for q in QS:
            pk, s, z = group_compress(t, q)
            pk2, s2, z2 = group_compress_divide_roundf(t, q)
            d = (oracle.ref_unpack(pk, q).int() - oracle.ref_unpack(pk2, q).int()).abs()
            assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 5e-3
            assert torch.equal(s, s2)
            e = (group_decompress(pk, s, z, q).float() - t.float()).pow(2).mean().sqrt()
            e2 = (group_decompress_divide_roundf(pk2, s2, z2, q).float() - t.float()).pow(2).mean().sqrt()
            assert abs(float(e / e2) - 1) < 1e-3
