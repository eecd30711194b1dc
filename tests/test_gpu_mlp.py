"""tcgen05 GEMM path: plain GEMM against an fp32 product, the fused gate/up forward and grad_down
backward epilogues against the CPU oracle, and the whole MLP block forward/backward.
Tolerance of this path (north star): max |err| <= 1e-2 * max|ref|, cosine > 0.999.  Packed codes
are compared bit-exactly against the oracle quantizer applied to the main branches the kernel
emitted (a tensor-core sum differs from a CPU sum in the last bits, so codes are pinned to the
kernel's own bf16 main values, and those to the reference product within tolerance)."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16 = torch.bfloat16


def close(a, b, rel=1e-2, cos=0.999):
    a, b = a.float().cpu().flatten(), b.float().cpu().flatten()
    scale = b.abs().max().clamp(min=1e-30)
    c = torch.nn.functional.cosine_similarity(a, b, dim=0)
    return bool((a - b).abs().max() <= rel * scale) and bool(c > cos)


@pytest.fixture(scope="module")
def mlp():
    from hyc_lora_release_b200 import mlp as m
    return m


def _randn(g, *shape, scale=1.0):
    return (torch.randn(*shape, generator=g) * scale).to(BF16)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 512), (200, 512, 1024), (1024, 4096, 2752)])
@pytest.mark.parametrize("b_is_kn", [False, True])
def test_plain_gemm(mlp, M, N, K, b_is_kn):
    g = torch.Generator().manual_seed(M + N + K)
    a = _randn(g, M, K)
    b = _randn(g, K, N, scale=0.05) if b_is_kn else _randn(g, N, K, scale=0.05)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    d = mlp.gemm(a.to(DEV), b.to(DEV), b_is_kn=b_is_kn, status=st)
    mlp.check_status(st, "gemm")
    ref = a.float() @ (b.float() if b_is_kn else b.float().t())
    assert close(d, ref, rel=4e-3)


def test_gemm_two_segments_lora_residual(mlp):
    g = torch.Generator().manual_seed(5)
    M, N, K, K2, R = 256, 256, 256, 384, 16
    a, a2 = _randn(g, M, K), _randn(g, M, K2)
    b, b2 = _randn(g, K, N, scale=0.05), _randn(g, K2, N, scale=0.05)
    xa0, xa1 = _randn(g, M, R), _randn(g, M, R)
    w0 = _randn(g, R, N, scale=0.1)          # element (col, r) at r*N + col
    w1 = _randn(g, N, R, scale=0.1)          # element (col, r) at col*R + r
    res = _randn(g, M, N)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    t = lambda *v: [x.to(DEV) for x in v]
    a_, a2_, b_, b2_, xa0_, xa1_, w0_, w1_, res_ = t(a, a2, b, b2, xa0, xa1, w0, w1, res)
    d = mlp.gemm(a_, b_, b_is_kn=True, a2=a2_, b2=b2_, lora0=(xa0_, w0_, 1, N), lora1=(xa1_, w1_, R, 1),
                 residual=res_, status=st)
    mlp.check_status(st, "gemm")
    ref = a.float() @ b.float() + a2.float() @ b2.float() + xa0.float() @ w0.float() + xa1.float() @ w1.float().t() + res.float()
    assert close(d, ref, rel=6e-3)
    # the same LoRA products as a third, zero-padded K segment instead of epilogue terms
    a3 = torch.zeros(M, 64, dtype=BF16); a3[:, :R] = xa0; a3[:, R:2 * R] = xa1
    b3 = torch.zeros(64, N, dtype=BF16); b3[:R] = w0; b3[R:2 * R] = w1.t()
    d3 = mlp.gemm(a_, b_, b_is_kn=True, a2=a2_, b2=b2_, a3=a3.to(DEV), b3=b3.to(DEV), residual=res_, status=st)
    mlp.check_status(st, "gemm")
    assert close(d3, ref, rel=6e-3)


@pytest.mark.parametrize("q", (2, 4, 8))
@pytest.mark.parametrize("T,H,R2,ldg", [(64, 128, 16, 16), (300, 512, 32, 64), (1024, 4096, 32, 64), (257, 256, 64, 72)])
def test_lora_grad_a_with_dequant_inside(mlp, q, T, H, R2, ldg):
    """out = gm^T @ dequant(codes): against the oracle's de-quantizer followed by an fp32 product."""
    g = torch.Generator().manual_seed(T + H + q)
    x = _randn(g, 1, T, H)
    s = oracle.ref_scale_per_channel(x, q)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=BF16), s)
    codes = oracle.ref_compress(x, s, q)[0]
    xhat = oracle.ref_decompress(codes[None], s, q)[0]
    gm = torch.zeros(T, ldg, dtype=BF16)
    gm[:, :R2] = _randn(g, T, R2)
    gm[:, R2:] = 7.0                      # columns beyond R2 must be ignored
    out = mlp.lora_grad_a(codes.to(DEV), s.reshape(-1).to(DEV), gm.to(DEV), R2, q)
    ref = gm[:, :R2].float().t() @ xhat.float()
    assert out.shape == (R2, H) and close(out, ref, rel=4e-3)


def _mlp_problem(g, B, M, H, I, R=16):
    x = _randn(g, B, M, H)
    x[:, :, torch.randperm(H, generator=g)[: max(1, H // 200)]] *= 20
    w = dict(norm_w=(1 + 0.1 * torch.randn(H, generator=g)).to(BF16),
             wg=_randn(g, I, H, scale=0.02), wu=_randn(g, I, H, scale=0.02), wd=_randn(g, H, I, scale=0.02),
             ag=_randn(g, R, H, scale=0.02), bg=_randn(g, I, R, scale=0.02),
             au=_randn(g, R, H, scale=0.02), bu=_randn(g, I, R, scale=0.02),
             ad=_randn(g, R, I, scale=0.02), bd=_randn(g, H, R, scale=0.02))
    return x, w


@pytest.mark.parametrize("q", (2, 4, 8))
def test_gateup_and_graddown_epilogues(mlp, q):
    from hyc_lora_release_b200._lib import lib, ptr, check, stream_of
    g = torch.Generator().manual_seed(40 + q)
    T, H, I, R = 256, 256, 256, 16
    x = _randn(g, T, H)
    wg, wu, wd = _randn(g, I, H, scale=0.05), _randn(g, I, H, scale=0.05), _randn(g, H, I, scale=0.05)
    xa1, xa2 = _randn(g, T, R), _randn(g, T, R)
    bg, bu = _randn(g, I, R, scale=0.05), _randn(g, I, R, scale=0.05)
    main1_ref, main2_ref = (x.float() @ wg.float().t()), (x.float() @ wu.float().t())
    s1 = oracle.ref_scale_per_channel(main1_ref.to(BF16)[None], q).reshape(-1)
    s2 = oracle.ref_scale_per_channel(main2_ref.to(BF16)[None], q).reshape(-1)
    d = lambda v: v.to(DEV)
    xd, wgd, wud, wdd, xa1d, xa2d, bgd, bud, s1d, s2d = map(d, (x, wg, wu, wd, xa1, xa2, bg, bu, s1, s2))
    epp = 8 // q
    q1 = torch.empty(T, I // epp, dtype=torch.uint8, device=DEV); q2 = torch.empty_like(q1)
    o = torch.empty(T, I, dtype=BF16, device=DEV); m1 = torch.empty_like(o); m2 = torch.empty_like(o)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    check(lib.hyc_mlp_gateup_fwd_tcgen05(ptr(xd), ptr(wgd), ptr(wud), T, H, I, ptr(xa1d), ptr(bgd), 16, 1,
                                         ptr(xa2d), ptr(bud), 16, 1, ptr(s1d), ptr(s2d), ptr(q1), ptr(q2), ptr(o),
                                         ptr(m1), ptr(m2), q, ptr(st), stream_of(xd)), "gateup")
    mlp.check_status(st, "gateup")
    assert close(m1, main1_ref, rel=4e-3) and close(m2, main2_ref, rel=4e-3)
    # codes: bit-exact against the oracle quantizer on the emitted bf16 main branches
    oq1, oq2, oo = oracle.ref_fused_silu_forward(xa1[None], bg.t(), m1.cpu()[None], s1[None], xa2[None], bu.t(),
                                                 m2.cpu()[None], s2[None], q)
    assert torch.equal(q1.cpu(), oq1[0]) and torch.equal(q2.cpu(), oq2[0])
    assert close(o, oo[0])
    # backward epilogue
    gout = _randn(g, T, H)
    gdm, ad = _randn(g, T, R), _randn(g, R, I, scale=0.05)
    had = torch.empty(T, I, dtype=BF16, device=DEV); gg = torch.empty_like(had); gu = torch.empty_like(had)
    gdm64 = torch.zeros(T, 64, dtype=BF16); gdm64[:, :R] = gdm      # the LoRA part rides along as a padded K block
    ad64 = torch.zeros(64, I, dtype=BF16); ad64[:R] = ad
    goutd, gdmd, add = map(d, (gout, gdm64, ad64))
    grad_down = (gout.float() @ wd.float() + gdm.float() @ ad.float()).to(BF16)
    ob, ogg, ogu = oracle.ref_fused_silu_backward(xa1[None], bg.t(), q1.cpu()[None], s1[None], xa2[None], bu.t(),
                                                  q2.cpu()[None], s2[None], grad_down[None], q)
    # (a) LoRA terms of the recomputation inside the epilogue
    check(lib.hyc_mlp_graddown_bwd_tcgen05(ptr(goutd), ptr(wdd), T, H, I, ptr(gdmd), ptr(add), 64,
                                           ptr(xa1d), ptr(bgd), 16, 1, ptr(xa2d), ptr(bud), 16, 1,
                                           ptr(q1), ptr(s1d), ptr(q2), ptr(s2d), None, None, 0,
                                           ptr(had), ptr(gg), ptr(gu), q, ptr(st), stream_of(xd)), "graddown")
    mlp.check_status(st, "graddown")
    assert close(had, ob[0]) and close(gg, ogg[0]) and close(gu, ogu[0])
    # (b) LoRA terms prepared by one GEMM launch on the zero-padded rank-16 operands
    xa12 = torch.zeros(T, 128, dtype=BF16, device=DEV); xa12[:, :R] = xa1d; xa12[:, 64:64 + R] = xa2d
    bdiag = torch.zeros(2 * I, 128, dtype=BF16, device=DEV); bdiag[:I, :R] = bgd; bdiag[I:, 64:64 + R] = bud
    l12 = mlp.gemm(xa12, bdiag, status=st)
    assert close(l12[:, :I], xa1.float() @ bg.float().t(), rel=4e-3) and close(l12[:, I:], xa2.float() @ bu.float().t(), rel=4e-3)
    had2 = torch.empty_like(had); gg2 = torch.empty_like(had); gu2 = torch.empty_like(had)
    import ctypes
    check(lib.hyc_mlp_graddown_bwd_tcgen05(ptr(goutd), ptr(wdd), T, H, I, ptr(gdmd), ptr(add), 64,
                                           None, None, 0, 0, None, None, 0, 0,
                                           ptr(q1), ptr(s1d), ptr(q2), ptr(s2d),
                                           ptr(l12), ctypes.c_void_p(l12.data_ptr() + 2 * I), 2 * I,
                                           ptr(had2), ptr(gg2), ptr(gu2), q, ptr(st), stream_of(xd)), "graddown pre")
    mlp.check_status(st, "graddown pre")
    assert close(had2, ob[0]) and close(gg2, ogg[0]) and close(gu2, ogu[0])


@pytest.mark.parametrize("q", (2, 4, 8))
def test_linear_lora_save_epilogue(mlp, q):
    """LoRA projection with the quantized save of its main branch in the epilogue: codes bit-exact against the
    oracle quantizer on the emitted bf16 main branch, y and main within tolerance of fp32."""
    from hyc_lora_release_b200.operators import compress_function as cf
    g = torch.Generator().manual_seed(90 + q)
    T, K, N, R = 300, 512, 768, 16
    x = _randn(g, T, K)
    w, a, b = _randn(g, N, K, scale=0.05), _randn(g, R, K, scale=0.05), _randn(g, N, R, scale=0.05)
    main_ref = x.float() @ w.float().t()
    scale = oracle.ref_scale_per_channel(main_ref.to(BF16)[None], q).reshape(-1)
    scale = torch.where(scale == 0, torch.tensor(1e-3, dtype=BF16), scale)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    y, qm, xa, main = mlp.linear_lora_save(x.to(DEV), w.to(DEV), a.to(DEV), b.to(DEV), scale.to(DEV), q,
                                           want_main=True, status=st)
    mlp.check_status(st, "linear_lora_save")
    assert close(main, main_ref, rel=4e-3)
    assert torch.equal(qm.cpu(), oracle.ref_compress(main.cpu()[None], scale[None], q)[0])
    assert torch.equal(qm, cf.compression_quantization(main[None], scale.to(DEV), q)[0])
    y_ref = (main.cpu().float() + (xa.cpu().float() @ b.float().t()).to(BF16).float()).to(BF16)
    assert close(y, y_ref.float(), rel=4e-3)
    assert close(y, main_ref + (x.float() @ a.float().t()) @ b.float().t())


@pytest.mark.parametrize("q", (2, 4, 8))
def test_mlp_block_forward_backward(mlp, q):
    g = torch.Generator().manual_seed(7 + q)
    B, M, H, I = 2, 128, 512, 1024
    x, w = _mlp_problem(g, B, M, H, I)
    W = mlp.MLPWeights(**{k: v.to(DEV) for k, v in w.items()})
    state = mlp.MLPState(q_bit=q, layernorm_outlier_ratio=0.01)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    # oracle operands: weights transposed as the layer passes them ([in, out]; a: [in, r]; b: [r, out])
    ow = (w["norm_w"], w["wg"].t(), w["wu"].t(), w["wd"].t(), w["ag"].t(), w["bg"].t(), w["au"].t(), w["bu"].t(),
          w["ad"].t(), w["bd"].t())
    ref_out, ref_saved = oracle.ref_mlp_block_forward(x, *ow, q, 0.01)
    gout = _randn(g, B, M, H)
    ref_g = oracle.ref_mlp_block_backward(gout, ref_saved, *ow, q)
    for it in range(7):     # 5 calibration iterations, then the steady-state branch
        if it == 5:
            # steady state: the oracle takes the same calibrated statistics (running means) as the device
            sv = state.static_value
            static = dict(x_medium_idx=sv["x_medium"]["outlier_channel_index"].cpu(),
                          x_medium_scale=sv["x_medium"]["scale"].cpu().to(BF16),
                          gate_scale=sv["gate"]["scale"].cpu().to(BF16), up_scale=sv["up"]["scale"].cpu().to(BF16),
                          x_norm_2_scale=sv["x_norm_2"]["scale"].cpu().to(BF16))
            ref_out, ref_saved = oracle.ref_mlp_block_forward(x, *ow, q, 0.01, static=static)
            ref_g = oracle.ref_mlp_block_backward(gout, ref_saved, *ow, q)
        out, saved = mlp.mlp_forward(x.to(DEV), W, state, status=st)
        grads = mlp.mlp_backward(gout.to(DEV), saved, W, status=st)
        mlp.check_status(st, "mlp")
        assert close(out, ref_out), it
        assert torch.equal(saved["xm_q"].cpu(), ref_saved["xm_q"])
        assert torch.equal(saved["xm_o"].cpu(), ref_saved["xm_o"])
        assert close(grads["grad_x"], ref_g["grad_x"]), it
        for name in ("ag", "au", "ad"):     # oracle layout [in, r] -> weight layout [r, in]
            assert close(grads["grad_" + name], ref_g["grad_" + name].t(), rel=2e-2), (it, name)
        for name in ("bg", "bu", "bd"):     # oracle layout [r, out] -> weight layout [out, r]
            assert close(grads["grad_" + name], ref_g["grad_" + name].t(), rel=2e-2), (it, name)
    assert state.iteration == 7
