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
    a, b = a.double().cpu().flatten(), b.double().cpu().flatten()
    scale = b.abs().max().clamp(min=1e-30)
    c = torch.nn.functional.cosine_similarity(a, b, dim=0)
    ok = bool((a - b).abs().max() <= rel * scale) and bool(c > cos)
    if not ok:
        print("max rel err %.4g (bound %g), cosine %.6f (bound %g)" % (float((a - b).abs().max() / scale), rel, float(c), cos))
    return ok


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


@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (129, 256, 128), (257, 512, 192), (383, 256, 64), (2304, 4096, 512),
                                   (2500, 2048, 320)])
@pytest.mark.parametrize("b_is_kn", [False, True])
def test_gemm_ragged_rows_and_several_rounds_of_pairs(mlp, M, N, K, b_is_kn):
    """Row counts that leave the second CTA of a pair with one valid row, a few, or none (the products run as pairs
    of CTAs on 256-row tiles), and tile counts beyond one round of pairs, with a LoRA block and a residual."""
    g = torch.Generator().manual_seed(3 * M + N + K)
    a = _randn(g, M, K).to(DEV)
    b = (_randn(g, K, N, scale=0.05) if b_is_kn else _randn(g, N, K, scale=0.05)).to(DEV)
    a2 = _randn(g, M, 64).to(DEV)
    b2 = (_randn(g, 64, N, scale=0.05) if b_is_kn else _randn(g, N, 64, scale=0.05)).to(DEV)
    res = _randn(g, M, N).to(DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    from hyc_lora_release_b200._lib import lib, ptr, check, stream_of
    big = torch.full((M + 256, N), 7.0, dtype=BF16, device=DEV)       # the rows behind the result must stay untouched
    check(lib.hyc_gemm_bf16_tcgen05(ptr(a), ptr(b), M, N, K, 1 if b_is_kn else 0, ptr(a2), ptr(b2), 64, None, None, 0,
                                    None, None, 0, 0, None, None, 0, 0, ptr(res), ptr(big), ptr(st), stream_of(a)), "gemm")
    mlp.check_status(st, "gemm")
    op = (lambda t: t.float()) if b_is_kn else (lambda t: t.float().t())
    ref = a.float() @ op(b) + a2.float() @ op(b2) + res.float()
    assert close(big[:M], ref, rel=6e-3)
    assert bool((big[M:] == 7.0).all())


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


def _saved_for_oracle(saved, dev=None):
    """The device's saved tensors in the shapes the oracle's backward expects (on `dev`, default CPU)."""
    B, M, H = saved["shape"]
    to = (lambda t: t.cpu()) if dev is None else (lambda t: t.to(dev))
    out = {}
    for k in ("rstd", "xm_o", "xm_q", "xm_scale", "xm_idx", "xn_q", "xn_scale", "gate_q", "gate_scale", "up_q", "up_scale"):
        out[k] = to(saved[k])
    for k in ("xm_q", "xn_q", "gate_q", "up_q"):
        out[k] = out[k].reshape(B, M, -1)
    for k in ("gate_xa", "up_xa", "down_xa"):
        out[k] = to(saved[k]).reshape(B, M, -1)
    return out


def _flipped_codes(a, b, q):
    """Fraction of q-bit codes that differ between two packed tensors."""
    x = (a.cpu() ^ b.cpu()).to(torch.int32)
    n = 0
    for i in range(8 // q):
        n += int((((x >> (q * i)) & ((1 << q) - 1)) != 0).sum())
    return n / (a.numel() * (8 // q))


@pytest.mark.parametrize("q", (2, 4, 8))
def test_mlp_block_forward_backward(mlp, q):
    """Whole MLP half against the oracle, 5 calibration iterations and 2 steady-state ones.  Forward: output and the
    saved form of the INPUT (codes + outlier slab) against the oracle's forward.  The codes of COMPUTED tensors
    (x_norm, the gate/up main branches) are pinned elsewhere (operator tests: bit-exact against the oracle quantizer
    on the emitted tensor); here they may differ from the oracle's in the few places where the tensor-core sum and
    the CPU sum round differently -- the fraction is counted and bounded.  Backward: the oracle's backward is given
    the DEVICE's saved tensors, so that every gradient is compared at the path's tolerance (1e-2, cosine 0.999)."""
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
    for it in range(7):     # 5 calibration iterations, then the steady-state branch
        if it == 5:
            # steady state: the oracle takes the same calibrated statistics (running means) as the device
            sv = state.static_value
            static = dict(x_medium_idx=sv["x_medium"]["outlier_channel_index"].cpu(),
                          x_medium_scale=sv["x_medium"]["scale"].cpu().to(BF16),
                          gate_scale=sv["gate"]["scale"].cpu().to(BF16), up_scale=sv["up"]["scale"].cpu().to(BF16),
                          x_norm_2_scale=sv["x_norm_2"]["scale"].cpu().to(BF16))
            ref_out, ref_saved = oracle.ref_mlp_block_forward(x, *ow, q, 0.01, static=static)
        out, saved = mlp.mlp_forward(x.to(DEV), W, state, status=st)
        grads = mlp.mlp_backward(gout.to(DEV), saved, W, status=st)
        mlp.check_status(st, "mlp")
        assert close(out, ref_out), it
        assert torch.equal(saved["xm_q"].cpu(), ref_saved["xm_q"])
        assert torch.equal(saved["xm_o"].cpu(), ref_saved["xm_o"])
        for name in ("xn_q", "gate_q", "up_q"):
            flips = _flipped_codes(saved[name].reshape(B, M, -1), ref_saved[name], q)
            assert flips < 0.01, (it, name, flips)
        ref_g = oracle.ref_mlp_block_backward(gout, _saved_for_oracle(saved), *ow, q)
        assert close(grads["grad_x"], ref_g["grad_x"]), it
        for name in ("ag", "au", "ad", "bg", "bu", "bd"):     # oracle layout [in, r] / [r, out] -> the weight's layout
            assert close(grads["grad_" + name], ref_g["grad_" + name].t()), (it, name)
    assert state.iteration == 7


def _fp32_product_rows(a, b_t, rows):
    """fp32 statement of (a @ b_t^T)[rows] on the device (a checker: plain torch, TF32 off)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return a[rows].float() @ b_t.float().t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


@pytest.mark.parametrize("shape,q", [("llama", 4), ("mistral", 2), ("mistral", 4), ("mistral", 8)])
def test_mlp_block_full_size(mlp, shape, q):
    """The MLP half at the full sizes of the benchmark configurations (Llama-2-7B: 2048 tokens x 4096 x 11008, q 4;
    Mistral-7B: 8192 tokens x 4096 x 14336, q 2/4/8): multi-wave persistence of the tcgen05 kernels, 43 / 56 column
    tiles, 172 / 224 K blocks.  The checkers run on the GPU (plain torch in fp32 for the products, the oracle's own
    functions on CUDA tensors for the element-wise chains): emitted main branches against an fp32 product on row
    slices, codes bit-exact against the oracle quantizer on the emitted tensors, the backward against the oracle's
    backward on the device's saved tensors at 1e-2 / cosine 0.999."""
    from hyc_lora_release_b200._lib import check, lib, ptr, stream_of
    from hyc_lora_release_b200.operators import compress_function as cf
    B, M, H, I, n_out, amp, ratio = (4, 512, 4096, 11008, 20, 30, 0.005) if shape == "llama" else (1, 8192, 4096, 14336, 41, 20, 0.01)
    T, R = B * M, 16
    g = torch.Generator(device=DEV).manual_seed(100 + q + I)
    rn = lambda *sh, sc=1.0: (torch.randn(*sh, generator=g, device=DEV) * sc).to(BF16)
    x = torch.randn(B, M, H, generator=g, device=DEV)
    x[:, :, torch.randperm(H, generator=g, device=DEV)[:n_out]] *= amp
    x = x.to(BF16)
    w = dict(norm_w=(1 + 0.1 * torch.randn(H, generator=g, device=DEV)).to(BF16), wg=rn(I, H, sc=.02), wu=rn(I, H, sc=.02),
             wd=rn(H, I, sc=.02), ag=rn(R, H, sc=.02), bg=rn(I, R, sc=.02), au=rn(R, H, sc=.02), bu=rn(I, R, sc=.02),
             ad=rn(R, I, sc=.02), bd=rn(H, R, sc=.02))
    W = mlp.MLPWeights(**w)
    state = mlp.MLPState(q_bit=q, layernorm_outlier_ratio=ratio)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    gout = rn(B, M, H)
    for it in range(6):          # 5 calibration iterations, then the single-pass steady state
        out, saved = mlp.mlp_forward(x, W, state, status=st)
        grads = mlp.mlp_backward(gout, saved, W, status=st)
    mlp.check_status(st, "mlp full size")
    sv = state.static_value
    ow = (w["norm_w"], w["wg"].t(), w["wu"].t(), w["wd"].t(), w["ag"].t(), w["bg"].t(), w["au"].t(), w["bu"].t(),
          w["ad"].t(), w["bd"].t())
    # ---- forward: the main branches of the steady-state kernel, re-emitted with the calibrated scales
    from hyc_lora_release_b200.operators.rmsnorm_kernels import rmsnorm_forward
    x_norm = rmsnorm_forward(x, w["norm_w"], 1e-5)[0]
    assert close(x_norm, oracle.ref_rmsnorm_forward(x, w["norm_w"], 1e-5)[0], rel=4e-3)
    xn2 = x_norm.reshape(T, H)
    gs, us = saved["gate_scale"], saved["up_scale"]
    epp = 8 // q
    q1 = torch.empty(T, I // epp, dtype=torch.uint8, device=DEV); q2 = torch.empty_like(q1)
    had = torch.empty(T, I, dtype=BF16, device=DEV); m1 = torch.empty_like(had); m2 = torch.empty_like(had)
    check(lib.hyc_mlp_gateup_fwd_tcgen05(ptr(xn2), ptr(w["wg"]), ptr(w["wu"]), T, H, I, ptr(saved["gate_xa"]), ptr(w["bg"]), 16, 1,
                                         ptr(saved["up_xa"]), ptr(w["bu"]), 16, 1, ptr(gs), ptr(us), ptr(q1), ptr(q2), ptr(had),
                                         ptr(m1), ptr(m2), q, ptr(st), stream_of(x)), "gateup")
    mlp.check_status(st, "gateup full size")
    assert torch.equal(q1.reshape(B, M, -1), saved["gate_q"]) and torch.equal(q2.reshape(B, M, -1), saved["up_q"])
    rows = torch.cat([torch.arange(0, 256), torch.arange(T // 2 - 64, T // 2 + 64), torch.arange(T - 256, T)]).to(DEV)
    assert close(m1[rows], _fp32_product_rows(xn2, w["wg"], rows), rel=4e-3)
    assert close(m2[rows], _fp32_product_rows(xn2, w["wu"], rows), rel=4e-3)
    # codes: the device quantizer operator on the emitted tensor (itself bit-exact against the reference's kernel) on
    # everything, the CPU oracle on a slice of rows
    assert torch.equal(q1, cf.compression_quantization(m1[None], gs, q)[0])
    assert torch.equal(q2, cf.compression_quantization(m2[None], us, q)[0])
    sl = slice(T // 3, T // 3 + 64)
    assert torch.equal(q1[sl].cpu(), oracle.ref_compress(m1[sl].cpu()[None], gs.cpu()[None], q)[0])
    oq1, oq2, ohad = oracle.ref_fused_silu_forward(saved["gate_xa"][None], w["bg"].t(), m1[None], gs[None],
                                                   saved["up_xa"][None], w["bu"].t(), m2[None], us[None], q)
    assert torch.equal(oq1[0], q1) and torch.equal(oq2[0], q2) and close(had, ohad[0])
    # ---- the input's saved form and the output
    xm_o, xm_q = oracle.ref_compress_channel_base(x, sv["x_medium"]["scale"].to(BF16), sv["x_medium"]["outlier_channel_index"], q)
    assert torch.equal(saved["xm_q"], xm_q) and torch.equal(saved["xm_o"], xm_o)
    down = _fp32_product_rows(had, w["wd"], rows) + (saved["down_xa"][rows].float() @ w["bd"].float().t())
    assert close(out.reshape(T, H)[rows], x.reshape(T, H)[rows].float() + down)
    # ---- backward against the oracle's backward on the device's saved tensors (all on the GPU)
    ref_g = oracle.ref_mlp_block_backward(gout, _saved_for_oracle(saved, DEV), *ow, q)
    # the three element-wise intermediates (22 M / 117 M bf16 values each) and grad_x (8 M / 33 M) are the ends of
    # chains of bf16 roundings that start from GEMM results: somewhere a large element ends two bf16 steps
    # (2 x 2^-7 of its value) from the oracle's, so their bound is 2^-6; the LoRA gradients are held to 1e-2
    assert close(grads["hadamard"], ref_g["hadamard"], rel=2 ** -6) and close(grads["g_gate"], ref_g["g_gate"], rel=2 ** -6)
    assert close(grads["g_up"], ref_g["g_up"], rel=2 ** -6)
    assert close(grads["grad_x"], ref_g["grad_x"], rel=2 ** -6), "grad_x"
    for name in ("ag", "au", "ad", "bg", "bu", "bd"):
        assert close(grads["grad_" + name], ref_g["grad_" + name].t()), name
