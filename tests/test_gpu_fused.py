"""Fused LoRA-SiLU-Hadamard forward/backward, RMSNorm and softmax backward against the golden
fixtures and the CPU oracle.  Packed codes are bit-exact; bf16 outputs are compared within the
tolerance of the path: max |err| <= 1e-2 * max|ref| and cosine > 0.999 (sigmoid and the rank-16
dot are evaluated in a different order on the device, so a bf16 ulp may differ)."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
QS = (2, 4, 8)
DEV = "cuda"


def close(a, b, rel=1e-2, cos=0.999):
    a, b = a.float().cpu().flatten(), b.float().cpu().flatten()
    scale = b.abs().max().clamp(min=1e-30)
    c = torch.nn.functional.cosine_similarity(a, b, dim=0) if b.abs().sum() > 0 else torch.tensor(1.0)
    return bool((a - b).abs().max() <= rel * scale) and bool(c > cos)


@pytest.fixture(scope="module")
def ops():
    from hyc_lora_release_b200.operators import (
        rmsnorm_kernels, softmax_kernels,
        triton_fuse_lora_silu_hadamard_backward_kernels as bk,
        triton_fuse_lora_silu_hadamard_forward_kernels as fk)
    return fk.triton_fuse_silu_forward, bk.triton_fuse_silu_backward, rmsnorm_kernels, softmax_kernels


@pytest.mark.parametrize("q", QS)
def test_golden_fused(ops, golden, q):
    fwd, bwd, _, _ = ops
    d = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in golden[f"q{q}"].items()}
    q1, q2, o = fwd(d["f_xa1"], d["f_b1"], d["f_x1"], d["f_s1"], d["f_xa2"], d["f_b2"], d["f_x2"], d["f_s2"], q)
    assert torch.equal(q1, d["f_q1"]) and torch.equal(q2, d["f_q2"])
    assert close(o, d["f_o"])
    assert (o != d["f_o"]).float().mean() < 0.02          # almost every element identical
    bo, gg, gu = bwd(d["f_xa1"], d["f_b1"], q1, d["f_s1"], d["f_xa2"], d["f_b2"], q2, d["f_s2"], d["f_go"], q)
    assert close(bo, d["f_bo"]) and close(gg, d["f_ggate"]) and close(gu, d["f_gup"])
    # the backward recomputes the forward output from the saved codes
    assert (bo != d["f_bo"]).float().mean() < 0.02


@pytest.mark.parametrize("q", QS)
@pytest.mark.parametrize("shape", [(1, 16, 32), (2, 50, 96), (1, 37, 11008), (2, 128, 1024)])
def test_oracle_fused(ops, q, shape):
    fwd, bwd, _, _ = ops
    B, M, N = shape
    g = torch.Generator().manual_seed(B * M + N + q)
    R = 16
    xa1, xa2 = torch.randn(B, M, R, generator=g).bfloat16(), torch.randn(B, M, R, generator=g).bfloat16()
    # LoRA-B as the layers pass it: the transposed view of an [N, R] weight
    w1, w2 = (torch.randn(N, R, generator=g) * 0.05).bfloat16(), (torch.randn(N, R, generator=g) * 0.05).bfloat16()
    b1, b2 = w1.T, w2.T
    x1, x2 = torch.randn(B, M, N, generator=g).bfloat16(), torch.randn(B, M, N, generator=g).bfloat16()
    s1, s2 = oracle.ref_scale_per_channel(x1, q), oracle.ref_scale_per_channel(x2, q)
    s1 = torch.where(s1 == 0, torch.tensor(1e-3, dtype=torch.bfloat16), s1)
    s2 = torch.where(s2 == 0, torch.tensor(1e-3, dtype=torch.bfloat16), s2)
    go = torch.randn(B, M, N, generator=g).bfloat16()
    oq1, oq2, oo = oracle.ref_fused_silu_forward(xa1, b1, x1, s1, xa2, b2, x2, s2, q)
    t = lambda *a: [v.to(DEV) for v in a]
    q1, q2, o = fwd(*t(xa1, b1, x1, s1, xa2, b2, x2, s2), q)
    assert torch.equal(q1.cpu(), oq1) and torch.equal(q2.cpu(), oq2) and close(o, oo)
    # contiguous [R, N] LoRA-B (what the reference's wrapper makes) gives the same result
    q1c, q2c, oc = fwd(*t(xa1, b1.contiguous(), x1, s1, xa2, b2.contiguous(), x2, s2), q)
    assert torch.equal(q1c, q1) and torch.equal(oc, o)
    ob, ogg, ogu = oracle.ref_fused_silu_backward(xa1, b1, oq1, s1, xa2, b2, oq2, s2, go, q)
    bo, gg, gu = bwd(*t(xa1, b1, oq1, s1, xa2, b2, oq2, s2, go), q)
    assert close(bo, ob) and close(gg, ogg) and close(gu, ogu)


def test_fused_linearity_at_full_width(ops):
    """Size-independent properties at the Mistral width: grad_up is linear in grad_o, and a zero
    LoRA-B makes o = silu(dequant(q1)) * dequant(q2)."""
    fwd, bwd, _, _ = ops
    from hyc_lora_release_b200.operators import compress_function as cf
    g = torch.Generator().manual_seed(4)
    B, M, N, R, q = 1, 512, 14336, 16, 4
    xa = torch.randn(B, M, R, generator=g).bfloat16().to(DEV)
    bz = torch.zeros(R, N, dtype=torch.bfloat16, device=DEV)
    x1 = torch.randn(B, M, N, generator=g).bfloat16().to(DEV)
    x2 = torch.randn(B, M, N, generator=g).bfloat16().to(DEV)
    s1, s2 = cf.get_statistics_only_quant(x1, q, "per-channel"), cf.get_statistics_only_quant(x2, q, "per-channel")
    q1, q2, o = fwd(xa, bz, x1, s1, xa, bz, x2, s2, q)
    assert torch.equal(q1, cf.compression_quantization(x1, s1, q)) and torch.equal(q2, cf.compression_quantization(x2, s2, q))
    go = torch.randn(B, M, N, generator=g).bfloat16().to(DEV)
    bo, gg, gu = bwd(xa, bz, q1, s1, xa, bz, q2, s2, go, q)
    d1, d2 = cf.decompression_dequantization(q1, s1, q), cf.decompression_dequantization(q2, s2, q)
    sig = torch.sigmoid(d1.float()).bfloat16()
    want = ((d1 * sig) * d2)
    assert close(bo, want)
    _, _, gu2 = bwd(xa, bz, q1, s1, xa, bz, q2, s2, go * 2, q)
    assert torch.equal(gu2, gu * 2)


def test_fused_unaligned_tensors_take_the_narrow_kernel(ops):
    """Tensors that are only 4-byte aligned (a view into a larger buffer) go through the fragment-layout kernel;
    its results are bit-identical to the wide kernel's."""
    from hyc_lora_release_b200._lib import check, lib, ptr, stream_of
    import ctypes
    g = torch.Generator().manual_seed(3)
    rows, N, q = 45, 160, 4
    x1, x2 = torch.randn(rows, N, generator=g).bfloat16(), torch.randn(rows, N, generator=g).bfloat16()
    xa1, xa2 = torch.randn(rows, 16, generator=g).bfloat16(), torch.randn(rows, 16, generator=g).bfloat16()
    bt1, bt2 = (torch.randn(N, 16, generator=g) * 0.05).bfloat16(), (torch.randn(N, 16, generator=g) * 0.05).bfloat16()
    s1, s2 = oracle.ref_scale_per_channel(x1[None], q).reshape(-1), oracle.ref_scale_per_channel(x2[None], q).reshape(-1)
    d = lambda t: t.to(DEV)
    xa1d, xa2d, bt1d, bt2d, s1d, s2d, x2d = map(d, (xa1, xa2, bt1, bt2, s1, s2, x2))
    outs = []
    for shift in (0, 2):        # elements: 0 -> 16-byte aligned, 2 -> 4-byte aligned
        base = torch.zeros(rows * N + 8, dtype=torch.bfloat16, device=DEV)
        x1d = base[shift:shift + rows * N].view(rows, N)
        x1d.copy_(x1)
        q1 = torch.empty(rows, N // 2, dtype=torch.uint8, device=DEV); q2 = torch.empty_like(q1)
        o = torch.empty(rows, N, dtype=torch.bfloat16, device=DEV)
        check(lib.hyc_fused_lora_silu_hadamard_fwd(ptr(xa1d), ptr(bt1d), ctypes.c_void_p(x1d.data_ptr()), ptr(s1d), ptr(xa2d),
                                                   ptr(bt2d), ptr(x2d), ptr(s2d), ptr(q1), ptr(q2), ptr(o), rows, N, 16, q,
                                                   stream_of(o)), "fwd")
        outs.append((q1, q2, o))
    assert all(torch.equal(a, b) for a, b in zip(outs[0], outs[1]))


@pytest.mark.parametrize("shape", [(3, 64), (2, 7, 4096), (1, 33, 11008), (5, 16384)])
def test_rmsnorm(ops, shape):
    _, _, rn, _ = ops
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(shape[-1], generator=g)).bfloat16()
    y, mean, rstd, bs, nw = rn.rmsnorm_forward(x.to(DEV), w.to(DEV), 1e-5)
    oy, orstd = oracle.ref_rmsnorm_forward(x, w, 1e-5)
    assert torch.allclose(rstd.cpu(), orstd, rtol=1e-5, atol=0) and close(y, oy, rel=4e-3)
    dy = torch.randn(*shape, generator=g).bfloat16()
    dx, none = rn.rmsnorm_backward(dy.to(DEV), x.to(DEV), w.to(DEV), mean, rstd, True, 1e-5, nw, bs)
    assert none is None and close(dx, oracle.ref_rmsnorm_backward(dy, x, w, orstd), rel=4e-3)


def test_rmsnorm_and_softmax_backward_golden(ops, golden):
    """Against the reference's own kernels (fixtures made by running them through the Triton interpreter): the
    fp32 row sums are taken in another order on the device, so a result may land on the neighbouring bf16 value
    where it sits at a rounding boundary; everything else must be equal."""
    _, _, rn, sm = ops
    d = golden["rmsnorm"]
    y, mean, rstd, bs, nw = rn.rmsnorm_forward(d["x"].to(DEV), d["w"].to(DEV), d["eps"])
    assert ((rstd.cpu() - d["rstd"]).abs() <= d["rstd"].abs() * 1e-6).all()
    assert float((y.cpu() != d["y"]).float().mean()) < 2e-3 and close(y, d["y"], rel=4e-3)
    dx, _ = rn.rmsnorm_backward(d["dy"].to(DEV), d["x"].to(DEV), d["w"].to(DEV), mean, d["rstd"].to(DEV), True, d["eps"], nw, bs)
    assert float((dx.cpu() != d["dx"]).float().mean()) < 5e-3 and close(dx, d["dx"], rel=4e-3)
    s = golden["softmax_bwd"]
    o = sm.softmax_backward(s["y"].to(DEV), s["g"].to(DEV))
    assert float((o.cpu() != s["o"]).float().mean()) < 5e-3 and close(o, s["o"], rel=4e-3)


@pytest.mark.parametrize("q", (2, 4, 8))
@pytest.mark.parametrize("shape", [(3, 64), (2, 7, 4096), (1, 33, 11008), (5, 16384), (1, 300, 4128)])
def test_rmsnorm_fused_with_saves(ops, q, shape):
    """One-pass norm + saves and the backward on the packed x: bit-identical to the separate operators, which
    the other tests tie to the oracle; the packed x is also checked against the oracle directly."""
    from hyc_lora_release_b200.operators import compress_function as cf
    _, _, rn, _ = ops
    N = shape[-1]
    g = torch.Generator().manual_seed(sum(shape) + q)
    x = torch.randn(*shape, generator=g)
    n_out = max(1, N // 100)
    x[..., torch.randperm(N, generator=g)[:n_out]] *= 25.0
    x[..., 40:43] *= 30.0                       # three outlier channels inside one octet
    x = x.bfloat16().reshape(-1, shape[-2] if len(shape) > 1 else 1, N)
    w = (1 + 0.1 * torch.randn(N, generator=g)).bfloat16()
    xd, wd = x.to(DEV), w.to(DEV)
    ratio = 0.02
    idx, sx = cf.get_statistics_channel_base(xd, ratio, q, "per-channel")
    y0, _, rstd0, _, _ = rn.rmsnorm_forward(xd, wd, 1e-5)
    sy = cf.get_statistics_only_quant(y0, q, "per-channel")
    xo0, qx0 = cf.outlier_subtraction_fuse_compression_quantization(xd, sx, idx, q)
    qy0 = cf.compression_quantization(y0, sy, q)
    y, rstd, xo, qx, qy = rn.rmsnorm_forward_save(xd, wd, 1e-5, q, sx, idx, sy)
    assert torch.equal(y, y0) and torch.equal(rstd, rstd0.reshape(-1))
    assert torch.equal(qx, qx0) and torch.equal(xo, xo0) and torch.equal(qy, qy0)
    oxo, oqx = oracle.ref_compress_channel_base(x, sx.cpu(), idx.cpu(), q)
    assert torch.equal(qx.cpu(), oqx) and torch.equal(xo.cpu(), oxo)
    # without the second save and without outlier channels
    y1, rstd1, xo1, qx1, qy1 = rn.rmsnorm_forward_save(xd, wd, 1e-5, q, sx, None, None)
    assert qy1 is None and xo1.shape[-1] == 0 and torch.equal(y1, y0)
    assert torch.equal(qx1, cf.compression_quantization(xd, sx, q))
    # backward on the packed x
    dy = torch.randn(*x.shape, generator=g).bfloat16().to(DEV)
    res = torch.randn(*x.shape, generator=g).bfloat16().to(DEV)
    x_hat = cf.outlier_addition_fuse_decompression_dequantization(qx0, sx, xo0, idx, q)
    dx0, _ = rn.rmsnorm_backward(dy, x_hat, wd, None, rstd0, True, 1e-5, 0, 0)
    dx = rn.rmsnorm_backward_packed(dy, qx, sx, xo, idx, wd, rstd, q)
    assert torch.equal(dx, dx0)
    dx_r = rn.rmsnorm_backward_packed(dy, qx, sx, xo, idx, wd, rstd, q, residual_grad=res)
    assert torch.equal(dx_r, dx0 + res)


@pytest.mark.parametrize("q", (2, 4, 8))
@pytest.mark.parametrize("shape", [(1, 5, 32), (2, 33, 96), (1, 300, 4096), (1, 17, 11008)])
def test_dequant_lora_add(ops, q, shape):
    """decompression_dequantization + LoRA re-add in one kernel: bit-exact against the oracle's de-quantizer
    followed by a bf16 add of the bf16 LoRA term computed by the same tensor-core product as the fused kernels
    (checked here against fp32 within one bf16 rounding)."""
    from hyc_lora_release_b200.operators import compress_function as cf
    B, M, N = shape
    g = torch.Generator().manual_seed(sum(shape) + q)
    x = torch.randn(B, M, N, generator=g).bfloat16()
    xa = torch.randn(B, M, 16, generator=g).bfloat16()
    b = (torch.randn(16, N, generator=g) * 0.05).bfloat16()
    s = oracle.ref_scale_per_channel(x, q)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=torch.bfloat16), s)
    pk = oracle.ref_compress(x, s, q)
    y = cf.decompression_dequantization_lora_add(pk.to(DEV), s.to(DEV), xa.to(DEV), b.to(DEV), q)
    xh = oracle.ref_decompress(pk, s, q)
    lora = (xa.float() @ b.float()).to(torch.bfloat16)
    ref = (xh.float() + lora.float()).to(torch.bfloat16)
    yc = y.cpu()
    mism = (yc != ref)
    # the only freedom is the summation order of the rank-16 product before its bf16 rounding
    assert mism.float().mean() < 2e-3 and close(y, ref, rel=4e-3)
    plain = cf.decompression_dequantization(pk.to(DEV), s.to(DEV), q)
    zero = cf.decompression_dequantization_lora_add(pk.to(DEV), s.to(DEV), torch.zeros_like(xa).to(DEV), b.to(DEV), q)
    assert torch.equal(zero, plain)


@pytest.mark.parametrize("shape", [(1, 2, 8, 8), (2, 3, 100, 104), (1, 4, 512, 512), (1, 1, 16, 4096)])
def test_softmax_backward(ops, shape):
    _, _, _, sm = ops
    g = torch.Generator().manual_seed(sum(shape))
    y = torch.softmax(3 * torch.randn(*shape, generator=g), -1).bfloat16()
    gy = torch.randn(*shape, generator=g).bfloat16()
    o = sm.softmax_backward(y.to(DEV), gy.to(DEV))
    assert close(o, oracle.ref_softmax_backward(y, gy), rel=4e-3)
