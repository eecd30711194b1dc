"""Parity of the per-channel quantize/pack and unpack/dequantize kernels (called through the
C ABI by the Python operator layer) with the golden fixtures and the CPU oracle.
Codes, indices and outlier values are bit-exact."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
QS = (2, 4, 8)
DEV = "cuda"


@pytest.fixture(scope="module")
def cf():
    from hyc_lora_release_b200.operators import compress_function
    return compress_function


@pytest.mark.parametrize("q", QS)
def test_golden_scale_pack_dequant(cf, golden, q):
    d = golden[f"q{q}"]
    x = d["x"].to(DEV)
    assert torch.equal(cf.get_statistics_only_quant(x, q, "per-channel").cpu(), d["scale"])
    pk = cf.compression_quantization(x, d["scale_safe"].to(DEV), q)
    assert torch.equal(pk.cpu(), d["packed"])
    xr = cf.decompression_dequantization(pk, d["scale_safe"].to(DEV), q)
    assert torch.equal(xr.cpu(), d["dequant"])
    assert torch.equal(cf.get_statistics_only_quant(d["xh"].to(DEV), q, "per-channel").cpu(), d["xh_scale"])


@pytest.mark.parametrize("q", QS)
def test_golden_zero_point(cf, golden, q):
    d = golden[f"q{q}"]
    xz = d["xz"].to(DEV)
    s, z = cf.get_statistics_only_quant_zero_point(xz, q, "per-channel")
    assert torch.equal(s.cpu(), d["zp_scale"]) and torch.equal(z.cpu(), d["zp"])
    pk = cf.compression_quantization_with_zero_point(xz, s, z, q)
    assert torch.equal(pk.cpu(), d["zp_packed"])
    xr = cf.decompression_dequantization_with_zero_point(pk, s, z, q)
    assert torch.equal(xr.cpu(), d["zp_dequant"])


@pytest.mark.parametrize("q", QS)
def test_pack_quant_zp_base_calibration_and_static(cf, golden, q):
    """``compression_pack_quant_zp_base`` (compress_function.py:364-370): statistics while calibrating, the stored
    ones afterwards; both branches against the golden vectors of the zero-point kernels."""
    d = golden[f"q{q}"]
    xz = d["xz"].to(DEV)
    pk, s, z = cf.compression_pack_quant_zp_base(xz, q, "per-channel", 0, 5, None)
    assert torch.equal(s.cpu(), d["zp_scale"]) and torch.equal(z.cpu(), d["zp"]) and torch.equal(pk.cpu(), d["zp_packed"])
    static = {"scale": d["zp_scale"].to(DEV), "zero_point": d["zp"].to(DEV)}
    other = (xz.float() * 0.5).to(torch.bfloat16)         # its own statistics would differ: the stored ones must be used
    pk2, s2, z2 = cf.compression_pack_quant_zp_base(other, q, "per-channel", 7, 5, static)
    assert s2 is static["scale"] and z2 is static["zero_point"]
    assert torch.equal(pk2.cpu(), oracle.ref_compress(other.cpu(), d["zp_scale"], q, d["zp"]))
    assert torch.equal(cf.decompression_dequantization_with_zero_point(pk, s, z, q).cpu(), d["zp_dequant"])


@pytest.mark.parametrize("q", QS)
def test_golden_channel_base(cf, golden, q):
    d = golden[f"q{q}"]
    x = d["x"].to(DEV)
    idx, s = cf.get_statistics_channel_base(x, d["cb_ratio"], q, "per-channel")
    assert sorted(idx.tolist()) == sorted(d["cb_idx"].tolist())
    assert torch.equal(s.cpu(), d["cb_scale"])
    x_before = x.clone()
    xo, pk = cf.outlier_subtraction_fuse_compression_quantization(x, d["cb_scale"].to(DEV), d["cb_idx"].to(DEV), q)
    assert torch.equal(x, x_before)                       # input is not modified
    assert torch.equal(xo.cpu(), d["cb_outlier"]) and torch.equal(pk.cpu(), d["cb_packed"])
    xr = cf.outlier_addition_fuse_decompression_dequantization(pk, d["cb_scale"].to(DEV), xo, d["cb_idx"].to(DEV), q)
    assert torch.equal(xr.cpu(), d["cb_restored"])
    # the pack wrapper, calibration branch and static branch
    o, qq, ci, sc = cf.compression_pack_channel_base(x, d["cb_ratio"], q, "per-channel", 0, 5, None)
    o2, qq2, ci2, sc2 = cf.compression_pack_channel_base(
        x, d["cb_ratio"], q, "per-channel", 5, 5, {"outlier_channel_index": ci, "scale": sc})
    assert torch.equal(qq, qq2) and torch.equal(o, o2)


def _planted(B, M, N, n_out, mult, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, M, N, generator=g)
    ch = torch.randperm(N, generator=g)[:n_out]
    x[:, :, ch] *= mult
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("q", QS)
@pytest.mark.parametrize("shape", [(1, 1, 32), (2, 7, 96), (3, 33, 1024), (1, 130, 11008), (2, 5, 14336)])
def test_oracle_ragged_shapes(cf, q, shape):
    B, M, N = shape
    x = _planted(B, M, N, max(1, N // 100), 20.0, 11 + N + q)
    s = oracle.ref_scale_per_channel(x, q)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=torch.bfloat16), s)
    xd = x.to(DEV)
    assert torch.equal(cf.get_statistics_only_quant(xd, q, "per-channel").cpu(), oracle.ref_scale_per_channel(x, q))
    pk = cf.compression_quantization(xd, s.to(DEV), q)
    assert torch.equal(pk.cpu(), oracle.ref_compress(x, s, q))
    assert torch.equal(cf.decompression_dequantization(pk, s.to(DEV), q).cpu(), oracle.ref_decompress(pk.cpu(), s, q))
    # channel-base with k outliers, sequence-exact index order
    ratio = 0.02
    k = int(N * ratio)
    idx, sc = cf.get_statistics_channel_base(xd, ratio, q, "per-channel")
    oidx, osc = oracle.ref_statistics_channel_base(x, ratio, q)
    assert torch.equal(idx.cpu(), oidx) and torch.equal(sc.cpu(), osc) and idx.numel() == k
    xo, pk2 = cf.outlier_subtraction_fuse_compression_quantization(xd, sc, idx, q)
    oxo, opk = oracle.ref_compress_channel_base(x, osc, oidx, q)
    assert torch.equal(xo.cpu(), oxo) and torch.equal(pk2.cpu(), opk)
    xr = cf.outlier_addition_fuse_decompression_dequantization(pk2, sc, xo, idx, q)
    assert torch.equal(xr.cpu(), oracle.ref_decompress_channel_base(opk, osc, oxo, oidx, q))


@pytest.mark.parametrize("q", QS)
def test_clustered_outlier_channels(cf, q):
    """Outlier channels packed next to each other: single threads own 3..8 of them (more than they keep in
    registers), whole blocks of 32 columns are outliers, and the list is not sorted."""
    B, M, N = 2, 37, 2048
    g = torch.Generator().manual_seed(5 + q)
    x = torch.randn(B, M, N, generator=g).to(torch.bfloat16)
    cols = list(range(64, 72)) + [100, 101, 102] + list(range(512, 544)) + [1031, 1047, 1063, 1079] + [2047, 0, 33, 35, 37]
    idx = torch.tensor(cols, dtype=torch.int64)[torch.randperm(len(cols), generator=g)]
    s = oracle.ref_scale_per_channel(x, q)
    s = torch.where(s == 0, torch.tensor(1e-3, dtype=torch.bfloat16), s)
    xd, sd, idxd = x.to(DEV), s.to(DEV), idx.to(DEV)
    xo, pk = cf.outlier_subtraction_fuse_compression_quantization(xd, sd, idxd, q)
    oxo, opk = oracle.ref_compress_channel_base(x, s, idx, q)
    assert torch.equal(xo.cpu(), oxo) and torch.equal(pk.cpu(), opk)
    xr = cf.outlier_addition_fuse_decompression_dequantization(pk, sd, xo, idxd, q)
    assert torch.equal(xr.cpu(), oracle.ref_decompress_channel_base(opk, s, oxo, idx, q))


def test_config0_full_size(cf):
    """bf16 [4,512,4096], 0.5 % channels x30, ratio 0.005, q_bit 4 (the CPU-runnable config)."""
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(4, 512, 4096, generator=g)
    ch = torch.randperm(4096, generator=g)[:20]
    x[:, :, ch] *= 30
    x = x.to(torch.bfloat16)
    xd = x.to(DEV)
    o, q, idx, s = cf.compression_pack_channel_base(xd.clone(), 0.005, 4, "per-channel", 0, 5, None)
    oidx, os_ = oracle.ref_statistics_channel_base(x, 0.005, 4)
    assert sorted(idx.tolist()) == sorted(ch.tolist())
    assert torch.equal(idx.cpu(), oidx) and torch.equal(s.cpu(), os_)
    oxo, opk = oracle.ref_compress_channel_base(x, os_, oidx, 4)
    assert torch.equal(o.cpu(), oxo) and torch.equal(q.cpu(), opk)
    xr = cf.outlier_addition_fuse_decompression_dequantization(q, s, o, idx, 4)
    assert torch.equal(xr.cpu(), oracle.ref_decompress_channel_base(opk, os_, oxo, oidx, 4))
    # reconstruction error: within half a step per channel unless clipped; outlier columns exact
    err = (xr.float().cpu() - x.float()).abs()
    assert torch.equal(xr[:, :, idx].cpu(), x[:, :, oidx])
    clipped = (x.float() / os_.float()).abs() > 7.5
    assert (err[~clipped] <= 0.51 * os_.float().expand_as(err)[~clipped] + 0.02 * x.float().abs()[~clipped]).all()


@pytest.mark.parametrize("q", QS)
def test_all_byte_values_decode(cf, q):
    epp = 8 // q
    N = 32 * 8 * epp
    pk = torch.arange(256, dtype=torch.uint8).repeat(3, 5, N // epp // 256 + 1)[:, :, : N // epp].contiguous()
    g = torch.Generator().manual_seed(5)
    s = (torch.rand(1, N, generator=g) + 0.01).to(torch.bfloat16)
    z = torch.randint(-128, 128, (1, N), generator=g, dtype=torch.int8)
    assert torch.equal(cf.decompression_dequantization(pk.to(DEV), s.to(DEV), q).cpu(), oracle.ref_decompress(pk, s, q))
    assert torch.equal(cf.decompression_dequantization_with_zero_point(pk.to(DEV), s.to(DEV), z.to(DEV), q).cpu(),
                       oracle.ref_decompress(pk, s, q, z))


@pytest.mark.parametrize("q", QS)
def test_ties_clipping_and_extremes(cf, q):
    """Exact .5 quotients (both signs), values far outside the range, zeros, small and large
    scales.  (Quotients beyond the fp32 range are outside the kernel's domain.)"""
    N = 64
    half = 2 ** (q - 1)
    base = torch.arange(-half - 3, half + 3, dtype=torch.float32)
    vals = torch.cat([base + 0.5, base, base + 0.25, torch.tensor([0.0, -0.0, 1e4, -1e4, 3e30, -3e30, 1e-30])])
    scales = torch.tensor([1.0, 0.5, 2.0, 0.0625, 3.0, 1e-3, 0.75, 1e3] * (N // 8))
    x = (vals[:, None] * scales[None, :]).to(torch.bfloat16)[None]
    s = scales[None, :].to(torch.bfloat16)
    pk = cf.compression_quantization(x.to(DEV), s.to(DEV), q)
    assert torch.equal(pk.cpu(), oracle.ref_compress(x, s, q))


def test_empty_and_strided_inputs(cf):
    s = torch.ones(1, 64, dtype=torch.bfloat16, device=DEV)
    e = cf.compression_quantization(torch.empty(0, 4, 64, dtype=torch.bfloat16, device=DEV), s, 4)
    assert e.shape == (0, 4, 32)
    g = torch.Generator().manual_seed(3)
    big = torch.randn(2, 9, 256, generator=g).to(torch.bfloat16)
    view = big[:, :, 64:128]                    # row stride 256, offset 128 bytes
    view_t = big.transpose(0, 1)[:, :, :64]     # batch/sequence strides swapped
    bd = big.to(DEV)
    for v, vd in ((view, bd[:, :, 64:128]), (view_t, bd.transpose(0, 1)[:, :, :64])):
        assert not vd.is_contiguous()
        assert torch.equal(cf.compression_quantization(vd, s, 4).cpu(), oracle.ref_compress(v, s.cpu(), 4))
    # 4-D head layout goes through head_to_hidden (compress_function.py:181-183)
    xh = torch.randn(2, 4, 9, 16, generator=g).to(torch.bfloat16)
    pk = cf.compression_quantization(xh.to(DEV), s, 4)
    assert torch.equal(pk.cpu(), oracle.ref_compress(xh, s.cpu(), 4))
    xr = cf.decompression_dequantization(pk, s, 4, is_head=True, num_heads=4)
    assert xr.shape == (2, 4, 9, 16)


def test_idempotent_requantization(cf):
    """Size-independent property at the Mistral MLP width: quantizing a de-quantized tensor
    with the same scale reproduces the codes."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(2, 1024, 14336, generator=g).to(torch.bfloat16).to(DEV)
    for q in QS:
        s = cf.get_statistics_only_quant(x, q, "per-channel")
        pk = cf.compression_quantization(x, s, q)
        xr = cf.decompression_dequantization(pk, s, q)
        # bf16 rounding moves code*s by at most 2^-9 relative, i.e. less than half a step
        assert torch.equal(cf.compression_quantization(xr, s, q), pk)
