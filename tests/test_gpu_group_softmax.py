"""Group mode, attention-map threshold prune and per-row top-k against the CPU oracle."""
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


def _softmax_map(b, h, s, seed, causal=True):
    g = torch.Generator().manual_seed(seed)
    logits = 3 * torch.randn(b, h, s, s, generator=g)
    if causal:
        logits = logits + torch.triu(torch.full((s, s), float("-inf")), diagonal=1)
    return torch.softmax(logits, dim=-1).to(torch.bfloat16)


@pytest.mark.parametrize("q", QS)
@pytest.mark.parametrize("shape", [(1, 64), (5, 192), (7, 512), (3, 1088), (2, 4096), (9, 11008)])
def test_group_mode(cf, q, shape):
    rows, N = shape
    g = torch.Generator().manual_seed(rows * N + q)
    x = torch.randn(rows, N, generator=g) * torch.rand(rows, 1, generator=g) * 4 + torch.randn(rows, 1, generator=g)
    x[0, :64] = 0.375              # a constant group (zero range)
    x[-1, -64:] = 200.0 + torch.rand(64, generator=g)   # zero point saturates
    x = x.to(torch.bfloat16)
    pk, s, z = cf.compression_group(x.to(DEV), q)
    opk, os_, oz = oracle.group_compress(x, q)
    assert torch.equal(s.cpu(), os_) and torch.equal(z.cpu(), oz) and torch.equal(pk.cpu(), opk)
    assert torch.equal(cf.decompression_group(pk, s, z, q).cpu(), oracle.group_decompress(opk, os_, oz, q))


@pytest.mark.parametrize("q", QS)
def test_group_mode_strided_rows(cf, q):
    """Rows with a stride larger than N go through the C ABI directly (the Python operator always makes
    its input contiguous); they take the warp-per-512-columns kernels instead of the flat ones."""
    from hyc_lora_release_b200._lib import check, lib, ptr, stream_of
    rows, N, ld = 6, 576, 640
    g = torch.Generator().manual_seed(q)
    full = (torch.randn(rows, ld, generator=g) * 3).to(torch.bfloat16)
    x = full[:, :N]
    xd = full.to(DEV)
    pk = torch.empty(rows, N * q // 8, dtype=torch.uint8, device=DEV)
    s = torch.empty(rows, N // 64, dtype=torch.bfloat16, device=DEV)
    z = torch.empty(rows, N // 64, dtype=torch.int8, device=DEV)
    check(lib.hyc_group_quant_pack(ptr(xd), rows, N, ld, ptr(pk), ptr(s), ptr(z), q, stream_of(xd)), "quant")
    opk, os_, oz = oracle.group_compress(x.contiguous(), q)
    assert torch.equal(s.cpu(), os_) and torch.equal(z.cpu(), oz) and torch.equal(pk.cpu(), opk)
    out = torch.full((rows, ld), 7.0, dtype=torch.bfloat16, device=DEV)
    check(lib.hyc_group_unpack_dequant(ptr(pk), rows, N, ptr(s), ptr(z), ptr(out), ld, q, stream_of(xd)), "dequant")
    assert torch.equal(out[:, :N].cpu(), oracle.group_decompress(opk, os_, oz, q))
    assert (out[:, N:] == 7.0).all()


def test_softmax_prune_golden(cf, golden):
    d = golden["softmax"]
    a = d["a"].to(DEV)
    thr = cf.get_statistics_softmax(a, d["ratio"])
    assert torch.equal(thr.cpu(), d["thr"])
    for t, i, v in ((d["thr"], d["idx"], d["val"]), (d["thr2"], d["idx2"], d["val2"])):
        sp = cf.compression_softmax(a, t.to(DEV))
        assert sp.is_sparse and torch.equal(sp.indices().cpu(), i) and torch.equal(sp.values().cpu(), v)
    sp = cf.compression_softmax(a, d["thr"])
    assert torch.equal(sp.to_dense().reshape(a.shape).cpu(), d["dense"])              # what the layers call
    assert torch.equal(cf.decompression_softmax(sp).reshape(a.shape).cpu(), d["dense"])  # our restore kernel
    h, thr2 = cf.compression_pack_softmax_base(a, d["ratio"], 0, 5, None)
    assert torch.equal(thr2.cpu(), d["thr"]) and torch.equal(h.indices().cpu(), d["idx"])


@pytest.mark.parametrize("shape", [(1, 1, 8, 8), (2, 3, 100, 100), (1, 2, 512, 512), (1, 1, 1000, 1000)])
def test_softmax_prune_oracle(cf, shape):
    a = _softmax_map(*shape[:3], seed=sum(shape))
    thr = oracle.ref_softmax_threshold(a, 0.05)
    sp = cf.compression_softmax(a.to(DEV), thr)
    idx, val = oracle.ref_softmax_prune(a, thr)
    assert torch.equal(sp.indices().reshape(-1).cpu(), idx) and torch.equal(sp.values().cpu(), val)
    assert torch.equal(cf.decompression_softmax(sp).reshape(a.shape).cpu(), oracle.ref_softmax_restore(idx, val, a.shape))
    # nothing kept / everything kept
    none = cf.compression_softmax(a.to(DEV), 2.0)
    assert none.values().numel() == 0 and torch.equal(cf.decompression_softmax(none).cpu(), torch.zeros(a.numel(), dtype=torch.bfloat16))
    allk = cf.compression_softmax(a.to(DEV), -1.0)
    assert allk.values().numel() == int((a != 0).sum())


@pytest.mark.parametrize("numel", [1, 7, 4095, 4097, 3 * 4096 + 5, 9 * 4096 + 8 * 31 + 3, 70001])
def test_softmax_prune_ragged_sizes(cf, numel):
    """Element counts that end inside a 16-byte chunk, inside a warp trip and inside a tile; dense and sparse keeps."""
    g = torch.Generator().manual_seed(numel)
    a = torch.rand(numel, generator=g).to(torch.bfloat16)
    a[torch.rand(numel, generator=g) < 0.2] = 0
    for thr in (0.9, 0.5, -1.0):
        idx, val = oracle.ref_softmax_prune(a, torch.tensor(thr))
        sp = cf.compression_softmax(a.to(DEV), thr)
        assert torch.equal(sp.indices().reshape(-1).cpu(), idx) and torch.equal(sp.values().cpu(), val)
        assert torch.equal(cf.decompression_softmax(sp).cpu(), oracle.ref_softmax_restore(idx, val, a.shape))
        for ordered in (True, False):
            m = cf.compression_softmax_static(a.to(DEV), thr, capacity=numel, ordered=ordered)
            n = int(m.nnz.item())
            mi, mv = (m.idx[:n], m.val[:n]) if ordered else m.entries()
            assert n == idx.numel() and torch.equal(mi.cpu(), idx) and torch.equal(mv.cpu(), val)
            assert torch.equal(m.to_dense().cpu(), oracle.ref_softmax_restore(idx, val, a.shape))


@pytest.mark.parametrize("q", QS)
@pytest.mark.parametrize("shape", [(1, 1, 64, 64), (2, 2, 128, 128), (1, 2, 512, 512), (1, 1, 320, 320), (1, 1, 64, 2048),
                                   (1, 1, 13, 128), (1, 1, 5, 1024), (1, 3, 256, 256), (1, 1, 3, 4096)])
def test_topk_mode(cf, q, shape):
    b, h, r, s = shape
    if r == s:
        a = _softmax_map(b, h, s, seed=s + q)
    else:
        g = torch.Generator().manual_seed(s + q)
        a = torch.softmax(3 * torch.randn(b, h, r, s, generator=g), -1).to(torch.bfloat16)
    m = cf.compression_softmax_topk(a.to(DEV), 0.05, q)
    vals, cols, pk, sc, zp = oracle.topk_compress(a, 0.05, q)
    assert torch.equal(m.col.cpu().to(torch.int64) & 0xFFFF, cols)
    assert torch.equal(m.val.cpu(), vals)
    assert torch.equal(m.scale.cpu(), sc) and torch.equal(m.zp.cpu(), zp) and torch.equal(m.q.cpu(), pk)
    assert torch.equal(m.to_dense().cpu(), oracle.topk_decompress(vals, cols, pk, sc, zp, q, a.shape))


def test_topk_ties_and_signs(cf):
    """Many equal magnitudes (ties go to the lower column), negative values, all-zero rows."""
    g = torch.Generator().manual_seed(77)
    S = 256
    x = (torch.randint(-3, 4, (40, S), generator=g).float() * 0.25)
    x[0] = 0.0
    x[1] = 1.0
    x[2, ::2] = -2.0
    x = x.to(torch.bfloat16)
    for ratio in (0.05, 0.25, 0.0, 1.0):
        m = cf.compression_softmax_topk(x.to(DEV), ratio, 4)
        vals, cols, pk, sc, zp = oracle.topk_compress(x, ratio, 4)
        assert torch.equal(m.col.cpu().to(torch.int64) & 0xFFFF, cols) and torch.equal(m.val.cpu(), vals)
        assert torch.equal(m.q.cpu(), pk) and torch.equal(m.scale.cpu(), sc) and torch.equal(m.zp.cpu(), zp)
        assert torch.equal(m.to_dense().cpu(), oracle.topk_decompress(vals, cols, pk, sc, zp, 4, x.shape))


@pytest.mark.parametrize("S,rows", [(64, 37), (512, 7), (2048, 3)])
def test_topk_ties_lane_layout(cf, S, rows):
    """Few distinct magnitudes in rows of 64 * 2^n columns (one lane per group of 64): partial ties at the
    threshold inside a lane, across lanes, rows with fewer non-zeros than k, and a ragged last warp."""
    g = torch.Generator().manual_seed(S + rows)
    x = (torch.randint(-2, 3, (rows, S), generator=g).float() * 0.5)
    x[0] = 0.0
    x[1, : S // 2] = 0.0
    x[2] = -1.0
    x = x.to(torch.bfloat16)
    for ratio in (0.02, 0.05, 0.11):
        for q in (2, 4, 8):
            m = cf.compression_softmax_topk(x.to(DEV), ratio, q)
            vals, cols, pk, sc, zp = oracle.topk_compress(x, ratio, q)
            assert torch.equal(m.col.cpu().to(torch.int64) & 0xFFFF, cols) and torch.equal(m.val.cpu(), vals)
            assert torch.equal(m.q.cpu(), pk) and torch.equal(m.scale.cpu(), sc) and torch.equal(m.zp.cpu(), zp)
            assert torch.equal(m.to_dense().cpu(), oracle.topk_decompress(vals, cols, pk, sc, zp, q, x.shape))


def test_topk_reused_buffers(cf):
    """``out=`` writes into the buffers of an earlier handle / an existing dense tensor, bit-identically."""
    a = _softmax_map(1, 2, 512, seed=3).to(DEV)
    b = _softmax_map(1, 2, 512, seed=4).to(DEV)
    ha = cf.compression_softmax_topk(a, 0.05, 4)
    hb = cf.compression_softmax_topk(b, 0.05, 4)
    want = [t.clone() for t in hb.tensors()]
    dense_b = hb.to_dense().clone()
    h = cf.compression_softmax_topk(b, 0.05, 4, out=ha)
    assert h is ha and all(torch.equal(x, y) for x, y in zip(ha.tensors(), want))
    buf = torch.empty_like(a)
    assert ha.to_dense(out=buf) is buf and torch.equal(buf, dense_b)
    with pytest.raises(ValueError):
        cf.compression_softmax_topk(b, 0.1, 4, out=ha)
    with pytest.raises(ValueError):
        ha.to_dense(out=torch.empty(2, 512, 512, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("q", QS)
@pytest.mark.parametrize("shape", [(1, 2, 512, 512), (1, 1, 13, 128), (1, 1, 5, 2048), (1, 1, 320, 320)])
def test_topk_restore_fused_with_softmax_backward(cf, q, shape):
    """out = softmax_backward(restored map, grad) without the restored map in HBM; the last shape takes the
    two-kernel fallback.  Against the oracle (tolerance: the fp32 row sum has another order) and against the
    two separate device kernels."""
    from hyc_lora_release_b200.operators.softmax_kernels import softmax_backward
    b, h, r, s = shape
    g = torch.Generator().manual_seed(s + q + r)
    a = torch.softmax(3 * torch.randn(b, h, r, s, generator=g), -1).to(torch.bfloat16)
    grad = torch.randn(b, h, r, s, generator=g).to(torch.bfloat16)
    m = cf.compression_softmax_topk(a.to(DEV), 0.05, q)
    out = m.softmax_backward(grad.to(DEV))
    y = m.to_dense()
    ref = oracle.ref_softmax_backward(y.cpu(), grad)
    two = softmax_backward(y, grad.to(DEV))
    scale = ref.float().abs().max()
    assert (out.float().cpu() - ref.float()).abs().max() <= 1e-2 * scale
    assert (out.float() - two.float()).abs().max() <= 1e-2 * scale
    buf = torch.empty_like(y)
    assert m.softmax_backward(grad.to(DEV), out=buf) is buf and torch.equal(buf, out)
    # the optional output scale is a second bf16 operation on the unscaled result
    sc = 1.0 / 128 ** 0.5
    want = (out.float() * torch.tensor(sc, dtype=torch.float32)).to(torch.bfloat16)
    assert torch.equal(m.softmax_backward(grad.to(DEV), scale=sc), want)
    assert torch.equal(softmax_backward(y, grad.to(DEV), scale=sc), (two.float() * torch.tensor(sc, dtype=torch.float32)).to(torch.bfloat16))


def test_topk_config1_full_size_properties(cf):
    """[4,32,512,512] causal softmax map, ratio 0.05, q_bit 4: checked through size-independent
    properties plus the oracle on a slice."""
    a = _softmax_map(4, 32, 512, seed=1).to(DEV)
    m = cf.compression_softmax_topk(a, 0.05, 4)
    k = 25
    assert m.val.shape == (4 * 32 * 512, k)
    cols = m.col.to(torch.int64) & 0xFFFF
    assert (cols[:, 1:] > cols[:, :-1]).all()                      # strictly ascending columns
    a2 = a.reshape(-1, 512)
    assert torch.equal(torch.gather(a2, 1, cols), m.val)            # values are the map's own entries
    kth = torch.topk(a2.float(), k, dim=-1).values[:, -1:]
    assert (m.val.float() >= kth).all()                             # nothing below the k-th largest
    d = m.to_dense()
    assert torch.equal(torch.gather(d.reshape(-1, 512), 1, cols), m.val)   # outliers restored exactly
    assert (d.float() - a.float()).abs().max() <= 0.04
    # deterministic: a second compression and a second restore are bit-identical
    m2 = cf.compression_softmax_topk(a, 0.05, 4)
    assert all(torch.equal(x, y) for x, y in zip(m2.tensors(), m.tensors()))
    assert torch.equal(m.to_dense(), d)
    sl = slice(0, 2048)
    vals, oc, pk, sc, zp = oracle.topk_compress(a2[sl].cpu(), 0.05, 4)
    assert torch.equal(cols[sl].cpu(), oc) and torch.equal(m.q[sl].cpu(), pk) and torch.equal(m.scale[sl].cpu(), sc)
    assert m.nbytes() < 0.45 * a.numel() * 2


@pytest.mark.parametrize("ordered", [True, False])
def test_softmax_prune_with_the_count_left_on_the_device(cf, ordered):
    """``compression_softmax_static`` -> ``PrunedMap`` / ``TiledPrunedMap``: the same entries as the sparse-tensor form, restored without
    a host synchronisation; a capacity that is too small drops the tail and says so.  ordered=False is the one-pass
    kernel: the same SET of (index, value) pairs, dense restore bit-identical."""
    a = _softmax_map(2, 3, 256, seed=9).to(DEV)
    thr = float(cf.get_statistics_softmax(a, 0.05))
    sp = cf.compression_softmax(a, thr)
    nnz = sp.values().numel()
    m = cf.compression_softmax_static(a, thr, ratio=0.05, ordered=ordered)
    assert m.capacity >= nnz and int(m.nnz.item()) == nnz and not m.overflowed()
    if ordered:
        assert torch.equal(m.idx[:nnz], sp.indices().reshape(-1)) and torch.equal(m.val[:nnz], sp.values())
    else:
        mi, mv = m.entries()
        assert torch.equal(mi, sp.indices().reshape(-1)) and torch.equal(mv, sp.values())
        # 4-byte words (+ 8 bytes per 2048 elements) against int64 index + bf16 value, same capacity
        assert m.nbytes() < 0.5 * cf.compression_softmax_static(a, thr, ratio=0.05, ordered=True).nbytes()
    dense = cf.decompression_softmax(sp).reshape(a.shape)
    assert torch.equal(m.to_dense(), dense)
    buf = torch.full(a.shape, 3.0, dtype=torch.bfloat16, device=DEV)
    assert m.to_dense(out=buf) is buf and torch.equal(buf, dense)
    small = cf.compression_softmax_static(a, thr, capacity=nnz // 2, ordered=ordered)
    assert small.overflowed()
    got = small.to_dense().reshape(-1)
    if ordered:
        assert int(small.nnz.item()) == nnz
        part = torch.zeros(a.numel(), dtype=torch.bfloat16, device=DEV)
        part[sp.indices().reshape(-1)[: nnz // 2]] = sp.values()[: nnz // 2]
        assert torch.equal(got, part)
    else:       # nnz reports capacity + the number of dropped entries; what was kept has its own value, nothing else
        dropped = int(small.nnz.item()) - small.capacity
        kept = got != 0
        assert dropped > 0 and int(kept.sum()) == nnz - dropped and int(kept.sum()) <= small.capacity
        assert torch.equal(got[kept], dense.reshape(-1)[kept])


@pytest.mark.parametrize("numel,thr", [(99 * 99, 0.02), (4096 * 3 + 5, -1.0), (8, 0.5), (2048 * 37, 0.0)])
def test_softmax_prune_tiled_ragged_and_negative_threshold(cf, numel, thr):
    """Sizes that end inside a chunk, a negative threshold on a tensor with exact zeros (zeros are no entries), a
    zero threshold: the tiled form holds exactly the entries of the two-phase list, run after run."""
    g = torch.Generator().manual_seed(numel)
    x = torch.randn(numel, generator=g)
    x[torch.rand(numel, generator=g) < 0.3] = 0.0
    x = x.to(torch.bfloat16).to(DEV).reshape(1, 1, 1, numel)
    sp = cf.compression_softmax(x, thr)
    want_idx, want_val = sp.indices().reshape(-1), sp.values()
    for _ in range(2):
        m = cf.compression_softmax_static(x, thr, capacity=numel)
        n = int(m.nnz.item())
        assert n == want_idx.numel()
        mi, mv = m.entries()
        assert torch.equal(mi, want_idx) and torch.equal(mv, want_val)
        assert torch.equal(m.to_dense().reshape(-1), cf.decompression_softmax(sp).reshape(-1))


@pytest.mark.parametrize("q", QS)
@pytest.mark.parametrize("B,h,M,S,mask_kind", [(2, 4, 64, 64, "causal"), (1, 3, 128, 512, "causal"), (2, 2, 64, 1024, "batch"),
                                               (1, 2, 32, 2048, None), (1, 2, 17, 128, "causal"), (1, 1, 8, 4096, None)])
def test_softmax_forward_fused_with_the_topk_save(cf, q, B, h, M, S, mask_kind):
    """scale + mask + softmax + top-k save in one kernel: the probabilities against the two-kernel path (equal up to the
    last bf16 bit where the fp32 row sum rounds differently), and the saved map EXACTLY the stand-alone compression of
    the probabilities the fused kernel returned (so codes, indices and values stay bit-exact against the oracle through
    the stand-alone kernel's tests).  The last two shapes are outside the fused kernel and take the two kernels."""
    import math
    from hyc_lora_release_b200.operators.softmax_kernels import softmax_forward_scale_mask, softmax_forward_topk_save
    g = torch.Generator().manual_seed(S + M + q)
    sc = (torch.randn(B, h, M, S, generator=g) * 8).to(torch.bfloat16).to(DEV)
    mask = None
    if mask_kind == "causal":
        mask = torch.full((M, S), torch.finfo(torch.bfloat16).min).triu(1).to(torch.bfloat16).reshape(1, 1, M, S).to(DEV)
    elif mask_kind == "batch":
        mask = (torch.randn(B, 1, M, S, generator=g) * 3).to(torch.bfloat16).to(DEV)
    scale = 1.0 / math.sqrt(128)
    a_ref = softmax_forward_scale_mask(sc, scale, mask)
    a, m = softmax_forward_topk_save(sc, scale, mask, 0.05, q)
    assert a.shape == sc.shape and a.dtype == torch.bfloat16
    diff = (a.float() - a_ref.float()).abs()
    assert bool((diff <= a_ref.float().abs() * 2 ** -7 + 1e-30).all()) and float((a != a_ref).float().mean()) < 0.05
    m2 = cf.compression_softmax_topk(a, 0.05, q)
    assert all(torch.equal(x, y) for x, y in zip(m.tensors(), m2.tensors()))
    # in place: the scores buffer becomes the probabilities
    buf = sc.clone()
    a3, m3 = softmax_forward_topk_save(buf, scale, mask, 0.05, q, inplace=True)
    assert a3.data_ptr() == buf.data_ptr() and torch.equal(a3, a)
    assert all(torch.equal(x, y) for x, y in zip(m3.tensors(), m.tensors()))
    # and against the oracle on the probabilities it produced
    vals, cols, pk, s_, z_ = oracle.topk_compress(a.cpu(), 0.05, q)
    assert torch.equal(m.val.cpu(), vals) and torch.equal(m.q.cpu(), pk) and torch.equal(m.scale.cpu(), s_)
