"""GPU parity of the codec kernels (rotation, quantize, dequantize, append) through the
C ABI, against the CPU oracle and the reference-generated golden files.  Packed codes must
be bit-exact; sign bits must be bit-exact except where fp32 arithmetic cannot decide the
sign (oracle.sign_ambiguity); norms within 1e-6 relative; dequantised values within 1e-5."""
import pytest
import torch

import oracle as orc
from tests.helpers import load_golden, t, bf16, sha, config0_inputs, sign_mismatch_report

pytestmark = pytest.mark.gpu

NORM_RTOL = 1e-6
DEQ_ATOL = 1e-5


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(autouse=True, params=["tc", "warp", "scan"])
def quant_kernel_choice(request, monkeypatch):
    """Every case runs once per quantize kernel: the row-per-thread kernel with tcgen05 projections
    (OMNI_QUANT_KERNEL=tc), the 8-rows-per-warp kernel with mma.sync projections (=warp, the default) and the
    one-row-per-warp scan kernel (=scan)."""
    monkeypatch.setenv("OMNI_QUANT_KERNEL", request.param)
    return request.param


def k():
    from omnistack_rs_b200.kernels import quantize, hadamard
    return quantize, hadamard


def check_packed(got, want, resid=None, user_id=0):
    gn, gq, gr = [x.cpu() for x in got]
    wn, wq, wr = want
    assert gn.dtype == torch.uint8 and gq.dtype == torch.uint8 and gr.dtype == torch.float32
    assert torch.equal(gn, wn), f"{int((gn != wn).sum())} nibble bytes differ"
    if not torch.equal(gq, wq):
        assert resid is not None, "sign bits differ"
        n_diff, n_bad = sign_mismatch_report(gq, wq, orc.sign_ambiguity(resid, user_id))
        assert n_bad == 0, f"{n_bad} of {n_diff} differing sign bits are not fp32-ambiguous"
    assert torch.allclose(gr, wr, rtol=NORM_RTOL, atol=1e-30)


@pytest.mark.parametrize("rotate_kernel", ["rows8", "warp"])
def test_rotation_bit_exact(dev, rotate_kernel, monkeypatch):
    """Both stand-alone rotation kernels (8 rows per warp, the default; one row per warp) against the fixtures."""
    monkeypatch.setenv("OMNI_ROTATE_KERNEL", rotate_kernel)
    _, had = k()
    g = load_golden("rotation.npz")
    x = t(g["x"])
    assert torch.equal(had.rotate_queries(x.to(dev)).cpu(), t(g["y"]))
    assert torch.equal(had.rotate_queries(x.to(torch.bfloat16).to(dev)).cpu().view(torch.int16), t(g["y_bf16"]))
    assert torch.equal(had.rotate_queries(x.to(torch.float16).to(dev)).cpu().view(torch.int16), t(g["y_fp16"]))
    xk = torch.randn(2, 3, 5, 128)
    a, b = had.rotate_kv_cache(xk.to(dev), (2 * xk).to(dev))
    assert torch.equal(a.cpu(), orc.wht128(xk)) and torch.equal(b.cpu(), orc.wht128(2 * xk))
    for n in (1, 7, 8, 9, 1000):                                   # row counts around the 8-row groups, all dtypes
        for dt in (torch.float32, torch.bfloat16, torch.float16):
            xr = (torch.randn(n, 128, generator=torch.Generator().manual_seed(n)) * 3).to(dt)
            got = had.rotate_queries(xr.to(dev)).cpu()
            assert got.dtype == dt and torch.equal(got, orc.wht128(xr)), (n, dt)
    with pytest.raises(ValueError, match="head_dim"):
        had.rotate_queries(torch.zeros(2, 64, device=dev))


def test_rotation_properties_large(dev):
    _, had = k()
    x = torch.randn(1 << 16, 128, device=dev)
    y = had.rotate_queries(x)
    assert torch.allclose(had.rotate_queries(y), x, atol=2e-5)                      # involution
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)                # isometry
    z = torch.randn_like(x)
    assert torch.allclose(had.rotate_queries(x + z), y + had.rotate_queries(z), atol=2e-5)   # linearity
    assert x.data_ptr() != y.data_ptr()


def test_config0_codec(dev):
    quant, _ = k()
    g = load_golden("config0_codec.npz")
    K, V, _ = config0_inputs()
    if sha(K) != str(g["sha_K"]):
        pytest.skip("torch.randn stream differs from the fixtures'")
    cbs = t(g["codebooks"])
    for raw, key in ((K, "k"), (V, "v")):
        rot = orc.wht128(raw)
        wn, wq, wr, resid = orc.quantize_heads(rot, cbs, 0, return_residual=True)
        assert sha(wn) == str(g[f"sha_{key}_nib"]) and sha(wq) == str(g[f"sha_{key}_qjl"])
        before = rot.clone()
        x_dev = rot.to(dev)
        check_packed(quant.quantize_heads(x_dev, cbs.to(dev), 0), (wn, wq, wr), resid)
        assert torch.equal(x_dev.cpu(), before)                                   # input untouched
        check_packed(quant.quantize_heads(raw.to(dev), cbs.to(dev), 0, rotate=True), (wn, wq, wr), resid)
    # golden dequantised tensors of user 0
    kn, kq, kr = quant.quantize_heads(orc.wht128(K[:1]).to(dev), cbs.to(dev), 0)
    k_hat = quant.dequantize_heads(kn, kq, kr, cbs.to(dev), 0, True).cpu()[0]
    assert (k_hat - t(g["k_hat_u0"])).abs().max() <= DEQ_ATOL
    k_int4 = quant.dequantize_heads(kn, kq, kr, cbs.to(dev), 0, False).cpu()[0]
    assert torch.equal(k_int4, orc.dequantize_heads(kn.cpu(), kq.cpu(), kr.cpu(), cbs, 0, False)[0])


def test_bf16_heavy_tail_users(dev):
    quant, _ = k()
    g = load_golden("codec_bf16_users.npz")
    x, cb = bf16(g["x_bf16"]), t(g["codebook"])
    for b, uid in enumerate(g["user_ids"].tolist()):
        got = quant.quantize_heads(x[b:b + 1].to(dev), cb.to(dev), uid, rotate=True)
        assert torch.equal(got[0].cpu()[0], t(g["nib"])[b])
        assert torch.equal(got[1].cpu()[0], t(g["qjl"])[b])
        assert torch.allclose(got[2].cpu()[0], t(g["norms"])[b], rtol=NORM_RTOL)
    # one launch with a per-user id tensor gives the same rows
    ids = torch.tensor(g["user_ids"], dtype=torch.int32, device=dev)
    n_, q_, r_ = quant.quantize_heads(x.to(dev), cb.to(dev), ids, rotate=True)
    assert torch.equal(n_.cpu(), t(g["nib"])) and torch.equal(q_.cpu(), t(g["qjl"]))


def test_rows_variant(dev):
    quant, _ = k()
    g = load_golden("rows.npz")
    n_, q_, r_ = quant.quantize_rows(t(g["x"]).to(dev), t(g["codebook"]).to(dev), base_head_idx=3, user_id=77)
    assert n_.shape == (3, 7, 64) and q_.shape == (3, 7, 8) and r_.shape == (3, 7)
    assert torch.equal(n_.cpu(), t(g["nib"])) and torch.equal(q_.cpu(), t(g["qjl"]))
    assert torch.allclose(r_.cpu(), t(g["norms"]), rtol=NORM_RTOL)
    xh = quant.dequantize_rows(n_, q_, r_, t(g["codebook"]).to(dev), 3, 77, True)
    assert (xh.cpu() - t(g["x_hat"])).abs().max() <= DEQ_ATOL


def test_rows_variant_beyond_1024_keys(dev):
    """Row keys past 1,023 select MT19937 seeds above the 1,024 resident ones (the reference seeds one stream per
    row for any row count, kernels/quantize.py:486-492, :524-535)."""
    quant, _ = k()
    g = load_golden("rows_beyond_1024.npz")
    base, uid = int(g["base_head_idx"]), int(g["user_id"])
    cb = t(g["codebook"]).to(dev)
    n_, q_, r_ = quant.quantize_rows(t(g["x"]).to(dev), cb, base_head_idx=base, user_id=uid)
    assert torch.equal(n_.cpu(), t(g["nib"])) and torch.equal(q_.cpu(), t(g["qjl"]))
    assert torch.allclose(r_.cpu(), t(g["norms"]), rtol=NORM_RTOL)
    xh = quant.dequantize_rows(n_, q_, r_, cb, base, uid, True)
    assert (xh.cpu() - t(g["x_hat"])).abs().max() <= DEQ_ATOL
    # an ordinary call of the reference's own tests: (2, 8, 100, 128) = 1,600 rows, keys 0..1599, two seed blocks
    gen = torch.Generator().manual_seed(41)
    x = orc.wht128(torch.randn(2, 8, 100, 128, generator=gen))
    want = orc.quantize_rows(x, cb.cpu(), 0, 5)
    got = quant.quantize_rows(x.to(dev), cb, 0, 5)
    assert got[0].shape == (2, 8, 100, 64) and got[1].shape == (2, 8, 100, 8) and got[2].shape == (2, 8, 100)
    assert torch.equal(got[0].cpu(), want[0]) and torch.equal(got[1].cpu(), want[1])
    assert torch.allclose(got[2].cpu(), want[2], rtol=NORM_RTOL)
    back = quant.dequantize_rows(*got, cb, 0, 5, True)
    assert (back.cpu() - orc.dequantize_rows(*want, cb.cpu(), 0, 5, True)).abs().max() <= DEQ_ATOL
    # a key range that starts in a third block and is revisited: the extended tables are rebuilt and reused
    far = quant.quantize_rows(x[0, 0, :9].to(dev), cb, base_head_idx=5000, user_id=1029)
    want_far = orc.quantize_rows(x[0, 0, :9], cb.cpu(), 5000, 1029)
    assert torch.equal(far[1].cpu(), want_far[1])
    again = quant.quantize_rows(x.to(dev), cb, 0, 5)
    assert torch.equal(again[1].cpu(), want[1])


@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 2, 7), (2, 5, 33)])
def test_shapes_and_codebook_variants(dev, shape):
    quant, _ = k()
    B, H, T = shape
    gen = torch.Generator().manual_seed(B * 100 + T)
    x = orc.wht128(torch.randn(B, H, T, 128, generator=gen) * 1.5)
    per_head = torch.sort(torch.randn(H, 16, generator=gen), dim=1).values
    shared = torch.linspace(-3, 3, 16)
    for cb in (per_head, shared):
        want = orc.quantize_heads(x, cb, 11, return_residual=True)
        check_packed(quant.quantize_heads(x.to(dev), cb.to(dev), 11), want[:3], want[3], 11)
        wn, wq, wr = want[:3]
        got = quant.dequantize_heads(wn.to(dev), wq.to(dev), wr.to(dev), cb.to(dev), 11, True).cpu()
        assert (got - orc.dequantize_heads(wn, wq, wr, cb, 11, True)).abs().max() <= DEQ_ATOL
    with pytest.raises(AssertionError):
        quant.quantize_heads(x.to(dev), torch.zeros(H + 1, 16, device=dev))


def test_edge_values(dev):
    quant, _ = k()
    cb = torch.linspace(-2, 2, 16)
    x = torch.zeros(1, 1, 6, 128)
    x[0, 0, 1] = cb[5]                       # exactly a centroid: zero residual -> all signs 1
    x[0, 0, 2] = 1e10                        # |x| so large that every distance ties -> code 0
    x[0, 0, 3] = -1e10
    x[0, 0, 4] = (cb[3] + cb[4]) / 2         # midpoint tie -> lower index
    x[0, 0, 5, ::2] = 100.0
    want = orc.quantize_heads(x, cb, 0, return_residual=True)
    got = quant.quantize_heads(x.to(dev), cb.to(dev), 0)
    check_packed(got, want[:3], want[3])
    assert (got[1].cpu()[0, 0, 1] == 0xFF).all() and float(got[2][0, 0, 1]) == 0.0
    # unsorted codebook and duplicated centroids still follow first-index argmin
    for cb2 in (cb.flip(0), torch.tensor([0.0] * 4 + [1.0] * 4 + [-1.0] * 8)):
        y = orc.wht128(torch.randn(1, 1, 9, 128, generator=torch.Generator().manual_seed(2)))
        want = orc.quantize_heads(y, cb2, 3, return_residual=True)
        check_packed(quant.quantize_heads(y.to(dev), cb2.to(dev), 3), want[:3], want[3], 3)


@pytest.mark.parametrize("kind", ["tight_pair", "clustered", "tiny_gaps", "wide_tail"])
def test_codebooks_the_grid_cannot_resolve(dev, kind):
    """Codebooks whose thresholds crowd into one cell of the fast kernel's grid (or whose gaps are far below the
    range) must still give the reference's codes: the kernel falls back to the exact thresholds or the scan."""
    quant, _ = k()
    gen = torch.Generator().manual_seed(21)
    if kind == "tight_pair":
        cb = torch.linspace(-2.5, 2.5, 16)
        cb[8] = cb[7] + 1e-4
    elif kind == "clustered":
        cb = torch.cat([torch.linspace(-3, -2.9, 6), torch.linspace(-0.05, 0.05, 5), torch.linspace(2.0, 4.0, 5)])
    elif kind == "tiny_gaps":
        cb = torch.arange(16, dtype=torch.float32) * 3e-7 + 1.0
    else:
        cb = torch.cat([torch.linspace(-1, 1, 15), torch.tensor([1e6])])
    y = orc.wht128(torch.randn(2, 1, 40, 128, generator=gen))
    y[0, 0, 0, :16] = cb                                        # exact centroids
    y[0, 0, 1, :15] = (cb[1:] + cb[:-1]) / 2                    # fp32 midpoints
    y[1, 0, 2, :16] = torch.nextafter(cb, torch.full_like(cb, 1e9))
    want = orc.quantize_heads(y, cb, 9, return_residual=True)
    got = quant.quantize_heads(y.to(dev), cb.to(dev), 9)
    check_packed(got, want[:3], want[3], 9)


def test_empty_and_strided_inputs(dev):
    quant, _ = k()
    cb = torch.linspace(-3, 3, 16).to(dev)
    n_, q_, r_ = quant.quantize_heads(torch.zeros(0, 2, 4, 128, device=dev), cb)
    assert n_.shape == (0, 2, 4, 64) and q_.shape == (0, 2, 4, 8) and r_.shape == (0, 2, 4)
    n_, _, _ = quant.quantize_heads(torch.zeros(2, 2, 0, 128, device=dev), cb)
    assert n_.shape == (2, 2, 0, 64)
    base = torch.randn(4, 6, 3, 128, generator=torch.Generator().manual_seed(5))
    view = base[1:3, ::2]                                   # non-contiguous batch/head strides
    want = orc.quantize_heads(view.contiguous(), cb.cpu(), 1, return_residual=True)
    check_packed(quant.quantize_heads(base.to(dev)[1:3, ::2], cb, 1), want[:3], want[3], 1)
    tview = base.transpose(1, 2)                            # (4,3,6,128): token/head swapped
    want = orc.quantize_heads(tview.contiguous(), cb.cpu(), 1, return_residual=True)
    check_packed(quant.quantize_heads(base.to(dev).transpose(1, 2), cb, 1), want[:3], want[3], 1)


def test_append_at_offsets(dev):
    quant, _ = k()
    from omnistack_rs_b200.serving import QuantizedKVCache
    gen = torch.Generator().manual_seed(9)
    B, H, S_max = 3, 2, 40
    cb = torch.sort(torch.randn(H, 16, generator=gen), dim=1).values
    ids = torch.tensor([4, 1030, 77], dtype=torch.int32)
    cache = QuantizedKVCache(B, H, S_max, cb, dev, user_ids=ids)
    chunks = [torch.randn(B, H, n, 128, generator=gen).to(torch.bfloat16) for n in (7, 1, 16)]
    vchunks = [torch.randn(B, H, n, 128, generator=gen).to(torch.bfloat16) for n in (7, 1, 16)]
    for kc, vc in zip(chunks, vchunks):
        cache.append(kc.to(dev), vc.to(dev))
    assert cache.lens.tolist() == [24, 24, 24]
    k_all, v_all = torch.cat(chunks, dim=2), torch.cat(vchunks, dim=2)
    for b in range(B):
        wn, wq, wr = orc.rotate_quantize(k_all[b:b + 1], cb, int(ids[b]))
        assert torch.equal(cache.k_nib[b, :, :24].cpu(), wn[0]) and torch.equal(cache.k_qjl[b, :, :24].cpu(), wq[0])
        assert torch.allclose(cache.k_norms[b, :, :24].cpu(), wr[0], rtol=NORM_RTOL)
        vn, _, _ = orc.rotate_quantize(v_all[b:b + 1], cb, int(ids[b]))
        assert torch.equal(cache.v_nib[b, :, :24].cpu(), vn[0])
    assert int(cache.k_nib[:, :, 24:].max()) == 0          # rows past the length stay untouched
    with pytest.raises(ValueError):
        cache.append(torch.zeros(B, H, 17, 128, device=dev), torch.zeros(B, H, 17, 128, device=dev))


def test_cache_without_v_residual_allocates_nothing_per_append(dev):
    """A cache built with ``store_v_residual=False`` keeps no sign bits or norms for V (attention never reads
    them): the V rows are produced without the projections, bit-equal to the full codec's nibbles, and an append
    neither allocates scratch of the cache's extent nor moves the allocator's high-water mark."""
    from omnistack_rs_b200.serving import QuantizedKVCache
    gen = torch.Generator().manual_seed(10)
    B, H, S_max = 4, 3, 96
    cb = torch.sort(torch.randn(H, 16, generator=gen), dim=1).values
    ids = torch.tensor([1, 2, 3, 2000], dtype=torch.int32)
    cache = QuantizedKVCache(B, H, S_max, cb, dev, user_ids=ids, store_v_residual=False)
    assert cache.v_qjl is None and cache.bytes_per_key() == 140
    chunks = [(torch.randn(B, H, n, 128, generator=gen).to(torch.bfloat16).to(dev),
               torch.randn(B, H, n, 128, generator=gen).to(torch.bfloat16).to(dev)) for n in (5, 8, 1, 30)]
    cache.append(*chunks[0])
    torch.cuda.synchronize(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    before = torch.cuda.memory_allocated(dev)
    for kc, vc in chunks[1:]:
        cache.append(kc, vc)
    torch.cuda.synchronize(dev)
    assert torch.cuda.memory_allocated(dev) == before
    assert torch.cuda.max_memory_allocated(dev) - before < 64 * 1024          # a few small index tensors at most
    v_all = torch.cat([c[1] for c in chunks], dim=2).cpu()
    k_all = torch.cat([c[0] for c in chunks], dim=2).cpu()
    for b in range(B):
        vn, _, _ = orc.rotate_quantize(v_all[b:b + 1], cb, int(ids[b]))
        assert torch.equal(cache.v_nib[b, :, :44].cpu(), vn[0])
        kn, kq, _ = orc.rotate_quantize(k_all[b:b + 1], cb, int(ids[b]))
        assert torch.equal(cache.k_nib[b, :, :44].cpu(), kn[0]) and torch.equal(cache.k_qjl[b, :, :44].cpu(), kq[0])
    q = torch.randn(B, 2 * H, 1, 128, generator=gen).to(torch.bfloat16)
    out = cache.attend(q.to(dev)).cpu()
    for b in range(B):
        want = orc.decode_attention(q[b:b + 1], cache.k_nib[b:b + 1, :, :44].cpu(), cache.k_qjl[b:b + 1, :, :44].cpu(),
                                    cache.k_norms[b:b + 1, :, :44].cpu(), cache.v_nib[b:b + 1, :, :44].cpu(), cb, int(ids[b]))
        assert (out[b:b + 1] - want).abs().max() <= 3e-3


def test_quantize_append_config3_slice_and_roundtrip(dev):
    """64 users x 256 tokens x 8 heads, bf16, N(0,1) with 1% of values x10 (benchmark config 3
    shape, user subset): bit-exact against the oracle, and the encode -> decode round trip
    beats INT4-only reconstruction on the full slice."""
    quant, had = k()
    gen = torch.Generator().manual_seed(33)
    U, H, T = 64, 8, 256
    x = torch.randn(U, H, T, 128, generator=gen)
    x = torch.where(torch.rand(U, H, T, 128, generator=gen) < 0.01, x * 10, x).to(torch.bfloat16)
    cb = orc.lloyd_max_fit(orc.wht128(x[:4]).float().reshape(-1)[:200000], max_iters=30)
    ids = torch.arange(U, dtype=torch.int32) * 37
    n_, q_, r_ = quant.quantize_heads(x.to(dev), cb.to(dev), ids.to(dev), rotate=True)
    for b in range(0, U, 9):
        want = orc.quantize_heads(orc.wht128(x[b:b + 1]), cb, int(ids[b]), return_residual=True)
        check_packed((n_[b:b + 1], q_[b:b + 1], r_[b:b + 1]), want[:3], want[3], int(ids[b]))
    rot = had.rotate_queries(x.to(dev)).float()
    full = quant.dequantize_heads(n_, q_, r_, cb.to(dev), ids.to(dev), True)
    int4 = quant.dequantize_heads(n_, q_, r_, cb.to(dev), ids.to(dev), False)
    mse_full, mse_int4 = float(((full - rot) ** 2).mean()), float(((int4 - rot) ** 2).mean())
    assert mse_full < 0.95 * mse_int4, (mse_full, mse_int4)
    assert torch.allclose(r_, (rot - int4).norm(dim=-1), rtol=1e-5)           # norm is the residual norm
