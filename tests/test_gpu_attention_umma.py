"""GPU parity of the tcgen05 attention kernel (kv heads with many query columns: grouped queries over several
tokens) against the CPU oracle, 3e-3 max-abs like every attention test.  ``OMNI_QATTN_KERNEL=umma`` takes the
kernel for every shape it covers, so small column counts are exercised too."""
import pytest
import torch

import oracle as orc
from tests.test_gpu_attention import make_cache, to_dev, attn_mod, ATOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def force_umma(monkeypatch):
    monkeypatch.setenv("OMNI_QATTN_KERNEL", "umma")
    yield
    from omnistack_rs_b200 import _lib
    _lib.check_device_status(torch.device("cuda:0"))


@pytest.mark.parametrize("Hq,Hkv,T,S", [(4, 1, 1, 128), (8, 2, 1, 300), (8, 2, 4, 257), (8, 2, 8, 1000), (4, 1, 32, 129),
                                         (8, 1, 16, 640), (2, 1, 65, 200), (4, 2, 3, 1), (4, 2, 2, 100)])
def test_umma_matches_oracle(dev, Hq, Hkv, T, S):
    fa = attn_mod()
    kn, kq, kr, vn, cb, gen = make_cache(2, Hkv, S, seed=Hq * 100 + T + S, user_id=3, per_head=(Hkv > 1))
    q = torch.randn(2, Hq, T, 128, generator=gen).to(torch.bfloat16)
    want = orc.decode_attention(q, kn, kq, kr, vn, cb, 3)
    d = to_dev(dev, q, kn, kq, kr, vn, cb)
    out = fa.omni_attn(*d, user_id=3)
    assert (out.cpu() - want).abs().max() <= ATOL
    noq = fa.omni_attn(*d, user_id=3, with_qjl=False)
    assert (noq.cpu() - orc.decode_attention(q, kn, kq, kr, vn, cb, 3, None, False)).abs().max() <= ATOL
    for ns in (2, 3):
        sp = fa.omni_attn(*d, user_id=3, n_splits=ns)
        assert (sp.cpu() - want).abs().max() <= ATOL, ns


def test_umma_ragged_rotation_and_scale(dev):
    fa = attn_mod()
    kn, kq, kr, vn, cb, gen = make_cache(3, 2, 500, seed=5, user_id=1, outliers=True)
    q_raw = torch.randn(3, 8, 6, 128, generator=gen)
    lens = torch.tensor([500, 1, 333], dtype=torch.int32)
    cache = to_dev(dev, kn, kq, kr, vn, cb)
    got = fa.omni_attn(q_raw.to(dev), *cache, user_id=1, seq_lens=lens.to(dev), rotate_q=True, unrotate_out=True, scale=0.07).cpu()
    for b in range(3):
        n = int(lens[b])
        want = orc.wht128(orc.decode_attention(orc.wht128(q_raw[b:b + 1]), kn[b:b + 1, :, :n], kq[b:b + 1, :, :n],
                                               kr[b:b + 1, :, :n], vn[b:b + 1, :, :n], cb, 1, 0.07))
        assert (got[b:b + 1] - want).abs().max() <= ATOL, b
    # |q| x 200 (reference tests/unit/test_fused_attention.py:256-278 asks for a finite result): with scores of
    # several hundred, fp16 query operands move near-tied keys' weights visibly, so only finiteness is asserted
    # there; |q| x 3000 engages the power-of-two post-scale that keeps the fp16 operands below 2^10
    for mul in (200.0, 3000.0):
        big = fa.omni_attn((q_raw * mul).to(dev), *cache, user_id=1).cpu()
        assert torch.isfinite(big).all()
        assert float(big.abs().max()) <= float(cb.abs().max()) + 5e-3           # a convex combination of centroids
    # the rounding of fp16 query operands enters the scores in proportion to |q|: at three times the benchmark's
    # query norm the budget is three times as wide
    mid = fa.omni_attn((q_raw * 3).to(dev), *cache, user_id=1).cpu()
    assert (mid - orc.decode_attention(q_raw * 3, kn, kq, kr, vn, cb, 1)).abs().max() <= 4 * ATOL


def test_umma_is_the_default_for_many_columns(dev, monkeypatch):
    """Without the override the tcgen05 kernel serves calls with 49 or more query columns per kv head and agrees
    with the warp-level kernel that would otherwise serve them tile by tile."""
    fa = attn_mod()
    kn, kq, kr, vn, cb, gen = make_cache(2, 2, 700, seed=9, user_id=6)
    q = torch.randn(2, 8, 25, 128, generator=gen).to(torch.bfloat16)          # 100 columns per kv head
    d = to_dev(dev, q, kn, kq, kr, vn, cb)
    monkeypatch.delenv("OMNI_QATTN_KERNEL")
    auto = fa.omni_attn(*d, user_id=6)
    monkeypatch.setenv("OMNI_QATTN_KERNEL", "mma")
    tiles = fa.omni_attn(*d, user_id=6)
    want = orc.decode_attention(q, kn, kq, kr, vn, cb, 6)
    assert (auto.cpu() - want).abs().max() <= ATOL and (tiles.cpu() - want).abs().max() <= ATOL


@pytest.mark.parametrize("S", [1, 7, 8, 9, 127, 128, 129, 136, 250, 700])
def test_umma_reads_the_pair_layout_of_v(dev, S):
    """V rows in a resident cache's pair layout: the two threads of a key pair exchange their table lookups, the
    user's last incomplete group of eight stays in the reference layout.  Same bits as the reference-layout call,
    with ragged lengths, splits and several query tokens."""
    fa = attn_mod()
    kn, kq, kr, vn, cb, gen = make_cache(3, 2, S, seed=2000 + S, user_id=4)
    q = torch.randn(3, 8, 5, 128, generator=gen).to(torch.bfloat16)
    lens = torch.tensor([S, max(1, S // 2), max(1, S - 3)], dtype=torch.int64)
    d = to_dev(dev, q, kn, kq, kr, vn, cb)
    paired = d[4].clone()
    fa.pair_v_rows(paired, 0, lens.to(dev))
    for ns in (1, 3):
        ref = fa.omni_attn(*d, user_id=4, seq_lens=lens.to(dev), n_splits=ns)
        got = fa.omni_attn(d[0], d[1], d[2], d[3], paired, d[5], user_id=4, seq_lens=lens.to(dev), n_splits=ns, v_paired=True)
        assert torch.equal(got, ref), (S, ns)
    for b in range(3):
        n = int(lens[b])
        want = orc.decode_attention(q[b:b + 1], kn[b:b + 1, :, :n], kq[b:b + 1, :, :n], kr[b:b + 1, :, :n], vn[b:b + 1, :, :n], cb, 4)
        assert (got[b:b + 1].cpu() - want).abs().max() <= ATOL
