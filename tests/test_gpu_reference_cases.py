"""Cases taken over from the reference's own unit tests, run against the CUDA kernels.

Each test names the reference test it mirrors (tests/unit/*.py of the reference).  Expected values come from the
oracle or from properties the reference asserts; tolerances are the reference's unless the kernel is held tighter.
"""
import math

import pytest
import torch

import oracle as orc
from tests.test_gpu_attention import make_cache, to_dev, attn_mod, ATOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


# ---- tests/unit/test_multi_lora.py ---------------------------------------------------------------------------
def lora_case(seed, B=8, Hq=8, Hkv=2, S=96, hid=64, rank=16, n=8):
    kn, kq, kr, vn, cb, gen = make_cache(B, Hkv, S, seed=seed, user_id=1)
    q = torch.randn(B, Hq, 1, 128, generator=gen).to(torch.bfloat16)
    x = torch.randn(B, 1, hid, generator=gen)
    la = torch.randn(n, rank, hid, generator=gen) * 0.2
    lb = torch.randn(n, Hq * 128, rank, generator=gen) * 0.2
    return (q, kn, kq, kr, vn, cb), x, la, lb


def test_8_users_8_loras_match_individual_runs(dev):
    """test_8_users_8_loras_distinct_slots (:99), test_batched_matches_individual_runs (:401)."""
    fa = attn_mod()
    cache, x, la, lb = lora_case(41)
    d = to_dev(dev, *cache)
    idx = torch.arange(8, dtype=torch.int32)
    kw = dict(user_id=1, x=x.to(dev), lora_a=la.to(dev), lora_b=lb.to(dev), lora_alpha=0.5)
    out = fa.omni_attn(*d, lora_indices=idx.to(dev), **kw)
    q_eff = orc.apply_lora_to_q(cache[0], x, la, lb, idx, 0.5)
    assert (out.cpu() - orc.decode_attention(q_eff, *cache[1:], 1)).abs().max() <= 1e-3
    for b in (0, 3, 7):
        solo = fa.omni_attn(d[0][b:b + 1], d[1][b:b + 1], d[2][b:b + 1], d[3][b:b + 1], d[4][b:b + 1], d[5], user_id=1,
                            x=x[b:b + 1].to(dev), lora_a=la.to(dev), lora_b=lb.to(dev), lora_alpha=0.5,
                            lora_indices=idx[b:b + 1].to(dev))
        assert (solo[0] - out[b]).abs().max() <= 1e-4


def test_swapping_adapters_changes_only_those_users(dev):
    """test_swap_lora_indices_changes_output (:438), test_sentinel_user_unaffected_by_neighbor_lora (:472),
    test_all_sentinel_matches_base (:195)."""
    fa = attn_mod()
    cache, x, la, lb = lora_case(42)
    d = to_dev(dev, *cache)
    kw = dict(user_id=1, x=x.to(dev), lora_a=la.to(dev), lora_b=lb.to(dev), lora_alpha=0.5)
    idx1 = torch.tensor([0, 1, -1, 3, 4, 5, 6, 7], dtype=torch.int32)
    idx2 = torch.tensor([1, 0, -1, 3, 4, 5, 6, 7], dtype=torch.int32)
    o1 = fa.omni_attn(*d, lora_indices=idx1.to(dev), **kw)
    o2 = fa.omni_attn(*d, lora_indices=idx2.to(dev), **kw)
    assert not torch.equal(o1[0], o2[0]) and not torch.equal(o1[1], o2[1])
    assert torch.equal(o1[2:], o2[2:])
    base = fa.omni_attn(*d, user_id=1)
    assert torch.equal(o1[2], base[2])                                     # the sentinel user is the base output, bit for bit
    none = fa.omni_attn(*d, lora_indices=torch.full((8,), -1, dtype=torch.int32, device=dev), **kw)
    assert torch.equal(none, base)


def test_rank_padding_and_zero_adapter(dev):
    """test_rank4_padded_attention_output_matches (:325), test_zero_rank_adapter_is_identity (:361)."""
    fa = attn_mod()
    cache, x, la, lb = lora_case(43, rank=4)
    d = to_dev(dev, *cache)
    idx = (torch.arange(8, dtype=torch.int32) % 4).to(dev)
    la16 = torch.zeros(8, 16, 64); la16[:, :4] = la
    lb16 = torch.zeros(8, 8 * 128, 16); lb16[:, :, :4] = lb
    o4 = fa.omni_attn(*d, user_id=1, x=x.to(dev), lora_a=la.to(dev), lora_b=lb.to(dev), lora_indices=idx, lora_alpha=1.0)
    o16 = fa.omni_attn(*d, user_id=1, x=x.to(dev), lora_a=la16.to(dev), lora_b=lb16.to(dev), lora_indices=idx, lora_alpha=1.0)
    assert (o4 - o16).abs().max() <= 1e-5
    zero = fa.omni_attn(*d, user_id=1, x=x.to(dev), lora_a=la.to(dev), lora_b=torch.zeros_like(lb).to(dev),
                        lora_indices=idx, lora_alpha=1.0)
    assert torch.equal(zero, fa.omni_attn(*d, user_id=1))                   # B = 0: q + 0 is q


# ---- tests/unit/test_fused_attention.py ------------------------------------------------------------------------
def test_inputs_untouched_default_scale_and_dtype(dev):
    """test_input_tensors_not_modified (:437), test_default_scale (:425), test_output_dtype_float32 (:416),
    test_output_shape (:407)."""
    fa = attn_mod()
    kn, kq, kr, vn, cb, gen = make_cache(2, 2, 64, seed=51)
    q = torch.randn(2, 4, 4, 128, generator=gen)
    d = to_dev(dev, q, kn, kq, kr, vn, cb)
    before = [x.clone() for x in d]
    out = fa.omni_attn(*d)
    assert out.shape == (2, 4, 4, 128) and out.dtype == torch.float32
    assert all(torch.equal(a, b) for a, b in zip(before, d))
    assert torch.equal(out, fa.omni_attn(*d, scale=1.0 / math.sqrt(128)))


def test_int4_only_matches_dense_attention_on_dequantised_cache(dev):
    """test_int4_only_matches_dequantize_heads (:289), test_qjl_changes_output (:387),
    test_qkt_scale_applied (:206)."""
    from omnistack_rs_b200.attention import reference_attn
    from omnistack_rs_b200.kernels.quantize import dequantize_heads
    fa = attn_mod()
    kn, kq, kr, vn, cb, gen = make_cache(1, 2, 32, seed=52)
    q = torch.randn(1, 4, 4, 128, generator=gen) * 0.3
    d = to_dev(dev, q, kn, kq, kr, vn, cb)
    k_hat = dequantize_heads(d[1], d[2], d[3], d[5], 0, with_qjl=False)
    v_hat = dequantize_heads(d[4], d[2], d[3], d[5], 0, with_qjl=False)
    plain = fa.omni_attn(*d, with_qjl=False)
    assert (plain - reference_attn(d[0], k_hat, v_hat)).abs().max() <= 1e-3
    assert not torch.allclose(plain, fa.omni_attn(*d, with_qjl=True), atol=1e-4)
    assert not torch.allclose(fa.omni_attn(*d, scale=0.01), fa.omni_attn(*d, scale=0.5), atol=1e-3)


def test_per_group_codebooks_are_applied_per_head(dev):
    """test_per_group_codebooks_applied_correctly (:324): swapping the heads' codebooks changes the result, and
    each head equals the single-head call with its own codebook."""
    fa = attn_mod()
    kn, kq, kr, vn, cb, gen = make_cache(1, 4, 32, seed=53)
    cb = torch.stack([cb[0] * s for s in (0.5, 1.0, 2.0, 4.0)])
    q = torch.randn(1, 8, 4, 128, generator=gen) * 0.3
    want = orc.decode_attention(q, kn, kq, kr, vn, cb, 0)
    out = fa.omni_attn(*to_dev(dev, q, kn, kq, kr, vn, cb)).cpu()
    assert (out - want).abs().max() <= ATOL
    swapped = fa.omni_attn(*to_dev(dev, q, kn, kq, kr, vn, cb.flip(0))).cpu()
    assert (swapped - out).abs().max() > 1e-2


# ---- tests/unit/test_hadamard.py ---------------------------------------------------------------------------------
def test_rotation_preserves_dot_products_and_inputs(dev):
    """test_elementwise_dot_under_1e4 (:58), test_qkt_attention_matrix (:77), test_rotate_queries_does_not_modify_input
    (:211), shape / dtype preservation (:195-209)."""
    from omnistack_rs_b200.kernels.hadamard import rotate_queries, rotate_kv_cache
    gen = torch.Generator().manual_seed(61)
    q = torch.randn(4, 8, 16, 128, generator=gen).to(dev)
    k = torch.randn(4, 8, 16, 128, generator=gen).to(dev)
    q0 = q.clone()
    qr = rotate_queries(q)
    kr, vr = rotate_kv_cache(k, k * 2)
    assert torch.equal(q, q0) and qr.shape == q.shape and qr.dtype == q.dtype and vr.shape == k.shape
    assert ((qr * kr).sum(-1) - (q * k).sum(-1)).abs().max() <= 1e-4
    assert (qr @ kr.transpose(-1, -2) - q @ k.transpose(-1, -2)).abs().max() <= 1e-3
    h4 = torch.zeros(1, 128, device=dev); h4[0, :4] = torch.tensor([1.0, 2.0, 3.0, 4.0])
    y = rotate_queries(h4)[0] * math.sqrt(128.0)                            # test_known_small_case (:166): H4 block of H128
    assert torch.allclose(y[:4], torch.tensor([10.0, -2.0, -4.0, 0.0], device=dev), atol=1e-5)


# ---- tests/unit/test_attention.py ----------------------------------------------------------------------------------
def test_dense_anchor_tiles_masks_and_dtypes(dev):
    """test_tile_size_independence (:62), test_causal_mask_blocks_future (:254), test_output_dtype_matches_input (:188),
    test_no_overflow_with_large_scores (:126), test_gqa_mha_equivalence (:236)."""
    from omnistack_rs_b200.attention import reference_attn, repeat_kv
    gen = torch.Generator().manual_seed(71)
    q = torch.randn(2, 8, 12, 128, generator=gen).to(dev)
    k = torch.randn(2, 2, 100, 128, generator=gen).to(dev)
    v = torch.randn(2, 2, 100, 128, generator=gen).to(dev)
    base = reference_attn(q, k, v, tile_size=128)
    for tile in (1, 7, 32, 100, 512):
        assert (reference_attn(q, k, v, tile_size=tile) - base).abs().max() <= 1e-5
    assert (reference_attn(q, repeat_kv(k, 4), repeat_kv(v, 4)) - base).abs().max() <= 1e-6
    assert reference_attn(q.half(), k.half(), v.half()).dtype == torch.float16
    assert torch.isfinite(reference_attn(q * 1e3, k, v)).all()
    qs, ks, vs = q[:, :, :12], k[:, :, :12], v[:, :, :12]
    causal = torch.triu(torch.full((12, 12), float("-inf"), device=dev), diagonal=1)[None, None]
    out = reference_attn(qs, ks, vs, mask=causal)
    v2 = vs.clone(); v2[:, :, 6:] += 100.0                                    # changing future values leaves rows 0..5 alone
    assert torch.allclose(reference_attn(qs, ks, v2, mask=causal)[:, :, :6], out[:, :, :6], atol=1e-5)
