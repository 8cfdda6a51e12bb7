"""Pins the CPU oracle against (a) the known-answer vectors the reference's own
unit tests hold and (b) fixtures produced by running the reference itself
(tests/golden/make_golden.py)."""
import math

import numpy as np
import pytest
import torch

import oracle as orc
from tests.helpers import load_golden, t, bf16, sha, config0_inputs


# ---- known answers restated from the reference's unit tests ------------------

def test_nibble_pack_known_values():
    # tests/unit/test_quant.py:167-182 -- codes (5,3) -> 0x35 = 53; all 15 -> 0xFF
    codes = torch.zeros(128, dtype=torch.uint8)
    codes[0], codes[1] = 5, 3
    assert int(orc.pack_nibbles(codes)[0]) == 53
    assert (orc.pack_nibbles(torch.full((128,), 15, dtype=torch.uint8)) == 0xFF).all()


def test_nibble_unpack_known_first_word():
    # tests/unit/test_quant.py:422-441 -- bytes 53 24 71 A6 -> 3 5 4 2 1 7 6 10
    packed = torch.zeros(64, dtype=torch.uint8)
    packed[:4] = torch.tensor([0x53, 0x24, 0x71, 0xA6], dtype=torch.uint8)
    assert orc.unpack_nibbles(packed)[:8].tolist() == [3, 5, 4, 2, 1, 7, 6, 10]


def test_nibble_roundtrip():
    codes = torch.randint(0, 16, (9, 128), dtype=torch.uint8)
    assert torch.equal(orc.unpack_nibbles(orc.pack_nibbles(codes)), codes)


def test_seed_formula_and_aliasing():
    # tests/unit/test_quant.py:604-632
    assert orc.qjl_seed(0, 3) == 3
    assert orc.qjl_seed(5, 3) == (5 ^ 3)
    assert orc.qjl_seed(1024, 7) == orc.qjl_seed(0, 7)
    assert orc.qjl_seed(-1, 0) == 1023          # Python modulo is non-negative


def test_wht_h4_structure_and_involution():
    # tests/unit/test_hadamard.py:132-188 -- self-inverse, norm preserving, e0 -> constant
    x = torch.randn(16, 128)
    y = orc.wht128(x)
    assert torch.allclose(orc.wht128(y), x, atol=1e-5)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    e0 = torch.zeros(128); e0[0] = 1.0
    assert torch.allclose(orc.wht128(e0), torch.full((128,), 1 / math.sqrt(128)))
    e1 = torch.zeros(128); e1[1] = 1.0                      # row 1 of H: + - + - ...
    assert torch.equal(torch.sign(orc.wht128(e1)), torch.tensor([1.0, -1.0] * 64))
    with pytest.raises(ValueError, match="head_dim"):
        orc.wht128(torch.zeros(2, 64))


def test_sign_bit_order():
    s = torch.zeros(64, dtype=torch.bool)
    s[0] = s[9] = s[63] = True
    p = orc.pack_sign_bits(s)
    assert p.tolist() == [1, 2, 0, 0, 0, 0, 0, 128]
    assert torch.equal(orc.unpack_sign_bits(p).bool(), s)


# ---- fixtures produced by the reference ---------------------------------------

def test_mt19937_matches_reference_table():
    g = load_golden("rademacher.npz")
    for seed, key in ((0, "seed0"), (5, "seed5"), (1023, "seed1023")):
        assert np.array_equal(orc.rademacher_bits(seed), g[key])
    allbits = np.stack([orc.rademacher_bits(s) for s in range(0, 1024)])
    assert sha(torch.from_numpy(allbits)) == str(g["sha_all"])


def test_mt19937_matches_torch_generator():
    for seed in (1, 77, 1000):
        gen = torch.Generator().manual_seed(seed)
        ref = torch.randint(0, 2, (64, 128), generator=gen, dtype=torch.float32).numpy().astype(np.uint8)
        assert np.array_equal(orc.rademacher_bits(seed), ref)


def test_rotation_golden():
    g = load_golden("rotation.npz")
    x = t(g["x"])
    assert torch.equal(orc.wht128(x), t(g["y"]))
    assert torch.equal(orc.wht128(x.to(torch.bfloat16)).view(torch.int16), t(g["y_bf16"]))
    assert torch.equal(orc.wht128(x.to(torch.float16)).view(torch.int16), t(g["y_fp16"]))


@pytest.fixture(scope="module")
def config0_oracle():
    g = load_golden("config0_codec.npz")
    K, V, q = config0_inputs()
    if sha(K) != str(g["sha_K"]) or sha(V) != str(g["sha_V"]):
        pytest.skip("torch.randn stream differs from the one the fixtures were made with")
    cbs = t(g["codebooks"])
    Kr, Vr = orc.wht128(K), orc.wht128(V)
    return g, cbs, Kr, Vr, orc.quantize_heads(Kr, cbs, 0), orc.quantize_heads(Vr, cbs, 0), q


def test_config0_codec_bit_exact(config0_oracle):
    g, cbs, Kr, Vr, (kn, kq, kr), (vn, vq, vr), _ = config0_oracle
    assert sha(Kr) == str(g["sha_Krot"]) and sha(Vr) == str(g["sha_Vrot"])
    assert sha(kn) == str(g["sha_k_nib"]) and sha(vn) == str(g["sha_v_nib"])
    assert sha(kq) == str(g["sha_k_qjl"]) and sha(vq) == str(g["sha_v_qjl"])
    assert torch.equal(kn[:4], t(g["k_nib_u4"])) and torch.equal(kq[:4], t(g["k_qjl_u4"]))
    assert torch.allclose(kr, t(g["k_norms"]), rtol=5e-7, atol=0)
    assert torch.allclose(vr, t(g["v_norms"]), rtol=5e-7, atol=0)


def test_config0_dequant(config0_oracle):
    g, cbs, _, _, (kn, kq, kr), (vn, vq, vr), _ = config0_oracle
    k_hat = orc.dequantize_heads(kn[:1], kq[:1], kr[:1], cbs, 0, True)[0]
    v_hat = orc.dequantize_heads(vn[:1], vq[:1], vr[:1], cbs, 0, False)[0]
    assert (k_hat - t(g["k_hat_u0"])).abs().max() <= 1e-6
    assert torch.equal(v_hat, t(g["v_hat_u0"]))
    # INT4+QJL reconstructs better than INT4 alone (tests/unit/test_quant.py:270-341)
    k_rot = t(g["k_rot_u0"])
    k_int4 = orc.dequantize_heads(kn[:1], kq[:1], kr[:1], cbs, 0, False)[0]
    assert ((k_hat - k_rot) ** 2).mean() < 0.95 * ((k_int4 - k_rot) ** 2).mean()


def test_config1_attention(config0_oracle):
    g, cbs, _, _, (kn, kq, kr), (vn, _, _), q = config0_oracle
    a = load_golden("config1_attention.npz")
    assert torch.equal(q.view(torch.int16), t(a["q_bf16"]))
    out = orc.decode_attention(q, kn, kq, kr, vn, cbs, 0, None, True)
    assert out.dtype == torch.float32
    assert (out - t(a["out"])).abs().max() <= 2e-6
    out2 = orc.decode_attention(q, kn, kq, kr, vn, cbs, 0, None, False)
    assert (out2 - t(a["out_noqjl"])).abs().max() <= 2e-6


def test_codec_bf16_users_golden():
    g = load_golden("codec_bf16_users.npz")
    x = bf16(g["x_bf16"])
    xr = orc.wht128(x)
    assert torch.equal(xr.view(torch.int16), t(g["x_rot_bf16"]))
    cb = t(g["codebook"])
    for b, uid in enumerate(g["user_ids"].tolist()):
        n_, q_, r_ = orc.quantize_heads(xr[b:b + 1], cb, uid)
        assert torch.equal(n_[0], t(g["nib"])[b])
        assert torch.equal(q_[0], t(g["qjl"])[b])
        assert torch.allclose(r_[0], t(g["norms"])[b], rtol=5e-7, atol=0)


def test_rows_golden():
    g = load_golden("rows.npz")
    n_, q_, r_ = orc.quantize_rows(t(g["x"]), t(g["codebook"]), base_head_idx=3, user_id=77)
    assert torch.equal(n_, t(g["nib"])) and torch.equal(q_, t(g["qjl"]))
    assert torch.allclose(r_, t(g["norms"]), rtol=5e-7, atol=0)
    xh = orc.dequantize_rows(n_, q_, r_, t(g["codebook"]), 3, 77, True)
    assert (xh - t(g["x_hat"])).abs().max() <= 1e-6


def test_gqa_attention_golden():
    g = load_golden("gqa_attention.npz")
    cb = t(g["codebook"]); uid = int(g["user_id"])
    kn, kq, kr = orc.quantize_heads(t(g["k_rot"]), cb, uid)
    vn, _, _ = orc.quantize_heads(t(g["v_rot"]), cb, uid)
    assert torch.equal(kn, t(g["k_nib"])) and torch.equal(kq, t(g["k_qjl"])) and torch.equal(vn, t(g["v_nib"]))
    out = orc.decode_attention(bf16(g["q_bf16"]), kn, kq, kr, vn, cb, uid, None, True)
    assert (out - t(g["out"])).abs().max() <= 2e-6
    out3 = orc.decode_attention(bf16(g["q3_bf16"]), kn, kq, kr, vn, cb, uid, float(g["scale3"]), True)
    assert (out3 - t(g["out3"])).abs().max() <= 2e-6


def test_lora_golden():
    g = load_golden("lora_attention.npz")
    q_eff = orc.apply_lora_to_q(t(g["q"]), t(g["x"]), t(g["lora_a"]), t(g["lora_b"]), t(g["lora_indices"]),
                                float(g["lora_alpha"]))
    assert (q_eff - t(g["q_eff"])).abs().max() <= 1e-6
    assert torch.equal(q_eff[1], t(g["q"])[1])            # index -1: row untouched
    out = orc.decode_attention(q_eff, t(g["k_nib"]), t(g["k_qjl"]), t(g["k_norms"]), t(g["v_nib"]),
                               t(g["codebooks"]), int(g["user_id"]), None, True)
    assert (out - t(g["out"])).abs().max() <= 2e-6


def test_lloyd_max_matches_stored_codebooks(config0_oracle):
    """The oracle's fit on the samples the reference calibrated head 0 with (all 64 users x 50 tokens x 128 dims of
    the rotated K) reproduces the codebook the reference stored, run to the reference's own 300-iteration cap."""
    g, cbs, Kr, _, _, _, _ = config0_oracle
    fit = orc.lloyd_max_fit(Kr[:, 0].reshape(-1))
    assert fit.shape == (16,) and fit.dtype == torch.float32
    assert (fit[1:] >= fit[:-1]).all()
    assert (fit - cbs[0]).abs().max() <= 1e-6
    with pytest.raises(ValueError):
        orc.lloyd_max_fit(torch.zeros(3))


def test_rows_beyond_1024_golden():
    """Row keys 1000..1059: the rows past key 1023 use MT19937 seeds above the 1,024 per-head seeds."""
    g = load_golden("rows_beyond_1024.npz")
    base, uid = int(g["base_head_idx"]), int(g["user_id"])
    n_, q_, r_ = orc.quantize_rows(t(g["x"]), t(g["codebook"]), base_head_idx=base, user_id=uid)
    assert torch.equal(n_, t(g["nib"])) and torch.equal(q_, t(g["qjl"]))
    assert torch.allclose(r_, t(g["norms"]), rtol=5e-7, atol=0)
    xh = orc.dequantize_rows(n_, q_, r_, t(g["codebook"]), base, uid, True)
    assert (xh - t(g["x_hat"])).abs().max() <= 1e-6
    for seed in (1024, 1500, 70000):                                  # G of large seeds against torch's CPU generator
        gen = torch.Generator().manual_seed(seed)
        bits = torch.randint(0, 2, (64, 128), generator=gen).numpy().astype(np.uint8)
        assert np.array_equal(bits, orc.rademacher_bits(seed))


def test_wide_codebook_attention_golden():
    """Un-rotated cache with outlier channels (centroids out to +-20) and queries aligned with single keys."""
    g = load_golden("wide_codebook_attention.npz")
    assert float(np.abs(g["codebook"]).max()) > 16.0
    out = orc.decode_attention(bf16(g["q_bf16"]), t(g["k_nib"]), t(g["k_qjl"]), t(g["k_norms"]), t(g["v_nib"]),
                               t(g["codebook"]), int(g["user_id"]), None, True)
    assert (out - t(g["out"])).abs().max() <= 2e-6


def test_sign_ambiguity_is_rare(config0_oracle):
    _, cbs, Kr, _, _, _, _ = config0_oracle
    _, _, _, resid = orc.quantize_heads(Kr[:8], cbs, 0, return_residual=True)
    amb = orc.sign_ambiguity(resid, 0)
    assert amb.float().mean() < 1e-4
