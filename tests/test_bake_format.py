"""Baked cache file format (reference: scripts/run_criteo_benchmark.py:319-404)."""
import pytest
import torch

import oracle as orc


def test_load_rejects_foreign_files_and_reads_reference_layout(tmp_path):
    from omnistack_rs_b200.bake import load_baked_cache
    bad = tmp_path / "bad.pt"
    torch.save({"nibbles": torch.zeros(1)}, bad)
    with pytest.raises(ValueError, match="missing"):
        load_baked_cache(str(bad))
    # a file written the way the reference writes it (CPU tensors from the oracle's codec)
    x = orc.wht128(torch.randn(2, 2, 5, 128, generator=torch.Generator().manual_seed(0)))
    cb = torch.sort(torch.randn(2, 16), dim=1).values
    nib, qjl, nrm = orc.quantize_heads(x, cb, 7)
    good = tmp_path / "good.pt"
    torch.save({"nibbles": nib, "qjl": qjl, "norms": nrm, "codebooks": cb, "stats": {"n_users": 2}}, good)
    n2, q2, r2, c2, st = load_baked_cache(str(good))
    assert torch.equal(n2, nib) and torch.equal(q2, qjl) and torch.equal(r2, nrm) and torch.equal(c2, cb)
    assert st["n_users"] == 2


@pytest.mark.gpu
def test_bake_on_gpu_roundtrip(tmp_path):
    from omnistack_rs_b200.bake import bake_kv_cache, load_baked_cache
    from omnistack_rs_b200.kernels.fused_attention import omni_attn
    gen = torch.Generator().manual_seed(4)
    kv = torch.randn(6, 2, 50, 128, generator=gen)
    path = str(tmp_path / "bake.pt")
    nib, qjl, nrm, cbs, stats = bake_kv_cache(kv, path, seed=3, device="cuda:0")
    assert nib.shape == (6, 2, 50, 64) and nib.dtype == torch.uint8 and not nib.is_cuda
    assert qjl.shape == (6, 2, 50, 8) and nrm.shape == (6, 2, 50) and cbs.shape == (2, 16)
    assert stats["bits_per_element"] == 4.75 and stats["compression_ratio"] == 3.368
    # given the stored codebooks the packed tensors are what the reference codec produces
    wn, wq, wr = orc.quantize_heads(orc.wht128(kv), cbs, 3)
    assert torch.equal(nib, wn) and torch.equal(qjl, wq) and torch.allclose(nrm, wr, rtol=1e-6)
    again = bake_kv_cache(kv, path, seed=3)                     # second call loads the file
    assert torch.equal(again[0], nib)
    dn, dq, dr, dc, _ = load_baked_cache(path, "cuda:0")
    q = torch.randn(6, 4, 1, 128, generator=gen).to(torch.bfloat16)
    out = omni_attn(q.to("cuda:0"), dn, dq, dr, dn, dc, user_id=3)       # V aliased to K's nibbles, as the reference driver does
    want = orc.decode_attention(q, wn, wq, wr, wn, cbs, 3)
    assert (out.cpu() - want).abs().max() <= 3e-3
