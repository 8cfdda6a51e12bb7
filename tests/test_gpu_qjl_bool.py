"""Unpacked QJL API (``RademacherQJL``, ``qjl_encode``, ``qjl_reconstruct``) on the GPU against the oracle's G and
exact fp64 projections; the cases follow the reference's tests/unit/test_quant.py:197-243 (shapes, per-head
seeds, residual norm) and :604-660 (seed formula, user aliasing, user-id consistency)."""
import math

import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def qjl_mod():
    from omnistack_rs_b200.quantization import qjl
    return qjl


def exact_signs(err, seed):
    G = orc.rademacher_matrix(seed).double()                  # (64, 128) of +-1
    proj = err.double() @ G.t()
    l1 = err.double().abs().sum(dim=-1, keepdim=True)
    return proj >= 0, proj.abs() <= l1 * 2.0 ** -40            # second: ties that fp64 itself cannot order


@pytest.mark.parametrize("shape", [(128,), (1, 128), (5, 3, 128), (2, 4, 50, 128)])
def test_encode_matches_exact_projection_signs(dev, shape):
    q = qjl_mod().RademacherQJL(128, 64)
    err = torch.randn(*shape, generator=torch.Generator().manual_seed(len(shape))) * 0.3
    signs, norms = q.encode(err.to(dev), head_idx=3, user_id=1030)           # seed (1030 % 1024) ^ 3 = 5
    assert signs.dtype == torch.bool and signs.shape == shape[:-1] + (64,)
    assert norms.shape == shape[:-1] + (1,) and norms.dtype == torch.float32
    want, tie = exact_signs(err, 5)
    assert bool(((signs.cpu() == want) | tie).all())
    assert torch.allclose(norms.cpu(), err.norm(dim=-1, keepdim=True), rtol=1e-6, atol=0)
    # reconstruction: exact integer sum times one rounded coefficient
    rec = q.reconstruct(signs, norms, head_idx=3, user_id=1030).cpu()
    b = signs.cpu().float() * 2 - 1
    ref = (b @ orc.rademacher_matrix(5).float()) * (norms.cpu() * math.sqrt(2.0 / math.pi) / 128)
    assert rec.shape == shape and torch.allclose(rec, ref, rtol=2e-7, atol=0)


def test_seeds_heads_and_user_aliasing(dev):
    q = qjl_mod().RademacherQJL(128, 64)
    err = torch.randn(64, 128, generator=torch.Generator().manual_seed(9)).to(dev)
    s0, _ = q.encode(err, head_idx=0, user_id=0)
    s1, _ = q.encode(err, head_idx=1, user_id=0)
    su, _ = q.encode(err, head_idx=0, user_id=7)
    sa, _ = q.encode(err, head_idx=0, user_id=1024)
    assert not torch.equal(s0, s1) and not torch.equal(s0, su)              # heads and users draw different G
    assert torch.equal(s0, sa)                                              # user 1024 aliases to user 0
    with pytest.raises(NotImplementedError):
        q.encode(err, head_idx=1024, user_id=0)
    with pytest.raises(RuntimeError):
        q.encode(err.cpu(), head_idx=0)                                     # no CPU fallback


def test_bool_api_agrees_with_packed_codec(dev):
    """The packed sign bytes of ``quantize_heads`` are the bool signs of the same residual."""
    from omnistack_rs_b200.kernels.quantize import quantize_heads, dequantize_heads
    gen = torch.Generator().manual_seed(12)
    x = torch.randn(2, 3, 40, 128, generator=gen)
    cb = torch.sort(torch.randn(3, 16, generator=gen), dim=1).values
    nib, qjl_bytes, norms = quantize_heads(x.to(dev), cb.to(dev), user_id=6)
    base = dequantize_heads(nib, qjl_bytes, norms, cb.to(dev), user_id=6, with_qjl=False)
    full = dequantize_heads(nib, qjl_bytes, norms, cb.to(dev), user_id=6, with_qjl=True)
    for h in range(3):
        err, signs, nr = qjl_mod().qjl_encode(x[:, h].to(dev), base[:, h], head_idx=h, user_id=6)
        assert torch.equal(orc.pack_sign_bits(signs.cpu()), qjl_bytes[:, h].cpu())
        assert torch.allclose(nr.squeeze(-1), norms[:, h], rtol=1e-6, atol=0)
        rec = qjl_mod().qjl_reconstruct(base[:, h], signs, nr, head_idx=h, user_id=6)
        assert torch.allclose(rec, full[:, h], rtol=0, atol=1e-6)
        # the residual estimate lowers the error (reference test_quant.py:270-345)
        assert (rec - x[:, h].to(dev)).pow(2).mean() < (base[:, h] - x[:, h].to(dev)).pow(2).mean()
