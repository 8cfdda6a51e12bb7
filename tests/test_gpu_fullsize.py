"""Full-size runs of the benchmark configurations, checked through size-independent properties
(the CPU oracle only sees sampled users): quantize-append at configuration 3's size and the
box-serving step at configuration 4's per-GPU batch."""
import math

import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu

LLOYD_MAX_N01 = [-2.733, -2.069, -1.618, -1.256, -0.9424, -0.6568, -0.3881, -0.1284,
                 0.1284, 0.3881, 0.6568, 0.9424, 1.256, 1.618, 2.069, 2.733]


def test_quantize_append_config3_full_size():
    """4,096 users x 8 heads x 256 tokens, bf16, N(0,1) with 1 % of values x10, user id = user index."""
    from omnistack_rs_b200.kernels import quantize as qz, hadamard
    dev = torch.device("cuda:0")
    U, H, T = 4096, 8, 256
    gen = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(U, H, T, 128, generator=gen, device=dev)
    x = torch.where(torch.rand(U, H, T, 128, generator=gen, device=dev) < 0.01, x * 10, x).to(torch.bfloat16)
    cb = torch.tensor(LLOYD_MAX_N01, device=dev)
    ids = torch.arange(U, dtype=torch.int32, device=dev)
    nib, qjl, nrm = qz.quantize_heads(x, cb, ids, rotate=True)
    assert nib.shape == (U, H, T, 64) and qjl.shape == (U, H, T, 8) and nrm.shape == (U, H, T)
    # sampled users against the oracle: codes and sign bits bit for bit
    for u in (0, 1, 1023, 1024, 2500, 4095):
        wn, wq, wr = orc.rotate_quantize(x[u:u + 1].cpu(), cb.cpu(), u)
        assert torch.equal(nib[u:u + 1].cpu(), wn) and torch.equal(qjl[u:u + 1].cpu(), wq)
        assert torch.allclose(nrm[u:u + 1].cpu(), wr, rtol=1e-6)
    # properties over all 8.4 M rows, in slices to bound memory
    better, worse = 0.0, 0.0
    for u0 in range(0, U, 512):
        sl = slice(u0, u0 + 512)
        rot = hadamard.rotate_queries(x[sl]).float()
        full = qz.dequantize_heads(nib[sl], qjl[sl], nrm[sl], cb, ids[sl], True)
        int4 = qz.dequantize_heads(nib[sl], qjl[sl], nrm[sl], cb, ids[sl], False)
        assert torch.allclose(nrm[sl], (rot - int4).norm(dim=-1), rtol=1e-5)        # the norm is the residual norm
        assert int(nib[sl].max()) <= 255 and torch.isfinite(nrm[sl]).all()
        better += float(((full - rot) ** 2).sum())
        worse += float(((int4 - rot) ** 2).sum())
        # idempotence: re-quantizing the INT4 reconstruction gives the same codes and a zero residual
        n2, _, r2 = qz.quantize_heads(int4[:64], cb, ids[sl][:64])
        assert torch.equal(n2, nib[sl][:64]) and float(r2.max()) == 0.0
    assert better < 0.95 * worse                                                    # QJL improves on INT4 alone


def test_box_serving_step_config4_batch():
    """16,384 users per step x 32 heads x 2,048 keys (the per-GPU batch of configuration 4) over 1,024
    resident users; logical user u reads slot u mod 1,024."""
    from omnistack_rs_b200.kernels.quantize import quantize_heads
    from omnistack_rs_b200.kernels.fused_attention import omni_attn
    from omnistack_rs_b200 import _lib
    dev = torch.device("cuda:0")
    users, res, H, S = 16384, 1024, 32, 2048
    gen = torch.Generator(device=dev).manual_seed(4)
    cb = torch.tensor(LLOYD_MAX_N01, device=dev)
    kn = torch.empty(res, H, S, 64, dtype=torch.uint8, device=dev)
    kq = torch.empty(res, H, S, 8, dtype=torch.uint8, device=dev)
    kr = torch.empty(res, H, S, dtype=torch.float32, device=dev)
    vn = torch.empty(res, H, S, 64, dtype=torch.uint8, device=dev)
    for u0 in range(0, res, 64):
        xk = torch.randn(64, H, S, 128, generator=gen, device=dev, dtype=torch.bfloat16)
        kn[u0:u0 + 64], kq[u0:u0 + 64], kr[u0:u0 + 64] = quantize_heads(xk, cb, 0, rotate=True)
        xv = torch.randn(64, H, S, 128, generator=gen, device=dev, dtype=torch.bfloat16)
        vn[u0:u0 + 64] = quantize_heads(xv, cb, 0, rotate=True)[0]
    slots = (torch.arange(users, dtype=torch.int32, device=dev) % res)
    q = torch.randn(res, H, 1, 128, generator=gen, device=dev, dtype=torch.bfloat16).repeat(users // res, 1, 1, 1)
    out = omni_attn(q, kn, kq, kr, vn, cb, user_id=0, cache_slots=slots)
    _lib.check_device_status(dev)
    assert out.shape == (users, H, 1, 128) and torch.isfinite(out).all()
    # users that share a slot and a query get the same row, whichever warp served them
    assert torch.equal(out[:res], out[res:2 * res]) and torch.equal(out[:res], out[-res:])
    # sampled users against the oracle
    for u in (0, 517, 1023):
        want = orc.decode_attention(q[u:u + 1].cpu(), kn[u:u + 1].cpu(), kq[u:u + 1].cpu(), kr[u:u + 1].cpu(),
                                    vn[u:u + 1].cpu(), cb.cpu(), 0)
        assert (out[u:u + 1].cpu() - want).abs().max() <= 3e-3
    # softmax weights sum to one: a cache whose V rows all hold centroid 7 returns that centroid
    vn.fill_(0x77)
    out_c = omni_attn(q[:2048], kn, kq, kr, vn, cb, user_id=0, cache_slots=slots[:2048])
    assert torch.allclose(out_c, torch.full_like(out_c, LLOYD_MAX_N01[7]), atol=1e-3)
    # scale invariance of the softmax: doubling q and halving the scale leaves the result unchanged
    a = omni_attn(q[:256], kn, kq, kr, vn, cb, user_id=0, cache_slots=slots[:256], scale=0.05)
    b = omni_attn((q[:256].float() * 2).to(torch.bfloat16), kn, kq, kr, vn, cb, user_id=0, cache_slots=slots[:256], scale=0.025)
    assert (a - b).abs().max() <= 1e-3


def test_gqa_decode_config2_full_size():
    """Configuration 2 at its own size: 256 users, 32 query / 8 kv heads, context lengths
    torch.randint(1024, 8193, (256,)) from seed 1, K/V N(0,1) with 4 channels x8 before the rotation, one shared
    codebook fitted on a million rotated samples, the split count the library picks (ragged lengths: ticket
    scheduling).  Oracle check on 10 users that include the shortest and the longest cache; the reference call is
    kernels/fused_attention.py:435-466 on the same packed inputs."""
    from omnistack_rs_b200.kernels.quantize import quantize_heads
    from omnistack_rs_b200.kernels.hadamard import rotate_queries
    from omnistack_rs_b200.kernels.fused_attention import omni_attn, _auto_splits
    from omnistack_rs_b200.quantization import calibrate_codebook
    from omnistack_rs_b200 import _lib
    dev = torch.device("cuda:0")
    B, Hq, Hkv, S = 256, 32, 8, 8192
    lens = torch.randint(1024, 8193, (B,), generator=torch.Generator().manual_seed(1)).to(torch.int32)
    gen = torch.Generator(device=dev).manual_seed(2)
    chans = torch.randperm(128, generator=torch.Generator().manual_seed(1))[:4].to(dev)
    kn = torch.empty(B, Hkv, S, 64, dtype=torch.uint8, device=dev)
    kq = torch.empty(B, Hkv, S, 8, dtype=torch.uint8, device=dev)
    kr = torch.empty(B, Hkv, S, dtype=torch.float32, device=dev)
    vn = torch.empty(B, Hkv, S, 64, dtype=torch.uint8, device=dev)
    cb = None
    for u0 in range(0, B, 32):
        xk = torch.randn(32, Hkv, S, 128, generator=gen, device=dev)
        xk[..., chans] *= 8.0
        if cb is None:
            cb = calibrate_codebook(rotate_queries(xk[:1]).reshape(-1)[: 1 << 20].contiguous())
            assert float(cb.abs().max()) < 8.0            # after the rotation the outliers are spread out
        kn[u0:u0 + 32], kq[u0:u0 + 32], kr[u0:u0 + 32] = quantize_heads(xk, cb, 0, rotate=True)
        xv = torch.randn(32, Hkv, S, 128, generator=gen, device=dev)
        xv[..., chans] *= 8.0
        vn[u0:u0 + 32] = quantize_heads(xv, cb, 0, rotate=True)[0]
        del xk, xv
    q = torch.randn(B, Hq, 1, 128, generator=gen, device=dev, dtype=torch.bfloat16)
    assert _auto_splits(B, Hq, Hkv, 1, S, True) > 1
    out = omni_attn(q, kn, kq, kr, vn, cb, user_id=0, seq_lens=lens.to(dev))
    _lib.check_device_status(dev)
    assert out.shape == (B, Hq, 1, 128) and torch.isfinite(out).all()
    one = omni_attn(q, kn, kq, kr, vn, cb, user_id=0, seq_lens=lens.to(dev), n_splits=1)
    assert (out - one).abs().max() <= 1.5e-3               # the splits round their fp16 softmax weights against other maxima
    sample = sorted({int(lens.argmin()), int(lens.argmax()), 0, 1, 37, 100, 128, 200, 254, 255})
    for u in sample:
        n = int(lens[u])
        want = orc.decode_attention(q[u:u + 1].cpu(), kn[u:u + 1, :, :n].cpu(), kq[u:u + 1, :, :n].cpu(),
                                    kr[u:u + 1, :, :n].cpu(), vn[u:u + 1, :, :n].cpu(), cb.cpu(), 0)
        assert (out[u:u + 1].cpu() - want).abs().max() <= 3e-3, (u, n)
