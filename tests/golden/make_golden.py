"""Generate the golden fixtures in this directory from the reference itself.

Run once in a container that holds the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/Omnistack-RS

The script imports the reference's CPU (torch) code path with Triton hidden,
feeds it seeded inputs and stores inputs (or their seeds and checksums) and
outputs as ``.npz`` files.  Nothing else in the repository needs the reference
checkout: the tests replay the oracle and the CUDA library against these files.
"""
from __future__ import annotations

import argparse
import hashlib
import math
import os
import sys

import numpy as np


def sha(t) -> str:
    a = t.detach().contiguous().cpu()
    if a.dtype.is_floating_point and a.dtype.itemsize == 2:
        a = a.view(__import__("torch").int16)
    return hashlib.sha256(a.numpy().tobytes()).hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", nargs="*", default=None, help="write only these fixture files (default: all)")
    args = ap.parse_args()
    # Hide Triton so every reference routine takes its torch branch.
    sys.modules["triton"] = None
    sys.modules["triton.language"] = None
    sys.path.insert(0, args.reference)
    import torch
    from omnistack_rs.kernels.hadamard import _wht_torch
    from omnistack_rs.kernels.quantize import (quantize_heads, dequantize_heads, quantize_rows,
                                               dequantize_rows)
    from omnistack_rs.kernels.fused_attention import _fused_attn_python, _apply_lora_to_q, omni_attn
    from omnistack_rs.quantization.codebook import calibrate_per_group, calibrate_codebook

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    here = os.path.dirname(os.path.abspath(__file__))

    def save(name, **arrs):
        if args.only is not None and name not in args.only:
            return
        out = {}
        for k, v in arrs.items():
            if isinstance(v, torch.Tensor):
                if v.dtype == torch.bfloat16:
                    v = v.view(torch.int16)
                v = v.numpy()
            out[k] = np.asarray(v)
        np.savez_compressed(os.path.join(here, name), **out)
        print(name, {k: (a.shape, str(a.dtype)) for k, a in out.items()})

    # ---- Rademacher table: all 1024 seeds, stored as one checksum + 3 full seeds
    bits_all = []
    for seed in range(1024):
        g = torch.Generator().manual_seed(seed)
        bits_all.append(torch.randint(0, 2, (64, 128), generator=g, dtype=torch.float32).to(torch.uint8))
    bits_all = torch.stack(bits_all)
    save("rademacher.npz", sha_all=np.array(sha(bits_all)), seed0=bits_all[0], seed5=bits_all[5],
         seed1023=bits_all[1023])

    # ---- config 0: codec round trip, config 1: decode attention on that cache
    g = torch.Generator().manual_seed(0)
    K = torch.randn(64, 8, 50, 128, generator=g)
    V = torch.randn(64, 8, 50, 128, generator=g)
    q1 = torch.randn(64, 8, 1, 128, generator=g).to(torch.bfloat16)
    Kr, Vr = _wht_torch(K), _wht_torch(V)
    cbs = calibrate_per_group([Kr[:, h].reshape(-1) for h in range(8)])
    kn, kq, kr = quantize_heads(Kr, cbs, 0)
    vn, vq, vr = quantize_heads(Vr, cbs, 0)
    k_hat = dequantize_heads(kn, kq, kr, cbs, 0, True)
    v_hat = dequantize_heads(vn, vq, vr, cbs, 0, False)
    out1 = _fused_attn_python(q1.float(), kn, kq, kr, vn, cbs, 0, 1.0 / math.sqrt(128), True)
    out1_noqjl = _fused_attn_python(q1.float(), kn, kq, kr, vn, cbs, 0, 1.0 / math.sqrt(128), False)
    save("config0_codec.npz",
         sha_K=np.array(sha(K)), sha_V=np.array(sha(V)), sha_Krot=np.array(sha(Kr)), sha_Vrot=np.array(sha(Vr)),
         codebooks=cbs,
         sha_k_nib=np.array(sha(kn)), sha_k_qjl=np.array(sha(kq)),
         sha_v_nib=np.array(sha(vn)), sha_v_qjl=np.array(sha(vq)),
         k_nib_u4=kn[:4], k_qjl_u4=kq[:4], v_nib_u4=vn[:4], v_qjl_u4=vq[:4],
         k_norms=kr, v_norms=vr, k_hat_u0=k_hat[0], v_hat_u0=v_hat[0], k_rot_u0=Kr[0])
    save("config1_attention.npz", q_bf16=q1, out=out1, out_noqjl=out1_noqjl)

    # ---- small codec case: bf16 input with heavy tail, several user ids, rotation inside
    g = torch.Generator().manual_seed(3)
    xb = torch.randn(5, 8, 16, 128, generator=g)
    mask = torch.rand(5, 8, 16, 128, generator=g) < 0.01
    xb = torch.where(mask, xb * 10.0, xb).to(torch.bfloat16)
    xb_rot = _wht_torch(xb)
    cb_shared = calibrate_codebook(xb_rot.float().reshape(-1))
    uids = [0, 5, 1023, 1024, 2051]
    nibs, qjls, nrms = [], [], []
    for b, uid in enumerate(uids):
        n_, q_, r_ = quantize_heads(xb_rot[b:b + 1], cb_shared, uid)
        nibs.append(n_); qjls.append(q_); nrms.append(r_)
    save("codec_bf16_users.npz", x_bf16=xb, x_rot_bf16=xb_rot, codebook=cb_shared,
         user_ids=np.array(uids, dtype=np.int32), nib=torch.cat(nibs), qjl=torch.cat(qjls), norms=torch.cat(nrms))

    # ---- fp16 and fp32 rotation vectors
    g = torch.Generator().manual_seed(4)
    xr = torch.randn(64, 128, generator=g) * 3.0
    save("rotation.npz", x=xr, y=_wht_torch(xr), y_bf16=_wht_torch(xr.to(torch.bfloat16)),
         y_fp16=_wht_torch(xr.to(torch.float16)).view(torch.int16))

    # ---- row-seeded variant
    g = torch.Generator().manual_seed(6)
    xrows = _wht_torch(torch.randn(3, 7, 128, generator=g))
    rn, rq, rr = quantize_rows(xrows, cbs[2], base_head_idx=3, user_id=77)
    rhat = dequantize_rows(rn, rq, rr, cbs[2], base_head_idx=3, user_id=77, with_qjl=True)
    save("rows.npz", x=xrows, codebook=cbs[2], nib=rn, qjl=rq, norms=rr, x_hat=rhat)

    # ---- GQA decode with outlier channels, shared codebook, short prefill (T=3)
    g = torch.Generator().manual_seed(1)
    B, Hq, Hkv, S = 3, 8, 2, 333
    chans = torch.randperm(128, generator=g)[:4]
    Kg = torch.randn(B, Hkv, S, 128, generator=g); Vg = torch.randn(B, Hkv, S, 128, generator=g)
    Kg[..., chans] *= 8.0; Vg[..., chans] *= 8.0
    Kgr, Vgr = _wht_torch(Kg), _wht_torch(Vg)
    cbg = calibrate_codebook(Kgr.reshape(-1))
    gkn, gkq, gkr = quantize_heads(Kgr, cbg, 9)
    gvn, gvq, gvr = quantize_heads(Vgr, cbg, 9)
    qg = torch.randn(B, Hq, 1, 128, generator=g).to(torch.bfloat16)
    qg3 = torch.randn(B, Hq, 3, 128, generator=g).to(torch.bfloat16)
    og = _fused_attn_python(qg.float(), gkn, gkq, gkr, gvn, cbg, 9, 1.0 / math.sqrt(128), True)
    og3 = _fused_attn_python(qg3.float(), gkn, gkq, gkr, gvn, cbg, 9, 0.05, True)
    save("gqa_attention.npz", k_rot=Kgr, v_rot=Vgr, codebook=cbg, user_id=np.array(9),
         k_nib=gkn, k_qjl=gkq, k_norms=gkr, v_nib=gvn, q_bf16=qg, out=og, q3_bf16=qg3, out3=og3,
         scale3=np.array(0.05))

    # ---- LoRA query prologue through the public entry point
    g = torch.Generator().manual_seed(8)
    B, Hq, Hkv, S, hid, rank = 4, 4, 2, 40, 64, 16
    Kl = _wht_torch(torch.randn(B, Hkv, S, 128, generator=g)); Vl = _wht_torch(torch.randn(B, Hkv, S, 128, generator=g))
    cbl = calibrate_per_group([Kl[:, h].reshape(-1) for h in range(Hkv)])
    lkn, lkq, lkr = quantize_heads(Kl, cbl, 2)
    lvn, _, _ = quantize_heads(Vl, cbl, 2)
    ql = torch.randn(B, Hq, 1, 128, generator=g)
    xl = torch.randn(B, 1, hid, generator=g)
    la = torch.randn(3, rank, hid, generator=g) * 0.1
    lb = torch.randn(3, Hq * 128, rank, generator=g) * 0.1
    lidx = torch.tensor([0, -1, 2, 1], dtype=torch.int32)
    q_eff = _apply_lora_to_q(ql, xl, la, lb, lidx, 0.5)
    ol = omni_attn(ql, lkn, lkq, lkr, lvn, cbl, user_id=2, with_qjl=True,
                   x=xl, lora_a=la, lora_b=lb, lora_indices=lidx, lora_alpha=0.5)
    save("lora_attention.npz", k_nib=lkn, k_qjl=lkq, k_norms=lkr, v_nib=lvn, codebooks=cbl, user_id=np.array(2),
         q=ql, x=xl, lora_a=la, lora_b=lb, lora_indices=lidx, lora_alpha=np.array(0.5), q_eff=q_eff, out=ol)

    # ---- row-seeded variant with row keys on both sides of 1,024 (seeds beyond the 1,024 per-head seeds)
    g = torch.Generator().manual_seed(12)
    xw = _wht_torch(torch.randn(3, 20, 128, generator=g))
    wn, wq, wr = quantize_rows(xw, cbs[1], base_head_idx=1000, user_id=77)
    what = dequantize_rows(wn, wq, wr, cbs[1], base_head_idx=1000, user_id=77, with_qjl=True)
    save("rows_beyond_1024.npz", x=xw, codebook=cbs[1], base_head_idx=np.array(1000), user_id=np.array(77),
         nib=wn, qjl=wq, norms=wr, x_hat=what)

    # ---- attention over an UN-rotated cache with outlier channels: centroids far outside +-4, and queries aligned
    #      with single keys so that one key dominates the softmax
    g = torch.Generator().manual_seed(13)
    B, Hq, Hkv, S = 2, 4, 2, 160
    chans = torch.randperm(128, generator=g)[:4]
    Kw = torch.randn(B, Hkv, S, 128, generator=g); Vw = torch.randn(B, Hkv, S, 128, generator=g)
    Kw[..., chans] *= 8.0; Vw[..., chans] *= 8.0
    cbw = calibrate_codebook(torch.cat([Kw.reshape(-1), Vw.reshape(-1)]))
    wkn, wkq, wkr = quantize_heads(Kw, cbw, 11)
    wvn, _, _ = quantize_heads(Vw, cbw, 11)
    qw = torch.randn(B, Hq, 1, 128, generator=g) * 0.3
    for b in range(B):
        for h in range(Hq):
            qw[b, h, 0] += 0.9 * Kw[b, h // (Hq // Hkv), 17 * (h + 1) + b]
    qw = qw.to(torch.bfloat16)
    ow = _fused_attn_python(qw.float(), wkn, wkq, wkr, wvn, cbw, 11, 1.0 / math.sqrt(128), True)
    save("wide_codebook_attention.npz", codebook=cbw, user_id=np.array(11), k_nib=wkn, k_qjl=wkq, k_norms=wkr,
         v_nib=wvn, q_bf16=qw, out=ow)


if __name__ == "__main__":
    main()
