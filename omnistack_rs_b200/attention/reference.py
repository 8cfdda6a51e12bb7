"""Full-precision GQA attention over dense tensors (the numerical anchor).

Mirrors ``reference_attn`` (:72) and ``repeat_kv`` (:49) of the reference's
``omnistack_rs/attention/reference.py``: tile-wise running (max, sum, accumulator) update
in float32, additive ``mask``, result cast to ``q.dtype``.  It operates on dense K/V and
is independent of the quantized path: a check for the packed kernels, run with torch operations
on the CUDA device its inputs live on (host tensors raise, like everywhere in this package).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _lib


def repeat_kv(x: torch.Tensor, n_groups: int) -> torch.Tensor:
    if n_groups == 1:
        return x
    B, n_kv, S, d = x.shape
    return x.unsqueeze(2).expand(B, n_kv, n_groups, S, d).reshape(B, n_kv * n_groups, S, d)


def reference_attn(q, k, v, mask: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                   tile_size: int = 128) -> torch.Tensor:
    _lib.require_cuda(q, k, v, mask)
    n_groups = q.shape[1] // k.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    qf = q.float()
    kf, vf = repeat_kv(k, n_groups).float(), repeat_kv(v, n_groups).float()
    B, H, T, D = qf.shape
    run_max = qf.new_full((B, H, T, 1), float("-inf"))
    run_sum = qf.new_zeros(B, H, T, 1)
    acc = qf.new_zeros(B, H, T, D)
    for s0 in range(0, kf.shape[2], tile_size):
        s1 = min(s0 + tile_size, kf.shape[2])
        sc = torch.matmul(qf, kf[:, :, s0:s1].transpose(-2, -1)) * scale
        if mask is not None:
            sc = sc + mask[..., s0:s1].float()
        new_max = torch.maximum(run_max, sc.amax(dim=-1, keepdim=True))
        corr = torch.exp(run_max - new_max)
        p = torch.exp(sc - new_max)
        run_sum = corr * run_sum + p.sum(dim=-1, keepdim=True)
        acc = corr * acc + torch.matmul(p, vf[:, :, s0:s1])
        run_max = new_max
    return (acc / run_sum).to(q.dtype)
