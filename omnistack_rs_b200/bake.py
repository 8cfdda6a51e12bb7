"""Baked cache files: the on-disk format of the reference's codec bake.

Mirrors ``bake_kv_cache`` of the reference driver (scripts/run_criteo_benchmark.py:319-404): the
file is a ``torch.save`` dict ``{"nibbles", "qjl", "norms", "codebooks", "stats"}`` of CPU tensors
(loadable with ``weights_only=True``), with the reference's shapes, dtypes and stats keys, so caches
baked by either implementation can be read by the other.  Here the rotation and the codec run on the
GPU (one fused kernel); the Lloyd-Max fit runs with the reference's algorithm on the device.
"""
from __future__ import annotations

import os
from typing import Tuple

import torch

from .kernels.quantize import quantize_heads
from .kernels.hadamard import rotate_queries, HEAD_DIM
from .quantization.codebook import calibrate_per_group

_KEYS = ("nibbles", "qjl", "norms", "codebooks", "stats")


def load_baked_cache(bake_path: str, device="cpu"):
    """Read a baked cache file; tensors are moved to ``device``.  Returns
    ``(nibbles, qjl, norms, codebooks, stats)`` like the reference."""
    saved = torch.load(bake_path, map_location="cpu", weights_only=True)
    missing = [k for k in _KEYS if k not in saved]
    if missing:
        raise ValueError(f"{bake_path} is not a baked cache: missing {missing}")
    nib, qjl, norms, cbs = (saved[k].to(device) for k in _KEYS[:4])
    if nib.dtype != torch.uint8 or qjl.dtype != torch.uint8 or nib.shape[-1] != HEAD_DIM // 2 or qjl.shape[-1] != 8:
        raise ValueError(f"{bake_path}: unexpected packed tensor layout")
    return nib, qjl, norms.float(), cbs.float(), saved["stats"]


def bake_kv_cache(kv_raw: torch.Tensor, bake_path: str, force: bool = False, seed: int = 0,
                  device=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, dict]:
    """Rotate, calibrate one codebook per kv head, quantize with ``user_id=seed`` and persist.
    ``kv_raw``: (N, n_kv_heads, seq_len, 128).  Returns CPU tensors like the reference."""
    if os.path.exists(bake_path) and not force:
        return load_baked_cache(bake_path)
    dev = torch.device(device) if device is not None else (kv_raw.device if kv_raw.is_cuda else torch.device("cuda"))
    x = kv_raw.to(dev)
    N, H, S, D = x.shape
    rot = rotate_queries(x)
    codebooks = calibrate_per_group([rot[:, h].reshape(-1) for h in range(H)])
    nib, qjl, norms = quantize_heads(rot, codebooks, user_id=seed)
    n_elements = N * H * S * HEAD_DIM
    compressed = nib.numel() + qjl.numel() + norms.numel() * 4
    stats = {
        "n_users": N, "n_kv_heads": H, "seq_len": S, "bf16_bytes": n_elements * 2,
        "compressed_bytes": compressed, "compression_ratio": round(n_elements * 2 / compressed, 3),
        "bits_per_element": round(compressed * 8 / n_elements, 3),
    }
    out = {"nibbles": nib.cpu(), "qjl": qjl.cpu(), "norms": norms.cpu(), "codebooks": codebooks.cpu(), "stats": stats}
    torch.save(out, bake_path)
    return out["nibbles"], out["qjl"], out["norms"], out["codebooks"], stats
