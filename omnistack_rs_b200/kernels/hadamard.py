"""Normalised 128-point Walsh-Hadamard rotation on the GPU.

Mirrors ``omnistack_rs/kernels/hadamard.py`` of the reference (``rotate_queries`` :196,
``rotate_kv_cache`` :214, ``_wht_rotate`` :155): same names, same return convention (a
new tensor of the input's shape, dtype and device; the input is never modified), same
``ValueError`` mentioning ``head_dim`` for a wrong last dimension.  Results are
bit-identical to the reference's ``_wht_torch`` (:51-85).
"""
from __future__ import annotations

import math

import torch

from .. import _lib

HEAD_DIM: int = 128
LOG2_HEAD_DIM: int = 7
_SCALE: float = 1.0 / math.sqrt(HEAD_DIM)


def _wht_rotate(x: torch.Tensor) -> torch.Tensor:
    if x.shape[-1] != HEAD_DIM:
        raise ValueError(f"WHT rotation requires last dim = {HEAD_DIM} (head_dim), got {x.shape[-1]}.")
    dev = _lib.require_cuda(x)
    if x.dtype not in _lib.DTYPE_CODE:
        raise TypeError(f"unsupported dtype {x.dtype}; use float32, bfloat16 or float16")
    lib = _lib.ensure_init(dev)
    src = x.contiguous()
    out = torch.empty_like(src)
    with torch.cuda.device(dev):
        _lib.check(lib.omni_rotate(_lib.ptr(src), _lib.ptr(out), src.numel() // HEAD_DIM,
                                   _lib.DTYPE_CODE[x.dtype], _lib.stream_ptr(dev)))
    return out.view(x.shape)


def rotate_queries(q: torch.Tensor) -> torch.Tensor:
    """Rotate query projections ``(B, n_heads, T, 128)``."""
    return _wht_rotate(q)


def rotate_kv_cache(k: torch.Tensor, v: torch.Tensor):
    """Rotate key and value tensors ``(B, n_kv_heads, S, 128)``."""
    return _wht_rotate(k), _wht_rotate(v)
