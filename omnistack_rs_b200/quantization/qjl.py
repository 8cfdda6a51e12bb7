"""Unpacked (bool-sign) QJL residual coding.

Mirrors ``omnistack_rs/quantization/qjl.py`` of the reference (``RademacherQJL`` :46,
``qjl_encode`` :136, ``qjl_reconstruct`` :162).  G comes from the library's MT19937 table
(seed ``(user_id % 1024) ^ head_idx``), so it is the matrix the reference draws with a CPU
``torch.Generator`` whatever device the data is on.  The projections run as one dense
product on the device; the packed, fused form of the same arithmetic is
``kernels.quantize.quantize_heads``.
"""
from __future__ import annotations

import ctypes as C
import functools
import math

import numpy as np
import torch

from .. import _lib


@functools.lru_cache(maxsize=64)
def _g_bits(seed: int) -> torch.Tensor:
    """(64, 128) uint8 bits of G for one seed, from the C library's host table."""
    if not 0 <= seed < 1024:
        raise NotImplementedError(f"seed {seed} outside the 1024-seed table (head_idx must be < 1024)")
    words = np.empty((64, 4), dtype=np.uint32)
    _lib.check(_lib.load().omni_gtable_host(words.ctypes.data_as(C.c_void_p), seed, 1))
    bits = (words[:, :, None] >> np.arange(32, dtype=np.uint32)) & 1
    return torch.from_numpy(bits.reshape(64, 128).astype(np.uint8))


class RademacherQJL:
    def __init__(self, head_dim: int, qjl_dim: int) -> None:
        if head_dim != 128 or qjl_dim != 64:
            raise NotImplementedError("the B200 library is built for head_dim=128, qjl_dim=64")
        self.head_dim = head_dim
        self.qjl_dim = qjl_dim

    def _make_G(self, head_idx: int, device, dtype, user_id: int = 0) -> torch.Tensor:
        seed = (user_id % 1024) ^ head_idx
        return (_g_bits(seed).to(device=device, dtype=dtype) * 2 - 1)

    def encode(self, error: torch.Tensor, head_idx: int, user_id: int = 0):
        _lib.require_cuda(error)
        err = error.float()
        G = self._make_G(head_idx, error.device, torch.float64, user_id)
        signs = (err.double() @ G.t()) >= 0
        norms = err.norm(dim=-1, keepdim=True).to(error.dtype)
        return signs, norms

    def reconstruct(self, signs: torch.Tensor, norms: torch.Tensor, head_idx: int, user_id: int = 0):
        _lib.require_cuda(signs)
        G = self._make_G(head_idx, signs.device, torch.float32, user_id)
        b = signs.float() * 2.0 - 1.0
        return (b @ G) * (norms.float() * math.sqrt(2.0 / math.pi) / self.head_dim)


def qjl_encode(x_orig, x_dequant, head_idx: int, qjl_dim: int = 64, user_id: int = 0):
    qjl = RademacherQJL(head_dim=x_orig.shape[-1], qjl_dim=qjl_dim)
    error = x_orig.float() - x_dequant.float()
    signs, norms = qjl.encode(error, head_idx, user_id=user_id)
    return error, signs, norms


def qjl_reconstruct(x_dequant, signs, norms, head_idx: int, qjl_dim: int = 64, user_id: int = 0):
    qjl = RademacherQJL(head_dim=x_dequant.shape[-1], qjl_dim=qjl_dim)
    return x_dequant.float() + qjl.reconstruct(signs, norms, head_idx, user_id=user_id)
