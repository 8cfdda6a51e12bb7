"""Unpacked (bool-sign) QJL residual coding.

Mirrors ``omnistack_rs/quantization/qjl.py`` of the reference (``RademacherQJL`` :46,
``qjl_encode`` :136, ``qjl_reconstruct`` :162).  G comes from the library's MT19937 table
(seed ``(user_id % 1024) ^ head_idx``), so it is the matrix the reference draws with a CPU
``torch.Generator`` whatever device the data is on.  ``encode`` and ``reconstruct`` run the
``omni_qjl_encode_bool`` / ``omni_qjl_reconstruct_bool`` kernels; the packed, fused form of the
same arithmetic is ``kernels.quantize.quantize_heads``.
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

    @staticmethod
    def _seed(head_idx: int, user_id: int) -> int:
        seed = (int(user_id) % 1024) ^ int(head_idx)
        if not 0 <= seed < 1024:
            raise NotImplementedError(f"seed {seed} outside the 1024-seed table (head_idx must be < 1024)")
        return seed

    def encode(self, error: torch.Tensor, head_idx: int, user_id: int = 0):
        dev = _lib.require_cuda(error)
        lib = _lib.ensure_init(dev)
        if error.shape[-1] != self.head_dim:
            raise ValueError(f"last dim must be head_dim={self.head_dim}, got {error.shape[-1]}")
        err = error.float().contiguous()
        n = err.numel() // self.head_dim
        signs = torch.empty(*error.shape[:-1], self.qjl_dim, dtype=torch.uint8, device=dev)
        norms = torch.empty(*error.shape[:-1], 1, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            _lib.check(lib.omni_qjl_encode_bool(_lib.ptr(err), n, self._seed(head_idx, user_id), _lib.ptr(signs),
                                                _lib.ptr(norms), _lib.stream_ptr(dev)))
        return signs.view(torch.bool), norms.to(error.dtype)

    def reconstruct(self, signs: torch.Tensor, norms: torch.Tensor, head_idx: int, user_id: int = 0):
        dev = _lib.require_cuda(signs, norms)
        lib = _lib.ensure_init(dev)
        if signs.shape[-1] != self.qjl_dim:
            raise ValueError(f"last dim of signs must be qjl_dim={self.qjl_dim}, got {signs.shape[-1]}")
        sg = signs.to(torch.uint8).contiguous()
        nr = norms.float().contiguous()
        n = sg.numel() // self.qjl_dim
        if nr.numel() != n:
            raise ValueError("norms must hold one value per sign row")
        out = torch.empty(*signs.shape[:-1], self.head_dim, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            _lib.check(lib.omni_qjl_reconstruct_bool(_lib.ptr(sg), _lib.ptr(nr), n, self._seed(head_idx, user_id),
                                                     _lib.ptr(out), _lib.stream_ptr(dev)))
        return out


def qjl_encode(x_orig, x_dequant, head_idx: int, qjl_dim: int = 64, user_id: int = 0):
    qjl = RademacherQJL(head_dim=x_orig.shape[-1], qjl_dim=qjl_dim)
    error = x_orig.float() - x_dequant.float()
    signs, norms = qjl.encode(error, head_idx, user_id=user_id)
    return error, signs, norms


def qjl_reconstruct(x_dequant, signs, norms, head_idx: int, qjl_dim: int = 64, user_id: int = 0):
    qjl = RademacherQJL(head_dim=x_dequant.shape[-1], qjl_dim=qjl_dim)
    return x_dequant.float() + qjl.reconstruct(signs, norms, head_idx, user_id=user_id)
