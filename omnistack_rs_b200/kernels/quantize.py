"""Packed INT4 + QJL codec on the GPU.

Mirrors ``omnistack_rs/kernels/quantize.py`` of the reference: ``quantize_heads`` (:542),
``dequantize_heads`` (:593), ``quantize_rows`` (:456), ``dequantize_rows`` (:502) keep their
signatures, output shapes/dtypes and the ``AssertionError`` on a codebook of the wrong
shape.  ``rotate_quantize_append`` is additive: it fuses the rotation and writes into a
preallocated cache at a per-user offset, producing exactly what
``quantize_heads(_wht_torch(x))`` would.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from .. import _lib
from .hadamard import HEAD_DIM

QJL_DIM: int = 64
_NBYTES_NIBBLE: int = HEAD_DIM // 2
_NBYTES_QJL: int = QJL_DIM // 8
_WORDS_PER_ROW: int = HEAD_DIM // 8


def _make_qjl_seed(user_id: int, row_seed: int) -> int:
    """``(user_id % 1024) ^ row_seed`` (reference quantize.py:293)."""
    return (user_id % 1024) ^ row_seed


def _prep_codebooks(codebooks: torch.Tensor, n_heads: int, dev) -> Tuple[torch.Tensor, int]:
    per_head = codebooks.dim() == 2
    if per_head:
        assert codebooks.shape == (n_heads, 16), codebooks.shape
    else:
        assert codebooks.shape == (16,), codebooks.shape
    return _lib.as_device(codebooks, dev, torch.float32), int(per_head)


def _user_args(user_id: Union[int, torch.Tensor], B: int, dev):
    """A Python int applies to the whole batch (the reference contract); an int tensor of
    shape (B,) gives one id per user."""
    if isinstance(user_id, torch.Tensor):
        ids = user_id.to(device=dev, dtype=torch.int32).contiguous()
        if ids.shape != (B,):
            raise ValueError(f"user_id tensor must have shape ({B},), got {tuple(ids.shape)}")
        return ids, 0
    uid = int(user_id) % 1024
    return None, uid


def _quantize_into(x, codebooks, user_id, rotate, nib, qjl, norms, os_b, os_h, out_offsets, out_offset):
    B, H, T, D = x.shape
    if D != HEAD_DIM:
        raise ValueError(f"codec requires last dim = {HEAD_DIM} (head_dim), got {D}")
    dev = _lib.require_cuda(x, nib, qjl, norms)
    if x.dtype not in _lib.DTYPE_CODE:
        raise TypeError(f"unsupported dtype {x.dtype}")
    lib = _lib.ensure_init(dev)
    if x.stride(-1) != 1 or any(s % 4 for s in x.stride()[:-1]) or x.data_ptr() % 16:
        x = x.contiguous()
    cb, per_head = _prep_codebooks(codebooks, H, dev)
    ids, uid = _user_args(user_id, B, dev)
    offs = None
    if out_offsets is not None:
        offs = out_offsets.to(device=dev, dtype=torch.int64).contiguous()
    with torch.cuda.device(dev):
        _lib.check(lib.omni_quantize_heads(
            _lib.ptr(x), _lib.DTYPE_CODE[x.dtype], int(bool(rotate)), _lib.ptr(cb), per_head,
            _lib.ptr(ids), uid, B, H, T, x.stride(0), x.stride(1), x.stride(2),
            _lib.ptr(nib), _lib.ptr(qjl), _lib.ptr(norms), os_b, os_h, _lib.ptr(offs), int(out_offset),
            _lib.stream_ptr(dev)))


def quantize_heads(x: torch.Tensor, codebooks: torch.Tensor, user_id=0, *, rotate: bool = False):
    """(B, n_heads, T, 128) rotated activations -> (nibbles u8 (B,H,T,64), qjl u8 (B,H,T,8),
    norms f32 (B,H,T)).  ``rotate=True`` applies the Hadamard rotation first."""
    B, H, T, _ = x.shape
    dev = _lib.require_cuda(x)
    nib = torch.empty(B, H, T, _NBYTES_NIBBLE, dtype=torch.uint8, device=dev)
    qjl = torch.empty(B, H, T, _NBYTES_QJL, dtype=torch.uint8, device=dev)
    norms = torch.empty(B, H, T, dtype=torch.float32, device=dev)
    _quantize_into(x, codebooks, user_id, rotate, nib, qjl, norms, H * T, T, None, 0)
    return nib, qjl, norms


def rotate_quantize_append(x_new: torch.Tensor, cache_nib: torch.Tensor, cache_qjl: torch.Tensor,
                           cache_norms: torch.Tensor, offsets, codebooks: torch.Tensor, user_id=0,
                           *, rotate: bool = True) -> None:
    """Rotate + quantize ``x_new`` (B, H, T_new, 128) and write the packed rows into the
    caches ``(B, H, S_max, 64|8|-)`` starting at key index ``offsets[b]`` (int tensor (B,) or
    one int).  Equals ``quantize_heads(_wht_torch(x_new))`` stored at that offset.  ``cache_qjl`` and
    ``cache_norms`` may both be ``None``: only the nibble rows are produced then (V rows: attention reads
    neither their sign bits nor their norms) and the projections are skipped."""
    B, H, T, _ = x_new.shape
    S_max = cache_nib.shape[2]
    if (cache_qjl is None) != (cache_norms is None):
        raise ValueError("cache_qjl and cache_norms must both be given or both be None")
    if cache_nib.shape != (B, H, S_max, _NBYTES_NIBBLE) or (cache_qjl is not None and (
            cache_qjl.shape != (B, H, S_max, _NBYTES_QJL) or cache_norms.shape != (B, H, S_max))):
        raise ValueError("cache tensors must be (B,H,S_max,64), (B,H,S_max,8), (B,H,S_max)")
    if not (cache_nib.is_contiguous() and (cache_qjl is None or (cache_qjl.is_contiguous() and cache_norms.is_contiguous()))):
        raise ValueError("cache tensors must be contiguous")
    if isinstance(offsets, torch.Tensor):
        if int(offsets.max()) + T > S_max or int(offsets.min()) < 0:
            raise ValueError("append would run past the cache capacity")
        _quantize_into(x_new, codebooks, user_id, rotate, cache_nib, cache_qjl, cache_norms,
                       H * S_max, S_max, offsets, 0)
    else:
        if int(offsets) < 0 or int(offsets) + T > S_max:
            raise ValueError("append would run past the cache capacity")
        _quantize_into(x_new, codebooks, user_id, rotate, cache_nib, cache_qjl, cache_norms,
                       H * S_max, S_max, None, int(offsets))


def dequantize_heads(nibbles, qjl_packed, norms, codebooks, user_id=0, with_qjl: bool = True) -> torch.Tensor:
    """Inverse codec -> (B, n_heads, T, 128) float32."""
    B, H, T, _ = nibbles.shape
    dev = _lib.require_cuda(nibbles, qjl_packed, norms)
    lib = _lib.ensure_init(dev)
    cb, per_head = _prep_codebooks(codebooks, H, dev)
    ids, uid = _user_args(user_id, B, dev)
    nibbles, qjl_packed, norms = nibbles.contiguous(), qjl_packed.contiguous(), norms.contiguous().float()
    out = torch.empty(B, H, T, HEAD_DIM, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.omni_dequantize_heads(
            _lib.ptr(nibbles), _lib.ptr(qjl_packed), _lib.ptr(norms), _lib.ptr(cb), per_head,
            _lib.ptr(ids), uid, B, H, T, H * T, T, int(bool(with_qjl)), _lib.ptr(out), _lib.stream_ptr(dev)))
    return out


def quantize_rows(x: torch.Tensor, codebook: torch.Tensor, base_head_idx: int = 0, user_id: int = 0):
    """(..., 128) -> (nibbles (...,64), qjl (...,8), norms (...)); row i of the flattened
    input is seeded with ``(user_id % 1024) ^ (base_head_idx + i)``."""
    if x.shape[-1] != HEAD_DIM:
        raise ValueError(f"codec requires last dim = {HEAD_DIM} (head_dim), got {x.shape[-1]}")
    dev = _lib.require_cuda(x)
    lib = _lib.ensure_init(dev)
    flat = x.reshape(-1, HEAD_DIM).float().contiguous()
    n = flat.shape[0]
    cb = codebook.to(device=dev, dtype=torch.float32).contiguous()
    assert cb.shape == (16,), cb.shape
    nib = torch.empty(n, _NBYTES_NIBBLE, dtype=torch.uint8, device=dev)
    qjl = torch.empty(n, _NBYTES_QJL, dtype=torch.uint8, device=dev)
    norms = torch.empty(n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.omni_quantize_rows(_lib.ptr(flat), _lib.ptr(cb), int(base_head_idx), int(user_id) % 1024, n,
                                          _lib.ptr(nib), _lib.ptr(qjl), _lib.ptr(norms), _lib.stream_ptr(dev)))
    lead = x.shape[:-1]
    return nib.reshape(*lead, _NBYTES_NIBBLE), qjl.reshape(*lead, _NBYTES_QJL), norms.reshape(*lead)


def dequantize_rows(nibbles, qjl_packed, norms, codebook, base_head_idx: int = 0, user_id: int = 0,
                    with_qjl: bool = True) -> torch.Tensor:
    """Inverse of :func:`quantize_rows` -> (..., 128) float32."""
    dev = _lib.require_cuda(nibbles, qjl_packed, norms)
    lib = _lib.ensure_init(dev)
    lead = nibbles.shape[:-1]
    nf = nibbles.reshape(-1, _NBYTES_NIBBLE).contiguous()
    qf = qjl_packed.reshape(-1, _NBYTES_QJL).contiguous()
    rf = norms.reshape(-1).float().contiguous()
    cb = codebook.to(device=dev, dtype=torch.float32).contiguous()
    out = torch.empty(nf.shape[0], HEAD_DIM, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.omni_dequantize_rows(_lib.ptr(nf), _lib.ptr(qf), _lib.ptr(rf), _lib.ptr(cb),
                                            int(base_head_idx), int(user_id) % 1024, nf.shape[0],
                                            int(bool(with_qjl)), _lib.ptr(out), _lib.stream_ptr(dev)))
    return out.reshape(*lead, HEAD_DIM)
