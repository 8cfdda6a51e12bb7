"""Fused attention over the packed INT4 + QJL cache on the GPU.

Mirrors ``omnistack_rs/kernels/fused_attention.py`` of the reference: ``omni_attn`` (:537),
``OmniAttention`` (:471, 15 positional arguments, backward returns ``None`` for each) and
``make_g_matrix`` (:296) keep their signatures.  The result is float32 of shape
``(B, n_heads, T, 128)`` like the reference's GPU path (:361).

Numerics follow the reference's CPU path ``_fused_attn_python`` (:435-466): K = INT4 + QJL,
V = INT4 only, G seeded per (user, kv head) with ``(user_id % 1024) ^ head`` exactly as
the codec.  ``g_matrix`` is accepted for signature compatibility and not used: the
reference's ``make_g_matrix`` draws all heads from one stream and therefore disagrees with
its own codec for every head but the first.

Additive keyword arguments: ``seq_lens`` (per-user valid length), ``rotate_q`` /
``unrotate_out`` (fold the Hadamard rotation into the query / out of the result),
``n_splits`` (split-K over the key axis; chosen automatically when ``None``).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _lib
from .hadamard import HEAD_DIM
from .quantize import QJL_DIM, _NBYTES_NIBBLE, _NBYTES_QJL, _make_qjl_seed, _prep_codebooks, _user_args  # noqa: F401

BLOCK_T: int = 16
BLOCK_S: int = 64
_SM_COUNT = 148


def make_g_matrix(n_kv_heads: int, seed: int, device="cpu"):
    """(G_lo, G_hi) int64 ``(n_kv_heads, 64)``: bits 0..63 / 64..127 of each projection row,
    drawn from one MT19937 stream of shape (n_kv_heads, 64, 128) like the reference (:296-317)."""
    gen = torch.Generator().manual_seed(seed)
    bits = torch.randint(0, 2, (n_kv_heads, QJL_DIM, HEAD_DIM), generator=gen, dtype=torch.int64)
    weights = torch.ones(64, dtype=torch.int64) << torch.arange(64, dtype=torch.int64)
    g_lo = (bits[..., :64] * weights).sum(dim=-1)
    g_hi = (bits[..., 64:] * weights).sum(dim=-1)
    return g_lo.to(device), g_hi.to(device)


def _prep_lora(q, x, lora_a, lora_b, lora_indices, dev):
    """Validated fp32 / int32 device tensors of the per-user query update."""
    B, Hq, T, D = q.shape
    if lora_indices.device.type == "cpu" and lora_indices.numel() and int(lora_indices.max()) >= lora_a.shape[0]:
        raise IndexError("lora_indices refers to an adapter that does not exist")
    x = _lib.as_device(x, dev, torch.float32)
    la = _lib.as_device(lora_a, dev, torch.float32)
    lb = _lib.as_device(lora_b, dev, torch.float32)
    idx = _lib.as_device(lora_indices, dev, torch.int32)
    rank, hidden = la.shape[1], la.shape[2]
    if x.shape != (B, T, hidden) or lb.shape[1:] != (Hq * D, rank) or idx.shape != (B,):
        raise ValueError("LoRA tensors must be x (B,T,hidden), lora_a (n,rank,hidden), lora_b (n,n_heads*128,rank), lora_indices (B,)")
    return x, la, lb, idx


def _apply_lora_to_q(q, x, lora_a, lora_b, lora_indices, lora_alpha):
    """q[b] += alpha * ((x[b] @ A[idx]^T) @ B[idx]^T) reshaped to heads; idx < 0 leaves the
    row untouched (reference :401-430; the fused prologue :166-191).  Runs ``omni_lora_q``; returns float32.
    Indices held on the host are range-checked here; indices already on the device are checked by the kernel,
    which reports through the device status word (``_lib.check_device_status`` raises ``IndexError``)."""
    B, Hq, T, D = q.shape
    dev = _lib.require_cuda(q)
    lib = _lib.ensure_init(dev)
    if q.dtype not in _lib.DTYPE_CODE:
        raise TypeError(f"unsupported q dtype {q.dtype}")
    q = q.contiguous()
    x = x.to(device=dev, dtype=torch.float32).contiguous()
    la = lora_a.to(device=dev, dtype=torch.float32).contiguous()
    lb = lora_b.to(device=dev, dtype=torch.float32).contiguous()
    if lora_indices.device.type == "cpu" and lora_indices.numel() and int(lora_indices.max()) >= lora_a.shape[0]:
        raise IndexError("lora_indices refers to an adapter that does not exist")
    idx = lora_indices.to(device=dev, dtype=torch.int32).contiguous()
    rank, hidden = la.shape[1], la.shape[2]
    if x.shape != (B, T, hidden) or lb.shape[1:] != (Hq * D, rank) or idx.shape != (B,):
        raise ValueError("LoRA tensors must be x (B,T,hidden), lora_a (n,rank,hidden), lora_b (n,n_heads*128,rank), lora_indices (B,)")
    out = torch.empty(B, Hq, T, D, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.omni_lora_q(_lib.ptr(q), _lib.DTYPE_CODE[q.dtype], _lib.ptr(x), _lib.ptr(la), _lib.ptr(lb),
                                   _lib.ptr(idx), la.shape[0], float(lora_alpha), B, Hq, T, hidden, rank, _lib.ptr(out),
                                   _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)))
    return out


def _auto_splits(B: int, Hq: int, Hkv: int, T: int, S: int) -> int:
    """Key-axis splits from the shape alone (measured on B200, 148 SMs x 12 warps).  A work unit of the
    tensor-core kernel is one (user, kv head, tile of 8 query columns); a unit costs a fixed prologue, so units
    are kept at 512 keys or more while there are enough of them (about 12,000: a few per resident warp, which
    also evens out ragged cache lengths) and shrink to 64 keys only to
    reach about 1,024 units when the call is small (few users, long caches)."""
    if S < 128 and B * Hq * T < 1024:
        return 1                                   # the lane-per-key kernel's shapes
    units = max(1, B * Hkv * -(-((Hq // Hkv) * T) // 8))
    splits = max(1, min(-(-12288 // units), S // 512))
    if units * splits < 1024:
        splits = max(splits, min(-(-1024 // units), S // 64))
    return int(max(1, min(splits, 1024)))


def _qattn(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl,
           seq_lens=None, cache_slots=None, rotate_q=False, unrotate_out=False, n_splits=None, lora=None):
    """One call of ``omni_qattn_decode_lora``; ``lora`` = (x, lora_a, lora_b, lora_indices, lora_alpha) or None."""
    dev = _lib.require_cuda(q, k_nibbles, k_qjl, k_norms, v_nibbles)
    lib = _lib.ensure_init(dev)
    B, Hq, T, D = q.shape
    if D != HEAD_DIM:
        raise ValueError(f"attention requires last dim = {HEAD_DIM} (head_dim), got {D}")
    n_slots, Hkv, S, _ = k_nibbles.shape
    if Hq % Hkv:
        raise ValueError(f"n_heads={Hq} is not a multiple of n_kv_heads={Hkv}")
    if cache_slots is None and n_slots != B:
        raise ValueError(f"cache holds {n_slots} users but q has batch {B}")
    if q.dtype not in _lib.DTYPE_CODE:
        raise TypeError(f"unsupported q dtype {q.dtype}")
    q = q.contiguous()
    k_nibbles, k_qjl, v_nibbles = k_nibbles.contiguous(), k_qjl.contiguous(), v_nibbles.contiguous()
    k_norms = _lib.as_device(k_norms, dev, torch.float32)
    cb, per_head = _prep_codebooks(codebooks, Hkv, dev)
    ids, uid = _user_args(user_id, B, dev)
    lens = None if seq_lens is None else _lib.as_device(seq_lens, dev, torch.int32)
    slots = None if cache_slots is None else _lib.as_device(cache_slots, dev, torch.int32)
    if n_splits is None:
        n_splits = _auto_splits(B, Hq, Hkv, T, S)
    ws, ws_bytes, lora_arg = None, 0, None
    if lora is not None:
        x, la, lb, idx = _prep_lora(q, lora[0], lora[1], lora[2], lora[3], dev)
        lora_arg = C.byref(_lib.OmniLora(x.data_ptr(), la.data_ptr(), lb.data_ptr(), idx.data_ptr(), la.shape[0],
                                         la.shape[2], la.shape[1], float(lora[4])))
        ws_bytes = lib.omni_qattn_lora_workspace_bytes(B, Hq, T, n_splits)
    elif n_splits > 1:
        ws_bytes = lib.omni_qattn_workspace_bytes(B, Hq, T, n_splits)
    stream = _lib.stream_ptr(dev)
    if ws_bytes:
        ws = _lib.workspace(dev, stream, ws_bytes)
    out = torch.empty(B, Hq, T, HEAD_DIM, dtype=torch.float32, device=dev)
    with _lib.on_device(dev):
        _lib.check(lib.omni_qattn_decode_lora(
            _lib.ptr(q), _lib.DTYPE_CODE[q.dtype], _lib.ptr(k_nibbles), _lib.ptr(k_qjl), _lib.ptr(k_norms),
            _lib.ptr(v_nibbles), _lib.ptr(cb), per_head, _lib.ptr(ids), uid, _lib.ptr(lens), _lib.ptr(slots),
            B, Hq, Hkv, T, S, Hkv * S, S, float(scale), int(bool(with_qjl)), int(bool(rotate_q)),
            int(bool(unrotate_out)), int(n_splits), _lib.ptr(ws), ws_bytes, _lib.ptr(out), _lib.ptr(_lib.status_word(dev)),
            stream, lora_arg))
    return out


class OmniAttention(torch.autograd.Function):
    """Forward-only wrapper with the reference's argument list (inference path: the
    backward returns ``None`` for all 15 inputs, reference :530-534)."""

    @staticmethod
    def forward(ctx, q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl,
                g_matrix=None, x=None, lora_a=None, lora_b=None, lora_indices=None, lora_alpha=1.0):
        if scale is None:
            scale = 1.0 / math.sqrt(HEAD_DIM)
        lora = None if x is None else (x, lora_a, lora_b, lora_indices, lora_alpha)
        out = _qattn(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl, lora=lora)
        ctx.save_for_backward(q, out)
        ctx.scale, ctx.with_qjl = scale, with_qjl
        return out

    @staticmethod
    def backward(ctx, grad_out):
        return (None,) * 15


def omni_attn(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id=0, scale: Optional[float] = None,
              with_qjl: bool = True, g_matrix=None, x=None, lora_a=None, lora_b=None, lora_indices=None,
              lora_alpha: float = 1.0, *, seq_lens=None, cache_slots=None, rotate_q: bool = False,
              unrotate_out: bool = False, n_splits: Optional[int] = None) -> torch.Tensor:
    """Fused INT4 + QJL attention with the optional per-user LoRA query update."""
    plain = seq_lens is None and cache_slots is None and not rotate_q and not unrotate_out and n_splits is None
    if plain and torch.is_grad_enabled() and q.requires_grad:          # only then does the autograd node matter
        return OmniAttention.apply(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl,
                                   g_matrix, x, lora_a, lora_b, lora_indices, lora_alpha)
    if scale is None:
        scale = 1.0 / math.sqrt(HEAD_DIM)
    lora = None if x is None else (x, lora_a, lora_b, lora_indices, lora_alpha)
    return _qattn(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl,
                  seq_lens, cache_slots, rotate_q, unrotate_out, n_splits, lora)
