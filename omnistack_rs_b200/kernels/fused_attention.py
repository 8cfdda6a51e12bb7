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
import functools
import math
import weakref
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


_SPLIT_CANDIDATES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)
_WARP_SLOTS = _SM_COUNT * 12


@functools.lru_cache(maxsize=4096)
def _auto_splits(B: int, Hq: int, Hkv: int, T: int, S: int, ragged: bool = False) -> int:
    """Key-axis splits from the shape alone: the candidate with the lowest modelled time.  The model (fitted to a
    sweep over 1-256 users and 2 K-32 K keys on B200; its pick is within 10 % of the best measured split count
    for every swept shape): a work unit of the tensor-core kernel - one (user, kv head, tile of 8 query columns,
    split) - costs about 3 us plus 22 ns per key when it has an SM to itself, rising to 45 ns per key with
    twelve warps per SM; units run in rounds of 148 x 12; the merge costs 2 us plus its bytes at 1 TB/s.
    ``ragged`` (per-user cache lengths were given): at least 8 splits of 512 keys or more (4 where the library
    orders the users by length), so that the ticket scheduling can even the lengths out, unless every warp has many
    units anyway."""
    if S < 128 and B * Hq * T < 1024:
        return 1                                   # the lane-per-key kernel's shapes
    units = max(1, B * Hkv * -(-((Hq // Hkv) * T) // 8))
    rows = B * Hq * T
    best, best_cost, unsplit_cost = 1, float("inf"), float("inf")
    for s in _SPLIT_CANDIDATES:
        if s > 1 and S // s < 64:
            break
        n = units * s
        active = min(12.0, max(1.0, n / _SM_COUNT))
        ns_per_key = 22.0 + 23.0 * (active - 1.0) / 11.0
        rounds = math.ceil(n / _WARP_SLOTS) if n <= 2 * _WARP_SLOTS else n / _WARP_SLOTS + 0.5
        cost = rounds * (3.0 + (S / s) * ns_per_key * 1e-3)
        if s > 1:
            cost += 2.0 + rows * s * 528 / 1e6
        if s == 1:
            unsplit_cost = cost
        if cost < best_cost:
            best, best_cost = s, cost
    # the model is least certain about the fixed cost of a unit on a busy SM: split only for a clear gain
    if best_cost >= 0.8 * unsplit_cost:
        best = 1
    if ragged and units < 8 * _WARP_SLOTS:
        # calls the library serves longest user first (several query columns per kv head, enough work items for its
        # preparation launch, at most 16,384 users) balance with coarser splits: measured on configuration 2,
        # 0.310-0.312 ms with 3 to 6 splits against 0.317 with 8
        ordered = 1 < B <= 16384 and (Hq // Hkv) * T > 1 and units * 4 >= 2 * _WARP_SLOTS
        best = max(best, min(4 if ordered else 8, S // 512))
    return best


class _DecodeCall:
    """One ``omni_qattn_decode_lora`` call with everything that stays the same between calls on the same cache
    already checked and converted: devices, shapes, dtypes, contiguity, the split count, the workspace size and
    the C arguments of the cache, the codebooks and the flags.  ``run`` supplies what changes per call (the query,
    the LoRA inputs, the stream, the output)."""

    __slots__ = ("dev", "dev_index", "fn", "q_shape", "q_dtype", "q_code", "mid_args", "ws_bytes", "status_ptr",
                 "lora_const", "keep", "refs", "ptrs")

    def run(self, q, lora):
        dev = self.dev
        if q.device != dev:
            _lib.require_cuda(q)
            raise ValueError(f"tensors on different devices: {dev} and {q.device}")
        if not q.is_contiguous():
            q = q.contiguous()
        stream = torch._C._cuda_getCurrentRawStream(self.dev_index) or None
        ws_ptr = None
        if self.ws_bytes:
            ws = _lib.workspace(dev, stream, self.ws_bytes)
            ws_ptr = ws.data_ptr()
        lora_arg = None
        if self.lora_const is not None:
            la, lb, n_adapters, hidden, rank, alpha = self.lora_const
            if la is None:                                  # a kept entry: the caller's own (checked) adapter stacks
                la, lb = lora[1], lora[2]
            x, idx = lora[0], lora[3]
            if idx.device.type == "cpu" and idx.numel() and int(idx.max()) >= n_adapters:
                raise IndexError("lora_indices refers to an adapter that does not exist")
            x = _lib.as_device(x, dev, torch.float32)
            idx = _lib.as_device(idx, dev, torch.int32)
            B, _, T = self.q_shape[:3]
            if x.shape != (B, T, hidden) or idx.shape != (B,):
                raise ValueError("LoRA tensors must be x (B,T,hidden), lora_a (n,rank,hidden), lora_b (n,n_heads*128,rank), lora_indices (B,)")
            lora_arg = C.byref(_lib.OmniLora(x.data_ptr(), la.data_ptr(), lb.data_ptr(), idx.data_ptr(), n_adapters,
                                             hidden, rank, alpha))
        out = torch.empty(self.q_shape, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            _lib.check(self.fn(q.data_ptr(), self.q_code, *self.mid_args, ws_ptr, self.ws_bytes, out.data_ptr(),
                               self.status_ptr, stream, lora_arg))
        return out


# Prepared calls of the most recent (cache tensors, query shape, flags) combinations.  An entry refers to its tensors
# weakly and is used only while those very objects are alive and their storage is where it was, so it neither keeps
# a dropped cache in memory nor survives a recycled ``id``.
_PLANS: dict = {}
_MAX_PLANS = 64


def clear_prepared_calls() -> None:
    """Forget the prepared decode calls (they are rebuilt on demand)."""
    _PLANS.clear()


def _plan_key(q, tensors, user_id, scale, flags, n_splits, lora):
    return (tuple(id(t) for t in tensors), tensors[0].shape, q.shape, q.dtype,
            user_id if not isinstance(user_id, torch.Tensor) else None, scale, flags, n_splits,
            None if lora is None else float(lora[4]))


def _build_call(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl, seq_lens, cache_slots,
                rotate_q, unrotate_out, n_splits, lora, v_paired):
    """Checks and conversions of one decode call; returns the call and whether it may be kept for later calls
    (only when no argument had to be converted: a converted copy would not follow the caller's tensor)."""
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
    given = [k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, seq_lens, cache_slots]
    k_nibbles, k_qjl, v_nibbles = k_nibbles.contiguous(), k_qjl.contiguous(), v_nibbles.contiguous()
    k_norms = _lib.as_device(k_norms, dev, torch.float32)
    cb, per_head = _prep_codebooks(codebooks, Hkv, dev)
    if isinstance(user_id, torch.Tensor) and user_id.dtype is torch.int32 and user_id.device == dev and user_id.is_contiguous():
        if user_id.shape != (B,):
            raise ValueError(f"user_id tensor must have shape ({B},), got {tuple(user_id.shape)}")
        ids, uid = user_id, 0
    else:
        ids, uid = _user_args(user_id, B, dev)
    lens = None if seq_lens is None else _lib.as_device(seq_lens, dev, torch.int32)
    slots = None if cache_slots is None else _lib.as_device(cache_slots, dev, torch.int32)
    used = [k_nibbles, k_qjl, k_norms, v_nibbles, cb, ids if isinstance(user_id, torch.Tensor) else user_id, lens, slots]
    keepable = all(g is u for g, u in zip(given, used))
    if n_splits is None:
        n_splits = _auto_splits(B, Hq, Hkv, T, S, seq_lens is not None)
    call = _DecodeCall()
    call.lora_const = None
    ws_bytes = 0
    if lora is not None:
        x, la, lb, idx = _prep_lora(q, lora[0], lora[1], lora[2], lora[3], dev)
        keepable = keepable and la is lora[1] and lb is lora[2]
        call.lora_const = (la, lb, la.shape[0], la.shape[2], la.shape[1], float(lora[4]))
        ws_bytes = lib.omni_qattn_lora_workspace_bytes(B, Hq, T, n_splits)
    elif n_splits > 1:
        ws_bytes = lib.omni_qattn_workspace_bytes(B, Hq, T, n_splits)
    call.dev = dev
    call.dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
    call.fn = lib.omni_qattn_decode_lora
    call.q_shape, call.q_dtype, call.q_code = q.shape, q.dtype, _lib.DTYPE_CODE[q.dtype]
    call.mid_args = (_lib.ptr(k_nibbles), _lib.ptr(k_qjl), _lib.ptr(k_norms), _lib.ptr(v_nibbles), _lib.ptr(cb), per_head,
                     _lib.ptr(ids), uid, _lib.ptr(lens), _lib.ptr(slots), B, Hq, Hkv, T, S, Hkv * S, S, float(scale),
                     int(bool(with_qjl)), int(bool(rotate_q)), int(bool(unrotate_out)), int(bool(v_paired)), int(n_splits))
    call.ws_bytes = ws_bytes
    call.status_ptr = _lib.ptr(_lib.status_word(dev))
    call.keep = (k_nibbles, k_qjl, k_norms, v_nibbles, cb, ids, lens, slots)     # alive for the duration of this call
    return call, keepable


def _qattn(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl,
           seq_lens=None, cache_slots=None, rotate_q=False, unrotate_out=False, n_splits=None, lora=None,
           v_paired=False):
    """One call of ``omni_qattn_decode_lora``; ``lora`` = (x, lora_a, lora_b, lora_indices, lora_alpha) or None.
    ``v_paired``: the V nibble rows are in the pair layout of :func:`pair_v_rows` (a resident cache's own format).
    Calls that repeat on the same cache tensors (a serving loop) reuse the checked and converted argument block of
    the first one; only the query, the LoRA inputs, the stream and the output are handled per call."""
    tensors = [k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, seq_lens, cache_slots]
    if isinstance(user_id, torch.Tensor):
        tensors.append(user_id)
    if lora is not None:
        tensors += [lora[1], lora[2]]
    flags = (bool(with_qjl), bool(rotate_q), bool(unrotate_out), bool(v_paired))
    key = _plan_key(q, tensors, user_id, scale, flags, n_splits, lora)
    hit = _PLANS.get(key)
    if hit is not None:
        for t, r, p in zip(tensors, hit.refs, hit.ptrs):
            if t is None:
                if r is not None:
                    break
            elif r is None or r() is not t or t.data_ptr() != p:
                break
        else:
            return hit.run(q, lora)
        _PLANS.pop(key, None)
    call, keepable = _build_call(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl, seq_lens,
                                 cache_slots, rotate_q, unrotate_out, n_splits, lora, v_paired)
    out = call.run(q, lora)
    if keepable:
        call.refs = tuple(None if t is None else weakref.ref(t) for t in tensors)
        call.ptrs = tuple(None if t is None else t.data_ptr() for t in tensors)
        call.keep = None                                    # the entry must not keep the caller's cache alive
        if call.lora_const is not None:                     # nor the adapter stacks: re-read through the weak references
            call.lora_const = (None, None) + call.lora_const[2:]
        if len(_PLANS) >= _MAX_PLANS:
            _PLANS.pop(next(iter(_PLANS)), None)
        _PLANS[key] = call
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
              unrotate_out: bool = False, n_splits: Optional[int] = None, v_paired: bool = False) -> torch.Tensor:
    """Fused INT4 + QJL attention with the optional per-user LoRA query update."""
    plain = (seq_lens is None and cache_slots is None and not rotate_q and not unrotate_out and n_splits is None
             and not v_paired)
    if plain and torch.is_grad_enabled() and q.requires_grad:          # only then does the autograd node matter
        return OmniAttention.apply(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl,
                                   g_matrix, x, lora_a, lora_b, lora_indices, lora_alpha)
    if scale is None:
        scale = 1.0 / math.sqrt(HEAD_DIM)
    lora = None if x is None else (x, lora_a, lora_b, lora_indices, lora_alpha)
    return _qattn(q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, scale, with_qjl,
                  seq_lens, cache_slots, rotate_q, unrotate_out, n_splits, lora, v_paired)


def pair_v_rows(v_nibbles: torch.Tensor, lens_before=0, lens_after=None) -> None:
    """Convert, in place, the V nibble rows ``(n_users, n_kv_heads, S, 64)`` of a resident cache to the pair layout
    the tensor-core kernel reads without a shift-and-merge per lookup (``omni_v_pair_groups``): the groups of eight
    keys that became complete when the users' lengths grew from ``lens_before`` to ``lens_after`` (ints, or int64
    tensors of shape (n_users,); ``lens_after=None`` means the full capacity S).  Applying it again to the same
    groups restores the reference layout."""
    dev = _lib.require_cuda(v_nibbles)
    lib = _lib.ensure_init(dev)
    if not v_nibbles.is_contiguous():
        raise ValueError("the cache's nibble array must be contiguous")
    B, H, S, _ = v_nibbles.shape
    if lens_after is None:
        lens_after = S
    tensors = isinstance(lens_before, torch.Tensor) or isinstance(lens_after, torch.Tensor)
    if tensors:
        before = torch.as_tensor(lens_before, device=dev).to(torch.int64).expand(B).contiguous()
        after = torch.as_tensor(lens_after, device=dev).to(torch.int64).expand(B).contiguous()
        args = (_lib.ptr(before), 0, _lib.ptr(after), 0)
    else:
        args = (None, int(lens_before), None, int(lens_after))
    with _lib.on_device(dev):
        _lib.check(lib.omni_v_pair_groups(_lib.ptr(v_nibbles), B, H, S, H * S, S, *args, _lib.stream_ptr(dev)))
