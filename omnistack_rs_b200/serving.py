"""Per-user cache container, user sharding across GPUs, and the host-buffer decode step.

The reference has no cache object (its README lists a paged cache as planned) and no
multi-GPU code; its serving loop (scripts/run_criteo_benchmark.py:481-560) keeps the packed
tensors resident on one GPU and sends a fresh query per step.  This module provides the same
loop for one process per GPU: users are independent, so rank r of n simply owns a contiguous
block of users and no collective is needed on the data path.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import _lib
from .kernels.quantize import _NBYTES_NIBBLE, _NBYTES_QJL, _prep_codebooks, rotate_quantize_append
from .kernels.fused_attention import _qattn, _auto_splits, pair_v_rows

HEAD_DIM = 128


def shard_range(n_units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous block [begin, end) of ``n_units`` owned by ``rank``; the first
    ``n_units % world_size`` ranks get one extra unit."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(n_units, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_rows_to_rank0(local: torch.Tensor, n_units: int, group=None) -> Optional[torch.Tensor]:
    """Gather per-rank row blocks (sharded with :func:`shard_range`) to rank 0 in user order.
    Blocks are padded to a common height because ``gather`` needs equal shapes.  Returns the
    ``(n_units, ...)`` tensor on rank 0 and ``None`` elsewhere.  Verification only -- the
    data path itself has no collective."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    spans = [shard_range(n_units, world, r) for r in range(world)]
    height = max(e - b for b, e in spans)
    padded = local.new_zeros((height,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    bufs = [torch.empty_like(padded) for _ in range(world)] if rank == 0 else None
    dist.gather(padded, bufs, dst=0, group=group)
    if rank != 0:
        return None
    return torch.cat([buf[: e - b] for buf, (b, e) in zip(bufs, spans)])


class ShardLiveness:
    """Host-side liveness record of the ranks of a sharded serving job, kept in a key-value store
    (``torch.distributed.TCPStore`` or any object with ``set`` / ``get`` / ``check``).  The data path has no
    collective, so a rank that stops cannot hang its peers; this record is how they learn of it before they next
    depend on that rank (a verification gather, a barrier): every rank posts the number of the step it has
    finished, and a rank that leaves on purpose says so.  Nothing here touches a GPU."""

    def __init__(self, store, rank: int, world_size: int):
        self.store, self.rank, self.world = store, rank, world_size

    def beat(self, step: int) -> None:
        self.store.set(f"omni/beat/{self.rank}", str(int(step)))

    def leave(self) -> None:
        self.store.set(f"omni/left/{self.rank}", "1")

    def _step_of(self, r: int) -> int:
        key = f"omni/beat/{r}"
        return int(self.store.get(key)) if self.store.check([key]) else -1

    def missing(self, step: int, timeout_s: float = 2.0, poll_s: float = 0.02):
        """Ranks that have not finished ``step`` within ``timeout_s`` (or announced that they left)."""
        import time
        deadline = time.monotonic() + timeout_s
        waiting = [r for r in range(self.world) if r != self.rank]
        gone = []
        while waiting:
            for r in list(waiting):
                if self.store.check([f"omni/left/{r}"]):
                    waiting.remove(r); gone.append(r)
                elif self._step_of(r) >= step:
                    waiting.remove(r)
            if not waiting or time.monotonic() >= deadline:
                break
            time.sleep(poll_s)
        return sorted(gone + waiting)


def collect_rows_via_store(store, rank: int, world_size: int, local: torch.Tensor, n_units: int, missing=()):
    """Verification gather that survives absent ranks: every live rank posts its row block (sharded with
    :func:`shard_range`) to the store and rank 0 assembles them.  Returns, on rank 0,
    ``(rows, missing_spans)`` -- the ``(n_units, ...)`` tensor with the rows of absent ranks left at zero and
    the ``[begin, end)`` unit ranges nobody delivered -- and ``None`` elsewhere."""
    import io
    if rank != 0:
        buf = io.BytesIO()
        torch.save(local.cpu(), buf)
        store.set(f"omni/rows/{rank}", buf.getvalue())
        return None
    rows = local.new_zeros((n_units,) + tuple(local.shape[1:]), device="cpu")
    b0, e0 = shard_range(n_units, world_size, 0)
    rows[b0:e0] = local.cpu()
    missing_spans = []
    for r in range(1, world_size):
        b, e = shard_range(n_units, world_size, r)
        if r in missing:
            missing_spans.append((b, e))
            continue
        rows[b:e] = torch.load(io.BytesIO(store.get(f"omni/rows/{r}")))
    return rows, missing_spans


class QuantizedKVCache:
    """Preallocated packed K/V cache for ``n_users`` users on one device.

    K rows hold nibbles + sign bytes + norm (4.75 bits per element); V rows are stored the
    same way (the codec produces all three) although attention reads only V's nibbles.
    """

    def __init__(self, n_users: int, n_kv_heads: int, max_len: int, codebooks: torch.Tensor,
                 device, user_ids: Optional[torch.Tensor] = None, store_v_residual: bool = True,
                 pair_v: bool = False):
        self.device = torch.device(device)
        self.n_users, self.n_kv_heads, self.max_len = n_users, n_kv_heads, max_len
        self.codebooks = codebooks.to(device=self.device, dtype=torch.float32).contiguous()
        shape = (n_users, n_kv_heads, max_len)
        mk = lambda *s, dt=torch.uint8: torch.zeros(*s, dtype=dt, device=self.device)  # noqa: E731
        self.k_nib, self.k_qjl, self.k_norms = mk(*shape, _NBYTES_NIBBLE), mk(*shape, _NBYTES_QJL), mk(*shape, dt=torch.float32)
        self.v_nib = mk(*shape, _NBYTES_NIBBLE)
        if store_v_residual:
            self.v_qjl, self.v_norms = mk(*shape, _NBYTES_QJL), mk(*shape, dt=torch.float32)
        else:   # attention never reads V's sign bits or norms: they are neither stored nor computed
            self.v_qjl = self.v_norms = None
        # pair_v: V nibble rows are kept in the pair layout the tensor-core kernel reads fastest; every append
        # converts the groups of eight keys it completes (``v_nib`` is then not interchangeable with the reference's)
        self.pair_v = bool(pair_v)
        self.lens = torch.zeros(n_users, dtype=torch.int64, device=self.device)
        # the same lengths as the attention entry points take them (int32, same storage for the cache's lifetime, so
        # repeated ``attend`` calls reuse one prepared call)
        self.lens32 = torch.zeros(n_users, dtype=torch.int32, device=self.device)
        self.user_ids = (torch.arange(n_users, dtype=torch.int32, device=self.device) if user_ids is None
                         else user_ids.to(device=self.device, dtype=torch.int32).contiguous())

    def bytes_per_key(self) -> int:
        return 2 * (_NBYTES_NIBBLE + _NBYTES_QJL + 4) if self.v_qjl is not None else 2 * _NBYTES_NIBBLE + _NBYTES_QJL + 4

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor, rotate: bool = True) -> None:
        """Quantize-append ``(n_users, n_kv_heads, T_new, 128)`` keys and values for every
        user at its current length."""
        T = k_new.shape[2]
        if int(self.lens.max()) + T > self.max_len:
            raise ValueError("append would run past the cache capacity")
        rotate_quantize_append(k_new, self.k_nib, self.k_qjl, self.k_norms, self.lens, self.codebooks,
                               self.user_ids, rotate=rotate)
        rotate_quantize_append(v_new, self.v_nib, self.v_qjl, self.v_norms, self.lens, self.codebooks,
                               self.user_ids, rotate=rotate)
        if self.pair_v:
            pair_v_rows(self.v_nib, self.lens, self.lens + T)
        self.lens += T
        self.lens32.copy_(self.lens)

    def attend(self, q: torch.Tensor, scale: Optional[float] = None, with_qjl: bool = True,
               rotate_q: bool = False, unrotate_out: bool = False, n_splits: Optional[int] = None) -> torch.Tensor:
        """Decode attention of ``q`` (n_users, n_heads, T, 128) against each user's valid prefix."""
        if scale is None:
            scale = 1.0 / math.sqrt(HEAD_DIM)
        return _qattn(q, self.k_nib, self.k_qjl, self.k_norms, self.v_nib, self.codebooks, self.user_ids, scale,
                      with_qjl, seq_lens=self.lens32, rotate_q=rotate_q, unrotate_out=unrotate_out, n_splits=n_splits,
                      v_paired=self.pair_v)


class HostDecodeStep:
    """One serving step with HOST buffers (``omni_qattn_decode_host``): the query comes from host memory, the fused
    attention runs over the resident cache, the result lands in page-locked host memory.  With a page-locked query
    tensor the kernels read and write the host buffers themselves (``mode == "direct"``: the transfer overlaps the
    attention work, one launch); a pageable query tensor is staged through device buffers in user chunks whose
    copies and kernels overlap on two internal streams (``"staged"``; ``OMNI_HOST_STEP=staged`` forces it).  The
    cache tensors must be complete before the first call (the internal streams do not wait on the caller's
    stream)."""

    def __init__(self, k_nib, k_qjl, k_norms, v_nib, codebooks, n_heads: int, batch: int, q_dtype=torch.bfloat16,
                 user_id=0, seq_lens=None, cache_slots=None, scale: Optional[float] = None, with_qjl: bool = True,
                 T: int = 1, n_chunks: Optional[int] = None, n_splits: Optional[int] = None, v_paired: bool = False):
        self.dev = _lib.require_cuda(k_nib, k_qjl, k_norms, v_nib)
        self.lib = _lib.ensure_init(self.dev)
        self.k_nib, self.k_qjl, self.k_norms, self.v_nib = k_nib, k_qjl, k_norms, v_nib
        n_slots, self.Hkv, self.S, _ = k_nib.shape
        if cache_slots is None and n_slots != batch:
            raise ValueError(f"cache holds {n_slots} users but the step batch is {batch}")
        self.cb, self.per_head = _prep_codebooks(codebooks, self.Hkv, self.dev)
        self.B, self.Hq, self.T, self.q_dtype = batch, n_heads, T, q_dtype
        if isinstance(user_id, torch.Tensor):
            self.ids, self.uid = user_id.to(device=self.dev, dtype=torch.int32).contiguous(), 0
        else:
            self.ids, self.uid = None, int(user_id) % 1024
        self.lens = None if seq_lens is None else seq_lens.to(device=self.dev, dtype=torch.int32).contiguous()
        self.slots = None if cache_slots is None else cache_slots.to(device=self.dev, dtype=torch.int32).contiguous()
        self.scale = float(scale if scale is not None else 1.0 / math.sqrt(HEAD_DIM))
        if n_chunks is None:                       # chunks of at least ~2k users keep every SM busy
            n_chunks = max(1, min(8, batch // 2048))
        self.with_qjl, self.n_chunks, self.v_paired = int(bool(with_qjl)), int(n_chunks), int(bool(v_paired))
        per_chunk = -(-batch // self.n_chunks)
        self.n_splits = int(n_splits) if n_splits is not None else _auto_splits(per_chunk, n_heads, self.Hkv, T, self.S, seq_lens is not None)
        self.ws_bytes = 2 * self.lib.omni_qattn_workspace_bytes(per_chunk, n_heads, T, self.n_splits)
        self.ws = torch.empty(max(self.ws_bytes // 4, 1), dtype=torch.float32, device=self.dev)
        shape = (batch, n_heads, T, HEAD_DIM)
        self.q_stage = self.out_stage = None            # device staging: allocated when a step first needs it
        self.mode = None                                # "direct" / "staged": how the last step moved its data
        self.q_host = torch.empty(shape, dtype=q_dtype).pin_memory()
        self.out_host = torch.empty(shape, dtype=torch.float32).pin_memory()
        self.h2d_bytes = self.q_host.numel() * self.q_host.element_size()
        self.d2h_bytes = self.out_host.numel() * 4
        torch.cuda.synchronize(self.dev)

    def step(self, q_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs one step; returns the pinned host result tensor (overwritten by the next step)."""
        src = self.q_host if q_host is None else q_host
        if src.is_cuda or src.shape != self.q_host.shape or src.dtype != self.q_dtype or not src.is_contiguous():
            raise ValueError("q_host must be a contiguous CPU tensor of the step's shape and dtype")
        direct = src.is_pinned() and not os.environ.get("OMNI_HOST_STEP", "").startswith("s")
        self.mode = "direct" if direct else "staged"
        if not direct and self.q_stage is None:
            self.q_stage = torch.empty(self.q_host.shape, dtype=self.q_dtype, device=self.dev)
            self.out_stage = torch.empty(self.q_host.shape, dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            _lib.check(self.lib.omni_qattn_decode_host(
                _lib.ptr(src), _lib.DTYPE_CODE[self.q_dtype], _lib.ptr(self.q_stage),
                _lib.ptr(self.k_nib), _lib.ptr(self.k_qjl), _lib.ptr(self.k_norms), _lib.ptr(self.v_nib),
                _lib.ptr(self.cb), self.per_head, _lib.ptr(self.ids), self.uid, _lib.ptr(self.lens), _lib.ptr(self.slots),
                self.B, self.Hq, self.Hkv, self.T, self.S, self.Hkv * self.S, self.S, self.scale, self.with_qjl,
                self.v_paired, _lib.ptr(self.out_stage), _lib.ptr(self.out_host), self.n_chunks,
                self.n_splits, _lib.ptr(self.ws), self.ws_bytes, _lib.ptr(_lib.status_word(self.dev))))
        return self.out_host


class GraphedAttention:
    """``omni_attn`` on fixed device buffers, captured once into a CUDA graph and replayed per query.

    Small decode calls (the reference benchmark's 64-user query is 20 us of device work behind about as much host
    work: Python, two or three kernel launches) are bound by the host when issued one by one; a replayed graph costs
    one launch.  The query (and, with adapters, the hidden state and adapter indices) lives in buffers owned by this
    object: write into ``q`` / ``x`` / ``lora_indices`` (or pass tensors to ``__call__``, which copies them in) and
    read the result from ``out``, which the next replay overwrites.  Everything else -- cache tensors, codebooks,
    per-user lengths, adapter stacks -- is captured by address, so in-place changes of their contents are seen and the
    tensors must stay alive (this object keeps references)."""

    def __init__(self, q_shape, q_dtype, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id=0, *, hidden=None,
                 lora_a=None, lora_b=None, lora_alpha: float = 1.0, **attn_kwargs):
        from .kernels.fused_attention import omni_attn
        dev = _lib.require_cuda(k_nibbles, k_qjl, k_norms, v_nibbles)
        # a replay reads the addresses the capture saw: an argument the call would have to convert (other device,
        # dtype or layout) would be captured as a temporary copy, so every tensor must already be in its final form
        final = [("k_nibbles", k_nibbles, torch.uint8), ("k_qjl", k_qjl, torch.uint8), ("k_norms", k_norms, torch.float32),
                 ("v_nibbles", v_nibbles, torch.uint8), ("codebooks", codebooks, torch.float32),
                 ("lora_a", lora_a, torch.float32), ("lora_b", lora_b, torch.float32),
                 ("seq_lens", attn_kwargs.get("seq_lens"), torch.int32), ("cache_slots", attn_kwargs.get("cache_slots"), torch.int32),
                 ("user_id", user_id if isinstance(user_id, torch.Tensor) else None, torch.int32)]
        for name, t, dt in final:
            if t is not None and not (t.device == dev and t.dtype is dt and t.is_contiguous()):
                raise ValueError(f"GraphedAttention: {name} must be a contiguous {dt} tensor on {dev}")
        B, _, T, _ = q_shape
        self.q = torch.zeros(q_shape, dtype=q_dtype, device=dev)
        self.x = self.lora_indices = None
        lora = {}
        if lora_a is not None:
            self.x = torch.zeros(B, T, lora_a.shape[2] if hidden is None else hidden, dtype=torch.float32, device=dev)
            self.lora_indices = torch.full((B,), -1, dtype=torch.int32, device=dev)
            lora = dict(x=self.x, lora_a=lora_a, lora_b=lora_b, lora_indices=self.lora_indices, lora_alpha=lora_alpha)
        self._keep = (k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id, lora_a, lora_b, attn_kwargs)

        def call():
            return omni_attn(self.q, k_nibbles, k_qjl, k_norms, v_nibbles, codebooks, user_id=user_id, **lora, **attn_kwargs)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):                      # first-call set-up (kernel attributes, tensor maps, workspace) is not captured
                call()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = call()

    def __call__(self, q=None, x=None, lora_indices=None) -> torch.Tensor:
        if q is not None:
            self.q.copy_(q, non_blocking=True)
        if x is not None:
            self.x.copy_(x, non_blocking=True)
        if lora_indices is not None:
            self.lora_indices.copy_(lora_indices, non_blocking=True)
        self.graph.replay()
        return self.out
