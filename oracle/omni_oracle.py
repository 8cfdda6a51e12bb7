"""CPU restatement of the OmniStack-RS KV codec and quantized decode attention.

TEST INFRASTRUCTURE ONLY -- this module is the parity checker and the timed
CPU baseline; it is never imported by the shipped package.

Every function states which reference routine (path inside the reference
project : line) it restates.  The restatement is pinned against the reference
itself: ``tests/golden/make_golden.py`` imports the reference's CPU (torch)
path, runs it on seeded inputs and stores the results under ``tests/golden``;
``tests/test_oracle_golden.py`` replays this module against those files and
against the reference tests' known-answer vectors.

Arithmetic conventions that matter for bit-exactness (all restated from the
reference):
  * the rotation is the in-order radix-2 butterfly (h = 1, 2, ..., 64) in fp32
    followed by ONE fp32 multiply by float32(1/sqrt(128)); a bf16/fp16 input is
    rounded back to its dtype afterwards;
  * the INT4 code is the FIRST index minimising |y - c| evaluated in fp32;
  * the Rademacher matrix comes from MT19937 seeded with
    ``(user_id mod 1024) xor head`` -- element (i, d) is the least significant
    bit of draw number 128*i + d;
  * a projection that is exactly zero (or -0.0) yields sign bit 1.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

HEAD_DIM = 128
QJL_DIM = 64
N_CENTROIDS = 16
NIB_BYTES = HEAD_DIM // 2
QJL_BYTES = QJL_DIM // 8
#: fp32 value of 1/sqrt(128) used by the rotation (kernels/hadamard.py:46,85)
WHT_SCALE = float(np.float32(1.0 / math.sqrt(HEAD_DIM)))
#: sqrt(2/pi)/128, the QJL reconstruction coefficient (kernels/quantize.py:450)
QJL_COEF = math.sqrt(2.0 / math.pi) / HEAD_DIM

__all__ = [
    "HEAD_DIM", "QJL_DIM", "N_CENTROIDS", "NIB_BYTES", "QJL_BYTES", "WHT_SCALE", "QJL_COEF",
    "mt19937_draws", "qjl_seed", "rademacher_bits", "rademacher_matrix", "pack_g_words",
    "wht128", "nearest_centroid", "pack_nibbles", "unpack_nibbles", "pack_sign_bits",
    "unpack_sign_bits", "quantize_heads", "dequantize_heads", "quantize_rows", "dequantize_rows",
    "rotate_quantize", "sign_ambiguity", "repeat_kv", "attention", "decode_attention",
    "apply_lora_to_q", "lloyd_max_fit", "lloyd_max_per_group",
]


# --------------------------------------------------------------------------- #
# MT19937 and the Rademacher matrix
# --------------------------------------------------------------------------- #

def mt19937_draws(seed: int, n: int) -> np.ndarray:
    """First ``n`` 32-bit outputs of MT19937 after ``init_genrand(seed)``.

    This is the generator behind ``torch.Generator().manual_seed(seed)`` on the
    CPU, which the reference uses to draw G (kernels/quantize.py:410-414,
    quantization/qjl.py:71-76).  Third-party algorithm (Matsumoto & Nishimura,
    1998); restated from its published description.
    """
    N, M = 624, 397
    mt = np.empty(N, dtype=np.uint64)
    mt[0] = seed & 0xFFFFFFFF
    for i in range(1, N):
        prev = int(mt[i - 1])
        mt[i] = (1812433253 * (prev ^ (prev >> 30)) + i) & 0xFFFFFFFF
    mt = mt.astype(np.uint32)
    out = np.empty(((n + N - 1) // N) * N, dtype=np.uint32)
    UPPER, LOWER, MAG = np.uint32(0x80000000), np.uint32(0x7FFFFFFF), np.uint32(0x9908B0DF)

    def twist(cur, nxt, far):
        y = (cur & UPPER) | (nxt & LOWER)
        return far ^ (y >> np.uint32(1)) ^ np.where(y & np.uint32(1), MAG, np.uint32(0))

    for blk in range(out.size // N):
        # the in-place update is done in dependency-respecting slabs
        mt[0:227] = twist(mt[0:227], mt[1:228], mt[397:624])
        mt[227:454] = twist(mt[227:454], mt[228:455], mt[0:227])
        mt[454:623] = twist(mt[454:623], mt[455:624], mt[227:396])
        mt[623] = twist(mt[623:624], mt[0:1], mt[396:397])[0]
        y = mt.copy()
        y ^= y >> np.uint32(11)
        y ^= (y << np.uint32(7)) & np.uint32(0x9D2C5680)
        y ^= (y << np.uint32(15)) & np.uint32(0xEFC60000)
        y ^= y >> np.uint32(18)
        out[blk * N:(blk + 1) * N] = y
    return out[:n]


def qjl_seed(user_id: int, row_key: int) -> int:
    """``(user_id % 1024) ^ row_key`` with Python's non-negative modulo
    (kernels/quantize.py:293-295)."""
    return (int(user_id) % 1024) ^ int(row_key)


def rademacher_bits(seed: int) -> np.ndarray:
    """(64, 128) uint8 in {0,1}: bit (i, d) of G for this seed.

    ``torch.randint(0, 2, (64,128), generator=MT19937(seed))`` consumes one
    32-bit draw per element and keeps ``draw % 2`` (kernels/quantize.py:412).
    """
    return (mt19937_draws(seed, QJL_DIM * HEAD_DIM) & np.uint32(1)).astype(np.uint8).reshape(QJL_DIM, HEAD_DIM)


def rademacher_matrix(seed: int) -> torch.Tensor:
    """(64, 128) fp32 matrix of +-1: ``G = 2*bits - 1`` (kernels/quantize.py:414)."""
    return torch.from_numpy(rademacher_bits(seed).astype(np.float32) * 2.0 - 1.0)


def pack_g_words(bits: np.ndarray) -> np.ndarray:
    """(64,128) bits -> (64,4) uint32, bit d of row i at word d//32, position d%32."""
    b = bits.reshape(QJL_DIM, 4, 32).astype(np.uint64)
    return (b << np.arange(32, dtype=np.uint64)).sum(axis=2).astype(np.uint32)


# --------------------------------------------------------------------------- #
# Rotation
# --------------------------------------------------------------------------- #

def wht128(x: torch.Tensor) -> torch.Tensor:
    """Normalised 128-point Walsh-Hadamard transform of the last axis
    (kernels/hadamard.py:51-85): seven butterfly stages h = 1..64 on fp32
    copies, upper' = upper + lower, lower' = upper - lower, then one multiply
    by float32(1/sqrt(128)); the result is cast back to the input dtype."""
    if x.shape[-1] != HEAD_DIM:
        raise ValueError(f"rotation needs last dim = {HEAD_DIM} (head_dim), got {x.shape[-1]}")
    a = x.detach().to(torch.float32).reshape(-1, HEAD_DIM).clone()
    b = torch.empty_like(a)                       # the stages ping-pong between two buffers
    n = a.shape[0]
    h = 1
    while h < HEAD_DIM:
        va, vb = a.view(n, HEAD_DIM // (2 * h), 2, h), b.view(n, HEAD_DIM // (2 * h), 2, h)
        torch.add(va[:, :, 0, :], va[:, :, 1, :], out=vb[:, :, 0, :])
        torch.sub(va[:, :, 0, :], va[:, :, 1, :], out=vb[:, :, 1, :])
        a, b = b, a
        h *= 2
    return a.mul_(WHT_SCALE).reshape(x.shape).to(x.dtype)


# --------------------------------------------------------------------------- #
# INT4 codebook search and bit packing
# --------------------------------------------------------------------------- #

def nearest_centroid(y: torch.Tensor, cb: torch.Tensor, chunk: int = 1 << 15) -> Tuple[torch.Tensor, torch.Tensor]:
    """First-index argmin of |y - cb[c]| in fp32 and the chosen centroid
    (kernels/quantize.py:361-369; quantization/codebook.py:110-126).
    ``y``: (N,128) fp32, ``cb``: (16,) fp32.  Chunked so the (N,128,16)
    distance tensor of the reference never exceeds ``chunk`` rows."""
    cb = cb.to(torch.float32)
    codes = torch.empty(y.shape, dtype=torch.uint8)
    for s in range(0, y.shape[0], chunk):
        blk = y[s:s + chunk]
        d = (blk.unsqueeze(-1) - cb.view(1, 1, N_CENTROIDS)).abs()
        codes[s:s + chunk] = d.argmin(dim=-1).to(torch.uint8)
    deq = cb[codes.long()]
    return codes, deq


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """byte j = code[2j] | code[2j+1] << 4 (kernels/quantize.py:372-377)."""
    c = codes.to(torch.int32)
    return ((c[..., 0::2] & 0xF) | ((c[..., 1::2] & 0xF) << 4)).to(torch.uint8)


def unpack_nibbles(nib: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_nibbles` (kernels/quantize.py:380-395 produces the
    same order through 32-bit words: nibble k of little-endian word w is code 8w+k)."""
    p = nib.to(torch.int32)
    out = torch.empty(*nib.shape[:-1], nib.shape[-1] * 2, dtype=torch.uint8)
    out[..., 0::2] = (p & 0xF).to(torch.uint8)
    out[..., 1::2] = ((p >> 4) & 0xF).to(torch.uint8)
    return out


def pack_sign_bits(signs: torch.Tensor) -> torch.Tensor:
    """(..., 64) bool -> (..., 8) uint8, byte b bit k = sign[8b + k]
    (kernels/quantize.py:418-423)."""
    s = signs.to(torch.int32).reshape(*signs.shape[:-1], QJL_BYTES, 8)
    w = (s << torch.arange(8, dtype=torch.int32)).sum(dim=-1)
    return w.to(torch.uint8)


def unpack_sign_bits(packed: torch.Tensor) -> torch.Tensor:
    """(..., 8) uint8 -> (..., 64) fp32 in {0,1} (kernels/quantize.py:438-440)."""
    p = packed.to(torch.int32).unsqueeze(-1)
    bits = (p >> torch.arange(8, dtype=torch.int32)) & 1
    return bits.reshape(*packed.shape[:-1], QJL_DIM).to(torch.float32)


# --------------------------------------------------------------------------- #
# Codec
# --------------------------------------------------------------------------- #

def _head_codebook(codebooks: torch.Tensor, h: int, n_heads: int) -> torch.Tensor:
    if codebooks.dim() == 2:
        assert codebooks.shape == (n_heads, N_CENTROIDS), codebooks.shape
        return codebooks[h].to(torch.float32)
    return codebooks.to(torch.float32)


def quantize_heads(x: torch.Tensor, codebooks: torch.Tensor, user_id: int = 0,
                   return_residual: bool = False):
    """INT4 + QJL codec over (B, H, T, 128) ROTATED activations
    (kernels/quantize.py:542-590).  Per head h: codebook ``codebooks[h]`` (or the
    shared (16,) one), seed ``(user_id % 1024) ^ h``; outputs nibbles
    (B,H,T,64) u8, sign bytes (B,H,T,8) u8 and residual norms (B,H,T) fp32."""
    B, H, T, D = x.shape
    assert D == HEAD_DIM
    nib = torch.zeros(B, H, T, NIB_BYTES, dtype=torch.uint8)
    qjl = torch.zeros(B, H, T, QJL_BYTES, dtype=torch.uint8)
    nrm = torch.zeros(B, H, T, dtype=torch.float32)
    resid = torch.zeros(B, H, T, D, dtype=torch.float32) if return_residual else None
    for h in range(H):
        cb = _head_codebook(codebooks, h, H)
        rows = x[:, h].reshape(-1, D).to(torch.float32)
        codes, deq = nearest_centroid(rows, cb)
        err = rows - deq                                       # quantize.py:581
        G = rademacher_matrix(qjl_seed(user_id, h))            # quantize.py:583, 410-414
        proj = err @ G.t()                                     # quantize.py:415 (sgemm)
        nib[:, h] = pack_nibbles(codes).reshape(B, T, NIB_BYTES)
        qjl[:, h] = pack_sign_bits(proj >= 0).reshape(B, T, QJL_BYTES)
        nrm[:, h] = err.norm(dim=-1).reshape(B, T)             # quantize.py:582
        if return_residual:
            resid[:, h] = err.reshape(B, T, D)
    if return_residual:
        return nib, qjl, nrm, resid
    return nib, qjl, nrm


def dequantize_heads(nib: torch.Tensor, qjl: torch.Tensor, norms: torch.Tensor,
                     codebooks: torch.Tensor, user_id: int = 0, with_qjl: bool = True) -> torch.Tensor:
    """Inverse codec (kernels/quantize.py:593-640): cb[code] plus, when
    ``with_qjl``, ``(s @ G) * (norm * sqrt(2/pi)/128)`` with s = 2*bits-1
    (kernels/quantize.py:426-451)."""
    B, H, T, _ = nib.shape
    out = torch.zeros(B, H, T, HEAD_DIM, dtype=torch.float32)
    for h in range(H):
        cb = _head_codebook(codebooks, h, H)
        codes = unpack_nibbles(nib[:, h].reshape(-1, NIB_BYTES))
        deq = cb[codes.long()]
        if with_qjl:
            s = unpack_sign_bits(qjl[:, h].reshape(-1, QJL_BYTES)) * 2.0 - 1.0
            G = rademacher_matrix(qjl_seed(user_id, h))
            scale = norms[:, h].reshape(-1) * QJL_COEF
            deq = deq + (s @ G) * scale.unsqueeze(1)
        out[:, h] = deq.reshape(B, T, HEAD_DIM)
    return out


def quantize_rows(x: torch.Tensor, codebook: torch.Tensor, base_head_idx: int = 0, user_id: int = 0):
    """Row-seeded variant (kernels/quantize.py:456-499, torch branch): row i of the
    flattened input uses seed ``(user_id % 1024) ^ (base_head_idx + i)``."""
    flat = x.reshape(-1, HEAD_DIM).to(torch.float32)
    cb = codebook.to(torch.float32)
    codes, deq = nearest_centroid(flat, cb)
    err = flat - deq
    signs = torch.empty(flat.shape[0], QJL_DIM, dtype=torch.bool)
    for i in range(flat.shape[0]):
        G = rademacher_matrix(qjl_seed(user_id, base_head_idx + i))
        signs[i] = (G @ err[i]) >= 0                            # quantize.py:323-324
    lead = x.shape[:-1]
    return (pack_nibbles(codes).reshape(*lead, NIB_BYTES),
            pack_sign_bits(signs).reshape(*lead, QJL_BYTES),
            err.norm(dim=-1).reshape(*lead))


def dequantize_rows(nib, qjl, norms, codebook, base_head_idx: int = 0, user_id: int = 0,
                    with_qjl: bool = True) -> torch.Tensor:
    """Inverse of :func:`quantize_rows` (kernels/quantize.py:502-537)."""
    lead = nib.shape[:-1]
    nf = nib.reshape(-1, NIB_BYTES)
    cb = codebook.to(torch.float32)
    out = cb[unpack_nibbles(nf).long()]
    if with_qjl:
        qf = qjl.reshape(-1, QJL_BYTES)
        rf = norms.reshape(-1)
        for i in range(nf.shape[0]):
            G = rademacher_matrix(qjl_seed(user_id, base_head_idx + i))
            s = unpack_sign_bits(qf[i]) * 2.0 - 1.0
            out[i] = out[i] + (s @ G) * (float(rf[i]) * QJL_COEF)   # quantize.py:355-356
    return out.reshape(*lead, HEAD_DIM)


def rotate_quantize(x: torch.Tensor, codebooks: torch.Tensor, user_id: int = 0):
    """The bake step of the reference driver: ``quantize_heads(_wht_torch(x))``
    (scripts/run_criteo_benchmark.py:355,367)."""
    return quantize_heads(wht128(x), codebooks, user_id)


def sign_ambiguity(resid: torch.Tensor, user_id: int = 0) -> torch.Tensor:
    """(B,H,T,64) bool: True where the sign of a projection is not decided by
    fp32 arithmetic.  The reference computes the projection with a BLAS sgemm
    whose summation order is unspecified (kernels/quantize.py:415); a bit is
    called ambiguous when the exact (fp64) projection is smaller in magnitude
    than 2^-20 times the L1 norm of the residual row."""
    B, H, T, D = resid.shape
    amb = torch.zeros(B, H, T, QJL_DIM, dtype=torch.bool)
    for h in range(H):
        G = rademacher_matrix(qjl_seed(user_id, h)).double()
        e = resid[:, h].reshape(-1, D).double()
        proj = e @ G.t()
        bound = e.abs().sum(dim=1, keepdim=True) * (2.0 ** -20)
        amb[:, h] = (proj.abs() <= bound).reshape(B, T, QJL_DIM)
    return amb


# --------------------------------------------------------------------------- #
# Attention
# --------------------------------------------------------------------------- #

def repeat_kv(x: torch.Tensor, n_groups: int) -> torch.Tensor:
    """Tile each kv head ``n_groups`` times: q head j reads kv head j // n_groups
    (attention/reference.py:49-67)."""
    if n_groups == 1:
        return x
    B, Hkv, S, D = x.shape
    return x.unsqueeze(2).expand(B, Hkv, n_groups, S, D).reshape(B, Hkv * n_groups, S, D)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
              tile: int = 128) -> torch.Tensor:
    """fp32 GQA attention with the tile-wise running (max, sum, acc) update
    (attention/reference.py:72-177, no mask).  Returns fp32."""
    Hq, Hkv = q.shape[1], k.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    qf = q.to(torch.float32)
    kf = repeat_kv(k.to(torch.float32), Hq // Hkv)
    vf = repeat_kv(v.to(torch.float32), Hq // Hkv)
    B, _, T, D = qf.shape
    run_max = qf.new_full((B, Hq, T, 1), float("-inf"))
    run_sum = qf.new_zeros(B, Hq, T, 1)
    acc = qf.new_zeros(B, Hq, T, D)
    for s0 in range(0, kf.shape[2], tile):
        kt, vt = kf[:, :, s0:s0 + tile], vf[:, :, s0:s0 + tile]
        sc = torch.matmul(qf, kt.transpose(-2, -1)) * scale
        new_max = torch.maximum(run_max, sc.amax(dim=-1, keepdim=True))
        corr = torch.exp(run_max - new_max)
        p = torch.exp(sc - new_max)
        run_sum = corr * run_sum + p.sum(dim=-1, keepdim=True)
        acc = corr * acc + torch.matmul(p, vt)
        run_max = new_max
    return acc / run_sum


def decode_attention(q: torch.Tensor, k_nib, k_qjl, k_norms, v_nib, codebooks, user_id: int = 0,
                     scale: Optional[float] = None, with_qjl: bool = True) -> torch.Tensor:
    """Quantized-cache attention, CPU path of the reference
    (kernels/fused_attention.py:435-466): dequantise K (INT4 + QJL) and V (INT4
    only) to fp32, then :func:`attention`.  ``q`` is upcast to fp32 and the result
    stays fp32."""
    B, Hkv, S, _ = k_nib.shape
    if scale is None:
        scale = 1.0 / math.sqrt(HEAD_DIM)
    k_hat = dequantize_heads(k_nib, k_qjl, k_norms, codebooks, user_id, with_qjl)
    zeros_q = torch.zeros(B, Hkv, S, QJL_BYTES, dtype=torch.uint8)
    zeros_n = torch.zeros(B, Hkv, S, dtype=torch.float32)
    v_hat = dequantize_heads(v_nib, zeros_q, zeros_n, codebooks, user_id, False)
    return attention(q.to(torch.float32), k_hat, v_hat, scale)


def apply_lora_to_q(q, x, lora_a, lora_b, lora_indices, lora_alpha: float) -> torch.Tensor:
    """Per-user low-rank query update (kernels/fused_attention.py:401-430):
    ``q[b] += alpha * reshape((x[b] @ A[idx].T) @ B[idx].T)``; index -1 leaves the
    row untouched.  Returns fp32."""
    B, Hq, T, D = q.shape
    out = q.to(torch.float32).clone()
    for b in range(B):
        idx = int(lora_indices[b])
        if idx < 0:
            continue
        down = x[b].float() @ lora_a[idx].float().t()
        up = down @ lora_b[idx].float().t()
        out[b] += up.reshape(T, Hq, D).permute(1, 0, 2) * lora_alpha
    return out


# --------------------------------------------------------------------------- #
# Lloyd-Max calibration (offline, host side)
# --------------------------------------------------------------------------- #

def lloyd_max_fit(samples: torch.Tensor, max_iters: int = 300, tol: float = 1e-6) -> torch.Tensor:
    """16-level Lloyd-Max fit (quantization/codebook.py:64-108): equal-mass
    initialisation from the sorted sample, nearest-centroid assignment by
    first-index argmin of |x-c|, mean update (empty cells keep their value),
    stop when the largest centroid move is below ``tol``; returned sorted."""
    x = samples.reshape(-1).to(torch.float32)
    if x.numel() < N_CENTROIDS:
        raise ValueError(f"Need at least {N_CENTROIDS} samples; got {x.numel()}")
    xs = x.sort().values
    per = xs.shape[0] // N_CENTROIDS
    cent = torch.stack([xs[i * per:(i + 1) * per].mean() for i in range(N_CENTROIDS)])
    for _ in range(max_iters):
        assign = (x.unsqueeze(1) - cent.unsqueeze(0)).abs().argmin(dim=1)
        new = cent.clone()
        for c in range(N_CENTROIDS):
            sel = assign == c
            if sel.any():
                new[c] = x[sel].mean()
        move = (new - cent).abs().max().item()
        cent = new
        if move < tol:
            break
    return cent.sort().values.contiguous()


def lloyd_max_per_group(groups, max_iters: int = 300, tol: float = 1e-6) -> torch.Tensor:
    """One codebook per kv head (quantization/codebook.py:148-172)."""
    if len(groups) == 0:
        raise ValueError("samples_by_group must be non-empty")
    return torch.stack([lloyd_max_fit(g, max_iters, tol) for g in groups])
