"""Helpers shared by the CPU and GPU tests: golden-file access and seeded inputs."""
from __future__ import annotations

import functools
import hashlib
import math
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(t: torch.Tensor) -> str:
    a = t.detach().contiguous().cpu()
    if a.dtype in (torch.bfloat16, torch.float16):
        a = a.view(torch.int16)
    return hashlib.sha256(a.numpy().tobytes()).hexdigest()


@functools.lru_cache(maxsize=None)
def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN_DIR, name)) as z:
        return {k: z[k] for k in z.files}


def t(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))


def bf16(a) -> torch.Tensor:
    """int16 bit pattern -> bf16 tensor."""
    return t(a).view(torch.bfloat16)


@functools.lru_cache(maxsize=None)
def config0_inputs():
    """K, V (64,8,50,128) fp32 and q (64,8,1,128) bf16 of benchmark configs 0/1:
    i.i.d. N(0,1) from seed 0, drawn in this order from one generator."""
    g = torch.Generator().manual_seed(0)
    K = torch.randn(64, 8, 50, 128, generator=g)
    V = torch.randn(64, 8, 50, 128, generator=g)
    q = torch.randn(64, 8, 1, 128, generator=g).to(torch.bfloat16)
    return K, V, q


def sign_mismatch_report(got_qjl: torch.Tensor, want_qjl: torch.Tensor, ambiguous: torch.Tensor):
    """Count differing sign bits and how many of those are outside the
    ambiguity mask ((...,64) bool)."""
    x = (got_qjl.cpu().to(torch.int32) ^ want_qjl.cpu().to(torch.int32)).unsqueeze(-1)
    diff = ((x >> torch.arange(8, dtype=torch.int32)) & 1).reshape(*got_qjl.shape[:-1], 64).bool()
    return int(diff.sum()), int((diff & ~ambiguous).sum())


DEFAULT_SCALE = 1.0 / math.sqrt(128)
