"""Lloyd-Max codebook calibration (offline, once per model).

Mirrors ``omnistack_rs/quantization/codebook.py`` of the reference (``LloydMaxCalibrator``
:33, ``calibrate_codebook`` :129, ``calibrate_per_group`` :148): same class, methods, errors
and algorithm (equal-mass initialisation, first-index nearest-centroid assignment, mean
update, empty cells stay put, stop below ``convergence_tol``, sorted float32 output).  The
iteration runs with torch ops on whatever device the samples live on; it is host-side
set-up work, not part of the per-token path.
"""
from __future__ import annotations

import torch

N_CENTROIDS: int = 16
_DEFAULT_MAX_ITERS: int = 300
_DEFAULT_TOL: float = 1e-6


class LloydMaxCalibrator:
    def __init__(self, n_centroids: int = N_CENTROIDS, max_iters: int = _DEFAULT_MAX_ITERS,
                 convergence_tol: float = _DEFAULT_TOL) -> None:
        if n_centroids != 16:
            raise ValueError(f"n_centroids must be 16 for INT4 nibble packing; got {n_centroids}")
        self.n_centroids = n_centroids
        self.max_iters = max_iters
        self.convergence_tol = convergence_tol
        self._codebook = None

    @property
    def codebook(self) -> torch.Tensor:
        if self._codebook is None:
            raise RuntimeError("LloydMaxCalibrator.fit() must be called before accessing codebook")
        return self._codebook

    def fit(self, samples: torch.Tensor) -> "LloydMaxCalibrator":
        x = samples.reshape(-1).float()
        n = self.n_centroids
        if x.numel() < n:
            raise ValueError(f"Need at least {n} samples; got {x.numel()}")
        xs = x.sort().values
        per = xs.shape[0] // n
        cent = xs[: per * n].view(n, per).mean(dim=1)
        ids = torch.arange(n, device=x.device)
        for _ in range(self.max_iters):
            assign = (x.unsqueeze(1) - cent.unsqueeze(0)).abs().argmin(dim=1)
            onehot = assign.unsqueeze(1) == ids.unsqueeze(0)
            new = cent.clone()
            for c in range(n):
                sel = onehot[:, c]
                if bool(sel.any()):
                    new[c] = x[sel].mean()
            move = float((new - cent).abs().max())
            cent = new
            if move < self.convergence_tol:
                break
        self._codebook = cent.sort().values.contiguous()
        return self

    def quantize(self, x: torch.Tensor):
        cb = self.codebook
        flat = x.reshape(-1).float()
        idx = (flat.unsqueeze(1) - cb.unsqueeze(0)).abs().argmin(dim=1)
        return idx.to(torch.uint8).reshape(x.shape), cb[idx].reshape(x.shape)


def calibrate_codebook(samples: torch.Tensor, max_iters: int = _DEFAULT_MAX_ITERS,
                       convergence_tol: float = _DEFAULT_TOL) -> torch.Tensor:
    return LloydMaxCalibrator(max_iters=max_iters, convergence_tol=convergence_tol).fit(samples).codebook


def calibrate_per_group(samples_by_group, max_iters: int = _DEFAULT_MAX_ITERS,
                        convergence_tol: float = _DEFAULT_TOL) -> torch.Tensor:
    if len(samples_by_group) == 0:
        raise ValueError("samples_by_group must be non-empty")
    return torch.stack([calibrate_codebook(s, max_iters, convergence_tol) for s in samples_by_group])
