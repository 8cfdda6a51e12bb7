"""Lloyd-Max codebook calibration (offline, once per model).

Mirrors ``omnistack_rs/quantization/codebook.py`` of the reference (``LloydMaxCalibrator``
:33, ``calibrate_codebook`` :129, ``calibrate_per_group`` :148): same class, methods, errors
and algorithm (equal-mass initialisation, first-index nearest-centroid assignment, mean
update, empty cells stay put, stop below ``convergence_tol``, sorted float32 output).

The fit itself is ``omni_lloyd_max_fit``: the samples are sorted once on the device, and the whole
iteration then runs in one kernel launch on cell boundaries and prefix sums (all groups of
``calibrate_per_group`` in the same launch).  There is no host implementation.
"""
from __future__ import annotations

import torch

from .. import _lib

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
        if x.numel() < self.n_centroids:
            raise ValueError(f"Need at least {self.n_centroids} samples; got {x.numel()}")
        self._codebook = _fit_groups([x], self.max_iters, self.convergence_tol)[0].contiguous()
        return self

    def quantize(self, x: torch.Tensor):
        cb = self.codebook
        flat = x.reshape(-1).float()
        idx = (flat.unsqueeze(1) - cb.unsqueeze(0)).abs().argmin(dim=1)
        return idx.to(torch.uint8).reshape(x.shape), cb[idx].reshape(x.shape)


def _fit_groups(groups, max_iters: int, tol: float) -> torch.Tensor:
    """(n_groups, 16) codebooks of flat float32 sample tensors from one ``omni_lloyd_max_fit`` call.  Samples
    held on the host are copied to the current CUDA device and the codebooks come back to the host; without a
    CUDA device this raises (there is no host implementation)."""
    home = groups[0].device
    if not all(g.is_cuda for g in groups):
        if not torch.cuda.is_available():
            raise RuntimeError("omni_b200: Lloyd-Max calibration runs on a CUDA device only (no CPU fallback)")
        groups = [g.cuda() for g in groups]
    dev = _lib.require_cuda(*groups)
    lib = _lib.ensure_init(dev)
    sizes = [int(g.numel()) for g in groups]
    for n in sizes:
        if n < N_CENTROIDS:
            raise ValueError(f"Need at least {N_CENTROIDS} samples; got {n}")
    ordered = torch.cat([g.sort().values for g in groups]) if len(groups) > 1 else groups[0].sort().values
    offsets = torch.tensor([0] + sizes, dtype=torch.int64).cumsum(0).to(dev)
    total = sum(sizes)
    ws_bytes = lib.omni_lloyd_max_workspace_bytes(total)
    ws = torch.empty(ws_bytes // 8, dtype=torch.float64, device=dev)
    out = torch.empty(len(groups), N_CENTROIDS, dtype=torch.float32, device=dev)
    with _lib.on_device(dev):
        _lib.check(lib.omni_lloyd_max_fit(_lib.ptr(ordered), total, _lib.ptr(offsets), len(groups), int(max_iters),
                                          float(tol), _lib.ptr(ws), ws_bytes, _lib.ptr(out), None, _lib.stream_ptr(dev)))
    return out.to(home)


def calibrate_codebook(samples: torch.Tensor, max_iters: int = _DEFAULT_MAX_ITERS,
                       convergence_tol: float = _DEFAULT_TOL) -> torch.Tensor:
    return LloydMaxCalibrator(max_iters=max_iters, convergence_tol=convergence_tol).fit(samples).codebook


def calibrate_per_group(samples_by_group, max_iters: int = _DEFAULT_MAX_ITERS,
                        convergence_tol: float = _DEFAULT_TOL) -> torch.Tensor:
    if len(samples_by_group) == 0:
        raise ValueError("samples_by_group must be non-empty")
    return _fit_groups([s.reshape(-1).float() for s in samples_by_group], max_iters, convergence_tol)
