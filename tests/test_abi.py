"""CPU checks of the C-ABI boundary: the shared library builds, loads, exports every
symbol the header declares, and its host-only entry points agree with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle as orc
from omnistack_rs_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "omni_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(omni_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/omni_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table and header disagree"


def test_abi_version_and_error_string(lib):
    assert lib.omni_abi_version() == 3
    assert lib.omni_gtable_host(None, 0, 1) == _lib.ERR_ARG
    assert b"NULL" in lib.omni_last_error()
    buf = np.empty((1, 64, 4), dtype=np.uint32)
    assert lib.omni_gtable_host(buf.ctypes.data_as(C.c_void_p), 1020, 8) == _lib.ERR_ARG


def test_host_rademacher_table_matches_oracle(lib):
    buf = np.empty((1024, 64, 4), dtype=np.uint32)
    assert lib.omni_gtable_host(buf.ctypes.data_as(C.c_void_p), 0, 1024) == _lib.OK
    for seed in (0, 1, 5, 511, 1023):
        assert np.array_equal(buf[seed], orc.pack_g_words(orc.rademacher_bits(seed)))
    g = np.load(os.path.join(ROOT, "tests", "golden", "rademacher.npz"))
    bits = ((buf[:, :, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(1024, 64, 128).astype(np.uint8)
    import hashlib
    assert hashlib.sha256(bits.tobytes()).hexdigest() == str(g["sha_all"])


def test_cpu_tensors_are_rejected():
    import torch
    from omnistack_rs_b200.kernels.quantize import quantize_heads
    from omnistack_rs_b200.kernels.hadamard import rotate_queries
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        quantize_heads(torch.zeros(1, 1, 1, 128), torch.zeros(16))
    with pytest.raises(ValueError, match="head_dim"):
        rotate_queries(torch.zeros(1, 1, 1, 64))


def test_make_g_matrix_matches_reference_layout():
    import torch
    from omnistack_rs_b200.kernels.fused_attention import make_g_matrix
    lo, hi = make_g_matrix(2, 7)
    assert lo.shape == (2, 64) and lo.dtype == torch.int64
    gen = torch.Generator().manual_seed(7)
    bits = torch.randint(0, 2, (2, 64, 128), generator=gen, dtype=torch.int64)
    assert int((lo[1, 3] >> 5) & 1) == int(bits[1, 3, 5])
    assert int((hi[0, 9] >> 63) & 1) == int(bits[0, 9, 127])


def test_calibrator_host_logic():
    import torch
    from omnistack_rs_b200.quantization import LloydMaxCalibrator, calibrate_per_group
    x = torch.randn(4096, generator=torch.Generator().manual_seed(0))
    with pytest.raises(ValueError):
        LloydMaxCalibrator(n_centroids=8)
    with pytest.raises(RuntimeError):
        LloydMaxCalibrator().codebook
    with pytest.raises(ValueError):
        LloydMaxCalibrator().fit(torch.zeros(3))
    with pytest.raises(ValueError):
        calibrate_per_group([])
    if not torch.cuda.is_available():                       # the fit is a CUDA kernel: it must refuse, not fall back
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            LloydMaxCalibrator().fit(x)
