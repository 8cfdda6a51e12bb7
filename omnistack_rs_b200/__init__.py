"""omnistack_rs_b200 -- B200 (sm_100a) KV-cache codec and fused quantized decode attention.

Drop-in for the hot path of OmniStack-RS: the sub-packages ``kernels``, ``quantization``
and ``attention`` keep the reference's function names and signatures and run
hand-written CUDA through the C ABI in ``include/omni_b200.h``.
"""
from . import _lib  # noqa: F401

HEAD_DIM = 128
QJL_DIM = 64

__all__ = ["HEAD_DIM", "QJL_DIM", "install_as_omnistack_rs"]


def install_as_omnistack_rs() -> None:
    """Register this package under the reference's import names
    (``omnistack_rs.kernels.quantize`` ...) so its scripts run unmodified."""
    import importlib
    import sys
    names = ["", ".kernels", ".kernels.hadamard", ".kernels.quantize", ".kernels.fused_attention",
             ".quantization", ".quantization.codebook", ".quantization.qjl", ".attention", ".attention.reference"]
    for n in names:
        sys.modules["omnistack_rs" + n] = importlib.import_module(__name__ + n)
