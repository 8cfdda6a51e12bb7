"""ctypes binding of ``libomni_b200.so`` (declared in ``include/omni_b200.h``).

There is no CPU implementation behind this module: if the shared library is missing
or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import os
import threading

import torch


OK, ERR_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE_WAIT, ERR_NOT_INIT = range(6)
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

# name -> (restype, argtypes); mirrors include/omni_b200.h
_i32, _i64, _f32, _vp, _sz = C.c_int32, C.c_int64, C.c_float, C.c_void_p, C.c_size_t
SIGNATURES = {
    "omni_init": (_i32, [_i32]),
    "omni_shutdown": (_i32, []),
    "omni_last_error": (C.c_char_p, []),
    "omni_abi_version": (_i32, []),
    "omni_gtable_host": (_i32, [_vp, _i32, _i32]),
    "omni_rotate": (_i32, [_vp, _vp, _i64, _i32, _vp]),
    "omni_quantize_heads": (_i32, [_vp, _i32, _i32, _vp, _i32, _vp, _i32, _i64, _i32, _i64, _i64, _i64, _i64,
                                   _vp, _vp, _vp, _i64, _i64, _vp, _i64, _vp]),
    "omni_dequantize_heads": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i32, _i64, _i32, _i64, _i64, _i64, _i32,
                                     _vp, _vp]),
    "omni_quantize_rows": (_i32, [_vp, _vp, _i32, _i32, _i64, _vp, _vp, _vp, _vp]),
    "omni_dequantize_rows": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _i32, _vp, _vp]),
    "omni_qattn_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32]),
    "omni_qattn_decode": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _i32, _vp, _vp,
                                 _i64, _i32, _i32, _i32, _i64, _i64, _i64, _f32, _i32, _i32, _i32, _i32, _i32,
                                 _vp, _sz, _vp, _vp, _vp]),
    "omni_v_pair_groups": (_i32, [_vp, _i64, _i32, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "omni_lora_q": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _f32, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "omni_qattn_lora_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32]),
    "omni_qattn_decode_lora": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _i32, _vp, _vp,
                                      _i64, _i32, _i32, _i32, _i64, _i64, _i64, _f32, _i32, _i32, _i32, _i32, _i32,
                                      _vp, _sz, _vp, _vp, _vp, _vp]),
    "omni_qjl_encode_bool": (_i32, [_vp, _i64, _i32, _vp, _vp, _vp]),
    "omni_qjl_reconstruct_bool": (_i32, [_vp, _vp, _i64, _i32, _vp, _vp]),
    "omni_lloyd_max_workspace_bytes": (_sz, [_i64]),
    "omni_lloyd_max_fit": (_i32, [_vp, _i64, _vp, _i32, _i32, C.c_double, _vp, _sz, _vp, _vp, _vp]),
    "omni_qattn_noalloc_scratch_bytes": (_sz, []),
    "omni_qattn_decode_noalloc": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _i32, _vp, _vp,
                                         _i64, _i32, _i32, _i32, _i64, _i64, _i64, _f32, _i32, _i32, _i32, _i32, _i32,
                                         _vp, _vp]),
    "omni_qattn_decode_host": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _i32, _vp, _vp,
                                      _i64, _i32, _i32, _i32, _i64, _i64, _i64, _f32, _i32, _i32, _vp, _vp, _i32,
                                      _i32, _vp, _sz, _vp]),
    "omni_qattn_noalloc_status": (_i32, [_vp, _i32]),
    "omni_diag_bounded_wait": (_i32, [_i32, _vp, _vp]),
}

_lock = threading.Lock()
_lib = None
_inited = set()


LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "libomni_b200.so")


def lib_path() -> str:
    """Path of the shared library; OMNI_B200_LIB overrides the in-tree default."""
    return os.environ.get("OMNI_B200_LIB", LIB_PATH)


def load() -> C.CDLL:
    """Load the shared library (never builds implicitly; see ``omnistack_rs_b200.build``)."""
    global _lib
    with _lock:
        if _lib is None:
            path = lib_path()
            if not os.path.exists(path):
                raise RuntimeError(
                    f"{path} is missing: build it with `python -m omnistack_rs_b200.build` "
                    "(there is no CPU fallback for the omni_b200 kernels)")
            lib = C.CDLL(path)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            _lib = lib
        return _lib


_EXC = {ERR_ARG: ValueError, ERR_UNSUPPORTED: NotImplementedError, ERR_CUDA: RuntimeError,
        ERR_DEVICE_WAIT: RuntimeError, ERR_NOT_INIT: RuntimeError}


def check(status: int) -> None:
    if status != OK:
        msg = load().omni_last_error().decode("utf-8", "replace")
        raise _EXC.get(status, RuntimeError)(f"omni_b200 status {status}: {msg}")


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors must live on one CUDA device; returns it."""
    dev = None
    for x in tensors:
        if x is None:
            continue
        if not x.is_cuda:
            raise RuntimeError("omni_b200 runs on CUDA tensors only (no CPU fallback); got a tensor on "
                               f"{x.device}")
        if dev is None:
            dev = x.device
        elif x.device != dev:
            raise ValueError(f"tensors on different devices: {dev} and {x.device}")
    if dev is None:
        raise ValueError("no tensor given")
    return dev


def ensure_init(device: torch.device) -> C.CDLL:
    lib = load()
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _inited:
        check(lib.omni_init(idx))
        _inited.add(idx)
    return lib


class OmniLora(C.Structure):
    """``omni_lora_t`` of the C header."""
    _fields_ = [("x", C.c_void_p), ("lora_a", C.c_void_p), ("lora_b", C.c_void_p), ("lora_indices", C.c_void_p),
                ("n_adapters", C.c_int32), ("hidden", C.c_int32), ("rank", C.c_int32), ("alpha", C.c_float)]


_NULL_CONTEXT = contextlib.nullcontext()


def on_device(device: torch.device):
    """Context manager that makes ``device`` current (free when it already is)."""
    if device.index is None or torch.cuda.current_device() == device.index:
        return _NULL_CONTEXT
    return torch.cuda.device(device)


def ptr(x):
    """Address of a tensor's storage as ctypes takes it for a ``void*`` argument (None = NULL)."""
    return None if x is None else x.data_ptr()


def stream_ptr(device: torch.device):
    """Raw handle of torch's current stream on ``device``."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(idx) or None


_workspaces = {}


def workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """Grow-only scratch of at least ``nbytes`` bytes, one per (device, stream): calls on one stream run in order,
    so they can share it; calls on different streams get different buffers."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream or 0)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() * 4 < nbytes:
        buf = torch.empty(max((nbytes + 3) // 4, 1 << 16), dtype=torch.float32, device=device)
        _workspaces[key] = buf
    return buf


def as_device(x: torch.Tensor, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """``x`` as a contiguous tensor of ``dtype`` on ``device``; ``x`` itself when it already is one."""
    if x.dtype is dtype and x.device == device and x.is_contiguous():
        return x
    return x.to(device=device, dtype=dtype).contiguous()


_status_words = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word the kernels set when a bounded device-side wait expires."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[idx]


def check_device_status(device: torch.device) -> None:
    """Synchronises the device and raises if a kernel reported an expired wait (RuntimeError) or an
    adapter index past the adapter count (IndexError) since the last check."""
    w = status_word(device)
    torch.cuda.synchronize(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        if code == 7:
            raise IndexError("omni_b200: lora_indices refers to an adapter that does not exist")
        if code == 8:
            raise NotImplementedError("omni_b200: a codebook holds an infinite or NaN centroid")
        raise RuntimeError(f"omni_b200: a device-side bounded wait expired (status {code})")
