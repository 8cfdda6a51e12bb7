"""The allocation-free decode entry point (``omni_qattn_decode_noalloc``).

Some hosts of this library may not allocate device memory at call time: a serving process
or plugin host that owns the device heap and gives its plugins fixed buffers, or a loop
that cannot take the device-wide stall of an allocation.  For them the split-K scratch
lives inside the library image.  This test drives the entry point through the C ABI twice
in a row -- the second call with another shape and split count, so that it runs over the
stale partial states of the first -- and requires the same result as the regular entry
point, which gets its workspace from the caller.  It also checks that a request larger
than the built-in scratch is refused with a message instead of being run.

Collected last on purpose (file name): a run that stops at the first failure has then
already covered every other test.
"""
import math
import os
import subprocess
import sys

import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu

ATOL = 3e-3          # the tolerance of the attention parity tests


def _cache(B, Hkv, S, seed):
    gen = torch.Generator().manual_seed(seed)
    cb = torch.sort(torch.randn(Hkv, 16, generator=gen) * 1.1, dim=1).values
    kn, kq, kr = orc.quantize_heads(orc.wht128(torch.randn(B, Hkv, S, 128, generator=gen)), cb, 6)
    vn, _, _ = orc.quantize_heads(orc.wht128(torch.randn(B, Hkv, S, 128, generator=gen)), cb, 6)
    return kn, kq, kr, vn, cb, gen


def _call(lib, name, q, kn, kq, kr, vn, cb, lens, n_splits, workspace=None):
    from omnistack_rs_b200 import _lib
    B, Hq, T, _ = q.shape
    _, Hkv, S, _ = kn.shape
    out = torch.full((B, Hq, T, 128), float("nan"), dtype=torch.float32, device=q.device)
    common = [_lib.ptr(q), _lib.DTYPE_CODE[q.dtype], _lib.ptr(kn), _lib.ptr(kq), _lib.ptr(kr), _lib.ptr(vn),
              _lib.ptr(cb), 1, None, 6, _lib.ptr(lens), None, B, Hq, Hkv, T, S, Hkv * S, S,
              1.0 / math.sqrt(128), 1, 0, 0, 0, n_splits]
    stream = _lib.stream_ptr(q.device)
    if name == "noalloc":
        status = lib.omni_qattn_decode_noalloc(*common, _lib.ptr(out), stream)
    else:
        status = lib.omni_qattn_decode(*common, _lib.ptr(workspace), workspace.numel() * 4, _lib.ptr(out), None, stream)
    return status, out


def test_noalloc_entry_matches_regular_entry_twice():
    from omnistack_rs_b200 import _lib
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    dev = torch.device("cuda:0")
    lib = _lib.ensure_init(dev)                      # the regular entry point needs it; the new one does not
    assert lib.omni_qattn_noalloc_scratch_bytes() == 32 << 20
    with torch.cuda.device(dev):
        free_before = None
        # the last case (100 keys, 2 splits) takes the lane-per-key kernel and the merge over the built-in scratch
        for B, Hq, Hkv, S, n_splits, seed in ((5, 8, 4, 700, 6, 1), (3, 4, 2, 130, 3, 2), (2, 4, 2, 100, 2, 3)):
            kn, kq, kr, vn, cb, gen = _cache(B, Hkv, S, seed)
            q = torch.randn(B, Hq, 2, 128, generator=gen).to(torch.bfloat16)
            lens = torch.randint(1, S + 1, (B,), generator=gen).to(torch.int32)
            want = torch.cat([orc.decode_attention(q[b:b + 1], kn[b:b + 1, :, :n], kq[b:b + 1, :, :n],
                                                   kr[b:b + 1, :, :n], vn[b:b + 1, :, :n], cb, 6)
                              for b, n in enumerate(lens.tolist())])
            d = [x.to(dev) for x in (q, kn, kq, kr, vn, cb, lens)]
            ws = torch.empty(lib.omni_qattn_workspace_bytes(B, Hq, 2, n_splits) // 4, dtype=torch.float32, device=dev)
            st_ref, out_ref = _call(lib, "regular", *d, n_splits, ws)
            st_new, out_new = _call(lib, "noalloc", *d, n_splits)
            torch.cuda.synchronize(dev)
            assert st_ref == _lib.OK and st_new == _lib.OK, lib.omni_last_error()
            assert torch.isfinite(out_new).all()
            assert (out_new - out_ref).abs().max() <= ATOL
            assert (out_new.cpu() - want).abs().max() <= ATOL
            # no device allocation after the first call: the driver's free-memory figure does not move
            # (the tensors of this test come out of torch's cached pool, whose size the loop does not change)
            d2 = [x.clone() for x in d]
            torch.cuda.synchronize(dev)
            free_before = torch.cuda.mem_get_info(dev)[0]
            for _ in range(3):
                st_again, _ = _call(lib, "noalloc", *d2, n_splits)
                assert st_again == _lib.OK
            torch.cuda.synchronize(dev)
            assert torch.cuda.mem_get_info(dev)[0] >= free_before
        # the entry point's own status word (it takes no status argument): nothing to report after normal calls
        import ctypes as C
        value = C.c_int32(-1)
        assert lib.omni_qattn_noalloc_status(C.byref(value), 1) == _lib.OK and value.value == 0
        assert lib.omni_qattn_noalloc_status(None, 0) == _lib.ERR_ARG


def test_noalloc_entry_refuses_oversized_request():
    from omnistack_rs_b200 import _lib
    dev = torch.device("cuda:0")
    lib = _lib.load()
    kn, kq, kr, vn, cb, gen = _cache(1, 1, 64, 3)
    q = torch.zeros(1, 1, 1, 128, dtype=torch.bfloat16)
    d = [x.to(dev) for x in (q, kn, kq, kr, vn, cb)]
    out = torch.zeros(1, 1, 1, 128, dtype=torch.float32, device=dev)
    too_many = (32 << 20) // (132 * 4) + 1          # one partial state more than the scratch holds
    with torch.cuda.device(dev):
        status = lib.omni_qattn_decode_noalloc(
            _lib.ptr(d[0]), 1, _lib.ptr(d[1]), _lib.ptr(d[2]), _lib.ptr(d[3]), _lib.ptr(d[4]), _lib.ptr(d[5]), 1,
            None, 6, None, None, too_many, 1, 1, 1, 64, 64, 64, 0.1, 1, 0, 0, 0, 2, _lib.ptr(out), None)
    assert status == _lib.ERR_UNSUPPORTED
    msg = lib.omni_last_error().decode()
    assert "scratch" in msg and "n_splits" in msg


_FRESH = r"""
import math, sys
import torch
sys.path.insert(0, {root!r})
import oracle as orc
from omnistack_rs_b200 import _lib

dev = torch.device("cuda:0")
lib = _lib.load()                                   # omni_init is NOT called in this process
gen = torch.Generator().manual_seed(9)
B, Hq, Hkv, S, n_splits = 3, 4, 2, 300, 2
cb = torch.sort(torch.randn(Hkv, 16, generator=gen) * 1.1, dim=1).values
kn, kq, kr = orc.quantize_heads(orc.wht128(torch.randn(B, Hkv, S, 128, generator=gen)), cb, 6)
vn, _, _ = orc.quantize_heads(orc.wht128(torch.randn(B, Hkv, S, 128, generator=gen)), cb, 6)
q = torch.randn(B, Hq, 1, 128, generator=gen).to(torch.bfloat16)
want = orc.decode_attention(q, kn, kq, kr, vn, cb, 6)
d = [x.to(dev) for x in (q, kn, kq, kr, vn, cb)]
out = torch.full((B, Hq, 1, 128), float("nan"), dtype=torch.float32, device=dev)
torch.cuda.synchronize(dev)
side = torch.cuda.Stream(device=dev)                # a non-blocking stream: no implicit order with the legacy stream
with torch.cuda.device(dev), torch.cuda.stream(side):
    st = lib.omni_qattn_decode_noalloc(
        _lib.ptr(d[0]), 1, _lib.ptr(d[1]), _lib.ptr(d[2]), _lib.ptr(d[3]), _lib.ptr(d[4]), _lib.ptr(d[5]), 1,
        None, 6, None, None, B, Hq, Hkv, 1, S, Hkv * S, S, 1.0 / math.sqrt(128), 1, 0, 0, 0, n_splits,
        _lib.ptr(out), side.cuda_stream)
side.synchronize()
assert st == _lib.OK, lib.omni_last_error()
err = float((out.cpu() - want).abs().max())
assert err <= 3e-3, err
print("fresh-process first call ok", err)
"""


def test_noalloc_first_call_in_fresh_process_on_side_stream():
    """The very first call of a process -- no omni_init, nothing warmed up -- issued on a non-blocking stream must
    already see the complete built-in row table (its set-up waits for the device before publishing the table)."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", _FRESH.format(root=root)], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "fresh-process first call ok" in res.stdout
