"""Build the CUDA shared library in-tree with nvcc for sm_100a.

    python -m omnistack_rs_b200.build [--force] [-v]

The output is ``omnistack_rs_b200/csrc/libomni_b200.so``.  nvcc cross-compiles, so
this works on a machine without a GPU.  Translation units are compiled in parallel into
``csrc/_obj`` and only when they (or a header) changed; the link step follows.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
OBJ_DIR = os.path.join(CSRC, "_obj")
LIB_PATH = os.path.join(CSRC, "libomni_b200.so")
SOURCES = ["runtime.cu", "codec.cu", "codec_fast.cu", "qattn.cu", "qattn_mma.cu", "qattn_mma_lora.cu", "qattn_umma.cu", "lora_q.cu",
           "lloyd_max.cu", "qjl_bool.cu"]
# qattn_mma.cu is also a header: qattn_mma_lora.cu includes it
HEADERS = ["common.cuh", "qattn.cuh", "codec_fast.cuh", "codec_tc.cuh", "qattn_mma.cu", os.path.join("..", "..", "include", "omni_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the omni_b200 CUDA library cannot be built")
    return exe


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _newest_header() -> float:
    return max(os.path.getmtime(os.path.join(CSRC, h)) for h in HEADERS)


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in _sources() + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n" + res.stdout + res.stderr)
    return res.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu of the library and link one shared object; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr = _newest_header()
    todo = []
    for s in _sources():
        obj = os.path.join(OBJ_DIR, os.path.splitext(s)[0] + ".o")
        src_m = max(os.path.getmtime(os.path.join(CSRC, s)), hdr)
        if force or verbose or not os.path.exists(obj) or os.path.getmtime(obj) < src_m:
            todo.append(s)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        for s, log in zip(todo, pool.map(lambda s: _compile(s, verbose), todo)):
            if verbose:
                print(f"---- {s}\n{log}")
    objs = [os.path.join(OBJ_DIR, os.path.splitext(s)[0] + ".o") for s in _sources()]
    res = subprocess.run([_nvcc()] + LINK_FLAGS + objs + ["-o", LIB_PATH + ".tmp"], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
