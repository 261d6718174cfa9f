"""In-tree build of the sm_100a native library.

Every ``*.cu`` beside this file is compiled with ``nvcc -gencode
arch=compute_100a,code=sm_100a`` into an object file and linked into one
shared library, ``libsga_b200.so``, in this directory. The kernels expose
plain ``extern "C"`` launchers that take raw device pointers and a stream
handle, so no PyTorch headers are involved and a full rebuild takes seconds.
The library is loaded with ``ctypes`` by :mod:`sga_b200.csrc` (``lib()``).

The reference ships no native sources at all (its kernels are Triton JIT,
``sga/kernels.py:33-139``); this directory is their CUDA replacement.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libsga_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
# Files whose numerics must follow IEEE fp32 op for op (no fast-math, no
# implicit FMA contraction): the optimizer tails and the replay kernels.
STRICT_FP = {"optim.cu", "replay.cu", "replay_select.cu", "dense_sync.cu", "index_sync.cu"}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _digest(path: str, flags: list[str]) -> str:
    h = hashlib.sha1()
    h.update(" ".join(flags).encode())
    for dep in [path] + [os.path.join(HERE, f) for f in sorted(os.listdir(HERE)) if f.endswith(".cuh")]:
        with open(dep, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _flags_for(src: str, extra: list[str]) -> list[str]:
    flags = list(NVCC_FLAGS) + list(extra)
    if src in STRICT_FP:
        flags = [f for f in flags if f != "--use_fast_math"] + ["-fmad=false"]
    return flags


def _compile_one(src: str, extra: list[str], verbose: bool, objdir: str = "build") -> tuple[str, bool, str]:
    path = os.path.join(HERE, src)
    obj = os.path.join(HERE, objdir, src[:-3] + ".o")
    stamp = obj + ".sha1"
    flags = _flags_for(src, extra)
    dig = _digest(path, flags)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj, False, ""
    cmd = [_nvcc()] + flags + ["-I", HERE, "-c", path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    with open(stamp, "w") as fh:
        fh.write(dig)
    return obj, True, res.stdout + res.stderr


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, bounds: bool = False) -> str:
    """Compile (if stale) and link the library; returns its path. ``bounds`` builds the debug
    variant ``libsga_b200_bounds.so`` with ``-DSGA_BOUNDS`` (index checks in the index-following
    kernels) beside the production library."""
    objdir = "build_bounds" if bounds else "build"
    os.makedirs(os.path.join(HERE, objdir), exist_ok=True)
    if force:
        for f in os.listdir(os.path.join(HERE, objdir)):
            os.remove(os.path.join(HERE, objdir, f))
    extra = (["-Xptxas", "-v"] if ptxas_info else []) + (["-DSGA_BOUNDS"] if bounds else [])
    srcs = sources()
    objs, rebuilt, logs = [], False, []
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as pool:
        for obj, did, log in pool.map(lambda s: _compile_one(s, extra, verbose, objdir), srcs):
            objs.append(obj)
            rebuilt |= did
            if log.strip():
                logs.append(log)
    out = os.path.join(HERE, LIB_NAME.replace(".so", "_bounds.so") if bounds else LIB_NAME)
    if rebuilt or not os.path.exists(out):
        cmd = [_nvcc(), "-shared", "-o", out] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if (verbose or ptxas_info) and logs:
        print("\n".join(logs))
    return out


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv,
              bounds="--bounds" in sys.argv)
    print(p)
