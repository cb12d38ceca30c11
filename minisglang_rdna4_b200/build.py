"""In-tree build of the native libraries.

* ``ops/libmsgl_cuda.so``  — every sm_100a kernel (``csrc/*.cu``), compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a GPU).
* ``ops/libmsgl_cuda_checked.so`` — the same sources with ``-DMSGL_CHECK_BOUNDS`` (device-side index
  checks that record and skip instead of trapping); built by ``--checked`` and loaded when
  ``MSGL_CHECK_BOUNDS=1``.
* ``ops/libmsgl_host.so``  — host helpers (``csrc/host/*.cpp``).

Objects are cached under ``csrc/_obj`` keyed by a hash of the source, its headers and the
flags, so a rebuild only recompiles what changed. Run ``python -m minisglang_rdna4_b200.build``.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
OPS = os.path.join(HERE, "ops")
CUDA_LIB = os.path.join(OPS, "libmsgl_cuda.so")
CHECKED_LIB = os.path.join(OPS, "libmsgl_cuda_checked.so")
HOST_LIB = os.path.join(OPS, "libmsgl_host.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-march=x86-64-v3"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256(" ".join(flags).encode())
    for p in sorted(paths):
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def _headers() -> List[str]:
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]


def _compile(cmd: List[str], out: str, log: str) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as fh:
        fh.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return out


def build_cuda(verbose: bool = True, checked: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    flags = NVCC_FLAGS + (["-DMSGL_CHECK_BOUNDS=1"] if checked else [])
    out_lib = CHECKED_LIB if checked else CUDA_LIB
    variant = ".chk" if checked else ""
    sources = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = _headers()
    jobs, objs = [], []
    for src in sources:
        tag = _digest([src] + headers, flags)
        obj = os.path.join(OBJ, f"{os.path.basename(src)[:-3]}{variant}.{tag}.o")
        objs.append(obj)
        if not os.path.exists(obj):
            tu = ['-DMSGL_TU_NAME="%s"' % os.path.basename(src)] if checked else []
            jobs.append(([nvcc] + flags + tu + ["-c", src, "-o", obj], obj, obj[:-2] + ".log"))
    if jobs and verbose:
        print(f"[build] compiling {len(jobs)} CUDA source(s) for sm_100a", file=sys.stderr)
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(lambda j: _compile(*j), jobs))
    stamp = _digest(objs, ["link"])
    stamp_file = out_lib + ".stamp"
    if jobs or not os.path.exists(out_lib) or not os.path.exists(stamp_file) or open(stamp_file).read() != stamp:
        _compile([nvcc, "-shared", "-o", out_lib] + objs + ["-lcudart"], out_lib,
                 os.path.join(OBJ, f"link{variant}.log"))
        with open(stamp_file, "w") as fh:
            fh.write(stamp)
    # drop stale objects
    keep = {os.path.basename(o) for o in objs}
    for f in os.listdir(OBJ):
        if f.endswith(".o") and f not in keep and (".chk." in f) == checked:
            os.remove(os.path.join(OBJ, f))
    return out_lib


def build_host(verbose: bool = True) -> str:
    os.makedirs(OBJ, exist_ok=True)
    host_dir = os.path.join(CSRC, "host")
    sources = sorted(os.path.join(host_dir, f) for f in os.listdir(host_dir) if f.endswith(".cpp"))
    hdrs = [os.path.join(host_dir, f) for f in os.listdir(host_dir) if f.endswith((".h", ".hpp"))]
    tag = _digest(sources + hdrs, CXX_FLAGS)
    stamp_file = HOST_LIB + ".stamp"
    if os.path.exists(HOST_LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == tag:
        return HOST_LIB
    if verbose:
        print("[build] compiling host library", file=sys.stderr)
    _compile(["g++"] + CXX_FLAGS + ["-shared", "-o", HOST_LIB] + sources + ["-lpthread"], HOST_LIB,
             os.path.join(OBJ, "host.log"))
    with open(stamp_file, "w") as fh:
        fh.write(tag)
    return HOST_LIB


def build_all(verbose: bool = True, checked: bool = False) -> None:
    build_host(verbose)
    build_cuda(verbose)
    if checked:
        build_cuda(verbose, checked=True)


if __name__ == "__main__":
    build_all(checked="--checked" in sys.argv[1:])
    print(CUDA_LIB)
    if "--checked" in sys.argv[1:]:
        print(CHECKED_LIB)
    print(HOST_LIB)
