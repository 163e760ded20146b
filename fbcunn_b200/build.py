"""Builds libfbfftconv.so (the CUDA kernels and the C ABI) for sm_100a, in tree.

    python -m fbcunn_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is written next to this file so
that it travels with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfbfftconv.so")
SOURCES = ["fft_kernels.cu", "contract_simt.cu", "contract_tc.cu", "contract_stream.cu", "bias.cu", "peer.cu", "tiled.cu", "fft1d_lines.cu", "api.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _deps():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    out.append(os.path.join(os.path.dirname(HERE), "include", "fbfftconv.h"))
    return out


def _digest() -> str:
    h = hashlib.sha256()
    for path in sorted(_deps()):
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _up_to_date(digest: str) -> bool:
    stamp = LIB + ".stamp"
    if not (os.path.exists(LIB) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == digest


def build(force: bool = False, verbose: bool = False) -> str:
    """Rebuilds when the sources' content hash differs from the one the library was
    built from (file times do not survive a copy of the tree).  Safe to call from
    several processes at once (the ranks of a multi-GPU job): one of them builds
    under a file lock, the others wait and find the library up to date; the library
    appears under its name only when it is complete."""
    digest = _digest()
    if not force and _up_to_date(digest):
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    with open(os.path.join(OBJ, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and _up_to_date(digest):
                return LIB  # another process built it while this one waited
            _build_locked(digest, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


def _build_locked(digest: str, verbose: bool) -> None:
    stamp = LIB + ".stamp"
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    if os.path.exists(stamp):
        os.remove(stamp)  # no stamp while objects and library are in flux

    def compile_one(src):
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    tmp = os.path.join(OBJ, "libfbfftconv.so.tmp")
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB)
    with open(stamp + ".tmp", "w") as f:
        f.write(digest)
    os.replace(stamp + ".tmp", stamp)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
