"""Builds libtgdn_b200.so (sm_100a only) from csrc/*.cu with nvcc, in-tree.

    python -m cute_triadic_gdn_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects are cached under csrc/build/ and rebuilt when a source or header changes.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "libtgdn_b200.so")
BUILD = os.path.join(CSRC, "build")

# sm_100a (B200) is the target and the default.  TGDN_ARCHS="100a,103a" adds the B300 flavour of the same kernels to the
# library (the family-specific tcgen05 / TMA instructions need an architecture-specific build per member of the family;
# the device check of the library admits every compute capability 10.x).  The 103a flavour compiles here; it has not run.
ARCHS = [a.strip() for a in os.environ.get("TGDN_ARCHS", "100a").split(",") if a.strip()]
NVCC_FLAGS = [f for a in ARCHS for f in ("-gencode", f"arch=compute_{a},code=sm_{a}")] + \
             ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libtgdn_b200.so cannot be built")
    return exe


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest():
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for root in (CSRC, os.path.join(PKG, "..", "include")):
        for f in sorted(os.listdir(root)):
            if f.endswith((".cu", ".cuh", ".h")):
                with open(os.path.join(root, f), "rb") as fh:
                    h.update(f.encode() + fh.read())
    return h.hexdigest()


def up_to_date():
    """True when the library on disk was linked from the sources as they are now."""
    stamp = os.path.join(BUILD, "digest.txt")
    return os.path.exists(OUT) and os.path.exists(stamp) and open(stamp).read() == _digest()


def build(force=False, verbose=False):
    """Compile every .cu for sm_100a and link the shared library; returns its path.  Concurrent callers (one per rank) are
    serialised by a lock file; whoever comes second finds the work done."""
    if not force and up_to_date():
        return OUT
    os.makedirs(BUILD, exist_ok=True)
    import fcntl
    with open(os.path.join(BUILD, "lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and up_to_date():
                return OUT
            return _build_locked(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose):
    stamp = os.path.join(BUILD, "digest.txt")
    digest = _digest()
    nvcc = _nvcc()

    def compile_one(src):
        obj = os.path.join(BUILD, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        with open(os.path.join(BUILD, src[:-3] + ".log"), "w") as fh:
            fh.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    tmp = OUT + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, OUT)                               # atomic: a concurrent dlopen sees the old or the new file, never half of one
    with open(stamp, "w") as fh:
        fh.write(digest)
    return OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
