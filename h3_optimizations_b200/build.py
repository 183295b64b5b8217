"""In-tree build of the native library: nvcc -> ``_lib/libh3sparse.so``.

Only sm_100a code is generated.  The CUDA runtime is linked statically and the
driver API is resolved at run time, so the library loads on a machine without a
GPU driver (symbol checks) while every compute entry point still needs a B200.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "_lib"
LIB_PATH = LIB_DIR / "libh3sparse.so"
SOURCES = ("api.cu", "quant.cu", "router.cu", "attn_tc.cu", "attn_mma.cu", "qkv_gemm.cu")

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
)


def _nvcc():
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return found


def _existing_sources():
    return [CSRC / name for name in SOURCES if (CSRC / name).exists()]


def _fingerprint(sources):
    digest = hashlib.sha256()
    for path in sorted(list(sources) + list(CSRC.glob("*.cuh")) + [PACKAGE_DIR.parent / "include" / "h3sparse.h"]):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def build(force=False, verbose=False):
    """Compile every CUDA source for sm_100a and link the shared library.
    Returns the library path.  Skips the work when sources are unchanged."""
    sources = _existing_sources()
    LIB_DIR.mkdir(exist_ok=True)
    stamp = LIB_DIR / "build.stamp"
    fingerprint = _fingerprint(sources)
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text() == fingerprint:
        return LIB_PATH
    nvcc = _nvcc()
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)

    def compile_one(src):
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src.name, proc.stderr))
        if verbose:
            sys.stderr.write(proc.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources))
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH)]
    link += [str(o) for o in objects]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed:\n%s" % proc.stderr)
    stamp.write_text(fingerprint)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
