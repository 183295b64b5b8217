"""Stage the reference's own Python sources under ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py --reference /path/to/H3-Optimizations

The reference (Pizzawookiee/H3-Optimizations) is pure Python: there is nothing
to compile.  "Building" it means placing its ``h3_optimizations`` package and
its ``benchmarks`` directory, unmodified, where the checker can import them on
a machine that has no checkout of the reference (``oracle/_ref/`` is ignored by
git, so no reference source ever enters this repository's history).  The
package uses lazy exports, so the modules that need ComfyUI are never imported
as long as only these are touched:

    h3_optimizations.attention.sparse.router              SparseTileRouter
    h3_optimizations.attention.sparse.config              HybridSparseConfig, resolve_video_budget
    h3_optimizations.attention.sparse.triton_route        build_compact_absolute_route
    h3_optimizations.attention.sparse.sparse_sage         _quantize_blocks
    h3_optimizations.attention.sparse.triton_sparse_kernels   launch_int8_sparse (Triton, GPU only)
    benchmarks/bench_sparse_backends.py                   sparse_float_reference, absolute_lut

``oracle.ref_bridge`` imports them from the staged copy.  What is staged is
used as a checker and as the timed CPU baseline, never by the product package.
"""

from __future__ import annotations

import argparse
import hashlib
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
TREES = ("h3_optimizations", "benchmarks")


def _tree_digest(root):
    digest = hashlib.sha256()
    for path in sorted(root.rglob("*.py")):
        digest.update(str(path.relative_to(root)).encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def stage(reference, target=TARGET):
    """Copy the reference's Python trees to ``target``; returns the target."""
    reference = Path(reference)
    missing = [name for name in TREES if not (reference / name).is_dir()]
    if missing:
        raise FileNotFoundError("%s has no %s directory" % (reference, " / ".join(missing)))
    target.mkdir(exist_ok=True)
    stamp = target / "SOURCE.txt"
    digests = {name: _tree_digest(reference / name) for name in TREES}
    wanted = "".join("%s %s\n" % (name, digests[name]) for name in TREES)
    if stamp.exists() and stamp.read_text() == wanted and all((target / name).is_dir() for name in TREES):
        return target
    for name in TREES:
        destination = target / name
        if destination.exists():
            shutil.rmtree(destination)
        shutil.copytree(reference / name, destination, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    stamp.write_text(wanted)
    return target


def main():
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--reference", required=True, help="checkout of Pizzawookiee/H3-Optimizations")
    args = parser.parse_args()
    print(stage(args.reference))
    return 0


if __name__ == "__main__":
    sys.exit(main())
