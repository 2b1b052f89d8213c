"""Build libfold_b200.so in-tree with nvcc for sm_100a.

    python fold_attention_b200/build.py [--force] [--verbose]

(run it by path: importing the package loads the library)

Environment: FOLD_NVCC_FLAGS adds compiler flags (for instance
`-DFOLD_BWD_COUNTERS`, which makes the backward's main loop count where each
warp role's cycles go and `fold_bwd_counters` return them), FOLD_LIB_OUT names
another output file (an instrumented build beside the product one).

nvcc cross-compiles without a GPU. The library sits beside this file so it
travels with the source tree; nothing is installed into site-packages.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libfold_b200.so")
STAMP = os.path.join(HERE, "csrc", ".build_stamp")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
] + os.environ.get("FOLD_NVCC_FLAGS", "").split()
if os.environ.get("FOLD_LIB_OUT"):
    LIB = os.path.abspath(os.environ["FOLD_LIB_OUT"])
    STAMP = LIB + ".stamp"


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest():
    h = hashlib.sha256()
    files = _sources() + sorted(
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))
    ) + [os.path.join(ROOT, "include", "fold_b200.h")]
    for p in files:
        h.update(p.encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def nvcc_path():
    for p in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if p and (os.path.sep not in p or os.path.exists(p)):
            return p
    raise RuntimeError("nvcc not found")


def build(force=False, verbose=False):
    """Compile every csrc/*.cu into one shared library. Objects are cached by
    content hash, so a rebuild recompiles only what changed."""
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(STAMP):
        if open(STAMP).read().strip() == digest:
            return LIB
    objdir = os.path.join(HERE, "csrc", "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = nvcc_path()
    inc = ["-I", os.path.join(ROOT, "include"), "-I", CSRC]
    hdr = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h")):
            hdr.update(open(os.path.join(CSRC, f), "rb").read())
    hdr.update(open(os.path.join(ROOT, "include", "fold_b200.h"), "rb").read())
    hdr.update(" ".join(NVCC_FLAGS).encode())
    objs, procs = [], []
    for src in _sources():
        h = hashlib.sha256(hdr.digest() + open(src, "rb").read()).hexdigest()[:16]
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + "." + h + ".o")
        objs.append(obj)
        if os.path.exists(obj) and not force:
            continue
        cmd = [nvcc, *NVCC_FLAGS, *inc, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{out}\n")
        elif verbose or "warning" in out:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-lcudart"]
    subprocess.check_call(cmd)
    # drop objects of older source versions (a side build keeps the product's objects)
    keep = set(objs)
    for f in os.listdir(objdir):
        p = os.path.join(objdir, f)
        if p.endswith(".o") and p not in keep and not os.environ.get("FOLD_LIB_OUT"):
            os.remove(p)
    with open(STAMP, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
