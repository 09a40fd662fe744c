"""Build the CUDA library in-tree: nvcc for sm_100a only, one shared object `libdm_b200.so` next to this file.

    python -m delta_matching_b200.build [--force] [--verbose]

The library exports the C ABI declared in include/dm_b200.h and links only against the CUDA runtime (the driver entry
point for tensor-map encoding is resolved at run time), so it builds on a machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libdm_b200.so")
SOURCES = ("dm_abi.cu", "dm_quant.cu", "dm_fwd.cu", "dm_delta.cu", "dm_bwd.cu", "dm_bwd_p2.cu", "dm_probe.cu", "dm_static_scratch.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.isfile(cand)):
            return cand
    return "nvcc"


def source_files():
    out = []
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(CSRC, f))
    out.append(os.path.join(os.path.dirname(HERE), "include", "dm_b200.h"))
    return out


def code_sha() -> str:
    """12 hex characters of a hash over the kernel sources (the stamp kernel_version() reports)."""
    h = hashlib.sha256()
    for f in source_files():
        if os.path.isfile(f):
            h.update(os.path.basename(f).encode())
            h.update(open(f, "rb").read())
    return h.hexdigest()[:12]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link (skipped when the library is newer than a stamp of the sources' hash)."""
    obj_dir = OBJ
    lib = LIB
    os.makedirs(obj_dir, exist_ok=True)
    stamp = os.path.join(obj_dir, "stamp.txt")
    sha = code_sha()
    if not force and os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == sha:
        return lib
    srcs = list(SOURCES)
    nvcc = _nvcc()
    flags = NVCC_FLAGS

    def compile_one(src):
        obj = os.path.join(obj_dir, src[:-3] + ".o")
        cmd = [nvcc, *flags, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    r = subprocess.run([nvcc, "-shared", "-o", lib, *objs, "-lcudart"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as fh:
        fh.write(sha + "\n")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
