"""Build the CUDA library in-tree: ``python -m blockgtq_b200.build``.

Compiles every ``csrc/*.cu`` for sm_100a with nvcc and links one shared
library, ``blockgtq_b200/libbgtq.so``, exporting the C ABI of ``include/bgtq.h``.
nvcc cross-compiles without a GPU.  The library links only the CUDA runtime.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.environ.get("BGTQ_LIB") or os.path.join(PKG, "libbgtq.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math=false", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources() -> list:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        [os.path.join(os.path.dirname(PKG), "include", "bgtq.h")]
    return any(os.path.getmtime(d) > t for d in deps)


JIT_SOURCES = ["bgtq_common.cuh", "bgtq_plan.h", "bgtq_decode_kernel.cuh"]


def _embed_jit_sources(objdir: str) -> str:
    """The decode kernel is also compiled at run time from its own text: write each source file it consists of
    as a C++ raw string literal (``<name>.str``) for csrc/bgtq_decode_jit.cu to include."""
    out = os.path.join(objdir, "jit_src")
    os.makedirs(out, exist_ok=True)
    for name in JIT_SOURCES:
        text = open(os.path.join(CSRC, name)).read()
        lines = [ln for ln in text.splitlines()
                 if not ln.startswith("#pragma once") and not ln.startswith('#include "')]
        body = "\n".join(lines)
        assert ')BGTQSRC"' not in body
        with open(os.path.join(out, name + ".str"), "w") as f:
            f.write('R"BGTQSRC(' + body + '\n)BGTQSRC"\n')
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    jit_inc = _embed_jit_sources(objdir)
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + [f for f in NVCC_FLAGS if f != "--use_fast_math=false"] + \
            (["-Xptxas", "-v"] if verbose else []) + os.environ.get("BGTQ_NVCC_EXTRA", "").split() + \
            ["-I", jit_inc, "-c", src, "-o", obj]
        procs.append((obj, cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    objs = []
    for obj, cmd, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + out)
        if verbose:
            sys.stderr.write(out)
        objs.append(obj)
    tmp = LIB + ".tmp"
    cmd = [nvcc, "-shared", "-o", tmp] + objs + ["-cudart", "shared", "-ldl"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if r.returncode != 0:
        raise RuntimeError("link failed: " + r.stdout.decode())
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
