"""In-tree build of the sm_100a extension.

Every ``csrc/*.cu`` is compiled with nvcc for ``compute_100a/sm_100a`` and linked
into ``b200moe/_C/libb200moe.so``, which ``b200moe.ops.native`` loads through
ctypes.  The sources use only the CUDA runtime (the one driver entry point they
need, ``cuTensorMapEncodeTiled``, is resolved at run time), so the library
builds on a machine without a GPU or a driver.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
# B200MOE_DEBUG=1 selects the checked build: -DB200MOE_DEBUG (range checks on data-dependent indices, see
# csrc/debug.cuh), its own object directory and library name, loaded by b200moe.ops.native under the same variable.
DEBUG = os.environ.get("B200MOE_DEBUG", "0") not in ("", "0")
OUT = os.path.join(HERE, "_C", "debug") if DEBUG else os.path.join(HERE, "_C")
LIB = os.path.join(OUT, "libb200moe_debug.so" if DEBUG else "libb200moe.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v"] + (["-DB200MOE_DEBUG"] if DEBUG else [])


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found")
    return found


def _sources():
    return sorted(f for f in os.listdir(SRC) if f.endswith(".cu"))


def _digest(path: str) -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(SRC)):
        if name.endswith((".cuh", ".h")) or os.path.join(SRC, name) == path:
            with open(os.path.join(SRC, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(name: str, verbose: bool) -> str:
    src = os.path.join(SRC, name)
    obj = os.path.join(OUT, name[:-3] + ".o")
    stamp = obj + ".sha"
    digest = _digest(src)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest:
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = obj[:-2] + ".ptxas.log"
    with open(log, "w") as f:
        f.write(proc.stdout + proc.stderr)
    if proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"nvcc failed for {name}")
    with open(stamp, "w") as f:
        f.write(digest)
    if verbose:
        print(f"[b200moe.build] compiled {name}")
    return obj


def build_all(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    if force:
        for name in os.listdir(OUT):
            if name.endswith((".o", ".sha", ".so")):
                os.unlink(os.path.join(OUT, name))
    names = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(names) or 1)) as pool:
        objects = list(pool.map(lambda n: _compile(n, verbose), names))
    newest = max(os.path.getmtime(o) for o in objects)
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        cmd = [nvcc(), "-shared", "-o", LIB, *objects, "-Xcompiler", "-fPIC", "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("link failed")
        if verbose:
            print(f"[b200moe.build] linked {LIB}")
    return LIB


if __name__ == "__main__":
    build_all(verbose=True, force="--force" in sys.argv)
