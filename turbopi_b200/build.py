"""Build libturbopi_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m turbopi_b200.build [--force]

Every .cu under csrc/ is one translation unit; objects are compiled in parallel
into csrc/_obj/ and linked into lib/libturbopi_b200.so.  A unit is recompiled only
when it or a header it can see is newer than its object.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "_obj"
LIB = PKG / "lib" / "libturbopi_b200.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return exe


def _newest_header():
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src, force):
    obj = OBJ / (src.stem + ".o")
    if (not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime
            and obj.stat().st_mtime > _newest_header()):
        return src.name, "up to date", ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ / (src.stem + ".log")).write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stderr[-4000:]}")
    return src.name, "compiled", r.stderr


def build(force=False, verbose=False):
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError("no CUDA sources found")
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(lambda s: _compile(s, force), sources))
    changed = any(state == "compiled" for _, state, _ in results)
    if verbose:
        for name, state, _ in results:
            print(f"[turbopi_b200.build] {name}: {state}")
    objs = [str(OBJ / (s.stem + ".o")) for s in sources]
    stale = not LIB.exists() or any(os.path.getmtime(o) > LIB.stat().st_mtime for o in objs)
    if changed or stale:
        cmd = [_nvcc(), "-shared", "-cudart", "shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
        if verbose:
            print(f"[turbopi_b200.build] linked {LIB}")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
