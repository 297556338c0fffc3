#!/usr/bin/env python3
"""Compile the reference's own plugin kernels, from the sources where they lie, into oracle/_ref/.

    python oracle/build_ref.py <reference-root>      (default: $TURBOPI_REFERENCE, else the checkout beside this build)

Test infrastructure: the shared objects are used only by the `-m gpu` parity tests, as the checker for the
plugin quantisers (quantizeWeightToINT4 / dequantizeINT4ToBF16 of openpi/w4a16_plugin/src/w4a16_gemm_kernel.cu,
quantizeActivationToFP8 / quantizeWeightToNVFP4 of openpi/w4a8_plugin/src/w4a8_gemm_kernel.cu) and for the NVFP4 GEMV
(nvfp4_gemv_forward of openpi/nvfp4_packed_plugin/src/nvfp4_packed_kernel.cu).  Each file is one
translation unit built with nvcc against the CUTLASS headers the reference vendors
(openpi/external/cutlass_nvfp4_build/include); nothing of the reference's own build system runs and no source
is copied.  Only the plain-CUDA quantiser entry points are ever called: the files' CUTLASS GEMMs use thread-block
clusters tuned for another chip and stay untouched.  Outputs are git-ignored; an up-to-date output is kept.
"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_REFERENCE = "/root/reference"
OUT = HERE / "_ref"
UNITS = {
    "libref_w4a16.so": "openpi/w4a16_plugin/src/w4a16_gemm_kernel.cu",
    "libref_w4a8.so": "openpi/w4a8_plugin/src/w4a8_gemm_kernel.cu",
    # plain CUDA (no CUTLASS): the plugin's GEMV launcher nvfp4_gemv_forward and its kernels
    "libref_nvfp4_packed.so": "openpi/nvfp4_packed_plugin/src/nvfp4_packed_kernel.cu",
}


def _reference(ref_root):
    return Path(ref_root or os.environ.get("TURBOPI_REFERENCE", DEFAULT_REFERENCE))


def _build_unit(ref, name, rel, verbose):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    inc = ref / "openpi" / "external" / "cutlass_nvfp4_build"
    src, dst = ref / rel, OUT / name
    if dst.exists() and dst.stat().st_mtime > src.stat().st_mtime:
        return dst
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-Xcompiler", "-fPIC",
           "--expt-relaxed-constexpr", "-shared", "-cudart", "shared", "-I", str(inc / "include"),
           "-I", str(inc / "tools" / "util" / "include"), "-o", str(dst), str(src)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    (OUT / (name + ".log")).write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        if verbose:
            print(f"[oracle/build_ref] {rel} does not build here (see oracle/_ref/{name}.log); its entry points stay unpinned")
        return None
    if verbose:
        print(f"[oracle/build_ref] built {dst}")
    return dst


def build(ref_root=None, verbose=True):
    ref = _reference(ref_root)
    if not ref.exists():
        if verbose:
            print(f"[oracle/build_ref] {ref} not present: keeping whatever oracle/_ref/ already holds")
        return []
    OUT.mkdir(exist_ok=True)
    return [d for d in (_build_unit(ref, n, r, verbose) for n, r in UNITS.items()) if d is not None]


# The reference's torch extensions (pybind modules): its production GEMV (nvfp4_gemv_v5 / v6) and the fused QKV
# projection with in-place cache write.  Built with torch.utils.cpp_extension from the sources where they lie, with the
# flag the reference's own loader passes (--use_fast_math, openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:58),
# into oracle/_ref/<name>/; the tests import the finished .so directly (load_torch_ext), no reference checkout needed.
TORCH_EXTS = {
    "ref_nvfp4_gemv_v5": "openpi/nvfp4_packed_plugin/src/nvfp4_gemv_v5.cu",
    "ref_fused_qkv_fp4": "openpi/kv_fuse_plugin/src/fused_qkv_fp4.cu",
    "ref_nvfp4_packed_torch": "openpi/nvfp4_packed_plugin/src/nvfp4_packed_torch.cu",
}


def _build_ext(ref, name, rel, verbose):
    from torch.utils import cpp_extension
    src, bdir = ref / rel, OUT / name
    so = bdir / f"{name}.so"
    if so.exists() and so.stat().st_mtime > src.stat().st_mtime:
        return so
    bdir.mkdir(exist_ok=True)
    try:
        cpp_extension.load(name=name, sources=[str(src)], build_directory=str(bdir), verbose=False,
                           extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math"],
                           is_python_module=False)
    except Exception as e:                           # a checker that does not build leaves its row to the Python pins
        (OUT / (name + ".log")).write_text(str(e))
        if verbose:
            print(f"[oracle/build_ref] {rel} does not build here (see oracle/_ref/{name}.log)")
        return None
    if verbose:
        print(f"[oracle/build_ref] built {so}")
    return so


def build_torch_exts(ref_root=None, verbose=True):
    ref = _reference(ref_root)
    if not ref.exists():
        return []
    OUT.mkdir(exist_ok=True)
    return [d for d in (_build_ext(ref, n, r, verbose) for n, r in TORCH_EXTS.items()) if d is not None]


def build_all(ref_root=None, verbose=True):
    """Every checker, the translation units side by side (each is one compiler run of minutes; nothing is rebuilt
    while its output is newer than its source)."""
    from concurrent.futures import ThreadPoolExecutor
    ref = _reference(ref_root)
    if not ref.exists():
        if verbose:
            print(f"[oracle/build_ref] {ref} not present: keeping whatever oracle/_ref/ already holds")
        return []
    OUT.mkdir(exist_ok=True)
    jobs = [(_build_unit, n, r) for n, r in UNITS.items()] + [(_build_ext, n, r) for n, r in TORCH_EXTS.items()]
    with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
        done = list(pool.map(lambda j: j[0](ref, j[1], j[2], verbose), jobs))
    return [d for d in done if d is not None]


def load_torch_ext(name):
    """Import oracle/_ref/<name>/<name>.so (built by build_torch_exts) as a module, or return None."""
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    so = OUT / name / f"{name}.so"
    if not so.exists():
        return None
    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    build_all(sys.argv[1] if len(sys.argv) > 1 else None)
