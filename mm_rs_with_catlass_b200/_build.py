"""In-tree build of ``libcatcoc_b200.so`` with nvcc for sm_100a.

The library is a plain C-ABI shared object (no Python or torch headers), loaded through
ctypes by :mod:`mm_rs_with_catlass_b200._native`. Building takes a few seconds and needs no
GPU; the result is written next to the sources under ``_lib/`` so it travels with the tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "_lib"
LIB_PATH = LIB_DIR / "libcatcoc_b200.so"
STAMP_PATH = LIB_DIR / "build.stamp"
# the same sources with -DCATCOC_CHECKED: every workspace / peer / output / TMEM offset of the kernels is
# compared with the extent of its buffer, a violation is recorded in the status block and the access skipped
CHECKED_LIB_PATH = LIB_DIR / "libcatcoc_b200_checked.so"
CHECKED_STAMP_PATH = LIB_DIR / "build_checked.stamp"


def lib_path(checked: bool = False) -> Path:
    return CHECKED_LIB_PATH if checked else LIB_PATH

SOURCES = [
    "kernels/launch.cu",
    "kernels/inst/f16_single.cu",
    "kernels/inst/f16_pair.cu",
    "kernels/inst/i8_single.cu",
    "kernels/inst/i8_pair.cu",
    "kernels/inst/f8_single.cu",
    "kernels/inst/f8_pair.cu",
    "kernels/inst/mx_single.cu",
    "kernels/shmem_prims.cu",
    "kernels/no_alloc.cu",
    "kernels/blas_prims.cu",
    "kernels/small_allreduce.cu",
    "kernels/flash_attn.cu",
    "kernels/mla_decode.cu",
    "shmem/host.cu",
    "oracle/oracle.cpp",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def _extra_flags() -> list[str]:
    """Extra nvcc flags for experiments (``CATCOC_NVCC_EXTRA="-DFOO=1 -DBAR"``); part of the digest."""
    return os.environ.get("CATCOC_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    cand = os.environ.get("CATCOC_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set CATCOC_NVCC")
    return cand


def _existing_sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def source_digest() -> str:
    h = hashlib.sha256()
    files = sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))
                   + list(CSRC.rglob("*.cpp")))
    for f in files:
        h.update(str(f.relative_to(CSRC)).encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS + _extra_flags()).encode())
    return h.hexdigest()


def is_current(checked: bool = False) -> bool:
    lib, stamp = (CHECKED_LIB_PATH, CHECKED_STAMP_PATH) if checked else (LIB_PATH, STAMP_PATH)
    return lib.exists() and stamp.exists() and stamp.read_text().strip() == source_digest()


def _compile_one(src: Path, obj: Path, verbose: bool, checked: bool = False) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, *_extra_flags(), *(["-DCATCOC_CHECKED=1"] if checked else []),
           "-I", str(CSRC / "include"), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), proc.stderr[-8000:]))
    return proc.stderr


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    """Compile every CUDA source of the package for sm_100a and link one shared library. The
    translation units (one per kernel flavour) compile in parallel. ``checked`` builds the
    bounds-checked variant next to the normal one."""
    LIB_PATH, STAMP_PATH = (CHECKED_LIB_PATH, CHECKED_STAMP_PATH) if checked else (globals()["LIB_PATH"], globals()["STAMP_PATH"])
    if not force and is_current(checked):
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / ("obj%d%s" % (os.getpid(), "c" if checked else ""))
    obj_dir.mkdir(exist_ok=True)
    sources = _existing_sources()
    objs = [obj_dir / (s.relative_to(CSRC).as_posix().replace("/", "_") + ".o") for s in sources]
    tmp = LIB_PATH.with_suffix(".so.tmp%d" % os.getpid())
    try:
        workers = max(1, min(len(sources), os.cpu_count() or 1, int(os.environ.get("CATCOC_BUILD_JOBS", "8"))))
        with ThreadPoolExecutor(max_workers=workers) as pool:
            logs = list(pool.map(lambda so: _compile_one(so[0], so[1], verbose, checked), zip(sources, objs)))
        if verbose:
            sys.stderr.write("".join(logs))
        link = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
                *[str(o) for o in objs], "-o", str(tmp)]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (" ".join(link), proc.stderr[-8000:]))
        os.replace(tmp, LIB_PATH)
    finally:
        tmp.unlink(missing_ok=True)
        shutil.rmtree(obj_dir, ignore_errors=True)
    STAMP_PATH.write_text(source_digest())
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv))
