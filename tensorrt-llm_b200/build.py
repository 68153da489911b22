"""Builds libdecode_attn.so (the C-ABI library with every CUDA kernel) in-tree for sm_100a.

nvcc cross-compiles without a GPU, so this runs on a CPU-only box as well.  Objects are rebuilt
only when a source or header they include is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libdecode_attn.so"
CHECKED_BUILD_DIR = PKG_DIR / "build_checked"
CHECKED_LIB_PATH = PKG_DIR / "libdecode_attn_checked.so"

SOURCES = ["dx_attn.cu", "dx_mha_inst.cu", "dx_gqa_inst.cu", "dx_wide_inst.cu", "dx_tok_inst.cu", "dx_tokws_inst.cu",
           "dx_general_inst.cu", "dx_general_more_inst.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return exe


def _newest_dep_mtime() -> float:
    deps = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG_DIR.parent / "include" / "decode_attn.h"]
    return max(p.stat().st_mtime for p in deps)


def _compile(src: str, force: bool, build_dir: Path, extra: list) -> Path:
    obj = build_dir / (Path(src).stem + ".o")
    srcp = CSRC / src
    if not force and obj.exists() and obj.stat().st_mtime >= max(srcp.stat().st_mtime, _newest_dep_mtime()):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(srcp), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (build_dir / (Path(src).stem + ".ptxas.log")).write_text(res.stderr)
    if res.returncode != 0:
        sys.stderr.write(res.stderr)
        raise RuntimeError(f"nvcc failed for {src}")
    return obj


def build(force: bool = False, checked: bool = False) -> Path:
    """checked: the bounds-checked variant (-DDECODE_ATTN_BOUNDS_CHECK, libdecode_attn_checked.so): every block-table
    look-up of the kernels validates index and pointer, records the first violation in the status word and redirects
    the access to a spare block.  A debugging build; the regular library has none of it."""
    build_dir = CHECKED_BUILD_DIR if checked else BUILD_DIR
    lib_path = CHECKED_LIB_PATH if checked else LIB_PATH
    extra = ["-DDECODE_ATTN_BOUNDS_CHECK"] if checked else []
    build_dir.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, build_dir, extra), SOURCES))
    if force or not lib_path.exists() or any(o.stat().st_mtime > lib_path.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(lib_path)]
        cmd += [str(o) for o in objs]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stderr)
            raise RuntimeError("link failed")
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, checked="--checked" in sys.argv))
