"""Builds libpaged_attention_b200.so (the product) and libpaged_attention_b200_test_aids.so
(test and measurement aids) in-tree with nvcc for sm_100a.

Usage: ``python -m flash_attention_factory_b200.build [--force] [--verbose]``.
The library is plain CUDA C++ behind a C ABI (include/paged_attention_b200.h);
it does not link against torch.  Each launcher is its own translation unit so
the files compile in parallel.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
INCLUDE = REPO_ROOT / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libpaged_attention_b200.so"
AIDS_LIB_PATH = PKG_DIR / "libpaged_attention_b200_test_aids.so"

SOURCES = [
    "host_common.cu",
    "c_api.cu",
    "host_step.cu",
    "multi_gpu.cu",
    "launch_kernels_loop.cu",
    "launch_kernels_reduce.cu",
    "launch_kernels_fp8_loop.cu",
    "launch_kernels_fp8_reduce.cu",
    "cache_write.cu",
]
# the aid library links its own copy of the shared host pieces and nothing of the product
AIDS_SOURCES = ["host_common.cu", "test_aids.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def find_nvcc() -> str:
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return nvcc


def _newest_mtime(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def needs_build() -> bool:
    if not LIB_PATH.exists() or not AIDS_LIB_PATH.exists():
        return True
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h*"))
    return _newest_mtime(deps) > min(LIB_PATH.stat().st_mtime, AIDS_LIB_PATH.stat().st_mtime)


def _compile_one(nvcc: str, src: str, verbose: bool, defines=(), build_dir: Path = BUILD_DIR) -> Path:
    obj = build_dir / (Path(src).stem + ".o")
    cmd = [nvcc, *NVCC_FLAGS, *defines, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(CSRC / src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles and links the shared library; returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = find_nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    every = list(dict.fromkeys(SOURCES + AIDS_SOURCES))
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(every)) as pool:
        objs = dict(zip(every, pool.map(lambda s: _compile_one(nvcc, s, verbose), every)))
    for target, sources in ((LIB_PATH, SOURCES), (AIDS_LIB_PATH, AIDS_SOURCES)):
        link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                "-o", str(target), *(str(objs[s]) for s in sources)]
        res = subprocess.run(link, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


def build_variant(name: str, defines) -> Path:
    """Builds the product library once more with extra -D flags as
    libpaged_attention_b200_<name>.so (measuring aids such as -DPA_TIMELINE, tuning builds with
    -DPA_TUNING_KNOBS); `PA_B200_LIBRARY_VARIANT=<name>` makes the package load it."""
    nvcc = find_nvcc()
    bdir = PKG_DIR / f"build_{name}"
    bdir.mkdir(exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(lambda s: _compile_one(nvcc, s, False, list(defines), bdir), SOURCES))
    target = PKG_DIR / f"libpaged_attention_b200_{name}.so"
    res = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(target),
                          *map(str, objs)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return target


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / smem usage")
    ap.add_argument("--timeline", action="store_true",
                    help="also build libpaged_attention_b200_timeline.so (-DPA_TIMELINE: per-CTA time stamps)")
    ap.add_argument("--bounds", action="store_true",
                    help="also build libpaged_attention_b200_bounds.so (-DPA_DEBUG_BOUNDS: range-checked indices)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    if a.timeline:
        print(build_variant("timeline", ["-DPA_TIMELINE"]))
    if a.bounds:
        print(build_variant("bounds", ["-DPA_DEBUG_BOUNDS"]))


if __name__ == "__main__":
    main()
