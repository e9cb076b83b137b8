"""Builds libsnnb200.so (sm_100a only) from csrc/*.cu with nvcc.

Usage: ``python -m triton_snn_fusion_b200.build [--force] [--verbose]``.
The objects go to ``csrc/build/`` and the shared library next to this file, so
the built library travels with the source tree.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = CSRC / "build"
LIB_PATH = PKG_DIR / "libsnnb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    # no --use_fast_math and no -fmad override: the LIF update uses explicit
    # round-to-nearest intrinsics where contraction would change results.
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG_DIR.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool, ptxas_v: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if ptxas_v:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    out = (proc.stdout + proc.stderr).strip()
    if verbose and out:
        print(f"--- {src.name}\n{out}")
    return out


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link libsnnb200.so. Returns its path."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _headers_mtime()
    src_m = max((s.stat().st_mtime for s in _sources()), default=0.0)
    if not force and not ptxas_v and LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= max(src_m, hdr_m):
        return LIB_PATH   # the library is newer than every source (object files may be absent: they need not travel)
    jobs = []
    objs = []
    for src in _sources():
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or ptxas_v or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, verbose, ptxas_v) for s, o in jobs]
            for f in futs:
                f.result()
    need_link = bool(jobs) or not LIB_PATH.exists() or any(o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs)
    if need_link:
        # link beside the target and rename: a reader never sees a half-written library
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart", "-ldl"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        tmp.replace(LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_v="--ptxas-v" in sys.argv)
    print(path)
