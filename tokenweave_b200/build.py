"""In-tree build of the native library ``tokenweave_b200/_C.so`` for sm_100a.

Every ``csrc/*.cu`` is compiled by nvcc with ``-gencode arch=compute_100a,code=sm_100a`` and the
objects are linked into one shared library next to the package, so the library travels with the
source tree. The kernels expose plain C launchers (``csrc/tw_kernels.h``); Python reaches them
through ctypes (``tokenweave_b200/ops/_native.py``), so no PyTorch header is compiled and a full
rebuild takes seconds.

Usage: ``python -m tokenweave_b200.build [--force] [--verbose]``
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
LIB_PATH = PKG_DIR / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    if cand.exists():
        return str(cand)
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found (set CUDA_HOME)")
    return found


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, obj: Path, log: Path, verbose: bool) -> None:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what changed and link ``_C.so``. Returns the library path."""
    nvcc = _nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    digest = _headers_digest()
    stamp = BUILD_DIR / "headers.sha256"
    headers_changed = force or not stamp.exists() or stamp.read_text() != digest
    jobs = []
    objs = []
    for src in _sources():
        obj = BUILD_DIR / (src.stem + ".o")
        objs.append(obj)
        if headers_changed or not obj.exists() or obj.stat().st_mtime < src.stat().st_mtime:
            jobs.append((src, obj, BUILD_DIR / (src.stem + ".log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, l, verbose) for s, o, l in jobs]
            for f in futs:
                f.result()
    need_link = bool(jobs) or not LIB_PATH.exists() or any(
        o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs)
    if need_link:
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode",
               "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, LIB_PATH)
    stamp.write_text(digest)
    return LIB_PATH


def resource_usage() -> str:
    """Registers / spills / shared memory per kernel as reported by ``ptxas -v`` at build time."""
    out = []
    for log in sorted(BUILD_DIR.glob("*.log")):
        out.append(f"== {log.stem}")
        out.append(log.read_text())
    return "\n".join(out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))
