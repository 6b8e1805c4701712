"""Builds ``libaeris_b200.so`` in-tree from the ``csrc/*.cu`` sources with plain nvcc for sm_100a.

The library exposes a C ABI (``csrc/api.h``) and is loaded with ctypes, so no torch headers are compiled and a
full rebuild takes seconds. Cross-compilation needs no GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
# AERIS_BOUNDS_CHECK=1 selects the checking build (-DAERIS_BOUNDS_CHECK): every gather code and push owner is
# validated on the device, a bad one is recorded in the status word and the access skipped. It stands in for a
# memory checker on machines where none can be run; it is a library of its own so both can sit side by side.
CHECKED = os.environ.get("AERIS_BOUNDS_CHECK") == "1"
LIB_PATH = CSRC / ("libaeris_b200_chk.so" if CHECKED else "libaeris_b200.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
] + (["-DAERIS_BOUNDS_CHECK"] if CHECKED else [])


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def needs_build() -> bool:
    stamp = CSRC / ("build_chk" if CHECKED else "build") / "digest.txt"
    return not (LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == _digest())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu to an object (in parallel) and link the shared library. Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    out_dir = CSRC / ("build_chk" if CHECKED else "build")
    out_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: Path) -> tuple[Path, str]:
        obj = out_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(_sources()) or 1)) as ex:
        results = list(ex.map(compile_one, _sources()))
    log = "\n".join(f"== {o.name}\n{err}" for o, err in results)
    (out_dir / "ptxas.log").write_text(log)
    if verbose:
        print(log)
    objs = [str(o) for o, _ in results]
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    (out_dir / "digest.txt").write_text(_digest())
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
