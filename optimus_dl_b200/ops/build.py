"""Builds the native sm_100a kernel library of this package, in-tree.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``
into ``ops/lib/obj/*.o`` (in parallel) and linked into ``ops/lib/libob_kernels.so``.
The library exposes a plain C ABI (``extern "C"`` launchers that take raw device
pointers and a ``cudaStream_t``) and is loaded with ``ctypes`` by ``ops/_lib.py``; it
needs no GPU to build.

Run as ``python -m optimus_dl_b200.ops.build`` (add ``-v`` for ptxas statistics).
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

OPS_DIR = Path(__file__).resolve().parent
CSRC = OPS_DIR / "csrc"
LIB_DIR = OPS_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libob_kernels.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str | None:
    cand = shutil.which("nvcc")
    if cand:
        return cand
    for p in ("/usr/local/cuda/bin/nvcc",):
        if os.path.exists(p):
            return p
    return None


def _digest(path: Path, headers: list[Path]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(path.read_bytes())
    for hd in headers:
        h.update(hd.read_bytes())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, headers: list[Path], verbose: bool) -> tuple[Path, bool, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    dig = _digest(src, headers)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj, False, ""
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(dig)
    return obj, True, res.stderr


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile (if stale) and link the kernel library; returns its path."""
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for f in OBJ_DIR.glob("*.sha"):
            f.unlink()
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    with ThreadPoolExecutor(max_workers=min(8, max(1, os.cpu_count() or 1))) as ex:
        results = list(ex.map(lambda s: _compile_one(nvcc, s, headers, verbose), sources))
    objs = [r[0] for r in results]
    changed = any(r[1] for r in results)
    if verbose:
        for r in results:
            if r[2]:
                print(r[2])
    if changed or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


def main() -> None:
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))


if __name__ == "__main__":
    main()
