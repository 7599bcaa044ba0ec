"""Build recipe for libpi05_b200.so (sm_100a only).

Each .cu under csrc/ is compiled to an object in csrc/build/ (parallel nvcc
processes) and linked into apxinf_b200/libpi05_b200.so, in-tree. nvcc
cross-compiles without a GPU. Run as `python -m apxinf_b200.build`.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "libpi05_b200.so"
BENCH_EXE = PKG / "pi05_bench"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-O3,-pthread",
    "--expt-relaxed-constexpr",
]
# extra compiler flags for experiments (e.g. -DNAME, -Xptxas -v); never set for the library that
# is shipped
NVCC_FLAGS += os.environ.get("PI05_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libpi05_b200.so cannot be built")
    return exe


def _deps_digest(src: Path) -> str:
    """Digest of a source and every header beside it (cheap whole-dir rule)."""
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for header in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
                         + list((PKG.parent / "include").glob("*.h"))
                         + list(CSRC.glob("*.inc"))):
        h.update(header.read_bytes())
    return h.hexdigest()


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    stamp = OBJ / (src.stem + ".sha")
    digest = _deps_digest(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    stamp.write_text(digest)
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for stale in OBJ.glob("*.sha"):
            stale.unlink()
    lib_sources = sorted(p for p in CSRC.glob("*.cu"))
    cli_sources = sorted(p for p in CSRC.glob("*.cc"))
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), lib_sources))
    newest = max(o.stat().st_mtime for o in objs)
    if not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *[str(o) for o in objs],
               "-Xcompiler", "-fPIC", "-Xlinker", "--no-undefined", "-lpthread", "-ldl"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    for src in cli_sources:
        exe = PKG / src.stem
        if not exe.exists() or exe.stat().st_mtime < max(src.stat().st_mtime, LIB.stat().st_mtime):
            cmd = ["g++", "-O2", "-std=c++17", "-I", str(PKG.parent / "include"), str(src),
                   "-o", str(exe), "-L", str(PKG), "-lpi05_b200", "-Wl,-rpath,$ORIGIN", "-lpthread"]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"g++ failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(path)
