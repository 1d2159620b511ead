"""In-tree build of the native library.

Every ``.cu`` / ``.cpp`` under ``idrak_b200/csrc`` is compiled for sm_100a with
nvcc and linked into ``idrak_b200/lib/libidrak_b200.so``. The library exports a
flat C ABI (``extern "C"``) that ``idrak_b200._native`` loads with ctypes, so the
kernels do not depend on the PyTorch C++ headers and a file compiles in seconds.

Objects are rebuilt only when their source (or a header) is newer than the
object. ``python -m idrak_b200.build`` builds from the command line.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "lib"
OBJDIR = LIBDIR / "obj"
LIBNAME = "libidrak_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-DNDEBUG",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("IDRAK_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set IDRAK_NVCC")


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.hpp"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, obj: Path, verbose: bool) -> tuple[Path, int, str]:
    cmd = [nvcc_path(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    return src, proc.returncode, proc.stdout + proc.stderr


def build(force: bool = False, verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile what is stale and link the shared library. Returns its path."""
    OBJDIR.mkdir(parents=True, exist_ok=True)
    lib = LIBDIR / LIBNAME
    hdr = _newest_header()
    todo = []
    objs = []
    for src in sources():
        obj = OBJDIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr):
            todo.append((src, obj))
    if todo:
        jobs = jobs or min(len(todo), os.cpu_count() or 4)
        with ThreadPoolExecutor(max_workers=jobs) as pool:
            for src, rc, out in pool.map(lambda so: _compile(so[0], so[1], verbose), todo):
                if verbose and out.strip():
                    print(f"--- {src.name}\n{out}", file=sys.stderr)
                if rc != 0:
                    raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    if todo or not lib.exists():
        cmd = [nvcc_path(), "-shared", "-o", str(lib), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart", "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}{proc.stderr}")
    return lib


def is_built() -> bool:
    return (LIBDIR / LIBNAME).exists()


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
