"""In-tree build of the C-ABI shared library (nvcc, sm_100a only).

`python -m sglang_security_b200.build` compiles every `csrc/*.cu` into
`sglang_security_b200/lib/libb200hotpath.so`.  nvcc cross-compiles without a GPU, so the
same command is the "does it build" check on the CPU box; the resulting .so is git-ignored but
travels to the GPU box with the working tree.
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
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = PKG_DIR.parent / "build" / "b200_obj"
LIB_PATH = LIB_DIR / "libb200hotpath.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: cannot build libb200hotpath.so")
    return cand


def _newest_dep_mtime() -> float:
    deps = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG_DIR.parent / "include" / "b200_hotpath.h"]
    return max(p.stat().st_mtime for p in deps if p.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    dep_mtime = _newest_dep_mtime()

    def compile_one(src: Path):
        obj = OBJ_DIR / (src.stem + ".o")
        if (not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime
                and obj.stat().st_mtime > dep_mtime):
            return obj, False
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        return obj, True

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [o for o, _ in results]
    rebuilt = any(r for _, r in results)
    if rebuilt or force or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(LIB_PATH), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


def ensure_built() -> Path:
    """Build the library if it is missing or older than its sources (first use in a fresh checkout)."""
    if LIB_PATH.exists():
        newest = max([p.stat().st_mtime for p in CSRC.glob("*.cu")] + [_newest_dep_mtime()])
        if LIB_PATH.stat().st_mtime >= newest:
            return LIB_PATH
    return build()


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(path)
