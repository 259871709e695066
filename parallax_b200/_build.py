"""In-tree build of the sm_100a kernel library (``parallax_b200/_C/libpxl_kernels.so``).

The kernel sources under ``csrc/`` expose a C ABI and include no PyTorch headers, so each
translation unit compiles in a few seconds with plain ``nvcc``; the Python side binds the
symbols with ``ctypes``. The library is kept inside the package directory so that a source
checkout carries its own binaries from the build machine to the GPU machine.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parent.parent
CSRC = REPO_ROOT / "csrc"
OUT_DIR = Path(__file__).resolve().parent / "_C"
LIB_NAME = "libpxl_kernels.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(paths: list[Path]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path() -> Path:
    return OUT_DIR / LIB_NAME


def is_fresh() -> bool:
    stamp = OUT_DIR / "build.stamp"
    if not lib_path().exists() or not stamp.exists():
        return False
    deps = _sources() + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    return stamp.read_text().strip() == _digest(deps)


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link them into one shared library."""
    if not force and is_fresh():
        return lib_path()
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    srcs = _sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    hdr_digest = _digest(headers)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        tag = obj_dir / (src.stem + ".tag")
        want = _digest([src]) + hdr_digest
        if not force and obj.exists() and tag.exists() and tag.read_text() == want:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}")
        tag.write_text(want)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    link = [nvcc, "-shared", "-o", str(lib_path()), *map(str, objs)]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link of libpxl_kernels.so failed")
    (OUT_DIR / "build.stamp").write_text(_digest(srcs + headers))
    return lib_path()


if __name__ == "__main__":
    p = build_kernels(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(p)
