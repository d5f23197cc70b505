"""Build the sm_100a extension in-tree: ``gdnet_b200/_C.so``.

``python -m gdnet_b200.build`` compiles every ``csrc/*.cu`` with nvcc for
``compute_100a/sm_100a`` (cross-compiles without a GPU), the binding file with the host
compiler, and links one shared library next to the package. Nothing is installed into
site-packages and no JIT cache is used, so the library travels with the source tree.
Object files are rebuilt only when their source (or a header) is newer.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "_build"
TARGET = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; the sm_100a extension cannot be built")
    return cand


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str], log: Path) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    BUILD.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    cu_files = sorted(CSRC.glob("*.cu"))
    cpp_files = sorted(CSRC.glob("*.cpp"))
    cuda_inc = str(_cuda_home() / "include")
    torch_inc = cpp_extension.include_paths()
    torch_lib = Path(torch.__file__).resolve().parent / "lib"

    jobs = []
    objs = []
    for src in cu_files:
        obj = BUILD / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append(([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                         BUILD / (src.stem + ".log")))
    for src in cpp_files:
        obj = BUILD / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C",
                   f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
                   "-I", str(CSRC), "-I", cuda_inc]
            for inc in torch_inc:
                cmd += ["-isystem", inc]
            cmd += ["-c", str(src), "-o", str(obj)]
            jobs.append((cmd, BUILD / (src.stem + ".log")))

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda j: _run(*j), jobs))
    if jobs or not TARGET.exists():
        link = ["g++", "-shared", "-o", str(TARGET), *map(str, objs),
                f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
                f"-L{_cuda_home() / 'lib64'}", "-lcudart", f"-Wl,-rpath,{torch_lib}"]
        _run(link, BUILD / "link.log")
    if verbose:
        for log in sorted(BUILD.glob("*.log")):
            for line in log.read_text().splitlines():
                if "registers" in line or "spill" in line and "0 bytes spill" not in line:
                    print(f"[{log.stem}] {line.strip()}")
    return TARGET


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
