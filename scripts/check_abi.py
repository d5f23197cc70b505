"""Environment check: versions, GPU capability, extension build and a one-kernel smoke test.

    python scripts/check_abi.py [--build]

Reports python / torch / CUDA / NCCL versions, the GPUs and whether they are sm_100 (the kernels are
built for sm_100a only), whether ``gdnet_b200/_C.so`` exists and loads, and on a GPU box launches one
tensor-core GEMM and one quantiser and compares them with PyTorch. Exit code 0 = usable.
Reference counterpart: scripts/check_abi.py and scripts/check-env.sh.
"""

from __future__ import annotations

import argparse
import os
import platform
import shutil
import subprocess
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--build", action="store_true", help="build the extension first")
    args = ap.parse_args()
    ok = True
    import torch

    print(f"python   {platform.python_version()}")
    print(f"torch    {torch.__version__}  (cuda {torch.version.cuda}, nccl {'.'.join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else 'n/a'})")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if os.path.exists(nvcc):
        print("nvcc     " + subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.strip().splitlines()[-1])
    else:
        print("nvcc     not found (needed only to build)")
    for mod in ("yaml", "numpy", "pynvml", "tiktoken", "datasets", "wandb"):
        try:
            __import__(mod)
            print(f"{mod:<8} ok")
        except Exception as exc:
            print(f"{mod:<8} missing ({type(exc).__name__}) - optional" if mod in ("tiktoken", "datasets", "wandb", "pynvml") else f"{mod:<8} MISSING")
            ok = ok and mod in ("tiktoken", "datasets", "wandb", "pynvml")

    from gdnet_b200 import _ext

    if args.build:
        from gdnet_b200.build import build

        print(f"built    {build()}")
    print(f"ext      {_ext.lib_path()} {'present' if _ext.available() else 'ABSENT: run python -m gdnet_b200.build'}")
    if not torch.cuda.is_available():
        print("gpu      none visible: CPU paths only")
        return 0 if ok else 1
    for i in range(torch.cuda.device_count()):
        cap = torch.cuda.get_device_capability(i)
        name = torch.cuda.get_device_name(i)
        good = cap[0] == 10
        ok = ok and good
        print(f"gpu[{i}]   {name} sm_{cap[0]}{cap[1]} {'ok' if good else 'UNSUPPORTED: kernels are sm_100a only'}")
    if not _ext.available():
        return 1
    from gdnet_b200.ops import cuda as cu

    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    err = (cu.gemm_bf16(a, b).float() - a.float() @ b.float().t()).abs().max().item()
    q, s = cu.quantize_rows(a)
    torch.cuda.synchronize()
    _ext.check_status(a)
    print(f"smoke    tcgen05 GEMM max err {err:.3f}, quantiser scales {tuple(s.shape)}")
    return 0 if ok and err < 1.0 else 1


if __name__ == "__main__":
    sys.exit(main())
