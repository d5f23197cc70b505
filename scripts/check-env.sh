#!/usr/bin/env bash
# Environment check for gdnet_b200: toolchain, PyTorch, GPU architecture, the built extension, a kernel smoke run.
# Reference counterpart: scripts/check-env.sh. Exit code 0 = everything needed for training on a B200 is there.
set -u
fail=0
say() { printf '%-34s %s\n' "$1" "$2"; }

py=${PYTHON:-python}
say "python" "$($py -c 'import sys; print(sys.version.split()[0])' 2>&1)"
say "torch" "$($py -c 'import torch; print(torch.__version__, "cuda", torch.version.cuda)' 2>&1)"
if command -v nvcc >/dev/null 2>&1; then
  say "nvcc" "$(nvcc --version | tail -n 2 | head -n 1)"
else
  say "nvcc" "MISSING (needed to build gdnet_b200/_C.so)"; fail=1
fi
if command -v nvidia-smi >/dev/null 2>&1; then
  say "gpu" "$(nvidia-smi --query-gpu=name,compute_cap,memory.total --format=csv,noheader | head -n 1)"
else
  say "gpu" "nvidia-smi not found (CPU-only checks)"
fi

root="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
if [ -f "$root/gdnet_b200/_C.so" ]; then
  say "extension" "gdnet_b200/_C.so present"
else
  say "extension" "not built: run  python gdnet_b200/build.py"; fail=1
fi

$py "$root/scripts/check_abi.py" || fail=1

$py - <<PY || fail=1
import sys
sys.path.insert(0, "$root")
import torch
from gdnet_b200.layer import GDLayer, apply_hard_sn, freeze_sn_iteration
layer = apply_hard_sn(GDLayer(64, 4))
x = torch.randn(1, 16, 64)
with freeze_sn_iteration(layer):
    f, s = layer.fwd_step(x, torch.zeros_like(x))
assert f.shape == x.shape and s.shape == x.shape
print("%-34s %s" % ("layer step (CPU)", "ok"))
if torch.cuda.is_available():
    major, minor = torch.cuda.get_device_capability()
    ok = (major, minor) >= (10, 0)
    print("%-34s %s" % ("tcgen05 / sm_100a kernels", "ok" if ok else "this GPU is sm_%d%d: the kernels need sm_100a" % (major, minor)))
    sys.exit(0 if ok else 1)
PY

if [ "$fail" -eq 0 ]; then echo "environment OK"; else echo "environment INCOMPLETE"; fi
exit "$fail"
