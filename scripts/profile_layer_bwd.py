"""A few forward+backward passes of one fused layer step, for wrapping in a profiler
(reference: scripts/profile_layer_bwd.py and scripts/profile_gate_w2_bwd.py):

    ncu --set full --clock-control none -k regex:gate_update_bwd -c 1 python scripts/profile_layer_bwd.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.layer import GDLayer  # noqa: E402
from gdnet_b200.utils.fp8 import convert_to_fp8  # noqa: E402

if __name__ == "__main__":
    B, T, d, k = (int(v) for v in (sys.argv[1] if len(sys.argv) > 1 else "8,4096,1024,4").split(","))
    dev = "cuda"
    torch.manual_seed(0)
    layer = convert_to_fp8(GDLayer(d, k).to(dev))
    x = torch.randn(B, T, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    s = torch.randn(B, T, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    for _ in range(3):
        fo, so, gm = layer._step("fwd", x, s, return_gate="mean")
        (fo.float().mean() + so.float().mean() + gm).backward()
    torch.cuda.synchronize()
    print("done")
