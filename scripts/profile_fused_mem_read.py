"""Fused CAM read against the einsum formulation: time and correctness at three sizes
(reference: scripts/profile_fused_mem_read.py). With ``--once`` it launches the kernel a few times on
one size so that a profiler can capture it:

    ncu --set full --clock-control none -k regex:mem_read -c 2 python scripts/profile_fused_mem_read.py --once
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.ops import functional as ops  # noqa: E402
from gdnet_b200.ops import reference as ref  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--once", action="store_true")
    args = ap.parse_args()
    dev = "cuda"
    sizes = [(64, 32, 256, 512)] if args.once else [(8, 32, 128, 256), (64, 32, 256, 512), (256, 64, 512, 1024)]
    for B, S, ds, dc in sizes:
        q, gam, e = torch.randn(B, ds, device=dev), torch.rand(B, ds, device=dev), torch.randn(S, ds, device=dev)
        tags, vals, al = torch.randn(B, S, ds, device=dev), torch.randn(B, S, dc, device=dev), torch.tensor([0.5], device=dev)
        out, w = ops.fused_mem_read(q, gam, e, tags, vals, al)
        out_r, w_r = ref.fused_mem_read(q, gam, e, tags, vals, al)
        err = (out - out_r).abs().max().item()

        def t(fn, n=50):
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n * 1000

        fused = t(lambda: ops.fused_mem_read(q, gam, e, tags, vals, al))
        plain = t(lambda: ref.fused_mem_read(q, gam, e, tags, vals, al))
        print(f"B={B} S={S} d_sig={ds} d_c={dc}: fused {fused:.1f} us, einsum {plain:.1f} us, max err {err:.2e}")


if __name__ == "__main__":
    main()
