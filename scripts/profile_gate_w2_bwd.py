"""Time the backward of the gate path of one layer step kernel by kernel (CUDA events).

    python scripts/profile_gate_w2_bwd.py [--B 4] [--T 512] [--d 512] [--iters 50]

What the reference's ``gate_w2_bwd`` (one elementwise kernel, a recomputed RMSNorm and two cuBLAS GEMMs,
gdnet/kernel/gated_causal_depthwise_conv/gate_norm.py:193-237; profiled by scripts/profile_gate_w2_bwd.py) does
is here: the two stream-update backward kernels (row statistics; outputs and column sums), the weight gradient
``dq^T h`` (bf16, operands read in place), the un-folding of the norm weight, and the data gradient with the
RMSNorm / silu backward in its epilogue.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from gdnet_b200.ops import cuda as cu

    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=4)
    ap.add_argument("--T", type=int, default=512)
    ap.add_argument("--d", type=int, default=512)
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    dev, bf, f32 = "cuda", torch.bfloat16, torch.float32
    M, d = args.B * args.T, args.d
    torch.manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device=dev, dtype=bf)  # noqa: E731
    dF, dS, g_pre, z, c, s, h, hg_pre = (rnd(M, d) for _ in range(8))
    W2 = rnd(d, d) * 0.05
    gnw, w_r, b2 = torch.ones(d, device=dev), torch.ones(d, device=dev), torch.full((d,), 2.0, device=dev)
    rstd = torch.rand(M, device=dev) + 0.5
    parts = (d + 127) // 128
    ssq = torch.rand(M, parts, device=dev) * d / parts
    dq, dz, dsc = torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, 2 * d, device=dev, dtype=bf)
    rowcoef = torch.empty(M, device=dev)
    acc = [torch.zeros(d, device=dev) for _ in range(4)]
    W2w = (W2.float() * gnw).to(bf)
    dW2w, dW2 = torch.zeros(d, d, device=dev, dtype=f32), torch.zeros(d, d, device=dev, dtype=f32)
    dh = torch.empty(M, d, device=dev, dtype=bf)

    stages = {
        "stream-update backward (2 kernels)": lambda: cu.K.gate_update_bwd(dF, dS, g_pre, z, c, s, w_r, b2, rstd, ssq, 1e-6, None,
                                                                          dq, dz, dsc, rowcoef, acc[0], acc[1], acc[2]),
        "weight gradient dq^T h (bf16, fp32 accumulate)": lambda: cu.gemm_bf16(dq, h, a_mn=True, b_mn=True, out=dW2w, accumulate=True),
        "un-fold norm weight (dW2, dw_norm)": lambda: cu.K.unscale_cols_bwd(dW2w, W2, gnw, dW2, acc[3]),
        "data gradient dq W2 with RMSNorm/silu backward epilogue": lambda: cu.gemm_bf16(dq, W2w, b_mn=True, out=dh, aux=hg_pre,
                                                                                         aux_mode=cu.AUX_RMS_SILU_BWD, rowcoef=rowcoef),
    }
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for name, fn in stages.items():
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / args.iters * 1e3
        total += us
        print(f"{name:58s} {us:9.1f} us")
    print(f"{'total':58s} {total:9.1f} us   (rows = {M}, d = {d})")


if __name__ == "__main__":
    main()
