"""Launch one GEMM kernel a few times on a fixed shape, for an ncu capture of a small case.

    python benchmarks/profile_one_gemm.py --kind fp8|bf16|wgrad --shape M,K,N [--iters 4]
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from gdnet_b200.ops import cuda as cu

    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="fp8", choices=["fp8", "mx", "bf16", "wgrad"])
    ap.add_argument("--shape", default="32768,1024,1024")
    ap.add_argument("--iters", type=int, default=4)
    args = ap.parse_args()
    M, K, N = (int(v) for v in args.shape.split(","))
    dev = "cuda"
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    if args.kind == "fp8":
        x8, sx = cu.quantize_rows(x)
        qw = cu.quantize_weight(w)
        fn = lambda: cu.gemm_fp8(x8, sx, qw.q, qw.s, out=out)
    elif args.kind == "mx":
        pa = cu.packed_buffer(M, K, dev)
        x8, sx = cu.quantize_rows(x, pow2=True, packed=pa)
        wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=dev)
        ws = torch.empty(N // 128, K // 128, device=dev)
        pb = cu.packed_buffer(N, K, dev)
        cu.K.quant_tile(w, False, wq, ws, cu.Q_BLOCK, None, None, cu.Q_BLOCK, True, pb, None)
        fn = lambda: cu.gemm_fp8_mx(x8, pa, wq, pb, out=out)
    elif args.kind == "bf16":
        fn = lambda: cu.gemm_bf16(x, w, out=out)
    else:
        dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        acc = torch.zeros(N, K, device=dev)
        fn = lambda: cu.gemm_bf16(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.iters
    print(f"{args.kind} {M}x{K}x{N}: {ms * 1000:.1f} us, {2.0 * M * N * K / ms / 1e9:.0f} TFLOP/s")


if __name__ == "__main__":
    main()
