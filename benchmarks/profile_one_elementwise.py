"""Launch one memory-bound kernel a few times on the training shape, for an ncu capture of a small case.

    python benchmarks/profile_one_elementwise.py --kernel conv_fwd|conv_bwd|gate_fwd|gate_bwd|quant_rows|quant_tile|rmsnorm|cross_entropy|mem_read|adamw|gemv
                                                 [--B 8] [--T 4096] [--d 1024] [--iters 3]

Inputs of one launch are a few hundred MB (larger than L2); nothing else runs before the kernel of interest
except the allocation fills.
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from gdnet_b200.ops import cuda as cu

    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--d", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    B, T, d = args.B, args.T, args.d
    M = B * T
    dev, bf = "cuda", torch.bfloat16
    K = cu.K
    rnd = lambda *s: torch.randn(*s, device=dev, dtype=bf)  # noqa: E731
    kb = d // 128
    if args.kernel == "conv_fwd":
        x, w, out = rnd(B, T, d), torch.randn(4, d, device=dev), torch.empty(B, T, d, device=dev, dtype=bf)
        q = torch.empty(M, d, dtype=torch.float8_e4m3fn, device=dev)
        s, p = torch.empty(kb, M, device=dev), cu.packed_buffer(M, d, dev)
        fn = lambda: K.dwconv_fwd(x, None, w, out, q, s, p)
    elif args.kernel == "conv_bwd":
        x, dc, w = rnd(B, T, d), rnd(B, T, d), torch.randn(4, d, device=dev)
        dx, dw = torch.empty(B, T, d, device=dev, dtype=bf), torch.zeros(d, 4, device=dev)
        fn = lambda: K.dwconv_bwd(dc, x, None, w, None, dx, None, dw)
    elif args.kernel in ("gate_fwd", "gate_bwd"):
        gp, z, c, s2, dF, dS = (rnd(M, d) for _ in range(6))
        wr, b2 = torch.ones(d, device=dev), torch.zeros(d, device=dev)
        rstd = torch.rand(M, device=dev) + 0.5
        if args.kernel == "gate_fwd":
            fo, so = torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, d, device=dev, dtype=bf)
            q = torch.empty(M, d, dtype=torch.float8_e4m3fn, device=dev)
            s, p = torch.empty(kb, M, device=dev), cu.packed_buffer(M, d, dev)
            fn = lambda: K.gate_update_fwd(gp, z, c, s2, wr, fo, so, None, rstd, None, 1e-6, q, s, p)
        else:
            parts = (d + 127) // 128
            ssq = torch.rand(M, parts, device=dev) * d / parts
            dq, dz, dsc = torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, 2 * d, device=dev, dtype=bf)
            rc = torch.empty(M, device=dev)
            acc = [torch.zeros(d, device=dev) for _ in range(3)]
            fn = lambda: K.gate_update_bwd(dF, dS, gp, z, c, s2, wr, b2, rstd, ssq, 1e-6, None, dq, dz, dsc, rc, *acc)
    elif args.kernel == "quant_rows":
        x = rnd(M, d)
        fn = lambda: cu.quantize_rows_mx(x)
    elif args.kernel == "quant_tile":
        x = rnd(M, d)
        fn = lambda: cu.quantize_both_mx(x, cu.Q_COLS)
    elif args.kernel == "rmsnorm":
        x, w = rnd(M, d), torch.ones(d, device=dev)
        y, rstd = torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, device=dev)
        fn = lambda: K.rmsnorm_fwd(x, w, y, rstd, 1e-6)
    elif args.kernel == "cross_entropy":
        V = 32000
        rows = 4096
        logits = rnd(rows, V)
        tgt = torch.randint(0, V, (rows,), device=dev)
        loss, inv = torch.empty(rows, device=dev), torch.full((1,), 1.0 / rows, device=dev)
        fn = lambda: K.cross_entropy(logits, tgt, loss, inv, V, -100, 1.0, True)
    elif args.kernel == "mem_read":
        Bq, S, dsig, dc = 4096, 64, 128, 128
        f = lambda *s: torch.randn(*s, device=dev)  # noqa: E731
        q, gamma, e, tags, vals, alpha = f(Bq, dsig), f(Bq, 1), f(S, dsig), f(Bq, S, dsig), f(Bq, S, dc), f(1)
        wts, out = torch.empty(Bq, S, device=dev), torch.empty(Bq, dc, device=dev)
        fn = lambda: K.mem_read_fwd(q, gamma, e, tags, vals, alpha, wts, out)
    elif args.kernel == "adamw":
        n = 128 * 1024 * 1024
        p_ = torch.zeros(n, device=dev, dtype=bf)
        gt, gi, m_, v_ = (torch.randn(n, device=dev) for _ in range(4))
        v_.abs_()
        scal = torch.tensor([0.1, 1.0], device=dev)
        fn = lambda: K.projected_adamw(p_, gt, gi, m_, v_, scal, 0.1, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1)
    elif args.kernel == "gemv":
        mats = [rnd(d, 2 * d) for _ in range(96)]
        vecs = [torch.nn.functional.normalize(torch.randn(2 * d, device=dev), dim=0) for _ in mats]
        fn = lambda: cu.sigma_estimates(mats, vecs)
    else:
        raise SystemExit(f"unknown kernel {args.kernel}")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(f"{args.kernel}: {e0.elapsed_time(e1) / args.iters * 1e3:.1f} us per call")


if __name__ == "__main__":
    main()
