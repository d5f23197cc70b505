"""Launch one memory-bound kernel a few times on the training shape, for an ncu capture of a small case.

    python benchmarks/profile_one_elementwise.py --kernel conv_fwd|conv_bwd|gate_fwd|gate_bwd|quant_rows|quant_tile|rmsnorm|cross_entropy|mem_read|adamw|gemv
                                                          |mem_read_bwd|rmsnorm_bwd|quant_tensor|colsum|unscale_cols|gate_mix|cam_blend
                                                          |gemm_fp8_aux|gemm_bf16_aux|fused_update|max_allreduce|gather_jobs
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
    elif args.kernel == "mem_read_bwd":
        Bq, S, dsig, dc = 4096, 64, 128, 128
        f = lambda *s: torch.randn(*s, device=dev)  # noqa: E731
        q, gamma, e, tags, vals, alpha = f(Bq, dsig), f(Bq, dsig), f(S, dsig), f(Bq, S, dsig), f(Bq, S, dc), f(1)
        wts = torch.softmax(f(Bq, S), dim=-1)
        d_out = f(Bq, dc)
        outs = [torch.empty_like(q), torch.empty_like(gamma), torch.zeros_like(e), torch.empty_like(tags), torch.empty_like(vals),
                torch.zeros(1, device=dev)]
        fn = lambda: K.mem_read_bwd(d_out, q, gamma, e, tags, vals, wts, alpha, *outs)
    elif args.kernel == "rmsnorm_bwd":
        x, dy, w = rnd(M, d), rnd(M, d), torch.ones(d, device=dev)
        rstd, dx, dw = torch.rand(M, device=dev) + 0.5, torch.empty(M, d, device=dev, dtype=bf), torch.zeros(d, device=dev)
        fn = lambda: K.rmsnorm_bwd(dy, x, w, rstd, dx, dw)
    elif args.kernel == "quant_tensor":
        x, scale = rnd(M, d), torch.full((1,), 100.0, device=dev)
        fn = lambda: cu.quantize_fp8_tensor(x, scale, True)
    elif args.kernel == "colsum":
        x, out = rnd(M, d), torch.zeros(d, device=dev)
        fn = lambda: K.colsum(x, out)
    elif args.kernel == "unscale_cols":
        W2, g = rnd(4 * d, 4 * d), torch.randn(4 * d, 4 * d, device=dev)
        colw, dW2, dcol = torch.ones(4 * d, device=dev), torch.zeros(4 * d, 4 * d, device=dev), torch.zeros(4 * d, device=dev)
        fn = lambda: K.unscale_cols_bwd(g, W2, colw, dW2, dcol)
    elif args.kernel == "gate_mix":
        gp, c, s2, R = rnd(M, d), rnd(M, d), rnd(M, d), torch.rand(M, d, device=dev).to(bf)
        fo, so = torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, d, device=dev, dtype=bf)
        fn = lambda: K.gate_mix_fwd(gp, c, s2, R, fo, so)
    elif args.kernel == "cam_blend":
        z, f2, retr = rnd(M, d), rnd(M, d), rnd(B, d)
        out, rstd = torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, device=dev)
        fn = lambda: K.cam_blend_fwd(z, f2, retr, torch.ones(d, device=dev), T, 1e-6, out, rstd)
    elif args.kernel in ("gemm_fp8_aux", "gemm_bf16_aux"):
        # the pair GEMMs with an auxiliary input and a second output (the <true> instantiations): layer shapes
        a, w = rnd(M, d), rnd(d, d) * 0.05
        aux, pre, bias = rnd(M, d), torch.empty(M, d, device=dev, dtype=bf), torch.zeros(d, device=dev)
        out = torch.empty(M, d, device=dev, dtype=bf)
        if args.kernel == "gemm_fp8_aux":
            a8, _, pa = cu.quantize_rows_mx(a)
            qw = cu.quantize_weight(w)
            fn = lambda: cu.gemm_fp8_mx(a8, pa, qw.q, qw.p, out=out, bias=bias, aux=aux, aux_mode=cu.AUX_ADD, pre_out=pre, act=cu.ACT_SILU)
        else:
            fn = lambda: cu.gemm_bf16(a, w, out=out, bias=bias, aux=aux, aux_mode=cu.AUX_ADD, pre_out=pre, act=cu.ACT_SILU)
    elif args.kernel in ("fused_update", "max_allreduce", "gather_jobs"):
        # the peer-memory kernels with a world of one: every "peer" table holds this GPU's own buffer, nothing waits
        tab = lambda t: torch.tensor([t.data_ptr()], dtype=torch.int64, device=dev)  # noqa: E731
        if args.kernel == "fused_update":
            n = 64 * 1024 * 1024
            gt, gi = torch.randn(n, device=dev), torch.randn(n, device=dev)
            p_, m_, v_ = torch.zeros(n, device=dev, dtype=bf), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            flags, scal, sums = torch.zeros(1024, dtype=torch.int32, device=dev), torch.tensor([0.1, 1.0], device=dev), torch.zeros(8, device=dev)
            seq = [0]

            def fn():
                seq[0] += 1
                K.allreduce_adamw(tab(gt), tab(gi), tab(p_), tab(flags), m_, v_, scal, n, 0, 1, seq[0], 0, True, 0.1, 1e-3, 0.9,
                                  0.999, 1e-8, 0.01, 1, sums)
        elif args.kernel == "max_allreduce":
            area, fl, vec = torch.zeros(2 * 4096, device=dev), torch.zeros(64, dtype=torch.int32, device=dev), torch.rand(4096, device=dev)
            seq = [0]

            def fn():
                seq[0] += 1
                K.max_allreduce(vec, tab(area), tab(fl), 4096, 0, 1, seq[0])
        else:
            n = 256 * 1024 * 1024
            src, dst = torch.randint(0, 255, (n,), dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
            rows = [[src.data_ptr() + o, dst.data_ptr() + o, 0, 65536 // 16] for o in range(0, n, 65536)]
            table = torch.tensor(rows, dtype=torch.int64, device=dev)
            fn = lambda: K.gather_jobs(table)
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
