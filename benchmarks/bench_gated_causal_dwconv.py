"""Microbenchmarks of the memory-bound kernels of a layer step, each against its roofline.

    python benchmarks/bench_gated_causal_dwconv.py [--shape B,T,d,k] [--json out.json] [--reference]

Default shape: B=8, T=8192 (L), d=2048, k=4, bf16 (the kernel microbenchmark configuration), plus the
training shape B=8, T=4096, d=1024. For every kernel: CUDA-event time (5 warm-up, 20 timed, inputs
rotated through > 126 MB so L2 does not serve them), the algorithmic bytes it must move and the
fraction of the measured copy bandwidth (MEASURED_PEAKS.json, else 6650 GB/s) that this corresponds to.
Reference counterpart: benchmarks/bench_gated_causal_dwconv.py (pyperf over nine sub-kernels).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def timeit(fn, warm=5, iters=20):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench(B, T, d, k, hbm_gbs):
    from gdnet_b200.ops import cuda as cu

    dev, bf = "cuda", torch.bfloat16
    M = B * T
    unit = M * d * 2  # bytes of one (M, d) bf16 tensor
    n_sets = max(2, int(400e6 // (4 * unit)) + 1)
    mk = lambda: [torch.randn(B, T, d, device=dev, dtype=bf) for _ in range(n_sets)]
    x, s, gp, z, dF, dS = mk(), mk(), mk(), mk(), mk(), mk()
    w = torch.randn(k, d, device=dev)      # the kernels read the taps transposed
    out = torch.empty(B, T, d, device=dev, dtype=bf)
    out2 = torch.empty_like(out)
    rows = []

    def add(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        rows.append(dict(kernel=name, shape=f"{B}x{T}x{d} k={k}", ms=round(ms, 4), gbytes=round(nbytes / 1e9, 3),
                         gbs=round(gbs, 1), frac_of_measured_hbm=round(gbs / hbm_gbs, 3)))

    K = cu.K
    add("dwconv_fwd", timeit(lambda i: K.dwconv_fwd(x[i % n_sets], None, w, out)), 2 * unit)
    dw = torch.zeros(d, k, device=dev)
    add("dwconv_bwd", timeit(lambda i: K.dwconv_bwd(dF[i % n_sets], x[i % n_sets], None, w, None, out, None, dw)), 3 * unit)
    wr = torch.ones(d, device=dev)
    rstd = torch.empty(M, device=dev)
    gs = torch.zeros((), device=dev)
    add("gate_update_fwd", timeit(lambda i: K.gate_update_fwd(gp[i % n_sets].view(M, d), z[i % n_sets].view(M, d),
                                                              x[i % n_sets].view(M, d), s[i % n_sets].view(M, d), wr,
                                                              out.view(M, d), out2.view(M, d), None, rstd, gs, 1e-6)), 6 * unit)
    add("gate_stream_update_fwd (R given)", timeit(lambda i: K.gate_mix_fwd(gp[i % n_sets].view(M, d), x[i % n_sets].view(M, d),
                                                                           s[i % n_sets].view(M, d), z[i % n_sets].view(M, d),
                                                                           out.view(M, d), out2.view(M, d))), 6 * unit)
    parts = (d + 127) // 128
    ssq = torch.rand(M, parts, device=dev) * d / parts
    b2 = torch.zeros(d, device=dev)
    dq, dz = torch.empty(M, d, device=dev, dtype=bf), torch.empty(M, d, device=dev, dtype=bf)
    dsc = torch.empty(M, 2 * d, device=dev, dtype=bf)
    rc = torch.empty(M, device=dev)
    acc = [torch.zeros(d, device=dev) for _ in range(3)]
    add("gate_update_bwd", timeit(lambda i: K.gate_update_bwd(dF[i % n_sets].view(M, d), dS[i % n_sets].view(M, d),
                                                              gp[i % n_sets].view(M, d), z[i % n_sets].view(M, d),
                                                              x[i % n_sets].view(M, d), s[i % n_sets].view(M, d), wr, b2,
                                                              rstd, ssq, 1e-6, None, dq, dz, dsc, rc, *acc)), 10 * unit)
    q = torch.empty(M, d, dtype=torch.float8_e4m3fn, device=dev)
    sc = torch.empty(parts, M, device=dev)
    add("quant_rows_1x128", timeit(lambda i: cu.quantize_rows(x[i % n_sets].view(M, d), q=q, s=sc)), 1.5 * unit)
    add("quant_rows+transposed", timeit(lambda i: cu.quantize_rows_and_transposed(x[i % n_sets].view(M, d), cu.Q_COLS)), 2 * unit)
    add("quant_rows+transposed mx", timeit(lambda i: cu.quantize_both_mx(x[i % n_sets].view(M, d), cu.Q_COLS)), 2 * unit)
    add("quant_transposed_block mx", timeit(lambda i: cu.quantize_transposed_mx(x[i % n_sets].view(M, d), cu.Q_BLOCK)), 1.5 * unit)
    y = torch.empty(M, d, device=dev, dtype=bf)
    add("rmsnorm_fwd", timeit(lambda i: K.rmsnorm_fwd(x[i % n_sets].view(M, d), wr, y, rstd, 1e-6)), 2 * unit)
    cs = torch.zeros(d, device=dev)
    add("colsum", timeit(lambda i: K.colsum(x[i % n_sets].view(M, d), cs)), unit)
    return rows


def bench_reference(B, T, d, k, hbm_gbs):
    """The unmodified reference's Triton kernels (``baseline/_ref``) on the same shapes and with the same timing:
    gdnet/kernel/gated_causal_depthwise_conv/conv.py:182-281 (conv forward / backward),
    gate_norm.py:133-183 (RMSNorm forward, stream update with the recovery gate given)."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "gdnet")):
        return [dict(kernel="reference", unavailable="baseline/_ref is not installed")]
    sys.path.insert(0, ref_root)
    from gdnet.kernel.gated_causal_depthwise_conv.conv import causal_dwconv_bwd, causal_dwconv_fwd
    from gdnet.kernel.gated_causal_depthwise_conv.gate_norm import gate_stream_update_fwd, rmsnorm_fwd

    dev, bf = "cuda", torch.bfloat16
    M = B * T
    unit = M * d * 2
    n_sets = max(2, int(400e6 // (4 * unit)) + 1)
    mk = lambda: [torch.randn(B, T, d, device=dev, dtype=bf) for _ in range(n_sets)]     # noqa: E731
    x, s, gp, R = mk(), mk(), mk(), mk()
    w = torch.randn(d, k, device=dev)
    block_t = min(1 << (T - 1).bit_length(), 64)
    rows = []

    def add(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        rows.append(dict(kernel=name, impl="reference (Triton)", shape=f"{B}x{T}x{d} k={k}", ms=round(ms, 4),
                         gbytes=round(nbytes / 1e9, 3), gbs=round(gbs, 1), frac_of_measured_hbm=round(gbs / hbm_gbs, 3)))

    add("dwconv_fwd", timeit(lambda i: causal_dwconv_fwd(x[i % n_sets], w, T, k, block_t)), 2 * unit)
    # the reference's backward writes dX in fp32 (4 bytes per element) and zero-fills it first
    add("dwconv_bwd", timeit(lambda i: causal_dwconv_bwd(gp[i % n_sets], x[i % n_sets], w, T, k, block_t)), 3 * unit)
    add("gate_stream_update_fwd (R given)", timeit(lambda i: gate_stream_update_fwd(
        gp[i % n_sets].view(M, d), x[i % n_sets].view(M, d), s[i % n_sets].view(M, d), R[i % n_sets].view(M, d), d)), 6 * unit)
    wn = torch.ones(d, device=dev, dtype=bf)
    add("rmsnorm_fwd", timeit(lambda i: rmsnorm_fwd(x[i % n_sets].view(M, d), wn, 1e-6, d)), 2 * unit)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="")
    ap.add_argument("--json", default="")
    ap.add_argument("--reference", action="store_true", help="also time the reference's Triton kernels (baseline/_ref)")
    args = ap.parse_args()
    hbm = 6650.0
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        hbm = float(json.load(open(pk))["hbm_gbs"])
    shapes = [tuple(int(v) for v in args.shape.split(","))] if args.shape else [(8, 8192, 2048, 4), (8, 4096, 1024, 4)]
    rows = []
    for shp in shapes:
        rows += bench(*shp, hbm)
        if args.reference:
            rows += bench_reference(*shp, hbm)
    for r in rows:
        print(json.dumps(r))
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
