"""GEMM microbenchmark on the training shapes: the sm_100a hardware block-scaled FP8 kernel (1x128 activation /
128x128 weight scales, power-of-two, applied by the tensor core) and the bf16 kernel against cuBLASLt
``torch._scaled_mm`` (per-tensor scales, what the reference's FP8Linear calls: gdnet/kernel/fp8_linear/linear.py:38-72)
and cuBLAS ``F.linear`` / ``torch.mm``, for the three GEMMs of a linear layer:

    forward   y  (M, N) = x  (M, K) . W^T (K, N)
    dgrad     dx (M, K) = dy (M, N) . W   (N, K)
    wgrad     dW (N, K) = dy^T (N, M) . x (M, K)      (this framework: bf16 operands read in place, fp32 accumulation)

    python benchmarks/bench_fp8_gemm.py [--shapes cfg2|train|all] [--json out.json] [--md out.md]

Timing: CUDA events on the launching stream, 5 warm-up + 20 timed launches, operands rotated through enough
buffer sets to exceed L2 (126 MB) between reuse. Reference harness: benchmarks/bench_fp8_gemm.py:28-95.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

CFG2 = [(16384, 2048, 2048), (16384, 2048, 8192), (16384, 8192, 2048)]            # (M tokens, K, N)
TRAIN = [(32768, 1024, 1024), (32768, 2048, 1024), (16384, 4096, 2048), (32768, 1024, 32000)]
FP8 = torch.float8_e4m3fn


def timeit(fn, n_sets, warm=5, iters=20):
    for i in range(warm):
        fn(i % n_sets)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i % n_sets)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _entry(row, key, t, flops):
    row[f"{key}_ms"] = t
    row[f"{key}_tflops"] = flops / t / 1e9


def bench_shape(M, K, N):
    from gdnet_b200.ops import cuda as cu

    dev = "cuda"
    flops = 2.0 * M * N * K
    per_set = (M * K + N * K + M * N) * 2
    n_sets = max(2, int(300e6 // per_set) + 1)
    xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
    ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(n_sets)]
    dys = [torch.randn(M, N, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    dx = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
    dw = torch.zeros(N, K, device=dev)
    row = {"M": M, "K": K, "N": N, "sets": n_sets}
    one = torch.ones(1, device=dev)

    # ---- bf16
    _entry(row, "fwd_cublas_bf16", timeit(lambda i: torch.nn.functional.linear(xs[i], ws[i]), n_sets), flops)
    _entry(row, "fwd_ours_bf16", timeit(lambda i: cu.gemm_bf16(xs[i], ws[i], out=y), n_sets), flops)
    _entry(row, "dgrad_cublas_bf16", timeit(lambda i: torch.mm(dys[i], ws[i]), n_sets), flops)
    _entry(row, "dgrad_ours_bf16", timeit(lambda i: cu.gemm_bf16(dys[i], ws[i], b_mn=True, out=dx), n_sets), flops)
    _entry(row, "wgrad_cublas_bf16", timeit(lambda i: torch.mm(dys[i].t(), xs[i]), n_sets), flops)
    _entry(row, "wgrad_ours_bf16", timeit(lambda i: cu.gemm_bf16(dys[i], xs[i], a_mn=True, b_mn=True, out=dw, accumulate=True),
                                          n_sets), flops)

    # ---- fp8 (needs every size a multiple of 128)
    if M % 128 == 0 and K % 128 == 0 and N % 128 == 0:
        qx = [cu.quantize_rows_mx(x) for x in xs]                       # (x8, scales, packed)
        qdy = [cu.quantize_rows_mx(t) for t in dys]
        qw = [cu.quantize_weight(w) for w in ws]                        # q/p for forward, qt/pt for dgrad
        _entry(row, "fwd_ours_fp8", timeit(lambda i: cu.gemm_fp8_mx(qx[i][0], qx[i][2], qw[i].q, qw[i].p, out=y), n_sets), flops)
        _entry(row, "dgrad_ours_fp8", timeit(lambda i: cu.gemm_fp8_mx(qdy[i][0], qdy[i][2], qw[i].qt, qw[i].pt, out=dx), n_sets), flops)
        try:
            _entry(row, "fwd_cublaslt_fp8", timeit(lambda i: torch._scaled_mm(qx[i][0], qw[i].q.t(), scale_a=one, scale_b=one,
                                                                              out_dtype=torch.bfloat16), n_sets), flops)
            _entry(row, "dgrad_cublaslt_fp8", timeit(lambda i: torch._scaled_mm(qdy[i][0], qw[i].qt.t(), scale_a=one, scale_b=one,
                                                                                out_dtype=torch.bfloat16), n_sets), flops)
            # the reference's wgrad: e4m3 transposed copies of dy and x (their cost is not in this number)
            dyt = [t.t().contiguous().to(FP8) for t in dys[:2]]
            xt = [t.t().contiguous().to(FP8) for t in xs[:2]]
            _entry(row, "wgrad_cublaslt_fp8", timeit(lambda i: torch._scaled_mm(dyt[i % 2], xt[i % 2].t(), scale_a=one, scale_b=one,
                                                                                out_dtype=torch.bfloat16), n_sets), flops)
        except Exception as exc:                                        # noqa: BLE001
            row["cublaslt_fp8_error"] = str(exc)[:120]
        t = timeit(lambda i: cu.quantize_rows_mx(xs[i], q=qx[i][0], s=qx[i][1], p=qx[i][2]), n_sets)
        row["quant_rows_ms"], row["quant_rows_gbs"] = t, (M * K * 3 + M * K / 32) / t / 1e6
    return row


def to_markdown(rows, peaks) -> str:
    out = ["| M x K x N | op | cuBLAS bf16 | ours bf16 | cuBLASLt fp8 (per tensor) | ours fp8 (block scaled) | ours / cuBLASLt |",
           "|---|---|---|---|---|---|---|"]
    for r in rows:
        for op in ("fwd", "dgrad", "wgrad"):
            cb, ob = r.get(f"{op}_cublas_bf16_tflops"), r.get(f"{op}_ours_bf16_tflops")
            cf, of = r.get(f"{op}_cublaslt_fp8_tflops"), r.get(f"{op}_ours_fp8_tflops")
            f = lambda v: f"{v:.0f}" if v else "-"                       # noqa: E731
            ours_best = of if of else ob
            ratio = f"{ours_best / cf:.2f}" if cf and ours_best else "-"
            out.append(f"| {r['M']} x {r['K']} x {r['N']} | {op} | {f(cb)} | {f(ob)} | {f(cf)} | {f(of)} | {ratio} |")
    note = "TFLOP/s, CUDA events, operands rotated over more than 126 MB."
    if peaks:
        note += f" Measured cuBLAS bf16 peak of this pool: {peaks['bf16_tflops']:.0f} burst / {peaks['bf16_tflops_sustained']:.0f} sustained."
    return "\n".join(out) + "\n\n" + note + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="all", choices=["cfg2", "train", "all"])
    ap.add_argument("--json", default="")
    ap.add_argument("--md", default="")
    args = ap.parse_args()
    peaks = None
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    shapes = CFG2 if args.shapes == "cfg2" else TRAIN if args.shapes == "train" else CFG2 + TRAIN
    rows = []
    for s in shapes:
        rows.append(bench_shape(*s))
        torch.cuda.empty_cache()
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in rows[-1].items()}), flush=True)
    md = to_markdown(rows, peaks)
    print(md)
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)
    if args.md:
        open(args.md, "w").write(md)


if __name__ == "__main__":
    main()
