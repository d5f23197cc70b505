"""GEMM microbenchmark on the training shapes: the sm_100a block-scaled FP8 and bf16 tensor-core
kernels against cuBLASLt ``torch._scaled_mm`` (per-tensor scales, what the reference's FP8Linear
calls) and cuBLAS ``F.linear``.

    python benchmarks/bench_fp8_gemm.py [--shapes cfg2|train|all] [--json out.json]

Timing: CUDA events on the launching stream, 5 warm-up + 20 timed launches, inputs rotated through
enough buffers to exceed L2 (126 MB) between reuse. Reference harness: benchmarks/bench_fp8_gemm.py.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

CFG2 = [(16384, 2048, 2048), (16384, 2048, 8192), (16384, 8192, 2048)]            # (M, K, N)
TRAIN = [(32768, 1024, 1024), (32768, 2048, 1024), (32768, 1024, 32000), (16384, 2048, 2048), (16384, 4096, 2048)]
WGRAD = [(1024, 32768, 1024), (1024, 32768, 2048), (2048, 16384, 2048)]             # reduction over tokens


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


def bench_shape(M, K, N, peaks):
    from gdnet_b200.ops import cuda as cu

    dev = "cuda"
    bytes_per_set = M * K * 2 + N * K * 2 + M * N * 2
    n_sets = max(2, int(300e6 // bytes_per_set) + 1)
    xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
    ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(n_sets)]
    outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
    flops = 2.0 * M * N * K
    row = {"M": M, "K": K, "N": N}

    t = timeit(lambda i: torch.nn.functional.linear(xs[i], ws[i]), n_sets)
    row["cublas_bf16_ms"], row["cublas_bf16_tflops"] = t, flops / t / 1e9
    t = timeit(lambda i: cu.gemm_bf16(xs[i], ws[i], out=outs[i]), n_sets)
    row["ours_bf16_ms"], row["ours_bf16_tflops"] = t, flops / t / 1e9

    if K % 128 == 0 and N % 128 == 0:
        q = [cu.quantize_rows(x) for x in xs]
        qw = []
        for w in ws:
            wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=dev)
            sw = torch.empty((N + 127) // 128, (K + 127) // 128, device=dev)
            cu.K.quant_tile(w, False, wq, sw, cu.Q_BLOCK, None, None, cu.Q_BLOCK)
            qw.append((wq, sw))
        t = timeit(lambda i: cu.gemm_fp8(q[i][0], q[i][1], qw[i][0], qw[i][1], out=outs[i]), n_sets)
        row["ours_fp8_ms"], row["ours_fp8_tflops"] = t, flops / t / 1e9
        t = timeit(lambda i: cu.quantize_rows(xs[i], q=q[i][0], s=q[i][1]), n_sets)
        row["quant_rows_ms"] = t
        row["quant_rows_gbs"] = (M * K * 3 + M * K / 32) / t / 1e6
        one = torch.ones(1, device=dev)
        x8 = [a[0] for a in q]
        w8 = [b[0] for b in qw]
        try:
            t = timeit(lambda i: torch._scaled_mm(x8[i], w8[i].t(), scale_a=one, scale_b=one,
                                                   out_dtype=torch.bfloat16), n_sets)
            row["cublaslt_fp8_ms"], row["cublaslt_fp8_tflops"] = t, flops / t / 1e9
        except Exception as exc:
            row["cublaslt_fp8_error"] = str(exc)[:100]
    if peaks:
        row["ours_bf16_frac_of_measured"] = row["ours_bf16_tflops"] / peaks["bf16_tflops"]
    return row


def bench_wgrad(N, M, K):
    """dW (N,K) = dy^T (N,M) x (M,K): both operands read MN-major (no transposed copy) vs cuBLAS."""
    from gdnet_b200.ops import cuda as cu

    dev = "cuda"
    n_sets = 3
    dy = [torch.randn(M, N, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
    x = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
    out = torch.zeros(N, K, device=dev)
    flops = 2.0 * M * N * K
    row = {"wgrad_N": N, "tokens": M, "K": K}
    t = timeit(lambda i: torch.mm(dy[i].t(), x[i]), n_sets)
    row["cublas_bf16_ms"], row["cublas_bf16_tflops"] = t, flops / t / 1e9
    t = timeit(lambda i: cu.gemm_bf16(dy[i], x[i], a_mn=True, b_mn=True, out=out, accumulate=True), n_sets)
    row["ours_bf16_ms"], row["ours_bf16_tflops"] = t, flops / t / 1e9
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="all", choices=["cfg2", "train", "all"])
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    peaks = None
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    shapes = CFG2 if args.shapes == "cfg2" else TRAIN if args.shapes == "train" else CFG2 + TRAIN
    rows = [bench_shape(*s, peaks) for s in shapes]
    rows += [bench_wgrad(*s) for s in WGRAD]
    for r in rows:
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}))
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
