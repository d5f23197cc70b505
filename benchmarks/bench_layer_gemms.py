"""Time every GEMM variant of one GDLayer step (forward, data gradient, weight gradient; bf16 gate path and
block-scaled FP8 recovery path) at the training shape, with CUDA events.

    python benchmarks/bench_layer_gemms.py [--rows 32768] [--d 1024] [--iters 20] [--json out.json]

Each variant runs on a ring of operand sets whose total size exceeds the L2 cache, so no launch finds its
inputs cached by the previous one. Reports microseconds and TFLOP/s per variant.
"""

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from gdnet_b200.ops import cuda as cu

    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--d", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ring", type=int, default=4)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    M, d, R = args.rows, args.d, args.ring
    dev = "cuda"
    bf, f32 = torch.bfloat16, torch.float32

    def rnd(*shape, scale=1.0):
        return torch.randn(*shape, device=dev, dtype=bf) * scale

    acts = [rnd(M, d) for _ in range(R)]
    acts2 = [rnd(M, 2 * d) for _ in range(R)]
    grads = [rnd(M, d, scale=0.01) for _ in range(R)]
    w1 = [rnd(d, d, scale=0.03) for _ in range(R)]
    w1r = [rnd(d, 2 * d, scale=0.03) for _ in range(R)]
    outs = [torch.empty(M, d, device=dev, dtype=bf) for _ in range(R)]
    outs2 = [torch.empty(M, 2 * d, device=dev, dtype=bf) for _ in range(R)]
    dw = [torch.zeros(d, d, device=dev, dtype=f32) for _ in range(R)]
    dw2 = [torch.zeros(d, 2 * d, device=dev, dtype=f32) for _ in range(R)]
    bias = torch.zeros(d, device=dev, dtype=f32)

    # FP8 operands (power-of-two scales, packed chunks)
    a8 = [cu.quantize_rows_mx(x) for x in acts]                       # (q, s, p) of (M, d)
    u8 = [cu.quantize_rows_mx(x) for x in acts2]                      # (M, 2d)
    g8 = [cu.quantize_both_mx(g, cu.Q_COLS) for g in grads]           # (q, p, qt, pt)
    at8 = [cu.quantize_transposed_mx(x, cu.Q_BLOCK) for x in acts]    # (qt (d, M), st, pt)
    ut8 = [cu.quantize_transposed_mx(x, cu.Q_BLOCK) for x in acts2]   # (2d, M)
    qw = [cu.quantize_weight(w) for w in w1]
    qwr = [cu.quantize_weight(w) for w in w1r]

    variants = {
        # gate path, bf16
        "bf16 fprop  (M,d)x(d,d)  +bias+silu+pre_out": (
            2.0 * M * d * d,
            lambda i: cu.gemm_bf16(acts[i], w1[i], out=outs[i], bias=bias, pre_out=outs[(i + 1) % R], act=cu.ACT_SILU)),
        "bf16 fprop  (M,d)x(d,d)  plain": (2.0 * M * d * d, lambda i: cu.gemm_bf16(acts[i], w1[i], out=outs[i])),
        "bf16 dgrad  (M,d)x(d,d)  weight read MN-major": (
            2.0 * M * d * d, lambda i: cu.gemm_bf16(grads[i], w1[i], b_mn=True, out=outs[i])),
        "bf16 wgrad  (d,M)x(M,d)  fp32 accumulate": (
            2.0 * M * d * d, lambda i: cu.gemm_bf16(grads[i], acts[i], a_mn=True, b_mn=True, out=dw[i], accumulate=True)),
        "bf16 wgrad  (d,M)x(M,d)  fp32 fresh": (
            2.0 * M * d * d, lambda i: cu.gemm_bf16(grads[i], acts[i], a_mn=True, b_mn=True, out=dw[i])),
        # recovery path, FP8 with hardware block scaling
        "mx   fprop  (M,2d)x(2d,d)": (
            4.0 * M * d * d, lambda i: cu.gemm_fp8_mx(u8[i][0], u8[i][2], qwr[i].q, qwr[i].p, out=outs[i])),
        "mx   fprop  (M,d)x(d,d)": (
            2.0 * M * d * d, lambda i: cu.gemm_fp8_mx(a8[i][0], a8[i][2], qw[i].q, qw[i].p, out=outs[i])),
        "mx   dgrad  (M,d)x(d,d)": (
            2.0 * M * d * d, lambda i: cu.gemm_fp8_mx(g8[i][0], g8[i][1], qw[i].qt, qw[i].pt, out=outs[i])),
        "mx   dgrad  (M,d)x(d,2d) +aux add": (
            4.0 * M * d * d,
            lambda i: cu.gemm_fp8_mx(g8[i][0], g8[i][1], qwr[i].qt, qwr[i].pt, out=outs2[i], aux=outs2[i],
                                     aux_mode=cu.AUX_ADD)),
        "mx   wgrad  (d,M)x(M,d)  fp32 accumulate": (
            2.0 * M * d * d,
            lambda i: cu.gemm_fp8_mx(g8[i][2], g8[i][3], at8[i][0], at8[i][2], out=dw[i], accumulate=True)),
        "mx   wgrad  (d,M)x(M,2d) fp32 accumulate": (
            4.0 * M * d * d,
            lambda i: cu.gemm_fp8_mx(g8[i][2], g8[i][3], ut8[i][0], ut8[i][2], out=dw2[i], accumulate=True)),
    }

    # the same GEMMs with the epilogues the fused layer step gives them
    FP8 = torch.float8_e4m3fn
    q8s = [torch.empty(M, d, dtype=FP8, device=dev) for _ in range(R)]
    p8s = [cu.packed_buffer(M, d, dev) for _ in range(R)]
    ssq = [torch.empty(M, (d + 127) // 128, dtype=f32, device=dev) for _ in range(R)]
    rowc = torch.zeros(M, dtype=f32, device=dev)
    variants.update({
        "mx   fprop  (M,2d)x(2d,d) bias+silu+pre_out+q8 (train)": (
            4.0 * M * d * d,
            lambda i: cu.gemm_fp8_mx(u8[i][0], u8[i][2], qwr[i].q, qwr[i].p, out=outs[i], bias=bias,
                                     pre_out=outs[(i + 1) % R], act=cu.ACT_SILU, q8=q8s[i], q8_p=p8s[i])),
        "mx   fprop  (M,2d)x(2d,d) bias+q8(silu) only (no-grad)": (
            4.0 * M * d * d,
            lambda i: cu.gemm_fp8_mx(u8[i][0], u8[i][2], qwr[i].q, qwr[i].p, out=outs[i], bias=bias, q8=q8s[i],
                                     q8_p=p8s[i], q8_silu=True, store_out=False)),
        "mx   fprop  (M,d)x(d,d)  bias": (
            2.0 * M * d * d, lambda i: cu.gemm_fp8_mx(a8[i][0], a8[i][2], qw[i].q, qw[i].p, out=outs[i], bias=bias)),
        "mx   dgrad  (M,d)x(d,d)  aux silu' + q8": (
            2.0 * M * d * d,
            lambda i: cu.gemm_fp8_mx(g8[i][0], g8[i][1], qw[i].qt, qw[i].pt, out=outs[i], aux=acts[i],
                                     aux_mode=cu.AUX_MUL_SILU_GRAD, q8=q8s[i], q8_p=p8s[i])),
        "bf16 fprop  (M,d)x(d,d)  bias+silu+pre_out+ssq_out (train)": (
            2.0 * M * d * d,
            lambda i: cu.gemm_bf16(acts[i], w1[i], out=outs[i], bias=bias, pre_out=outs[(i + 1) % R], act=cu.ACT_SILU,
                                   ssq_out=ssq[i])),
        "bf16 fprop  (M,d)x(d,d)  bias+silu+ssq_out (no-grad)": (
            2.0 * M * d * d,
            lambda i: cu.gemm_bf16(acts[i], w1[i], out=outs[i], bias=bias, act=cu.ACT_SILU, ssq_out=ssq[i])),
        "bf16 fprop  (M,d)x(d,d)  bias + row scale from ssq": (
            2.0 * M * d * d,
            lambda i: cu.gemm_bf16(acts[i], w1[i], out=outs[i], bias=bias, ssq_in=ssq[i], norm_dim=d, norm_eps=1e-6)),
        "bf16 dgrad  (M,d)x(d,d)  aux rms/silu backward": (
            2.0 * M * d * d,
            lambda i: cu.gemm_bf16(grads[i], w1[i], b_mn=True, out=outs[i], aux=acts[i],
                                   aux_mode=cu.AUX_RMS_SILU_BWD, rowcoef=rowc)),
        "bf16 dgrad  (M,d)x(d,d)  aux add in place": (
            2.0 * M * d * d,
            lambda i: cu.gemm_bf16(grads[i], w1[i], b_mn=True, out=outs[i], aux=outs[i], aux_mode=cu.AUX_ADD)),
    })

    results = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, (flops, fn) in variants.items():
        for i in range(R):
            fn(i)
        torch.cuda.synchronize()
        e0.record()
        for it in range(args.iters):
            fn(it % R)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / args.iters * 1000.0
        tf = flops / us / 1e6
        results.append({"variant": name, "us": round(us, 1), "tflops": round(tf, 0)})
        print(f"{name:52s} {us:8.1f} us  {tf:7.0f} TFLOP/s")
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"rows": M, "d": d, "results": results}, f, indent=1)


if __name__ == "__main__":
    main()
