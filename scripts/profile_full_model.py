"""Per-kernel time breakdown of one training step (torch.profiler, CUDA activities).

    python scripts/profile_full_model.py [--config 350m|tiny] [--steps 1] [--out profiles/step_kernels.txt]

Prints the kernels of a projected step sorted by total device time with their launch counts and
shares, the peak memory, and optionally writes a chrome trace. Numbers taken under the profiler
are for *shares* only; throughput is measured by bench.py. Reference counterpart:
scripts/profile_full_model.py (torch.profiler + cProfile over five steps).
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import bench

    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="350m", choices=sorted(bench.CONFIGS))
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--out", default="")
    ap.add_argument("--trace", default="")
    ap.add_argument("--top", type=int, default=40)
    args = ap.parse_args()
    cfg = bench.CONFIGS[args.config]
    dev = torch.device("cuda", 0)
    step, _ = bench.build_ours(cfg, dev, 1)
    batches = bench.make_batches(cfg, args.warmup + args.steps, seed=1)

    def run(b):
        seq, wc = b[0].to(dev), (b[1].to(dev) if b[1] is not None else None)
        return step(seq[:, :-1], seq[:, 1:], wc)

    for b in batches[: args.warmup]:
        run(b)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for b in batches[args.warmup :]:
            run(b)
        torch.cuda.synchronize()
    rows = [(e.key, e.device_time_total, e.count) for e in prof.key_averages() if e.device_time_total > 0
            and e.device_type == torch.autograd.DeviceType.CUDA]
    rows.sort(key=lambda r: -r[1])
    total = sum(r[1] for r in rows)
    lines = [f"config {args.config}: {args.steps} step(s), device time {total / 1e3 / args.steps:.1f} ms/step, "
             f"peak memory {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB",
             f"{'share':>6} {'ms/step':>9} {'calls/step':>10}  kernel"]
    for name, t, n in rows[: args.top]:
        lines.append(f"{100 * t / total:6.2f} {t / 1e3 / args.steps:9.3f} {n / args.steps:10.0f}  {name[:110]}")
    # where the device waits for the host: idle time between consecutive kernels, charged to the kernel that
    # follows the gap (only gaps above 5 us; under the profiler the host is slower than in a plain run)
    evs = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                  if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end > e.time_range.start),
                 key=lambda t: t[0])
    gaps: dict[str, list] = {}
    idle = 0.0
    busy_until = evs[0][1] if evs else 0.0
    for start, end, name in evs[1:]:
        gap = start - busy_until
        if gap > 5.0:
            idle += gap
            g = gaps.setdefault(name, [0.0, 0])
            g[0] += gap
            g[1] += 1
        busy_until = max(busy_until, end)
    lines.append(f"device idle between kernels: {idle / 1e3 / args.steps:.1f} ms/step; largest waits before:")
    for name, (t, n) in sorted(gaps.items(), key=lambda kv: -kv[1][0])[:12]:
        lines.append(f"       {t / 1e3 / args.steps:9.3f} ms {n / args.steps:8.0f} gaps  {name[:100]}")
    text = "\n".join(lines)
    print(text)
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        open(args.out, "w").write(text + "\n")
    if args.trace:
        prof.export_chrome_trace(args.trace)


if __name__ == "__main__":
    main()
