"""Per-kernel time breakdown of one training step (torch.profiler, CUDA activities).

    python scripts/profile_full_model.py [--config 350m|tiny] [--steps 1] [--out profiles/step_kernels.txt]

Prints the kernels of a projected step sorted by total device time with their launch counts and
shares, the peak memory, and optionally writes a chrome trace. Numbers taken under the profiler
are for *shares* only; throughput is measured by bench.py.

The host side of the reference's script (scripts/profile_full_model.py:163-211) is here too:
``--cprofile`` runs the same steps under cProfile and prints the top functions by cumulative time (where the
Python driver of the step spends its time between launches); ``--memory FILE`` records the allocator's history
over the profiled steps and writes a snapshot for torch's memory visualiser plus the peak allocated / reserved
figures; ``--audit`` lists the hidden-copy sites (``.contiguous()``, ``.to()``, ``.clone()``, ``cat`` / ``stack``)
in the model's hot files by walking their syntax trees (scripts/audit_copies.py), which answers the question the
reference put to a bytecode listing of ``GDNet.forward``.
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
    ap.add_argument("--cprofile", action="store_true", help="also profile the Python side of the steps with cProfile")
    ap.add_argument("--memory", default="", help="write an allocator-history snapshot (pickle) to this file")
    ap.add_argument("--audit", action="store_true", help="list hidden-copy sites in the hot files")
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
    host_lines: list[str] = []
    if args.cprofile:
        import cProfile
        import io
        import pstats

        pr = cProfile.Profile()
        pr.enable()
        for b in batches[args.warmup :]:
            run(b)
        torch.cuda.synchronize()
        pr.disable()
        buf = io.StringIO()
        pstats.Stats(pr, stream=buf).sort_stats("cumulative").print_stats(40)
        host_lines += ["", "cProfile, top 40 by cumulative time (host side of the profiled steps):", buf.getvalue()]
    if args.memory:
        torch.cuda.memory._record_memory_history(max_entries=200_000)
        for b in batches[args.warmup :]:
            run(b)
        torch.cuda.synchronize()
        torch.cuda.memory._dump_snapshot(args.memory)
        torch.cuda.memory._record_memory_history(enabled=None)
        host_lines += ["", f"allocator history written to {args.memory} (open with torch's memory visualiser); "
                       f"peak allocated {torch.cuda.max_memory_allocated() / 2**30:.2f} GiB, "
                       f"peak reserved {torch.cuda.max_memory_reserved() / 2**30:.2f} GiB"]
    if args.audit:
        import subprocess

        out = subprocess.run([sys.executable, os.path.join(ROOT, "scripts", "audit_copies.py")], capture_output=True, text=True)
        host_lines += ["", "hidden-copy sites in the hot files (scripts/audit_copies.py):", out.stdout[-6000:]]
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
    text = "\n".join(lines + host_lines)
    print(text)
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        open(args.out, "w").write(text + "\n")
    if args.trace:
        prof.export_chrome_trace(args.trace)


if __name__ == "__main__":
    main()
