"""Training throughput over a grid of (batch, sequence) configurations.

    python scripts/throughput.py [--precision fp32|bf16|fp8] [--cam on|off|both] [--sp-size N] [--model ref|350m|1.3b]
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 scripts/throughput.py --precision fp8

Same grid, model (d_embed 512, d 2048, 8 layers, 2 cycles, k 9, vocab 100277) and step as the
reference's scripts/throughput.py; with several ranks the sequence is split over ``--sp-size`` ranks
(default: all of them) and the batch over the rest. Per configuration: 5 warm-up and 30 timed
projected steps; reported are device-timed ms/step (CUDA events, max over ranks), tokens/s and peak
memory. Out-of-memory configurations are reported as such and the sweep continues. On a terminal the results and a
read-only NVML view of the GPUs (utilisation, memory, power, SM clock) are shown as live tables (``--plain`` for lines).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.loss import projected_step  # noqa: E402
from gdnet_b200.model import GDNet  # noqa: E402
from gdnet_b200.utils.distributed import (destroy, get_dp_group, get_sp_group, get_world_size,  # noqa: E402
                                          init_distributed, init_process_groups, is_main_process)
from gdnet_b200.utils.fp8 import cast_for_precision, update_fp8_scales  # noqa: E402
from gdnet_b200.utils.sp import clear_symm_handles  # noqa: E402

N_WRITE = 4
GRID = [(b, t) for t in (512, 1024, 2048, 4096, 8192) for b in (4, 8, 16, 32, 64)] + [(4, 16384), (8, 16384), (4, 32768)]
MODELS = {
    "ref": dict(vocab_size=100_277, d_embed=512, d=2048, n_layers=8, n_cycles=2, kernel_size=9),
    "350m": dict(vocab_size=32000, d_embed=1024, d=1024, n_layers=24, n_cycles=2, kernel_size=4),
    "1.3b": dict(vocab_size=32000, d_embed=2048, d=2048, n_layers=24, n_cycles=2, kernel_size=4),
}


def run_config(B, T, args, sp_group, dp_group, device, n_warmup=5, n_steps=30):
    sp = dist.get_world_size(sp_group) if sp_group is not None else 1
    dp = dist.get_world_size(dp_group) if dp_group is not None else 1
    T_loc, B_loc = T // sp, B // dp
    spec = MODELS[args.model]
    model = GDNet(chunk_size=T_loc, **spec).to(device)
    n_params = sum(p.numel() for p in model.parameters())
    cast_for_precision(model, args.precision)
    model.cam_enabled = args.cam_now
    on_gpu = device.type == "cuda"
    if on_gpu and args.precision != "fp32":
        from gdnet_b200.train.engine import TrainEngine

        runner = TrainEngine(model, lr=1e-3, precision=args.precision, sp_group=sp_group if sp > 1 else None)
        params, opt = None, None
    else:
        runner, params = model, list(model.parameters())
        opt = torch.optim.AdamW(params, lr=1e-3)
    V = spec["vocab_size"]
    tok = torch.randint(0, V, (B_loc, T_loc), device=device)
    tgt = torch.randint(0, V, (B_loc, T_loc), device=device)
    wc = torch.randint(0, V, (B_loc, N_WRITE, T_loc), device=device) if args.cam_now else None

    def one(i):
        projected_step(runner, params, opt, tok, tgt, precision=args.precision, write_chunks=wc,
                       sp_group=sp_group if sp > 1 else None)
        if args.precision == "fp8" and i % 16 == 0:
            update_fp8_scales(model)

    for i in range(n_warmup):
        one(i)
    if on_gpu:
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    import time

    t0 = time.perf_counter()
    for i in range(n_steps):
        one(i)
    if on_gpu:
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / n_steps
        mem = torch.cuda.max_memory_allocated(device) / 2**30
    else:
        ms, mem = (time.perf_counter() - t0) * 1000 / n_steps, 0.0
    if dist.is_initialized():
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    del runner, model
    if on_gpu:
        torch.cuda.empty_cache()
    if sp > 1:
        clear_symm_handles()
    return ms, B * T / (ms / 1000.0), n_params, mem


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--precision", choices=["fp32", "bf16", "fp8"], default="fp8")
    ap.add_argument("--cam", choices=["on", "off", "both"], default="on")
    ap.add_argument("--sp-size", type=int, default=None)
    ap.add_argument("--model", choices=sorted(MODELS), default="ref")
    ap.add_argument("--only", default="", help="comma list like 8x4096,4x8192")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--json", default="")
    ap.add_argument("--plain", action="store_true", help="plain lines instead of the live tables")
    ap.add_argument("--no-monitor", action="store_true", help="do not sample the GPUs through NVML")
    args = ap.parse_args()

    init_distributed()
    world = get_world_size()
    init_process_groups(args.sp_size if args.sp_size is not None else world)
    sp_group, dp_group = (get_sp_group(), get_dp_group()) if world > 1 else (None, None)
    sp = dist.get_world_size(sp_group) if sp_group is not None else 1
    dp = dist.get_world_size(dp_group) if dp_group is not None else 1
    on_gpu = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if on_gpu else torch.device("cpu")
    grid = GRID
    if args.only:
        grid = [tuple(int(v) for v in item.split("x")) for item in args.only.split(",")]
    rows = []
    monitor, tables = None, None
    if is_main_process() and on_gpu and not args.no_monitor:
        from gdnet_b200.runtime.monitor import GpuMonitor

        monitor = GpuMonitor()
        monitor.start()
    try:
        for cam in ([True, False] if args.cam == "both" else [args.cam == "on"]):
            args.cam_now = cam
            if is_main_process():
                from gdnet_b200.runtime.monitor import LiveTables

                if tables is not None:
                    tables.close()
                tables = LiveTables(f"precision={args.precision} cam={'on' if cam else 'off'} gpus={world} sp={sp} dp={dp} "
                                    f"model={args.model}", monitor, force_plain=args.plain)
            for B, T in grid:
                if T % sp or B % dp:
                    continue
                try:
                    ms, tps, n_params, mem = run_config(B, T, args, sp_group, dp_group, device, n_steps=args.steps)
                    row = dict(B=B, T=T, ms=ms, tok_s=tps, params=n_params, mem_gib=mem, cam=cam)
                except torch.cuda.OutOfMemoryError:
                    torch.cuda.empty_cache()
                    row = dict(B=B, T=T, ms=float("nan"), tok_s=float("nan"), params=0, mem_gib=0.0, cam=cam, oom=True)
                rows.append(row)
                if tables is not None:
                    tables.add(row)
    finally:
        if tables is not None:
            tables.close()
        if monitor is not None:
            monitor.stop()
        if args.json and is_main_process():
            json.dump(rows, open(args.json, "w"), indent=1)
        destroy()


if __name__ == "__main__":
    main()
