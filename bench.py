"""Flagship benchmark: GDNet ~350M training throughput (tokens/s) on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 350m|1.3b|1.3b-sp|tiny|...]

Config: d_model 1024, 24 layers, 2 cycles, dwconv width 4, vocab 32000,
seq_len 4096, micro-batch 8 per GPU, FP8 e4m3 linears, AdamW, projected-gradient step with 4
memory write chunks (as the reference's scripts/throughput.py:218-316 runs it), data parallel over
N GPUs (weak scaling). Synthetic packed tokens (geometric document lengths, EOS=0), random-init
weights. Prints ONE JSON line on rank 0.

Two measurements per run, both over exactly K steps after W warm-up steps:
* ``value``: device-timed (CUDA events, max over ranks); inputs already on the device. Between steps
  the working set (activations of 32768 tokens x 96 layer steps, > 50 GB) is far larger than L2.
* ``e2e``: the same step driven through the public API with the step's tokens copied from pinned
  host memory every step and the loss read back to the host every step.

``--impl reference`` runs the unmodified reference package (installed under baseline/_ref) through
its own ``projected_step`` for the same config and prints the same line with ``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
BASELINE_TOK_S = None  # the reference publishes no throughput number

CONFIGS = {
    "350m": dict(vocab_size=32000, d_embed=1024, d=1024, n_layers=24, n_cycles=2, kernel_size=4, seq_len=4096,
                 micro_batch=8, n_write=4),
    "tiny": dict(vocab_size=4096, d_embed=256, d=256, n_layers=2, n_cycles=2, kernel_size=4, seq_len=512,
                 micro_batch=2, n_write=2),
    # ~1.3B fully sharded: every large layer matrix (bf16 master, fp32 gradients, AdamW moments) lives on one owner
    # rank; the GEMMs of a layer step gather the operands they need from the owners over NVLink (the copies ride on
    # the tensor-core kernels), the weight-gradient epilogues add into the owner's shard, the update kernel does
    # projection + AdamW on the shard
    "1.3b": dict(vocab_size=32000, d_embed=2048, d=2048, n_layers=24, n_cycles=2, kernel_size=4, seq_len=8192,
                 micro_batch=2, n_write=4, shard="full"),
    # ~1.3B, one 65536-token sequence split into contiguous shards over the ranks (sequence parallel): conv halos
    # and their gradients cross ranks inside the conv kernels, every shard reads a memory that holds the summaries
    # of the shards before it, and the layer matrices are sharded over the same ranks (gathered by the GEMMs)
    "1.3b-sp": dict(vocab_size=32000, d_embed=2048, d=2048, n_layers=24, n_cycles=2, kernel_size=4, seq_len=65536,
                    micro_batch=1, n_write=4, mode="sp", shard="full"),
    # the two 1.3B configurations with 2 instead of 24 layers: same shapes per layer, for quick checks on few GPUs
    "1.3b-l2": dict(vocab_size=32000, d_embed=2048, d=2048, n_layers=2, n_cycles=2, kernel_size=4, seq_len=8192,
                    micro_batch=2, n_write=4, shard="full"),
    "1.3b-sp-l2": dict(vocab_size=32000, d_embed=2048, d=2048, n_layers=2, n_cycles=2, kernel_size=4, seq_len=16384,
                       micro_batch=1, n_write=4, mode="sp", shard="full"),
    "tiny-sp": dict(vocab_size=4096, d_embed=256, d=256, n_layers=2, n_cycles=2, kernel_size=4, seq_len=2048,
                    micro_batch=1, n_write=2, mode="sp", shard="full"),
    "tiny-shard": dict(vocab_size=4096, d_embed=256, d=256, n_layers=2, n_cycles=2, kernel_size=4, seq_len=512,
                       micro_batch=2, n_write=2, shard="full"),
}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = 0
        self._halt = threading.Event()

    def run(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            names = {
                pynvml.nvmlClocksEventReasonSwPowerCap: "sw_power_cap",
                pynvml.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
                pynvml.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
                pynvml.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                pynvml.nvmlClocksEventReasonHwPowerBrakeSlowdown: "hw_power_brake",
            }
            while not self._halt.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                time.sleep(self.period)
        except Exception as exc:  # NVML missing or not permitted: report, never fail the bench
            self.reasons.add(f"nvml_unavailable:{type(exc).__name__}")

    def stop(self) -> dict:
        self._halt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz or None,
                "reasons": sorted(self.reasons)}


def make_batches(cfg, n_batches: int, seed: int, rank: int = 0, world: int = 1):
    """Pinned host tensors: per step ``seq (B, T+1)`` and write chunks ``(B, n_write, T)`` (or None).

    Sequence-parallel configs: every rank draws the same global sequence (one document of uniform tokens)
    and keeps its contiguous shard plus the one token that follows it (the last target)."""
    import torch

    from gdnet_b200.data.synthetic import synthetic_packed_batch

    g = torch.Generator().manual_seed(seed)
    B, T, V, W = cfg["micro_batch"], cfg["seq_len"], cfg["vocab_size"], cfg["n_write"]
    pin = torch.cuda.is_available()
    out = []
    for _ in range(n_batches):
        if cfg.get("mode") == "sp":
            full = torch.randint(1, V, (B, T + 1), generator=g)
            tl = T // world
            seq = full[:, rank * tl : (rank + 1) * tl + 1].contiguous()
            wc = None
            if W > 0:       # earlier sequences of the same stream, cut into the same shards
                wc = torch.randint(1, V, (B, W, T), generator=g)[:, :, rank * tl : (rank + 1) * tl].contiguous()
                wc = wc.pin_memory() if pin else wc
        else:
            seq, _, _ = synthetic_packed_batch(B, T, V, 1024.0, g)
            wc = None
            if W > 0:
                wc, _, _ = synthetic_packed_batch(B * W, T - 1, V, 1024.0, g)
                wc = wc.view(B, W, T)
                wc = wc.pin_memory() if pin else wc
        seq = seq.pin_memory() if pin else seq
        out.append((seq, wc))
    return out


def build_ours(cfg, device, world):
    import torch

    from gdnet_b200.model import GDNet
    from gdnet_b200.train.engine import TrainEngine
    from gdnet_b200.utils.fp8 import cast_for_precision

    torch.manual_seed(0)
    model = GDNet(vocab_size=cfg["vocab_size"], d_embed=cfg["d_embed"], d=cfg["d"], n_layers=cfg["n_layers"],
                  n_cycles=cfg["n_cycles"], kernel_size=cfg["kernel_size"], chunk_size=cfg["seq_len"]).to(device)
    cast_for_precision(model, "fp8")
    sp_group = None
    if cfg.get("mode") == "sp" and world > 1:
        import torch.distributed as dist

        sp_group = dist.group.WORLD
    share = os.environ.get("GDNET_SHARE_FP8", "1" if cfg.get("share_fp8") else "0") == "1"
    engine = TrainEngine(model, lr=1e-3, precision="fp8", sp_group=sp_group,
                         comm=os.environ.get("GDNET_COMM", cfg.get("comm", "fused")), share_fp8_weights=share,
                         fused_ce=os.environ.get("GDNET_FUSED_CE", "1") == "1",
                         shard=os.environ.get("GDNET_SHARD", cfg.get("shard", "none")))

    def step(tokens, targets, write_chunks):
        return engine.projected_step(tokens, targets, write_chunks=write_chunks)

    def launches():
        from gdnet_b200.ops import cuda as cu

        return cu.launch_count()

    step.engine = engine
    return step, launches


def build_reference(cfg, device, world, local_rank):
    import torch

    ref_root = os.path.join(ROOT, "baseline", "_ref")
    sys.path.insert(0, ref_root)
    if not os.path.exists(os.path.join(ref_root, "gdnet", "kernel", "fp8_linear", "gemm.py")):
        # The reference's SM90 CuTe-DSL GEMM (gdnet/kernel/fp8_linear/gemm.py) is left out of snapshots
        # that run on 2 or more GPUs. The reference marks it "Unused for now" and its FP8 linear never
        # calls it (it uses torch._scaled_mm); only the package __init__ imports the name. Provide the
        # name so the rest of the unmodified package imports.
        import types

        stub = types.ModuleType("gdnet.kernel.fp8_linear.gemm")

        def fp8_gemm(*_a, **_k):
            raise NotImplementedError("the reference's SM90 fp8_gemm is not part of this snapshot")

        stub.fp8_gemm = fp8_gemm
        sys.modules["gdnet.kernel.fp8_linear.gemm"] = stub
    from gdnet.loss import projected_step  # noqa: E402  (the unmodified reference package)
    from gdnet.model import GDNet
    from gdnet.utils.distributed import get_dp_group, init_process_groups
    from gdnet.utils.fp8 import convert_to_fp8, update_fp8_scales

    torch.set_float32_matmul_precision("high")
    torch.manual_seed(0)
    sp = cfg.get("mode") == "sp" and world > 1
    # sequence parallel as the reference's scripts/throughput.py:218-252 sets it up: all ranks in one SP group,
    # the model's chunk size is the local shard, DDP over the (single-rank) data-parallel group
    chunk = cfg["seq_len"] // world if sp else cfg["seq_len"]
    model = GDNet(vocab_size=cfg["vocab_size"], d_embed=cfg["d_embed"], d=cfg["d"], n_layers=cfg["n_layers"],
                  n_cycles=cfg["n_cycles"], kernel_size=cfg["kernel_size"], chunk_size=chunk).to(device)
    model.embed.weight.data = model.embed.weight.data.bfloat16()
    convert_to_fp8(model)
    base = model
    sp_group = None
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP

        init_process_groups(world if sp else 1)
        if sp:
            from gdnet.utils.distributed import get_sp_group

            sp_group = get_sp_group()
        model = DDP(model, device_ids=[local_rank], process_group=get_dp_group(), static_graph=True,
                    bucket_cap_mb=200, broadcast_buffers=False)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-3)
    params = list(model.parameters())
    counter = {"i": 0}

    def step(tokens, targets, write_chunks):
        loss = projected_step(model, params, optimizer, tokens, targets, precision="fp8", write_chunks=write_chunks,
                              sp_group=sp_group)
        if counter["i"] % 16 == 0:
            update_fp8_scales(base)
        counter["i"] += 1
        return loss

    return step, (lambda: 0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=sorted(CONFIGS), default="350m")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]

    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "gdnet")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/gdnet is not installed"}))
        return

    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    try:
        if args.impl == "ours":
            step, launches = build_ours(cfg, device, world)
        else:
            step, launches = build_reference(cfg, device, world, local_rank)
    except Exception as exc:  # the reference may be unable to run here; say why in one line
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}))
            return
        raise

    W, K = max(args.warmup, 0), args.steps
    sp = cfg.get("mode") == "sp"
    batches = make_batches(cfg, W + 2 * K, seed=1234 + (0 if sp else rank), rank=rank, world=world)
    T = cfg["seq_len"]

    def to_device(b):
        seq = b[0].to(device, non_blocking=True)
        wc = b[1].to(device, non_blocking=True) if b[1] is not None else None
        return seq[:, :-1], seq[:, 1:], wc

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # warm-up (also JIT / autotune / cache fill)
    first = None
    for i in range(W):
        tok, tgt, wc = to_device(batches[i])
        out = step(tok, tgt, wc)
        if i == 0:
            first = float(out)      # loss of the very first step: the same on both arms when they compute the same model
    sync_all()

    # (1) device-timed, inputs resident on the device
    dev_batches = [to_device(b) for b in batches[W : W + K]]
    sync_all()
    n0 = launches()
    eng = getattr(step, "engine", None)
    if eng is not None:
        eng.time_updates = True
    ws = getattr(eng, "weight_stream", None) if eng is not None else None
    gathered0 = ws.gathered_bytes if ws is not None else 0
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for tok, tgt, wc in dev_batches:
        step(tok, tgt, wc)
    ev1.record()
    sync_all()
    clocks = sampler.stop()
    n_launch = launches() - n0
    gathered = (ws.gathered_bytes - gathered0) / K if ws is not None else None
    ms_dev = ev0.elapsed_time(ev1) / K
    update_ms = None
    breakdown = None
    if eng is not None:
        ts = sorted(eng.update_times_ms())
        breakdown = eng.update_breakdown_ms()
        eng.time_updates = False
        update_ms = ts[len(ts) // 2] if ts else None

    # (2) end to end through the public step call: H2D of the step's inputs, D2H of its loss
    sync_all()
    t0 = time.perf_counter()
    last = 0.0
    for b in batches[W + K : W + 2 * K]:
        tok, tgt, wc = to_device(b)
        last = float(step(tok, tgt, wc))
    sync_all()
    ms_e2e = (time.perf_counter() - t0) * 1000.0 / K

    t = torch.tensor([ms_dev, ms_e2e, update_ms if update_ms is not None else -1.0], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = float(t[0]), float(t[1])
    update_ms = float(t[2]) if float(t[2]) >= 0 else None
    global_batch = cfg["micro_batch"] * (1 if sp else world)     # sequences per step over the whole job
    value = global_batch * T / (ms_dev / 1000.0)
    e2e = global_batch * T / (ms_e2e / 1000.0)
    h2d = batches[0][0].numel() * 8 + (batches[0][1].numel() * 8 if batches[0][1] is not None else 0)
    comm = os.environ.get("GDNET_COMM", cfg.get("comm", "fused")) if world > 1 else "local"

    if rank == 0:
        print(json.dumps({
            "impl": args.impl,
            "metric": "train tokens/sec/box (device, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "strong" if sp else "weak",
            "vs_baseline": (value / BASELINE_TOK_S) if BASELINE_TOK_S else None,
            "dtype": "fp8-e4m3 linears / bf16 activations", "data": "synthetic packed tokens, random-init weights",
            "config": {"model": f"gdnet-{args.config} d={cfg['d']} L={cfg['n_layers']} cycles={cfg['n_cycles']} "
                                f"k={cfg['kernel_size']} vocab={cfg['vocab_size']}",
                       "global_batch": global_batch, "seq_len": T,
                       "parallelism": f"sp{world}" if sp else f"dp{world}",
                       "comm": comm if args.impl == "ours" else "nccl",
                       "step": f"projected_step, {cfg['n_write']} CAM write chunks, AdamW",
                       "l2": f"inputs larger than L2: every step touches {torch.cuda.max_memory_allocated() / 1e9:.1f} GB "
                             "of live tensors (peak allocated), L2 is 0.126 GB"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": n_launch,
            # device time of the update phase per step (gradient collective + projection + AdamW + parameter
            # all-gather, waits for slower ranks included), max over ranks; on one GPU it is the optimizer alone
            "update_phase_ms": update_ms,
            # rank 0's last update kernel, by device timestamps: wait for the slowest rank at its opening barrier,
            # pulling the peers' gradients + projection + AdamW + storing the parameters to all ranks, closing barrier
            "update_breakdown_ms": breakdown,
            # bytes of parameters, gradient buffers and AdamW moments resident on rank 0, and (fully sharded layer
            # matrices) the bytes of GEMM operands it pulled from their owner ranks per step
            "resident_bytes": eng.resident_bytes() if eng is not None else None,
            "gathered_bytes_per_step": gathered,
            "first_loss": first,
            "last_loss": last,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
