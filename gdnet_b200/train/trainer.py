"""Pre-training loop: phases, data pipeline, interactive shell, logging, checkpoints.

Behavioural parity with the reference's ``scripts/training.py`` (same config keys, same batch
geometry ``B = token_budget // T`` sliced by DP rank along the batch and by SP rank along time,
``n_write`` previous batches as CAM write chunks, WSD learning-rate schedule, rank-0 shell with
``status | eta | gpu | save | stop | lr [val] | help``, checkpoints ``step_XXXXXXX.pt`` /
``_manual`` / ``_final``). Differences: device-timed step time (CUDA events) next to wall time,
JSONL metrics, heartbeats for the watchdog, the data cursor stored in the checkpoint, a stat-poll
instead of an inotify library to wait for a token file, and AdamW from the flat-buffer engine
(or ``torch.optim.AdamW`` with ``engine: false``) instead of bitsandbytes' 8-bit AdamW.
"""

from __future__ import annotations

import dataclasses
import os
import sys
import threading
import time
from collections import deque
from pathlib import Path

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader

from ..config import Config, global_batch, wsd_lr
from ..data import (CopyTaskDataset, FineWebEduDataset, NemotronDataset, PackedTokenDataset,
                    SyntheticPackedDataset)
from ..models.gdnet import GDNet
from ..parallel import groups
from ..runtime.ckpt import load_ckpt, load_sharded, save_ckpt, save_sharded
from ..runtime.metrics import MetricsLog, StepTimer
from ..runtime.watchdog import Heartbeat, Watchdog
from ..utils.fp8 import cast_for_precision, update_fp8_scales
from .step import projected_step


@dataclasses.dataclass
class State:
    step: int = 0
    total_steps: int = 0
    loss: float = float("nan")
    lr: float = 0.0
    tok_per_sec: float = 0.0
    ms_per_step: float = 0.0
    device_ms_per_step: float = float("nan")
    phase: str = ""


class Shell(threading.Thread):
    """Rank-0 command prompt on stdin; commands act between steps."""

    HELP = "status  eta  gpu  save  stop  lr [val]  help"

    def __init__(self, state: State, set_lr, get_lr, stop_event, save_event, stream_in=None, stream_out=None):
        super().__init__(daemon=True)
        self.state, self.set_lr, self.get_lr = state, set_lr, get_lr
        self.stop_event, self.save_event = stop_event, save_event
        self.inp = stream_in if stream_in is not None else sys.stdin
        self.out = stream_out if stream_out is not None else sys.stdout

    def say(self, text: str) -> None:
        self.out.write(text)
        self.out.flush()

    def run(self) -> None:
        while not self.stop_event.is_set():
            try:
                self.say(">> ")
                line = self.inp.readline()
            except (EOFError, OSError, ValueError):
                return
            if not line:
                return
            self.handle(line.strip())

    def handle(self, line: str) -> None:
        words = line.split()
        if not words:
            return
        cmd, args, s = words[0], words[1:], self.state
        if cmd == "status":
            pct = 100.0 * s.step / max(s.total_steps, 1)
            self.say(f"phase      : {s.phase}\nstep       : {s.step}/{s.total_steps}  ({pct:.1f}%)\n"
                     f"loss       : {s.loss:.4f}\nlr         : {s.lr:.2e}\n"
                     f"throughput : {s.tok_per_sec:,.0f} tok/s\nms/step    : {s.ms_per_step:.1f} "
                     f"(device {s.device_ms_per_step:.1f})\n")
        elif cmd == "eta":
            left = s.total_steps - s.step
            if s.ms_per_step > 0 and left > 0:
                secs = int(left * s.ms_per_step / 1000)
                self.say(f"eta: {secs // 3600}h {secs % 3600 // 60}m {secs % 60}s  ({left} steps)\n")
            else:
                self.say("eta: unknown\n")
        elif cmd == "gpu":
            self.say(gpu_report())
        elif cmd == "save":
            self.save_event.set()
            self.say("checkpoint queued\n")
        elif cmd == "stop":
            self.stop_event.set()
            self.say("stopping after current step...\n")
        elif cmd == "lr":
            if not args:
                self.say(f"lr = {self.get_lr():.2e}\n")
            else:
                try:
                    self.set_lr(float(args[0]))
                    self.say(f"lr -> {float(args[0]):.2e}\n")
                except ValueError:
                    self.say(f"bad value: {args[0]}\n")
        elif cmd == "help":
            self.say(self.HELP + "\n")
        else:
            self.say(f"unknown: {cmd}\n")


def gpu_report() -> str:
    """Utilisation and memory of every visible GPU through NVML (read-only queries)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        lines = []
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            util, mem = pynvml.nvmlDeviceGetUtilizationRates(h), pynvml.nvmlDeviceGetMemoryInfo(h)
            used, total = mem.used / 2**30, mem.total / 2**30
            lines.append(f"gpu[{i}]  util={util.gpu}%  mem={used:.1f}/{total:.1f} GB  ({100 * used / total:.1f}%)\n")
        return "".join(lines) or "no GPUs\n"
    except Exception as exc:
        return f"NVML unavailable: {exc}\n"


class CudaPrefetcher:
    """Copies the next batch to the device on a side stream while the current step computes
    (reference: scripts/training.py:220-255). Batches are pinned first so the copy is asynchronous."""

    def __init__(self, loader, device: torch.device) -> None:
        self._it, self._device = iter(loader), device
        self._stream = torch.cuda.Stream(device) if device.type == "cuda" else None
        self._next = None
        self._fetch()

    def _fetch(self) -> None:
        try:
            batch = next(self._it)
        except StopIteration:
            self._next = None
            return
        if self._stream is None:
            self._next = batch
            return
        with torch.cuda.stream(self._stream):
            move = lambda t: (t if t.is_pinned() else t.pin_memory()).to(self._device, non_blocking=True)
            self._next = tuple(move(t) for t in batch) if isinstance(batch, (tuple, list)) else move(batch)

    def __iter__(self):
        return self

    def __next__(self):
        if self._stream is not None:
            torch.cuda.current_stream(self._device).wait_stream(self._stream)
        batch = self._next
        if batch is None:
            raise StopIteration
        self._fetch()
        return batch


def wait_for_file(path: str, rank: int = 0, poll_s: float = 2.0, timeout_s: float | None = None) -> None:
    """Block until ``path`` exists and is non-empty (the tokeniser may still be writing later phases)."""
    p = Path(path)
    t0 = time.time()
    told = False
    while not (p.exists() and p.stat().st_size > 0):
        if not told and rank == 0:
            print(f"[data] waiting for {path} ...", flush=True)
            told = True
        if timeout_s is not None and time.time() - t0 > timeout_s:
            raise TimeoutError(f"{path} did not appear within {timeout_s} s")
        time.sleep(poll_s)


def make_dataset(phase: dict, cfg: Config, start_window: int = 0):
    source = phase.get("dataset", "fineweb-edu")
    seq_len = phase["seq_len"]
    path = phase.get("path")
    if path and Path(path).exists():
        return PackedTokenDataset(paths=path, seq_len=seq_len, start_window=start_window)
    if source == "packed":
        raise FileNotFoundError(f"packed dataset not found: {path}")
    if source == "synthetic":
        return SyntheticPackedDataset(seq_len, cfg.vocab_size, phase.get("mean_doc_len", 1024.0), cfg.seed)
    if source == "copy":
        return CopyTaskDataset(seq_len, phase.get("n_copy", 64), cfg.vocab_size, cfg.seed)
    if source == "fineweb-edu":
        return FineWebEduDataset(seq_len=seq_len, min_int_score=phase["min_int_score"],
                                 max_int_score=phase["max_int_score"], encoding=cfg.tokenizer,
                                 subset=phase.get("subset", "sample-10BT"), seed=cfg.seed)
    if source == "nemotron":
        return NemotronDataset(seq_len=seq_len, encoding=cfg.tokenizer, subset=phase.get("subset", "everything"),
                               min_chars=phase.get("min_chars", 0), seed=cfg.seed)
    raise ValueError(f"unknown dataset source '{source}'")


def build_model(cfg: Config, device: torch.device, sp_size: int) -> GDNet:
    max_seq = max(p["seq_len"] for p in cfg.phases)
    if max_seq % sp_size:
        raise ValueError(f"max seq_len {max_seq} must be divisible by sp_size {sp_size}")
    torch.manual_seed(cfg.seed)
    model = GDNet(vocab_size=cfg.vocab_size, d_embed=cfg.d_embed, d=cfg.d, n_layers=cfg.n_layers,
                  n_cycles=cfg.n_cycles, chunk_size=max_seq // sp_size, kernel_size=cfg.kernel_size,
                  n_slots=cfg.n_slots).to(device)
    return cast_for_precision(model, cfg.precision, cfg.fp8_recipe)


def train(cfg: Config, interactive: bool = True) -> State:
    """Run every phase of ``cfg``. Returns the final :class:`State` (rank 0's view)."""
    if not cfg.phases:
        raise ValueError("config must define at least one phase")
    groups.init_distributed()
    world, rank = groups.get_world_size(), groups.get_rank()
    sp_size = cfg.sp_size if world > 1 else 1
    groups.init_process_groups(sp_size)
    sp_group, dp_group = (groups.get_sp_group(), groups.get_dp_group()) if world > 1 else (None, None)
    sp_rank = dist.get_rank(sp_group) if sp_group is not None else 0
    dp_size = dist.get_world_size(dp_group) if dp_group is not None else 1
    dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
    if sp_size == 1:
        sp_group = None
    main_proc = rank == 0
    on_gpu = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if on_gpu else torch.device("cpu")

    model = build_model(cfg, device, sp_size)
    use_engine = cfg.engine and on_gpu and cfg.precision != "fp32"
    if use_engine:
        from .engine import TrainEngine

        runner = TrainEngine(model, lr=cfg.lr, betas=(cfg.beta1, cfg.beta2), weight_decay=cfg.weight_decay,
                             precision=cfg.precision, sp_group=sp_group, comm=cfg.comm, shard=cfg.shard)
        optimizer, params = None, None
        set_lr, get_lr = runner.set_lr, (lambda: runner.lr)
    else:
        runner = model
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP

            runner = DDP(model, device_ids=[device.index] if on_gpu else None, process_group=dp_group,
                         broadcast_buffers=False)
        params = list(runner.parameters())
        optimizer = torch.optim.AdamW(params, lr=cfg.lr, betas=(cfg.beta1, cfg.beta2), weight_decay=cfg.weight_decay)

        def set_lr(v):
            for pg in optimizer.param_groups:
                pg["lr"] = v

        get_lr = lambda: optimizer.param_groups[0]["lr"]

    # With several GPUs the engine keeps AdamW moments (and, fully sharded, the layer matrices) only for its own
    # shard, so a checkpoint is a directory to which every rank writes its part; one GPU writes the single file.
    sharded_ckpt = use_engine and world > 1
    step, cursor = 0, {}
    if cfg.resume:
        if Path(cfg.resume).is_dir():
            if not use_engine:
                raise ValueError("a sharded checkpoint directory can only be resumed by the training engine")
            step, cursor = load_sharded(Path(cfg.resume), runner)
        else:
            step, cursor = load_ckpt(Path(cfg.resume), model, optimizer)
            if use_engine and cursor.get("engine_optim"):
                runner.load_state_dict_optim(cursor["engine_optim"])

    ckpt_dir = Path(cfg.ckpt_dir)
    state = State(total_steps=cfg.total_steps, step=step)
    stop_event, save_event = threading.Event(), threading.Event()
    metrics = MetricsLog(cfg.metrics_file if main_proc else "", cfg.project if main_proc else "", cfg.run,
                         dataclasses.asdict(cfg))
    heartbeat = Heartbeat(cfg.heartbeat_dir, rank) if cfg.heartbeat_dir else None
    watchdog = None
    if main_proc:
        ckpt_dir.mkdir(parents=True, exist_ok=True)
        if interactive and sys.stdin is not None and sys.stdin.isatty():
            Shell(state, set_lr, get_lr, stop_event, save_event).start()
        if cfg.heartbeat_dir and world > 1:
            watchdog = Watchdog(cfg.heartbeat_dir, world,
                                on_failure=lambda r: print(f"[watchdog] ranks not advancing: {r}", flush=True))
            watchdog.start()

    def checkpoint(tag: str, windows_done: int, phase_idx: int) -> None:
        """Every rank calls this at the same step. One GPU: the reference's single file, written by the only
        rank. Several GPUs with the engine: a directory with one shard file per rank."""
        if sharded_ckpt:
            extra = {"phase": phase_idx, "windows_done": windows_done}
            save_sharded(ckpt_dir / f"step_{step:07d}{tag}", step, runner, extra)
            return
        if not main_proc:
            return
        extra = {"phase": phase_idx, "windows_done": windows_done, "rng": torch.get_rng_state()}
        if use_engine:
            extra["engine_optim"] = runner.state_dict_optim()
        save_ckpt(ckpt_dir / f"step_{step:07d}{tag}.pt", step, model, optimizer, None, extra)

    def agree(flags: list[bool]) -> list[bool]:
        """Rank 0's decisions (stop, manual save), made known to every rank: they come from its console."""
        if world == 1:
            return flags
        t = torch.tensor([int(f) for f in flags], device=device, dtype=torch.int32)
        dist.broadcast(t, src=0)
        return [bool(x) for x in t.tolist()]

    windows_done, phase_idx = 0, 0
    stopping, clean_exit = False, False
    try:
        phase_start = 0
        for phase_idx, phase in enumerate(cfg.phases):
            phase_end = phase_start + phase["steps"]
            if step >= phase_end:
                phase_start = phase_end
                continue
            T = phase["seq_len"]
            if T % sp_size:
                raise ValueError(f"phase seq_len {T} must be divisible by sp_size {sp_size}")
            T_local = T // sp_size
            B = global_batch(cfg, T, dp_size)
            state.phase = f"{phase.get('dataset', 'fineweb-edu')}  seq_len={T}  B={B}  steps {phase_start}-{phase_end}"
            if phase.get("path"):
                wait_for_file(phase["path"], rank)
            resume_here = cursor.get("phase") == phase_idx
            windows_done = int(cursor.get("windows_done", 0)) if resume_here else 0
            ds = make_dataset(phase, cfg, start_window=windows_done)
            nw = cfg.num_data_workers
            loader = DataLoader(ds, batch_size=B, num_workers=nw, pin_memory=on_gpu,
                                prefetch_factor=2 if nw > 0 else None, persistent_workers=nw > 0)
            write_buf: deque = deque(maxlen=max(cfg.n_write, 1))
            timer = StepTimer(device)
            timer.start()
            b_per = B // dp_size
            rows = slice(dp_rank * b_per, (dp_rank + 1) * b_per)
            cols = slice(sp_rank * T_local, (sp_rank + 1) * T_local)

            for batch in CudaPrefetcher(loader, device):
                if step >= phase_end or stopping:
                    break
                mask = None
                if isinstance(batch, (tuple, list)):          # copy task: (tokens, targets, loss mask)
                    tokens, targets, mask = (t[rows][:, cols] for t in batch)
                else:                                           # packed windows of seq_len + 1 ids
                    tokens, targets = batch[rows, :-1][:, cols], batch[rows, 1:][:, cols]
                write_chunks = None
                if cfg.n_write > 0 and model.cam_enabled and len(write_buf) == cfg.n_write:
                    write_chunks = torch.stack(list(write_buf), dim=1)
                write_buf.append(tokens.clone())

                set_lr(cfg.lr * wsd_lr(step, cfg))
                loss = projected_step(runner, params, optimizer, tokens, targets, beta=cfg.beta_proj,
                                      precision=cfg.precision, write_chunks=write_chunks, sp_group=sp_group,
                                      grad_clip=cfg.grad_clip, accum_steps=cfg.accum_steps, loss_mask=mask)
                step += 1
                windows_done += B
                state.step = step
                if cfg.precision == "fp8" and step % 16 == 0:
                    update_fp8_scales(model)
                if heartbeat is not None:
                    heartbeat.beat(step)

                if step % cfg.log_every == 0:
                    loss_val = float(loss)                     # the only host sync of the window
                    dev_ms, wall_ms = timer.stop(cfg.log_every)
                    state.loss, state.lr = loss_val, get_lr()
                    state.ms_per_step, state.device_ms_per_step = wall_ms, dev_ms
                    state.tok_per_sec = B * T / (wall_ms / 1000.0)
                    if main_proc:
                        metrics.log(step, loss=loss_val, lr=state.lr, tok_per_sec=state.tok_per_sec,
                                    ms_per_step=wall_ms, device_ms_per_step=dev_ms)
                    timer.start()
                if step % cfg.ckpt_every == 0:
                    checkpoint("", windows_done, phase_idx)
                if step % cfg.log_every == 0 or world == 1:
                    # the console commands of rank 0 take effect on all ranks at the same step
                    stopping, manual = agree([stop_event.is_set(), save_event.is_set()])
                    if manual:
                        save_event.clear()
                        checkpoint("_manual", windows_done, phase_idx)
            if stopping:
                break
            phase_start = phase_end
        clean_exit = True
    finally:
        # after an error the ranks are no longer in step: each writes what it can on its own, which for a sharded
        # checkpoint is its own shard file (the manifest comes from rank 0)
        try:
            checkpoint("_final", windows_done, phase_idx)
        except Exception as exc:                      # never mask the error that ended the run
            if clean_exit:
                raise
            print(f"[rank {rank}] final checkpoint failed: {exc}", flush=True)
        if main_proc:
            stop_event.set()
            metrics.close()
            if watchdog is not None:
                watchdog.stop()
        groups.destroy()
    return state
