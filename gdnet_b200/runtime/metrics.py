"""Step metrics: device-timed step time (CUDA events), tokens/s, JSONL sink, optional wandb."""

from __future__ import annotations

import json
import time
from pathlib import Path


class StepTimer:
    """CUDA-event timing of a window of steps without synchronising every step."""

    def __init__(self, device=None):
        import torch

        self.torch = torch
        self.on_gpu = torch.cuda.is_available() and (device is None or getattr(device, "type", "cuda") == "cuda")
        self._t0 = None
        self._ev0 = None

    def start(self) -> None:
        if self.on_gpu:
            self._ev0 = self.torch.cuda.Event(enable_timing=True)
            self._ev0.record()
        self._t0 = time.perf_counter()

    def stop(self, n_steps: int) -> tuple[float, float]:
        """Returns ``(device_ms_per_step, wall_ms_per_step)``; synchronises once."""
        dev_ms = float("nan")
        if self.on_gpu and self._ev0 is not None:
            ev1 = self.torch.cuda.Event(enable_timing=True)
            ev1.record()
            ev1.synchronize()
            dev_ms = self._ev0.elapsed_time(ev1) / max(n_steps, 1)
        wall_ms = (time.perf_counter() - self._t0) * 1000.0 / max(n_steps, 1)
        return dev_ms, wall_ms


class MetricsLog:
    def __init__(self, path: str = "", wandb_project: str = "", run: str = "", config: dict | None = None):
        self._fh = None
        if path:
            Path(path).parent.mkdir(parents=True, exist_ok=True)
            self._fh = open(path, "a")
        self._wandb = None
        if wandb_project:
            try:
                import wandb

                wandb.init(project=wandb_project, name=run or None, config=config or {}, resume="allow")
                self._wandb = wandb
            except Exception as exc:  # no network / not installed: keep training
                print(f"[metrics] wandb disabled: {exc}")

    def log(self, step: int, **values) -> None:
        if self._fh is not None:
            self._fh.write(json.dumps({"step": step, "time": time.time(), **values}) + "\n")
            self._fh.flush()
        if self._wandb is not None:
            self._wandb.log(values, step=step)

    def close(self) -> None:
        if self._fh is not None:
            self._fh.close()
        if self._wandb is not None:
            self._wandb.finish()
