"""Query-only GPU monitor and live result tables for the throughput sweep.

``GpuMonitor`` samples utilisation, memory, power and SM clock of every visible GPU through NVML on a background
thread (reference: the ``Monitor`` thread of scripts/throughput.py:152-197). It only *reads*: no clock, power or
mode setting of a GPU is touched. ``LiveTables`` renders the rows measured so far and the last GPU sample with
``rich`` when the output is a terminal, and falls back to plain lines otherwise (reference: scripts/throughput.py:85-149).
"""

from __future__ import annotations

import threading
import time


class GpuMonitor(threading.Thread):
    def __init__(self, period: float = 0.5, nvml=None):
        super().__init__(daemon=True)
        self.period = period
        self._nvml = nvml            # injectable for tests (any object with the few pynvml calls used below)
        self._halt = threading.Event()
        self.latest: list[dict] = []
        self.peak_mem_gib: dict[int, float] = {}
        self.error: str | None = None

    def _lib(self):
        if self._nvml is None:
            import pynvml

            self._nvml = pynvml
        return self._nvml

    def sample(self) -> list[dict]:
        nv = self._lib()
        out = []
        for i in range(nv.nvmlDeviceGetCount()):
            h = nv.nvmlDeviceGetHandleByIndex(i)
            util = nv.nvmlDeviceGetUtilizationRates(h)
            mem = nv.nvmlDeviceGetMemoryInfo(h)
            row = {"index": i, "util": int(util.gpu), "mem_gib": mem.used / 2**30, "mem_total_gib": mem.total / 2**30,
                   "power_w": nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                   "sm_mhz": int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))}
            self.peak_mem_gib[i] = max(self.peak_mem_gib.get(i, 0.0), row["mem_gib"])
            out.append(row)
        return out

    def run(self):
        try:
            self._lib().nvmlInit()
            while not self._halt.is_set():
                self.latest = self.sample()
                time.sleep(self.period)
        except Exception as exc:          # NVML missing or not permitted: the sweep goes on without the GPU table
            self.error = f"{type(exc).__name__}: {exc}"

    def stop(self):
        self._halt.set()
        self.join(timeout=2)


class LiveTables:
    """Result rows plus the GPU table, redrawn in place on a terminal; plain lines elsewhere."""

    COLUMNS = (("B", "{:>4}"), ("T", "{:>6}"), ("ms/step", "{:>10.1f}"), ("tok/s", "{:>12,.0f}"), ("params(M)", "{:>10.1f}"),
               ("mem(GiB)", "{:>9.1f}"))

    def __init__(self, title: str, monitor: GpuMonitor | None = None, force_plain: bool = False, stream=None):
        import sys

        self.title, self.monitor = title, monitor
        self.rows: list[dict] = []
        self.stream = stream or sys.stdout
        self._live = None
        if not force_plain and getattr(self.stream, "isatty", lambda: False)():
            try:
                from rich.live import Live

                self._live = Live(self._render(), refresh_per_second=2, transient=False)
                self._live.start()
            except Exception:             # rich missing or the terminal refuses: plain lines
                self._live = None
        if self._live is None:
            print(title, file=self.stream)
            print(" ".join(f"{name:>{len(fmt.format(0))}}" for name, fmt in self.COLUMNS), file=self.stream)

    @staticmethod
    def _cells(row):
        vals = (row["B"], row["T"], row["ms"], row["tok_s"], row["params"] / 1e6, row["mem_gib"])
        return [fmt.format(v) for (_, fmt), v in zip(LiveTables.COLUMNS, vals)]

    def _render(self):
        from rich.console import Group
        from rich.table import Table

        res = Table(title=self.title)
        for name, _ in self.COLUMNS:
            res.add_column(name, justify="right")
        res.add_column("")
        for row in self.rows:
            res.add_row(*self._cells(row), "OOM" if row.get("oom") else "")
        parts = [res]
        if self.monitor is not None and self.monitor.latest:
            gpu = Table(title="GPUs (NVML, read only)")
            for name in ("gpu", "util %", "mem GiB", "power W", "SM MHz"):
                gpu.add_column(name, justify="right")
            for g in self.monitor.latest:
                gpu.add_row(str(g["index"]), str(g["util"]), f"{g['mem_gib']:.1f} / {g['mem_total_gib']:.0f}",
                            f"{g['power_w']:.0f}", str(g["sm_mhz"]))
            parts.append(gpu)
        return Group(*parts)

    def add(self, row: dict) -> None:
        self.rows.append(row)
        if self._live is not None:
            self._live.update(self._render())
        else:
            print(" ".join(self._cells(row)) + ("  OOM" if row.get("oom") else ""), file=self.stream, flush=True)

    def close(self) -> None:
        if self._live is not None:
            self._live.update(self._render())
            self._live.stop()
        elif self.monitor is not None and self.monitor.latest:
            for g in self.monitor.latest:
                print(f"gpu {g['index']}: util {g['util']} %, mem {g['mem_gib']:.1f} GiB (peak {self.monitor.peak_mem_gib.get(g['index'], 0):.1f}), "
                      f"{g['power_w']:.0f} W, SM {g['sm_mhz']} MHz", file=self.stream)
