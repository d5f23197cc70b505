"""Debug aids for the kernels of this package (the reference ships none: no sanitizer run, no assertions).

``RedZones``: while the mode is active every tensor that ``torch.empty`` / ``zeros`` / ``empty_like`` / ``new_empty``
and friends create on the watched device is carved out of a slightly larger allocation whose tail is filled with a
canary byte; ``check()`` verifies every tail written since the last check and raises ``RedZoneError`` naming the
tensor whose red zone was overwritten. The fused CUDA ops allocate all their outputs and scratch buffers through
exactly these calls, so a kernel that stores past the end of one of them is caught at the next check, on any
device and without a sanitizer. The mode keeps the buffers of one interval alive until they are checked: use it on
small shapes.

``engine_invariants``: what the peer-memory kernels must leave behind after a completed step, read back on the
host: a clean status word, block counters back at zero, and every peer's flag word exactly at the sequence number of
the last launch (a larger value means a rank ran ahead, a smaller one that a signal was lost).

    with RedZones(device) as rz:
        loss = engine.projected_step(tokens, targets)
        rz.check()
    engine_invariants(engine)          # all ranks, between steps
"""

from __future__ import annotations

import torch
from torch.utils._python_dispatch import TorchDispatchMode

CANARY = 0xA5
PAD = 256      # bytes behind every tensor

_ALLOC_OPS = None


def _alloc_ops():
    global _ALLOC_OPS
    if _ALLOC_OPS is None:
        a = torch.ops.aten
        _ALLOC_OPS = {
            a.empty.memory_format: False, a.empty_like.default: False, a.new_empty.default: False,
            a.empty_strided.default: False,
            a.zeros.default: True, a.zeros_like.default: True, a.new_zeros.default: True,
        }
    return _ALLOC_OPS


class RedZoneError(RuntimeError):
    """Bytes behind a tensor were overwritten."""


class RedZones(TorchDispatchMode):
    def __init__(self, device=None, pad: int = PAD):
        super().__init__()
        self.device = torch.device(device) if device is not None else None
        self.pad = int(pad)
        self._live: list = []          # (raw uint8 buffer, payload bytes, description)
        self._busy = False
        self.checked = 0

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        out = func(*args, **kwargs)
        zero = _alloc_ops().get(func)
        if zero is None or self._busy or not isinstance(out, torch.Tensor):
            return out
        if (self.device is not None and out.device != self.device) or out.numel() == 0 or not out.is_contiguous() \
                or out.device.type == "meta":
            return out
        self._busy = True
        try:
            nbytes = out.numel() * out.element_size()
            # the payload keeps the 16-byte alignment the kernels ask for; the red zone starts right behind it
            raw = torch.empty(nbytes + self.pad, dtype=torch.uint8, device=out.device)
            raw[nbytes:].fill_(CANARY)
            guarded = raw[:nbytes].view(out.dtype).view(out.shape)
            if zero:
                guarded.zero_()
            self._live.append((raw, nbytes, f"{tuple(out.shape)} {out.dtype} from {func}"))
        finally:
            self._busy = False
        return guarded

    def check(self) -> int:
        """Verify the red zones of everything allocated since the last check; returns how many were verified."""
        self._busy = True
        try:
            n = 0
            for raw, nbytes, what in self._live:
                tail = raw[nbytes:]
                bad = tail != CANARY
                if bool(bad.any()):
                    first = int(bad.nonzero()[0])
                    self._live.clear()
                    raise RedZoneError(f"{int(bad.sum())} byte(s) behind a tensor {what} were overwritten, the first "
                                       f"{first} byte(s) past its end")
                n += 1
            self._live.clear()
            self.checked += n
            return n
        finally:
            self._busy = False

    def __exit__(self, *exc):
        try:
            if exc[0] is None:
                self.check()
        finally:
            return super().__exit__(*exc)


def engine_invariants(engine) -> None:
    """Host-side check of what a completed training step leaves in the exchange areas of ``engine`` (see the module
    docstring). Every rank calls it between steps; with several ranks it synchronises them first so that no peer is
    already inside the next step."""
    import torch.distributed as dist

    from .. import _ext

    dev = next(engine.parameters()).device
    on_gpu = dev.type == "cuda"
    if on_gpu:
        torch.cuda.synchronize(dev)
        _ext.check_status(torch.empty(1, device=dev))
    for g in engine.groups:
        counter = g.sums[4:5].view(torch.int32)
        if int(counter) != 0:
            raise AssertionError(f"block counter of the update kernel is {int(counter)}, not 0: a launch did not finish")
    flags = getattr(engine, "_flags", None)
    if flags is None or engine.world == 1:
        return
    if on_gpu:
        dist.barrier(group=engine.pg)
        torch.cuda.synchronize(dev)
    words = flags.view(torch.int32, 3 * engine.world).tolist()
    last_gi = len(engine.groups) - 1
    expect = {0: engine.comm_seq * 8 + last_gi, 1: engine.comm_seq * 8 + last_gi}
    if getattr(engine, "task_seq", 0) and engine.overlap_task_reduce:
        expect[2] = engine.task_seq * 8 + last_gi
    if engine.comm not in ("fused", "scatter") or engine.comm_seq == 0:
        return
    for slot, want in expect.items():
        for writer in range(engine.world):
            if writer == engine.rank:
                continue
            got = words[slot * engine.world + writer]
            if got != want:
                raise AssertionError(f"flag of rank {writer} in slot {slot} on rank {engine.rank} is {got}, expected {want} "
                                     f"({'a rank ran ahead' if got > want else 'a signal is missing'})")
