"""Process-group bootstrap: one process per GPU, NCCL over NVLink for the plumbing.

Parity with the reference's ``gdnet/utils/distributed.py:31-98,181-290`` (same
function names and behaviour: env:// rendezvous, no-op when ``WORLD_SIZE`` is 1,
sequence-parallel groups are contiguous rank blocks and data-parallel groups are
strided). Additions: a ``gloo`` fallback is picked automatically when CUDA is absent,
and rendezvous defaults to 127.0.0.1.
"""

from __future__ import annotations

import logging
import os
from datetime import timedelta
from typing import Any, Callable

import torch
import torch.distributed as dist

log = logging.getLogger(__name__)

_SP_GROUP: dist.ProcessGroup | None = None
_DP_GROUP: dist.ProcessGroup | None = None
_SP_SIZE: int = 1


def sp_dp_ranks(world_size: int, sp_size: int) -> tuple[list[list[int]], list[list[int]]]:
    """Rank lists of every SP group (contiguous blocks) and DP group (strided)."""
    if sp_size < 1 or world_size % sp_size != 0:
        raise ValueError(f"world_size {world_size} not divisible by sp_size {sp_size}")
    dp_size = world_size // sp_size
    sp = [list(range(b * sp_size, (b + 1) * sp_size)) for b in range(dp_size)]
    dp = [list(range(s, world_size, sp_size)) for s in range(sp_size)]
    return sp, dp


def init_process_groups(sp_size: int = 1) -> None:
    """Create the SP and DP groups; every rank must call this with the same value."""
    global _SP_GROUP, _DP_GROUP, _SP_SIZE
    if not (dist.is_available() and dist.is_initialized()):
        return
    world, rank = dist.get_world_size(), dist.get_rank()
    sp_lists, dp_lists = sp_dp_ranks(world, sp_size)
    _SP_SIZE = sp_size
    for ranks in sp_lists:
        grp = dist.new_group(ranks)
        if rank in ranks:
            _SP_GROUP = grp
    for ranks in dp_lists:
        grp = dist.new_group(ranks)
        if rank in ranks:
            _DP_GROUP = grp


def init_distributed(backend: str | None = None, timeout_minutes: float = 30) -> None:
    """Initialise the default process group from RANK/WORLD_SIZE/MASTER_* (env://).

    Idempotent; a no-op for a single process. ``backend=None`` picks ``nccl`` when a GPU
    is visible and ``gloo`` otherwise.
    """
    if not dist.is_available():
        log.warning("torch.distributed is not available; running single-process")
        return
    if dist.is_initialized():
        return
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world == 1:
        return
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        if not torch.cuda.is_available():
            raise RuntimeError("the nccl backend needs CUDA; use backend='gloo' on CPU")
        torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", local_rank)
    dist.init_process_group(backend=backend, timeout=timedelta(minutes=timeout_minutes), **kwargs)
    log.info("distributed up: rank %d/%d local_rank %d backend %s", rank, world, local_rank, backend)


def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def is_main_process() -> bool:
    return get_rank() == 0


def get_sp_group() -> dist.ProcessGroup | None:
    """The caller's sequence-parallel group (WORLD if groups were never built)."""
    if not (dist.is_available() and dist.is_initialized()):
        return None
    return _SP_GROUP if _SP_GROUP is not None else dist.group.WORLD


def get_dp_group() -> dist.ProcessGroup | None:
    if not (dist.is_available() and dist.is_initialized()):
        return None
    return _DP_GROUP


def barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def destroy() -> None:
    global _SP_GROUP, _DP_GROUP
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
    _SP_GROUP = _DP_GROUP = None


def _worker(rank: int, world: int, fn: Callable, args: tuple, kwargs: dict, backend: str | None,
            timeout_minutes: float, master_addr: str, master_port: int) -> None:
    os.environ.update(
        RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
        MASTER_ADDR=master_addr, MASTER_PORT=str(master_port),
    )
    init_distributed(backend=backend, timeout_minutes=timeout_minutes)
    try:
        fn(*args, **kwargs)
    finally:
        destroy()


def launch(fn: Callable, *args: Any, devices: int | None = None, backend: str | None = None,
           timeout_minutes: float = 30, master_addr: str = "127.0.0.1", master_port: int = 29500,
           **kwargs: Any) -> None:
    """Run ``fn`` on ``devices`` spawned ranks (one per GPU; CPU ranks with gloo).

    ``fn`` must be importable at module level. With one device it is called inline.
    """
    if devices is None:
        devices = torch.cuda.device_count() if torch.cuda.is_available() else 1
    if devices <= 1:
        fn(*args, **kwargs)
        return
    from torch.multiprocessing.spawn import spawn

    spawn(_worker, nprocs=devices, join=True,
          args=(devices, fn, args, kwargs, backend, timeout_minutes, master_addr, master_port))
