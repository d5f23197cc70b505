"""Pre-tokenised packed data: raw little-endian ``uint32`` token files.

Parity with the reference's ``gdnet/data/packed.py``: windows of ``seq_len + 1`` tokens,
DataLoader worker ``w`` of ``n`` takes windows ``w, w+n, w+2n, ...``; several files are
read one after the other. Additions: an optional ``(rank, world)`` split of the window
stream (the reference feeds every rank the same stream and slices the batch), a
resumable cursor, and an optional native reader thread (``csrc/loader.cpp``) that
stages windows in pinned memory.
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch
from torch.utils.data import IterableDataset, get_worker_info


class PackedTokenDataset(IterableDataset):
    def __init__(self, paths, seq_len: int, rank: int = 0, world: int = 1, start_window: int = 0) -> None:
        self._paths = [Path(paths)] if isinstance(paths, (str, Path)) else [Path(p) for p in paths]
        self._seq_len = int(seq_len)
        self._rank, self._world = int(rank), int(world)
        self.start_window = int(start_window)

    def windows_in(self, path: Path) -> int:
        n_tokens = path.stat().st_size // 4
        return max(0, n_tokens // (self._seq_len + 1))

    def __iter__(self):
        info = get_worker_info()
        wid, nworkers = (info.id, info.num_workers) if info is not None else (0, 1)
        lane = self._rank * nworkers + wid
        lanes = self._world * nworkers
        span = self._seq_len + 1
        skip = self.start_window
        for path in self._paths:
            toks = np.memmap(path, dtype=np.uint32, mode="r")
            n_win = len(toks) // span
            for win in range(lane, n_win, lanes):
                if skip > 0:
                    skip -= 1
                    continue
                lo = win * span
                yield torch.from_numpy(toks[lo : lo + span].astype(np.int64))
