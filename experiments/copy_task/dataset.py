"""Synthetic recall tasks for the copy-with-gap study.

Vocabulary (reference: experiments/copy_task/dataset.py:6-9): signal tokens 0..9, noise tokens
10..49, the recall marker 50; size 52. A sample is the signal, a stretch of noise and the recall
marker; the label is the signal itself, to be named from the state at the recall marker.
"""

from __future__ import annotations

import torch
from torch.utils.data import Dataset

N_SIGNAL, N_NOISE = 10, 40
RECALL_TOKEN = N_SIGNAL + N_NOISE
VOCAB_SIZE = 52


def _noise(n: int, width: int, gen) -> torch.Tensor:
    return torch.randint(0, N_NOISE, (n, width), generator=gen) + N_SIGNAL


class _PairDataset(Dataset):
    inputs: torch.Tensor
    targets: torch.Tensor

    def __len__(self) -> int:
        return self.inputs.shape[0]

    def __getitem__(self, i):
        return self.inputs[i], self.targets[i]


class CopyWithGapDataset(_PairDataset):
    """``seq_len`` signal tokens, ``gap`` noise tokens, the recall marker.

    (reference: experiments/copy_task/dataset.py:12-35)
    """

    def __init__(self, n: int, seq_len: int = 3, gap: int = 8, generator: torch.Generator | None = None):
        sig = torch.randint(0, N_SIGNAL, (n, seq_len), generator=generator)
        self.inputs = torch.cat([sig, _noise(n, gap, generator), torch.full((n, 1), RECALL_TOKEN)], dim=1)
        self.targets = sig


class SelectiveCopyDataset(_PairDataset):
    """Every signal token is followed by ``distractor_ratio`` noise tokens; then the gap and the marker.

    (reference: experiments/copy_task/dataset.py:38-73)
    """

    def __init__(self, n: int, seq_len: int = 3, gap: int = 8, distractor_ratio: int = 1,
                 generator: torch.Generator | None = None):
        sig = torch.randint(0, N_SIGNAL, (n, seq_len), generator=generator)
        dis = _noise(n, seq_len * distractor_ratio, generator).view(n, seq_len, distractor_ratio)
        head = torch.cat([sig.unsqueeze(-1), dis], dim=-1).reshape(n, -1)
        self.inputs = torch.cat([head, _noise(n, gap, generator), torch.full((n, 1), RECALL_TOKEN)], dim=1)
        self.targets = sig
