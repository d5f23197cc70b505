"""Weighted infinite mixture of iterable datasets.

Parity with the reference's ``gdnet/data/mixed.py``: each draw picks a source with
probability proportional to its weight (seeded ``random.Random``), an exhausted source
restarts.
"""

from __future__ import annotations

import random

from torch.utils.data import IterableDataset


class MixedDataset(IterableDataset):
    def __init__(self, datasets, weights, seed: int = 42) -> None:
        if not datasets or len(datasets) != len(weights):
            raise ValueError("need as many weights as datasets, and at least one")
        total = float(sum(weights))
        self._sources = list(datasets)
        self._probs = [w / total for w in weights]
        self._seed = seed

    def __iter__(self):
        rng = random.Random(self._seed)
        its = [iter(s) for s in self._sources]
        ids = list(range(len(its)))
        while True:
            (j,) = rng.choices(ids, weights=self._probs)
            item = next(its[j], None)
            if item is None:
                its[j] = iter(self._sources[j])
                item = next(its[j])
            yield item
