"""Streaming text corpora tokenised on the fly and packed into fixed windows.

Parity with the reference's ``gdnet/data/fineweb_edu.py`` and ``gdnet/data/nemotron.py``:
Hugging Face streaming datasets, a 10k-document shuffle buffer, ``tiktoken``
``encode_ordinary`` + end-of-text per document, windows of ``seq_len + 1`` tokens with a
one-token overlap between consecutive windows. ``datasets`` and ``tiktoken`` are imported
lazily, so the rest of the package works without them (and without a network).
"""

from __future__ import annotations

from typing import Callable, Iterable, Iterator

import torch
from torch.utils.data import IterableDataset


def pack_token_stream(docs: Iterable[list[int]], seq_len: int) -> Iterator[torch.Tensor]:
    """Concatenate tokenised documents and cut windows of ``seq_len+1`` ids.

    The last id of a window is repeated as the first id of the next one, so every
    position is a target exactly once.
    """
    span = seq_len + 1
    buf: list[int] = []
    for ids in docs:
        buf.extend(ids)
        while len(buf) >= span:
            yield torch.tensor(buf[:span], dtype=torch.int64)
            del buf[:seq_len]


class _StreamingTextDataset(IterableDataset):
    text_key = "text"

    def __init__(self, seq_len: int, encoding: str = "cl100k_base", seed: int = 42,
                 shuffle_buffer: int = 10_000) -> None:
        self.seq_len, self.encoding, self.seed, self.shuffle_buffer = seq_len, encoding, seed, shuffle_buffer

    def _streams(self) -> list:
        raise NotImplementedError

    def _keep(self, row: dict) -> bool:
        return True

    def _token_docs(self):
        import tiktoken

        enc = tiktoken.get_encoding(self.encoding)
        eot = enc.eot_token
        for stream in self._streams():
            for row in stream.shuffle(seed=self.seed, buffer_size=self.shuffle_buffer):
                if self._keep(row):
                    yield enc.encode_ordinary(row[self.text_key]) + [eot]

    def __iter__(self):
        return pack_token_stream(self._token_docs(), self.seq_len)


class FineWebEduDataset(_StreamingTextDataset):
    """``HuggingFaceFW/fineweb-edu`` filtered by ``int_score`` (and ``token_count``)."""

    def __init__(self, seq_len: int, min_int_score: int = 3, max_int_score: int = 5,
                 encoding: str = "cl100k_base", subset: str = "sample-10BT", seed: int = 42,
                 min_tokens: int = 0) -> None:
        super().__init__(seq_len, encoding, seed)
        self.lo, self.hi, self.subset, self.min_tokens = min_int_score, max_int_score, subset, min_tokens

    def _streams(self):
        from datasets import load_dataset

        return [load_dataset("HuggingFaceFW/fineweb-edu", name=self.subset, split="train", streaming=True)]

    def _keep(self, row):
        score = row.get("int_score", self.lo)
        return self.lo <= score <= self.hi and row.get("token_count", self.min_tokens) >= self.min_tokens


class NemotronDataset(_StreamingTextDataset):
    """``nvidia/Nemotron-Pretraining-Specialized-v1.1``; ``subset="everything"`` chains all configs."""

    repo = "nvidia/Nemotron-Pretraining-Specialized-v1.1"

    def __init__(self, seq_len: int, encoding: str = "cl100k_base", subset: str = "everything",
                 min_chars: int = 0, seed: int = 42) -> None:
        super().__init__(seq_len, encoding, seed)
        self.subset, self.min_chars = subset, min_chars

    def _streams(self):
        from datasets import get_dataset_config_names, load_dataset

        names = get_dataset_config_names(self.repo) if self.subset == "everything" else [self.subset]
        return [load_dataset(self.repo, name=n, split="train", streaming=True) for n in names]

    def _keep(self, row):
        return len(row.get(self.text_key, "")) >= self.min_chars
