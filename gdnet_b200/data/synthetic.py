"""Synthetic data: packed random documents and the copy task.

``synthetic_packed_batch``: uniform-random token ids packed into windows, document
lengths drawn from a geometric distribution (mean ``mean_doc_len``), documents
separated by ``EOS = 0``; also returns the document index of every position and a mask
of targets that stay inside their document. The reference has no document-boundary
handling (its packed loader yields plain windows, gdnet/data/packed.py:26-38), so the
mask is optional input to the loss.

``copy_task_batch``: ``n_copy`` tokens uniform in ``[2, vocab)``, delimiter ``1``, the same
tokens again, padded with ``0``; the loss mask selects the copied half.
"""

from __future__ import annotations

import torch
from torch.utils.data import IterableDataset

EOS = 0


def synthetic_packed_batch(batch: int, seq_len: int, vocab_size: int, mean_doc_len: float = 1024.0,
                           generator: torch.Generator | None = None, single_document: bool = False):
    """Returns ``(seq (B, T+1) int64, doc_id (B, T+1) int32, target_mask (B, T) bool)``.

    ``seq[:, :-1]`` are the inputs and ``seq[:, 1:]`` the targets. ``target_mask[b, t]`` is
    False where the target is the first token of a new document's body, i.e. where
    predicting it would need information from across a boundary.
    """
    span = seq_len + 1
    seq = torch.randint(1, vocab_size, (batch, span), generator=generator, dtype=torch.int64)
    if single_document:
        doc_id = torch.zeros(batch, span, dtype=torch.int32)
        return seq, doc_id, torch.ones(batch, seq_len, dtype=torch.bool)
    # a position ends a document with probability 1/mean: geometric lengths
    ends = torch.rand(batch, span, generator=generator) < (1.0 / mean_doc_len)
    seq = torch.where(ends, torch.full_like(seq, EOS), seq)
    doc_id = torch.cumsum(ends.to(torch.int32), dim=1) - ends.to(torch.int32)
    target_mask = doc_id[:, 1:] == doc_id[:, :-1]
    return seq, doc_id.to(torch.int32), target_mask


class SyntheticPackedDataset(IterableDataset):
    """Endless stream of synthetic packed windows ``int64[seq_len+1]``."""

    def __init__(self, seq_len: int, vocab_size: int, mean_doc_len: float = 1024.0, seed: int = 0,
                 single_document: bool = False):
        self.seq_len, self.vocab_size, self.mean_doc_len = seq_len, vocab_size, mean_doc_len
        self.seed, self.single_document = seed, single_document

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed)
        while True:
            seq, _, _ = synthetic_packed_batch(64, self.seq_len, self.vocab_size, self.mean_doc_len, g,
                                               self.single_document)
            yield from seq


def copy_task_batch(batch: int, seq_len: int = 256, n_copy: int = 64, vocab_size: int = 258,
                    generator: torch.Generator | None = None):
    """Returns ``(tokens (B,T), targets (B,T), loss_mask (B,T))`` for next-token training.

    Layout of the underlying sequence: ``x_1..x_n, 1, x_1..x_n, 0, 0, ...``. The mask is True
    where the target is one of the copied tokens.
    """
    if 2 * n_copy + 1 > seq_len + 1:
        raise ValueError("sequence too short for the copy task")
    payload = torch.randint(2, vocab_size, (batch, n_copy), generator=generator, dtype=torch.int64)
    full = torch.zeros(batch, seq_len + 1, dtype=torch.int64)
    full[:, :n_copy] = payload
    full[:, n_copy] = 1
    full[:, n_copy + 1 : 2 * n_copy + 1] = payload
    tokens, targets = full[:, :-1].contiguous(), full[:, 1:].contiguous()
    mask = torch.zeros(batch, seq_len, dtype=torch.bool)
    mask[:, n_copy : 2 * n_copy] = True       # target index t holds full[t+1]
    return tokens, targets, mask


class CopyTaskDataset(IterableDataset):
    def __init__(self, seq_len: int = 256, n_copy: int = 64, vocab_size: int = 258, seed: int = 0):
        self.seq_len, self.n_copy, self.vocab_size, self.seed = seq_len, n_copy, vocab_size, seed

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed)
        while True:
            tok, tgt, m = copy_task_batch(32, self.seq_len, self.n_copy, self.vocab_size, g)
            for i in range(tok.shape[0]):
                yield tok[i], tgt[i], m[i]
