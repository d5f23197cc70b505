"""Key-value retrieval across chunks: synthetic data.

A sample is ``n_slots`` context chunks followed by one query chunk (reference:
experiments/retrieval/dataset.py). Tokens: keys 0..15, values 16..31, noise 32..47, SIGNAL 48,
QUERY 49. A signal chunk starts ``[SIGNAL, key, value]``, a query chunk ``[QUERY, key]``; everything
else is noise.

Conditions: 1 = the key is written once (first chunk); 2 = the key is written twice with different
values, ``ambiguous_k`` noise chunks apart, and the later value is the answer; 3 = the key is never
written. With ``value_in_query=True`` (the second version of the experiment, reference:
experiments/retrieval_v2/run.py:71-76,121-128) the query chunk of condition 3 also carries the value, so the
right behaviour is to answer from the local chunk and keep the memory gate shut.
"""

from __future__ import annotations

import torch
from torch.utils.data import Dataset

N_KEYS = N_VALUES = N_NOISE_VOCAB = 16
CHUNK_SIZE = 16
KEY_OFFSET, VALUE_OFFSET, NOISE_OFFSET = 0, N_KEYS, N_KEYS + N_VALUES
SIGNAL_TOKEN = NOISE_OFFSET + N_NOISE_VOCAB
QUERY_TOKEN = SIGNAL_TOKEN + 1
VOCAB_SIZE = QUERY_TOKEN + 1


class RetrievalDataset(Dataset):
    """``chunks`` (n, n_slots + 1, chunk_size) and ``targets`` (n,); target -1 = nothing to predict."""

    def __init__(self, n: int, n_slots: int, chunk_size: int = CHUNK_SIZE, condition: int = 1,
                 ambiguous_k: int = 2, seed: int = 0, value_in_query: bool = False):
        if condition not in (1, 2, 3):
            raise ValueError(f"unknown condition {condition}")
        if condition == 2 and ambiguous_k + 2 > n_slots:
            raise ValueError("ambiguous_k leaves no room for the second signal chunk")
        g = torch.Generator().manual_seed(seed)
        chunks = torch.randint(NOISE_OFFSET, NOISE_OFFSET + N_NOISE_VOCAB, (n, n_slots + 1, chunk_size), generator=g)
        key = torch.randint(0, N_KEYS, (n,), generator=g)
        val = torch.randint(0, N_VALUES, (n,), generator=g)
        target = val.clone()

        def put_signal(j, v):
            chunks[:, j, 0], chunks[:, j, 1], chunks[:, j, 2] = SIGNAL_TOKEN, KEY_OFFSET + key, VALUE_OFFSET + v

        if condition in (1, 2):
            put_signal(0, val)
        if condition == 2:
            newer = (val + torch.randint(1, N_VALUES, (n,), generator=g)) % N_VALUES      # never equal to val
            put_signal(ambiguous_k + 1, newer)
            target = newer
        chunks[:, n_slots, 0], chunks[:, n_slots, 1] = QUERY_TOKEN, KEY_OFFSET + key
        if condition == 3:
            if value_in_query:
                chunks[:, n_slots, 2] = VALUE_OFFSET + val
            else:
                target = torch.full((n,), -1)
        self.chunks, self.targets = chunks, target

    def __len__(self) -> int:
        return self.targets.shape[0]

    def __getitem__(self, i):
        return self.chunks[i], self.targets[i]
